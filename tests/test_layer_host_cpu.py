"""CPU: host-side decisions of the layer object (no kernel runs: the object is built around CPU
tensors and only asked which form a call of a given size would take)."""
import pytest
import torch

from oracle import workloads as wl


def _layer(native, cfg_name, dims, **kw):
    import vllm_xpu_kernels.fused_moe_interface as fmi
    cfg = wl.scaled(wl.CONFIGS[cfg_name], **dims)
    w = wl.make_weights(cfg, seed=0)
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    return cfg, fmi.XpuFusedMoe(w13, s13, w["w13_bias"], w2, s2, w["w2_bias"], cfg.K, cfg.activation, cfg.E, **kw)


def test_which_calls_fuse_the_activation_into_gemm1(native):
    rows = lambda layer, per_expert: layer.fuses_activation(per_expert * layer.num_experts)
    # 16-bit, SiLU, whole 128-feature tiles: fused at every size (one CTA up to 128-token tiles, a CTA pair beyond)
    _, bf16 = _layer(native, "cfg1_small_bf16", dict(H=256, I=256, E=4))
    assert [rows(bf16, r) for r in (1, 96, 97, 5000)] == ["epilogue"] * 4
    # ... other intermediate sizes: only where 128-token tiles are picked anyway
    _, odd = _layer(native, "cfg1_small_bf16", dict(H=256, I=208, E=4))
    assert [rows(odd, r) for r in (1, 96, 97, 5000)] == ["epilogue", "epilogue", None, None]
    _, off = _layer(native, "cfg1_small_bf16", dict(H=256, I=256, E=4), fuse_activation=False)
    assert rows(off, 8) is None
    # block-scaled fp8, SiLU: activation and 1x128 quantisation in the epilogue from 512 rows per expert
    _, fp8 = _layer(native, "cfg4_deepseek_fp8", dict(H=256, I=256, E=8))
    assert [rows(fp8, r) for r in (1, 511, 512, 4096)] == [None, None, "fp8", "fp8"]
    _, forced = _layer(native, "cfg4_deepseek_fp8", dict(H=256, I=256, E=8), fuse_activation=True)
    assert [rows(forced, r) for r in (11, 12)] == [None, "fp8"]
    # a hint about the rows actually in use (expert parallelism: buffers sized for the worst case) decides
    fp8.rows_hint = 512 * fp8.num_experts
    assert fp8.fuses_activation(100 * 512 * fp8.num_experts) == "fp8" and rows(fp8, 1) == "fp8"
    # MXFP4 with SwigluOAI: always in the epilogue
    _, mx = _layer(native, "cfg5_gptoss_mxfp4", dict(H=256, I=256, E=4))
    assert [rows(mx, r) for r in (1, 4096)] == ["epilogue"] * 2


def test_recipes_that_cannot_take_prequantised_inputs_say_so(native):
    _, bf16 = _layer(native, "cfg1_small_bf16", dict(H=256, I=256, E=4))
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        bf16.apply(torch.empty_like(x), x, torch.ones(2, 2), torch.zeros(2, 2, dtype=torch.int32),
                   a1q_scale=torch.ones(2, 2))
