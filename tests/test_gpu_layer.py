"""GPU parity of the whole fused-MoE layer through ``XpuFusedMoe.apply``:
reference-made golden vectors, scaled-down versions of the five benchmark
shapes against the CPU oracle, expert-parallel masks, and size-independent
properties at the full Mixtral shape."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV, topk_softmax
from oracle import torch_oracle as to
from oracle import workloads as wl

pytestmark = pytest.mark.gpu

TOL = {"bf16": 2e-2, "fp8block": 5e-2, "mxfp4": 1e-1}


def _run_layer(native, cfg, w, x, tw, ids, E_local=None, ep_rank=0, ep_size=1, fuse=False, clamp=None,
               mx=None):
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(w13), mv(s13), mv(w["w13_bias"]), mv(w2), mv(s2), mv(w["w2_bias"]),
                               cfg.K, cfg.activation, E_local or cfg.E, ep_rank=ep_rank, ep_size=ep_size,
                               gemm1_clamp_limit=clamp, fuse_activation=fuse, mxfp4_activations=mx)
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=DEV)
    layer.apply(out, x.to(DEV), tw.to(DEV), ids.to(DEV))
    return out.cpu()


def test_layer_reference_vectors_bf16(native):
    """tests/fused_moe/test_fused_moe.py of the reference: weights handed over as
    the [E,K,N] transposes, tolerance 2e-2."""
    for c in load_golden("layer_bf16.pt"):
        ep_rank, ep_size = c.get("ep_rank", 0), c.get("ep_size", 1)
        E_local = c["num_experts"]
        lo = ep_rank * E_local
        w13 = c["w13"][lo:lo + E_local].transpose(-1, -2).contiguous().to(DEV)
        w2 = c["w2"][lo:lo + E_local].transpose(-1, -2).contiguous().to(DEV)
        b13 = c["w13_bias"][lo:lo + E_local].to(DEV) if c["w13_bias"] is not None else None
        b2 = c["w2_bias"][lo:lo + E_local].to(DEV) if c["w2_bias"] is not None else None
        K = c["topk_ids"].shape[1]
        layer = native.XpuFusedMoe(w13, None, b13, w2, None, b2, K, "silu", E_local, ep_rank=ep_rank,
                                   ep_size=ep_size, gemm1_clamp_limit=c["clamp"])
        out = torch.empty_like(c["output"], device=DEV)
        layer.apply(out, c["x"].to(DEV), c["topk_weights"].to(DEV), c["topk_ids"].to(DEV))
        torch.testing.assert_close(out.cpu(), c["output"], rtol=2e-2, atol=2e-2)


def _mxfp8_layer(native, c, mode=None, dev_dtype=None):
    E = c["num_experts"]
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(c["w13"].view(torch.float8_e4m3fn)), mv(c["w13_scales"]), mv(c["w13_bias"]),
                               mv(c["w2"].view(torch.float8_e4m3fn)), mv(c["w2_scales"]), mv(c["w2_bias"]),
                               c["topk_ids"].shape[1], "silu", E, mxfp4_activations=mode)
    out = torch.empty_like(c["x"], device=DEV)
    layer.apply(out, c["x"].to(DEV), c["topk_weights"].to(DEV), c["topk_ids"].to(DEV))
    return layer, out.cpu()


def test_layer_mxfp8_reference_vectors_and_oracle(native):
    """mxfp8 weights: against the outputs of the reference's own eager simulation (its only
    implementation of this recipe, vllm_xpu_kernels/fused_moe_interface.py:27-31) and against
    the staged oracle, which differs from the kernels in summation order only."""
    for c in load_golden("layer_mxfp8.pt"):
        layer, out = _mxfp8_layer(native, c)
        assert layer.recipe == "mxfp8" and layer.mx_acts and layer.mx_planes == 1
        top = float(c["out"].float().abs().max())
        torch.testing.assert_close(out.float(), c["out"].float(), rtol=2e-2, atol=4e-2 * top)
        E = c["num_experts"]
        w13, w2 = c["w13"].view(torch.float8_e4m3fn), c["w2"].view(torch.float8_e4m3fn)
        w13d = torch.stack([to.dequant_mxfp8_wei(w13[e], c["w13_scales"][e]).t() for e in range(E)])
        w2d = torch.stack([to.dequant_mxfp8_wei(w2[e], c["w2_scales"][e]).t() for e in range(E)])
        for mode in ("mxfp8", "mxfp8x2", "bf16"):
            _, o = _mxfp8_layer(native, c, mode)
            ref = to.fused_moe_staged(c["x"], w13d, c["w13_bias"], w2d, c["w2_bias"], c["topk_weights"], c["topk_ids"],
                                      E, activation="silu", act_quant=False if mode == "bf16" else mode)
            torch.testing.assert_close(o.float(), ref.float(), rtol=2e-2, atol=2e-2 * top)


@pytest.mark.parametrize("name,dims", [("cfg2_mixtral_bf16", dict(H=512, I=256, E=4)),
                                       ("cfg4_deepseek_fp8", dict(H=512, I=256, E=8))])
@pytest.mark.parametrize("src,rows_per_seg", [(3, 5), (2, 70)])
def test_layer_apply_sorted_segments(native, name, dims, src, rows_per_seg):
    """apply_sorted: rows already grouped into src * E segments (source-major, expert-minor, the
    arrival order of an expert-parallel exchange); every row gets its expert's MLP, no
    permutation, no reduction.  Against the oracle run as a top-1 layer with unit weights."""
    cfg = wl.scaled(wl.CONFIGS[name], **dims)
    E = cfg.E
    w = wl.make_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(src * 100 + rows_per_seg)
    seg = torch.randint(0, 2 * rows_per_seg, (src * E,), generator=g, dtype=torch.int32)
    seg[1] = 0                                                   # an empty segment
    M = int(seg.sum())
    x = (torch.randn(M, cfg.H, generator=g) / 2).to(torch.bfloat16)
    ids = torch.repeat_interleave(torch.arange(src * E) % E, seg.long()).view(M, 1).int()
    d13, d2 = wl.dequant_weights(cfg, w)
    quant = cfg.recipe == "fp8block"
    ref = to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], torch.ones(M, 1), ids, E,
                              activation=cfg.activation, act_quant=quant)
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(w13), mv(s13), mv(w["w13_bias"]), mv(w2), mv(s2), mv(w["w2_bias"]), 1,
                               cfg.activation, E)
    out = torch.full((M, cfg.H), float("nan"), dtype=torch.bfloat16, device=DEV)
    if quant:
        q, sc = to.per_token_group_fp8_quant(x, 128, 1e-10)
        layer.apply_sorted(out, q.to(DEV), seg.to(DEV), a1q_scale=sc.to(DEV))
    else:
        layer.apply_sorted(out, x.to(DEV), seg.to(DEV))
    tol = TOL[cfg.recipe]
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=tol, atol=tol)


SMALL = [
    ("cfg1_small_bf16", dict(H=2048, I=1408, E=8), 64),     # the CPU-runnable config at full size
    ("cfg2_mixtral_bf16", dict(H=512, I=1792, E=8), 33),
    ("cfg3_qwen3_fp8", dict(H=512, I=256, E=128), 40),
    ("cfg4_deepseek_fp8", dict(H=896, I=256, E=256), 24),
    ("cfg5_gptoss_mxfp4", dict(H=576, I=576, E=32), 20),
]


@pytest.mark.parametrize("name,dims,T", SMALL)
def test_layer_against_oracle(native, name, dims, T):
    cfg = wl.scaled(wl.CONFIGS[name], **dims)
    w = wl.make_weights(cfg, seed=0)
    x, logits, bias = wl.make_inputs(cfg, T, seed=0)
    tw, ids = wl.route_cpu(cfg, logits, bias)
    d13, d2 = wl.dequant_weights(cfg, w)
    ref = to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E,
                              activation=cfg.activation, act_quant=cfg.recipe == "fp8block")
    out = _run_layer(native, cfg, w, x, tw, ids)
    tol = TOL[cfg.recipe]
    torch.testing.assert_close(out.float(), ref.float(), rtol=tol, atol=tol)
    if cfg.recipe == "bf16":
        # also against the reference's own whole-layer statement
        ref2 = to.fused_moe_bf16(x, w["w13"], None, w["w2"], None, tw, ids, cfg.E)
        torch.testing.assert_close(out.float(), ref2.float(), rtol=2e-2, atol=2e-2)
    # the fused-activation path computes the same layer
    out_f = _run_layer(native, cfg, w, x, tw, ids, fuse=True)
    torch.testing.assert_close(out_f.float(), ref.float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("T", [1, 20, 300])
def test_layer_mxfp4_activation_modes(native, T):
    """MXFP4 weights: the 16-bit-activation path (the reference's w4a16) and the
    two-plane block-scaled path against the w4a16 oracle at the bf16 tolerance
    (absolute part relative to the largest output);
    the one-plane path against an oracle that quantises the activations the
    same way, and against the w4a16 oracle at the MXFP4 tolerance relative to
    the largest output."""
    cfg = wl.scaled(wl.CONFIGS["cfg5_gptoss_mxfp4"], H=576, I=704, E=16)
    w = wl.make_weights(cfg, seed=3)
    x, logits, bias = wl.make_inputs(cfg, T, seed=3)
    tw, ids = wl.route_cpu(cfg, logits, bias)
    d13, d2 = wl.dequant_weights(cfg, w)
    ref16 = to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E, activation=cfg.activation)
    ref_mx = to.fused_moe_staged(x, d13, w["w13_bias"], d2, w["w2_bias"], tw, ids, cfg.E,
                                 activation=cfg.activation, act_quant="mxfp8")
    scale = float(ref16.float().abs().max())
    for fuse in (False, True):
        o16 = _run_layer(native, cfg, w, x, tw, ids, fuse=fuse, mx="bf16")
        torch.testing.assert_close(o16.float(), ref16.float(), rtol=2e-2, atol=2e-2 * max(1.0, scale))
        ox2 = _run_layer(native, cfg, w, x, tw, ids, fuse=fuse, mx="mxfp8x2")
        torch.testing.assert_close(ox2.float(), ref16.float(), rtol=2e-2, atol=2e-2 * max(1.0, scale))
        omx = _run_layer(native, cfg, w, x, tw, ids, fuse=fuse, mx="mxfp8")
        torch.testing.assert_close(omx.float(), ref_mx.float(), rtol=3e-2, atol=3e-2 * max(1.0, scale))
        torch.testing.assert_close(omx.float(), ref16.float(), rtol=1e-1, atol=1e-1 * scale)


@pytest.mark.parametrize("w_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("mode", ["mxfp8x2", "bf16"])
def test_layer_per_tensor_fp8(native, w_dtype, dtype, has_bias, mode):
    """tests/fused_moe/test_fused_moe.py:179-296 of the reference: per-tensor fp8 weights
    (e4m3 / e5m2) with power-of-two expert scales, weights handed over as [E,K,N],
    tolerance 2e-2 (bf16) / 1e-2 (fp16); on the block-scaled tensor-core path
    (default) and on the 16-bit-activation path."""
    T, H, I, E, K = 48, 256, 192, 8, 2
    g = torch.Generator().manual_seed(7)
    a = (torch.randn(T, H, generator=g) / 16).to(dtype)
    w13 = (torch.randn(E, 2 * I, H, generator=g) / 16).to(dtype)
    w2 = (torch.randn(E, H, I, generator=g) / 16).to(dtype)
    b13 = (torch.randn(E, 2 * I, generator=g) / 16).to(dtype) if has_bias else None
    b2 = (torch.randn(E, H, generator=g) / 16).to(dtype) if has_bias else None
    s13 = torch.exp2(torch.randint(-3, 4, (E,), generator=g).float())
    s2 = torch.exp2(torch.randint(-3, 4, (E,), generator=g).float())
    q13 = (w13.float() / s13.view(E, 1, 1)).to(w_dtype)
    q2 = (w2.float() / s2.view(E, 1, 1)).to(w_dtype)
    ref13 = (q13.to(dtype) * s13.view(E, 1, 1).to(dtype))
    ref2 = (q2.to(dtype) * s2.view(E, 1, 1).to(dtype))
    tw, ids = torch.topk(torch.randn(T, E, generator=g), k=K, dim=-1, sorted=False)
    ref = to.fused_moe_bf16(a, ref13, b13, ref2, b2, tw, ids.int(), E)
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(q13.transpose(-1, -2).contiguous()), mv(s13), mv(b13),
                               mv(q2.transpose(-1, -2).contiguous()), mv(s2), mv(b2), K, "silu", E,
                               mxfp4_activations=mode)
    assert layer.mx_acts == (mode != "bf16")
    out = torch.empty_like(a, device=DEV)
    layer.apply(out, a.to(DEV), tw.to(DEV), ids.int().to(DEV))
    tol = 1e-2 if dtype == torch.float16 else 2e-2
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layer_int4(native, has_bias, dtype):
    """tests/fused_moe/test_fused_moe.py:299-410 of the reference: uint4 weights [E,N,K/2]
    with zero point 8 and power-of-two group scales (group 128), handed over as uint8."""
    T, H, I, E, K, group = 40, 256, 128, 8, 2, 128
    g = torch.Generator().manual_seed(7)
    a = (torch.randn(T, H, generator=g) / 16).to(dtype)
    w13 = torch.randint(0, 255, (E, 2 * I, H // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    w2 = torch.randint(0, 255, (E, H, I // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    s13 = torch.exp2(torch.randint(-5, -4, (E, 2 * I, H // group), generator=g).float()).to(dtype)
    s2 = torch.exp2(torch.randint(-5, -4, (E, H, I // group), generator=g).float()).to(dtype)
    b13 = (torch.randn(E, 2 * I, generator=g) / 16).to(dtype) if has_bias else None
    b2 = (torch.randn(E, H, generator=g) / 16).to(dtype) if has_bias else None
    tw, ids = torch.topk(torch.randn(T, E, generator=g), k=K, dim=-1, sorted=False)
    ref = to.fused_moe_bf16(a, to.dequant_int4(w13, s13, group), b13, to.dequant_int4(w2, s2, group), b2, tw,
                            ids.int(), E)
    mv = lambda t: t.to(DEV) if t is not None else None
    w13_dev = mv(w13)
    layer = native.XpuFusedMoe(w13_dev, mv(s13), mv(b13), mv(w2), mv(s2), mv(b2), K, "silu", E)
    assert layer.is_int4 and torch.equal(w13_dev.cpu(), w13)        # caller's weights untouched
    out = torch.empty_like(a, device=DEV)
    layer.apply(out, a.to(DEV), tw.to(DEV), ids.int().to(DEV))
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_layer_expert_parallel_masks_sum_to_the_full_layer(native):
    """ep_size ranks, each holding E/ep experts and masking the others
    (tests/fused_moe/test_fused_moe.py:531-657): the partial outputs add up."""
    cfg = wl.scaled(wl.CONFIGS["cfg1_small_bf16"], H=256, I=128, E=8)
    w = wl.make_weights(cfg, seed=1)
    x, logits, _ = wl.make_inputs(cfg, 19, seed=1)
    tw, ids = wl.route_cpu(cfg, logits, None)
    full = _run_layer(native, cfg, w, x, tw, ids).float()
    acc = torch.zeros_like(full)
    for rank in range(4):
        sl = slice(rank * 2, rank * 2 + 2)
        wr = {k: (v[sl] if v is not None else None) for k, v in w.items()}
        part = _run_layer(native, cfg, wr, x, tw, ids, E_local=2, ep_rank=rank, ep_size=4)
        ref = to.fused_moe_bf16(x, w["w13"], None, w["w2"], None, tw, ids, 2, ep_rank=rank, ep_size=4)
        torch.testing.assert_close(part.float(), ref.float(), rtol=2e-2, atol=2e-2)
        acc += part.float()
    torch.testing.assert_close(acc, full, rtol=3e-2, atol=3e-2)


def test_layer_clamp_limit(native):
    cfg = wl.scaled(wl.CONFIGS["cfg1_small_bf16"], H=256, I=128, E=4)
    w = wl.make_weights(cfg, seed=2)
    x, logits, _ = wl.make_inputs(cfg, 16, seed=2)
    tw, ids = wl.route_cpu(cfg, logits, None)
    ref = to.fused_moe_bf16(x, w["w13"], None, w["w2"], None, tw, ids, cfg.E, gemm1_clamp_limit=0.3)
    for fuse in (False, True):
        out = _run_layer(native, cfg, w, x, tw, ids, clamp=0.3, fuse=fuse)
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_full_size_mixtral_properties(native):
    """At the benchmark's full Mixtral shape (H=4096, I=14336, E=8, top-2) the CPU
    oracle is out of reach, so check properties that hold at any size:
    permuting the tokens permutes the outputs bit for bit, zero routing weights
    give zeros, and the tensor-core GEMM agrees with the checking kernel."""
    H, I, E, K, T = 4096, 14336, 8, 2, 96
    g = torch.Generator(device=DEV).manual_seed(0)
    w13 = (torch.randn(E, H, 2 * I, generator=g, device=DEV, dtype=torch.float32) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, I, H, generator=g, device=DEV, dtype=torch.float32) * I ** -0.5).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=DEV)
    tw, ids, _ = topk_softmax(logits, K, True)
    layer = native.XpuFusedMoe(w13, None, None, w2, None, None, K, "silu", E)
    out = torch.empty_like(x)
    layer.apply(out, x, tw, ids)
    assert bool(torch.isfinite(out.float()).all()) and float(out.float().abs().mean()) > 1e-3
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(3)).to(DEV)
    out_p = torch.empty_like(x)
    layer.apply(out_p, x[perm].contiguous(), tw[perm].contiguous(), ids[perm].contiguous())
    assert torch.equal(out_p, out[perm])
    out_z = torch.empty_like(x)
    layer.apply(out_z, x, torch.zeros_like(tw), ids)
    assert float(out_z.float().abs().max()) == 0.0
    # a slice of gemm1 against the checking kernel
    rows = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    a = torch.randn(T * K, H, generator=g, device=DEV).to(torch.bfloat16)
    d1 = torch.empty(T * K, 2 * I, dtype=torch.bfloat16, device=DEV)
    d2 = torch.empty_like(d1)
    torch.ops._xpu_C.b200_grouped_gemm(a, None, w13, None, None, d1, rows, 2 * I, H, E, 2, 0, 1.702, 7.0, 0.0, 1, 0)
    torch.ops._xpu_C.b200_grouped_gemm(a, None, w13, None, None, d2, rows, 2 * I, H, E, 2, 0, 1.702, 7.0, 0.0, 2, 0)
    torch.testing.assert_close(d1.float(), d2.float(), rtol=1e-2, atol=1e-2)


def test_functional_entry_point_matches_the_oracle(native):
    """`xpu_fused_moe` (vllm_xpu_kernels/fused_moe_interface.py:421-619 of the reference): one call,
    recipe read off the weights, output allocated when not given."""
    for name, dims, T in (("cfg1_small_bf16", dict(H=512, I=256, E=8), 37),
                          ("cfg3_qwen3_fp8", dict(H=512, I=256, E=32), 29)):
        cfg = wl.scaled(wl.CONFIGS[name], **dims)
        w = wl.make_weights(cfg, seed=4)
        x, logits, bias = wl.make_inputs(cfg, T, seed=4)
        tw, ids = wl.route_cpu(cfg, logits, bias)
        d13, d2 = wl.dequant_weights(cfg, w)
        ref = to.fused_moe_staged(x, d13, None, d2, None, tw, ids, cfg.E, activation=cfg.activation,
                                  act_quant=cfg.recipe == "fp8block")
        w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
        mv = lambda t: t.to(DEV) if t is not None else None
        out = native.xpu_fused_moe(x.to(DEV), mv(w13), mv(s13), None, mv(w2), mv(s2), None, tw.to(DEV), ids.to(DEV),
                                   cfg.K, cfg.activation, cfg.E, is_block_fp8=cfg.recipe == "fp8block")
        assert out.shape == x.shape and out.dtype == x.dtype
        tol = TOL[cfg.recipe]
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=tol, atol=tol)
        given = torch.empty_like(x, device=DEV)
        back = native.xpu_fused_moe(x.to(DEV), mv(w13), mv(s13), None, mv(w2), mv(s2), None, tw.to(DEV),
                                    ids.to(DEV), cfg.K, cfg.activation, cfg.E, output=given)
        assert back is given and torch.equal(given, out)


def test_functional_entry_point_int4_converts_the_weights_once(native):
    T, H, I, E, K, group = 24, 256, 128, 4, 2, 128
    g = torch.Generator().manual_seed(9)
    a = (torch.randn(T, H, generator=g) / 16).to(torch.bfloat16)
    w13 = torch.randint(0, 255, (E, 2 * I, H // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    w2 = torch.randint(0, 255, (E, H, I // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    s13 = torch.exp2(torch.randint(-5, -4, (E, 2 * I, H // group), generator=g).float()).to(torch.bfloat16)
    s2 = torch.exp2(torch.randint(-5, -4, (E, H, I // group), generator=g).float()).to(torch.bfloat16)
    tw, ids = torch.topk(torch.randn(T, E, generator=g), k=K, dim=-1, sorted=False)
    ref = to.fused_moe_bf16(a, to.dequant_int4(w13, s13, group), None, to.dequant_int4(w2, s2, group), None, tw,
                            ids.int(), E)
    w13d, w2d = w13.to(DEV), w2.to(DEV)
    args = (a.to(DEV), w13d, s13.to(DEV), None, w2d, s2.to(DEV), None, tw.to(DEV), ids.int().to(DEV), K, "silu", E)
    out1 = native.xpu_fused_moe(*args, is_int4=True)
    conv = w13d._b200_signed_nibbles[1]
    out2 = native.xpu_fused_moe(*args, is_int4=True)
    assert w13d._b200_signed_nibbles[1] is conv, "the second call must reuse the converted weights"
    assert torch.equal(w13d.cpu(), w13), "the caller's weights stay as they were"
    torch.testing.assert_close(out1.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(out1, out2)


def test_layer_takes_prequantised_fp8_hidden_states(native):
    """`apply(..., a1q_scale=...)` with e4m3 hidden_states and their 1x128 scales
    (vllm_xpu_kernels/fused_moe_interface.py:273-281, 356-366 of the reference): the rows and
    scales are permuted as they are, so the result equals the layer quantising the 16-bit input
    itself, bit for bit."""
    cfg = wl.scaled(wl.CONFIGS["cfg3_qwen3_fp8"], H=512, I=256, E=32)
    w = wl.make_weights(cfg, seed=6)
    x, logits, bias = wl.make_inputs(cfg, 45, seed=6)
    tw, ids = wl.route_cpu(cfg, logits, bias)
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(w13), mv(s13), None, mv(w2), mv(s2), None, cfg.K, cfg.activation, cfg.E)
    out16 = torch.empty(x.shape, dtype=torch.bfloat16, device=DEV)
    layer.apply(out16, x.to(DEV), tw.to(DEV), ids.to(DEV))
    q, sc = to.per_token_group_fp8_quant(x, 128, 1e-10)
    outq = torch.full_like(out16, float("nan"))
    layer.apply(outq, q.to(DEV), tw.to(DEV), ids.to(DEV), a1q_scale=sc.to(DEV))
    assert torch.equal(outq, out16)
    d13, d2 = wl.dequant_weights(cfg, w)
    ref = to.fused_moe_staged(x, d13, None, d2, None, tw, ids, cfg.E, activation=cfg.activation, act_quant=True)
    torch.testing.assert_close(outq.cpu().float(), ref.float(), rtol=5e-2, atol=5e-2)


def test_prequantised_hidden_states_are_refused_for_other_recipes(native):
    cfg = wl.scaled(wl.CONFIGS["cfg5_gptoss_mxfp4"], H=576, I=576, E=8)
    w = wl.make_weights(cfg, seed=1)
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(w13), mv(s13), mv(w["w13_bias"]), mv(w2), mv(s2), mv(w["w2_bias"]), cfg.K,
                               cfg.activation, cfg.E)
    q = torch.zeros(4, cfg.H, dtype=torch.float8_e4m3fn, device=DEV)
    sc = torch.zeros(4, cfg.H // 32, dtype=torch.uint8, device=DEV)
    out = torch.empty(4, cfg.H, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(NotImplementedError, match="block-scaled fp8 weights only"):
        layer.apply(out, q, torch.zeros(4, cfg.K, device=DEV), torch.zeros(4, cfg.K, dtype=torch.int32, device=DEV),
                    a1q_scale=sc)


def test_a_bounded_wait_that_runs_out_reaches_the_caller(native):
    """The failure path of the tensor-core kernels, made on purpose without faulting anything: a
    small kernel waits with the kernels' own bounded wait, and a budget of about a millisecond,
    on an mbarrier that nobody arrives at; it gives up, returns and sets the device's status
    word.  The next status check - and the next grouped-GEMM call - raise, and clear it."""
    anchor = torch.zeros(1, device=DEV)
    X = torch.ops._xpu_C
    assert X.b200_check_status(anchor, True) == 0
    X.b200_selftest_bounded_wait(anchor, 2_000_000)
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        X.b200_check_status(anchor, True)
    assert X.b200_check_status(anchor, True) == 0          # cleared by the raise
    # the same through the op a layer calls
    X.b200_selftest_bounded_wait(anchor, 2_000_000)
    torch.cuda.synchronize()
    E, M, N, K = 2, 32, 128, 128
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    wt = torch.randn(E, K, N, device=DEV).to(torch.bfloat16)
    d = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    rows = torch.tensor([20, 12], dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="device-side wait timed out"):
        X.cutlass_grouped_gemm_interface(a, None, wt, None, None, d, rows, N, K, E)
    X.cutlass_grouped_gemm_interface(a, None, wt, None, None, d, rows, N, K, E)   # the context is intact
    torch.cuda.synchronize()
    ref = torch.cat([a[:20].float() @ wt[0].float(), a[20:].float() @ wt[1].float()])
    torch.testing.assert_close(d.float(), ref, rtol=2e-2, atol=2e-2)
    assert X.b200_check_status(anchor, True) == 0


@pytest.mark.parametrize("T", [40, 700])
def test_fp8_layer_fused_and_unfused_activation_agree_bit_for_bit(native, T):
    """Block-scaled fp8 layer: gemm1's epilogue can apply SiLU and the 1x128 quantisation (one kernel
    less, no [T*K, 2I] round trip; the default for many rows per expert, forced here) or the
    two-kernel form runs (fuse_activation=False, and below 12 rows per expert).  Same values either way."""
    cfg = wl.scaled(wl.CONFIGS["cfg3_qwen3_fp8"], H=512, I=384, E=16)
    w = wl.make_weights(cfg, seed=8)
    x, logits, bias = wl.make_inputs(cfg, T, seed=8)
    tw, ids = wl.route_cpu(cfg, logits, bias)
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    mv = lambda t: t.to(DEV) if t is not None else None
    outs = []
    for fuse in (True, False):
        layer = native.XpuFusedMoe(mv(w13), mv(s13), None, mv(w2), mv(s2), None, cfg.K, cfg.activation, cfg.E,
                                   fuse_activation=fuse, gemm1_clamp_limit=0.8)
        marks = []
        layer.stage_hook = marks.append
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=DEV)
        layer.apply(out, x.to(DEV), tw.to(DEV), ids.to(DEV))
        outs.append(out)
        assert "gemm1" in marks
    assert torch.equal(outs[0], outs[1])
    d13, d2 = wl.dequant_weights(cfg, w)
    ref = to.fused_moe_staged(x, d13, None, d2, None, tw, ids, cfg.E, activation=cfg.activation, act_quant=True,
                              gemm1_clamp_limit=0.8)
    torch.testing.assert_close(outs[0].cpu().float(), ref.float(), rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("name,dims,T", [("cfg3_qwen3_fp8", dict(H=512, I=256, E=32), 24),
                                         ("cfg5_gptoss_mxfp4", dict(H=576, I=576, E=16), 9)])
def test_layer_call_replays_from_a_cuda_graph(native, name, dims, T):
    """After one warm-up call the layer allocates nothing, reads nothing back and picks no
    launch parameter from device data, so a call can be captured in a CUDA graph (how serving
    engines run decode steps) and replayed on new inputs."""
    cfg = wl.scaled(wl.CONFIGS[name], **dims)
    w = wl.make_weights(cfg, seed=2)
    w13, s13, w2, s2 = wl.to_op_layout(cfg, w)
    mv = lambda t: t.to(DEV) if t is not None else None
    layer = native.XpuFusedMoe(mv(w13), mv(s13), mv(w["w13_bias"]), mv(w2), mv(s2), mv(w["w2_bias"]), cfg.K,
                               cfg.activation, cfg.E)
    ins = []
    for seed in (1, 2):
        x, logits, bias = wl.make_inputs(cfg, T, seed=seed)
        tw, ids = wl.route_cpu(cfg, logits, bias)
        ins.append((x.to(DEV), tw.to(DEV), ids.to(DEV)))
    eager = []
    for x, tw, ids in ins:
        out = torch.empty(T, cfg.H, dtype=torch.bfloat16, device=DEV)
        layer.apply(out, x, tw, ids)
        eager.append(out.clone())
    sx, stw, sids = (t.clone() for t in ins[0])
    sout = torch.empty(T, cfg.H, dtype=torch.bfloat16, device=DEV)
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.apply(sout, sx, stw, sids)
        with torch.cuda.graph(g, stream=side):
            layer.apply(sout, sx, stw, sids)
    torch.cuda.current_stream().wait_stream(side)
    for (x, tw, ids), ref in zip(ins, eager):
        sx.copy_(x); stw.copy_(tw); sids.copy_(ids)
        sout.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(sout, ref)
