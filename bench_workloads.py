"""The five benchmark layers: shapes, seeded synthetic inputs and on-device weights.

Shapes, dtypes and value distributions are the ones the benchmark configurations state
(a small CPU-runnable layer and Mixtral-8x7B-, Qwen3-30B-A3B-, DeepSeek-V3- and
gpt-oss-120b-shaped ones); the numbers are synthetic stand-ins - no dataset or checkpoint
is involved, as in the reference's own benchmarks, which draw ``torch.randn``
(benchmark/benchmark_cutlass_fused_moe.py of vllm-xpu-kernels).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

import torch


@dataclass
class MoeConfig:
    name: str
    H: int
    I: int
    E: int
    K: int
    recipe: str            # "bf16" | "fp8block" | "mxfp4"
    routing: str           # "softmax" | "grouped_sigmoid"
    activation: str = "silu"
    renormalize: bool = True
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    logit_offset_std: float = 0.0
    has_bias: bool = False
    tokens: tuple = field(default_factory=tuple)


CONFIGS = {
    "cfg1_small_bf16": MoeConfig("cfg1_small_bf16", 2048, 1408, 8, 2, "bf16", "softmax", tokens=(64,)),
    "cfg2_mixtral_bf16": MoeConfig("cfg2_mixtral_bf16", 4096, 14336, 8, 2, "bf16", "softmax",
                                   logit_offset_std=0.5, tokens=(1, 32, 512, 4096)),
    "cfg3_qwen3_fp8": MoeConfig("cfg3_qwen3_fp8", 2048, 768, 128, 8, "fp8block", "softmax",
                                tokens=(16, 256, 4096, 16384)),
    "cfg4_deepseek_fp8": MoeConfig("cfg4_deepseek_fp8", 7168, 2048, 256, 8, "fp8block",
                                   "grouped_sigmoid", n_group=8, topk_group=4,
                                   routed_scaling_factor=2.5, tokens=(64, 1024, 8192)),
    "cfg5_gptoss_mxfp4": MoeConfig("cfg5_gptoss_mxfp4", 2880, 2880, 128, 4, "mxfp4", "softmax",
                                   activation="swigluoai", has_bias=True, tokens=(1, 128, 2048)),
}


def scaled(cfg: MoeConfig, H=None, I=None, E=None) -> MoeConfig:
    """A smaller layer of the same kind."""
    return dataclasses.replace(cfg, H=H or cfg.H, I=I or cfg.I, E=E or cfg.E)


def make_inputs(cfg: MoeConfig, T: int, seed: int = 0):
    """-> x bf16 [T,H], router logits fp32 [T,E], routing bias fp32 [E] or None (CPU, seeded)."""
    gen = torch.Generator().manual_seed(seed * 1000 + 2)
    x = torch.randn((T, cfg.H), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn((T, cfg.E), generator=gen, dtype=torch.float32)
    if cfg.logit_offset_std > 0:
        logits = logits + (torch.randn((cfg.E,), generator=gen, dtype=torch.float32)
                           * cfg.logit_offset_std).unsqueeze(0)
    bias = None
    if cfg.routing == "grouped_sigmoid":
        bias = torch.randn((cfg.E,), generator=gen, dtype=torch.float32) * 0.1
    return x, logits, bias


def quant_fp8_block(w):
    """[N,K] float -> (e4m3 [N,K], fp32 scales [N/128,K/128] = block amax / 448)."""
    N, K = w.shape
    x = w.float().view(N // 128, 128, K // 128, 128)
    s = x.abs().amax(dim=(1, 3), keepdim=True).clamp(min=1e-12) / 448.0
    q = (x / s).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(N, K), s.reshape(N // 128, K // 128)


def make_device_weights(cfg: MoeConfig, num_experts: int, device, seed: int = 1234):
    """Random-init weights of `num_experts` experts in the layouts ``XpuFusedMoe`` takes, drawn on
    the device expert by expert: -> (w13, w13_scales, w13_bias, w2, w2_scales, w2_bias)."""
    g = torch.Generator(device=device).manual_seed(seed)
    E, H, I = num_experts, cfg.H, cfg.I
    if cfg.recipe == "bf16":     # [E,K,N]
        w13 = torch.empty(E, H, 2 * I, dtype=torch.bfloat16, device=device)
        w2 = torch.empty(E, I, H, dtype=torch.bfloat16, device=device)
        for e in range(E):
            w13[e] = (torch.randn(H, 2 * I, generator=g, device=device) * H ** -0.5).to(torch.bfloat16)
            w2[e] = (torch.randn(I, H, generator=g, device=device) * I ** -0.5).to(torch.bfloat16)
        return w13, None, None, w2, None, None
    if cfg.recipe == "fp8block":  # [E,N,K] e4m3 quantised from N(0, 1/fan_in)
        w13 = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device=device)
        w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=device)
        s13 = torch.empty(E, 2 * I // 128, H // 128, dtype=torch.float32, device=device)
        s2 = torch.empty(E, H // 128, I // 128, dtype=torch.float32, device=device)
        for e in range(E):
            w13[e], s13[e] = quant_fp8_block(torch.randn(2 * I, H, generator=g, device=device) * H ** -0.5)
            w2[e], s2[e] = quant_fp8_block(torch.randn(H, I, generator=g, device=device) * I ** -0.5)
        return w13, s13, None, w2, s2, None
    # mxfp4: uniform e2m1 codes, e8m0 exponents in [-10, -4], bf16 biases N(0, 0.02)
    def rnd(lo, hi, shape):
        return torch.randint(lo, hi, shape, generator=g, device=device, dtype=torch.int32).to(torch.uint8)
    w13 = rnd(0, 256, (E, 2 * I, H // 2)).view(torch.float4_e2m1fn_x2)
    w2 = rnd(0, 256, (E, H, I // 2)).view(torch.float4_e2m1fn_x2)
    s13 = rnd(117, 124, (E, 2 * I, H // 32))
    s2 = rnd(117, 124, (E, H, I // 32))
    b13 = (torch.randn(E, 2 * I, generator=g, device=device) * 0.02).to(torch.bfloat16)
    b2 = (torch.randn(E, H, generator=g, device=device) * 0.02).to(torch.bfloat16)
    return w13, s13, b13, w2, s2, b2


def weight_bytes_per_expert(cfg: MoeConfig) -> int:
    """Bytes of one expert's weights as stored (incl. scales and biases)."""
    n = 3 * cfg.H * cfg.I
    if cfg.recipe == "bf16":
        return 2 * n
    if cfg.recipe == "fp8block":
        return n + 4 * (n // (128 * 128))
    return n // 2 + n // 32 + (2 * (2 * cfg.I + cfg.H) if cfg.has_bias else 0)


def layer_bytes(cfg: MoeConfig, T: int, experts_active: int) -> int:
    """Algorithmic bytes of one layer call: the active experts' weights, x in, y out, router
    logits, ids + weights; intermediates are not counted."""
    return experts_active * weight_bytes_per_expert(cfg) + 2 * T * cfg.H * 2 + T * cfg.E * 4 + T * cfg.K * 8


def layer_flops(cfg: MoeConfig, T: int) -> float:
    return 6.0 * T * cfg.K * cfg.H * cfg.I
