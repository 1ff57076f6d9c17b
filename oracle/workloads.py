"""TEST INFRASTRUCTURE - seeded synthetic inputs for the five benchmark shapes.

The shapes, dtypes and value distributions are the ones the benchmark
configurations state (Mixtral-8x7B-, Qwen3-30B-A3B-, DeepSeek-V3- and
gpt-oss-120b-shaped layers plus a small CPU-runnable one); the numbers are
synthetic stand-ins drawn from a CPU ``torch.Generator`` with a fixed draw
order, so the oracle and the device see identical bits.  Weights are produced
in the logical ``[E, N, K]`` layout; ``to_op_layout`` converts them to what
``XpuFusedMoe`` takes.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import torch_oracle as to


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
    """A smaller layer of the same kind, for tests the CPU oracle can finish."""
    import dataclasses
    return dataclasses.replace(cfg, H=H or cfg.H, I=I or cfg.I, E=E or cfg.E)


def _randn(gen, shape, std=1.0, chunk_rows=None):
    return torch.randn(shape, generator=gen, dtype=torch.float32) * std


def make_weights(cfg: MoeConfig, seed: int = 0, num_experts=None, device="cpu"):
    """-> dict with logical-layout weights: w13 [E,2I,H], w2 [E,H,I] (+ scales, biases).
    Generated expert by expert to bound host memory."""
    E = num_experts or cfg.E
    H, I = cfg.H, cfg.I
    gen = torch.Generator().manual_seed(seed * 1000 + 1)
    out = {}
    if cfg.recipe == "bf16":
        w13 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=device)
        w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=device)
        for e in range(E):
            w13[e] = (_randn(gen, (2 * I, H), H ** -0.5)).to(torch.bfloat16).to(device)
            w2[e] = (_randn(gen, (H, I), I ** -0.5)).to(torch.bfloat16).to(device)
        out.update(w13=w13, w2=w2, w13_scale=None, w2_scale=None)
    elif cfg.recipe == "fp8block":
        w13 = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device=device)
        w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=device)
        s13 = torch.empty(E, 2 * I // 128, H // 128, dtype=torch.float32, device=device)
        s2 = torch.empty(E, H // 128, I // 128, dtype=torch.float32, device=device)
        for e in range(E):
            q, s = to.quant_fp8_block_wei(_randn(gen, (2 * I, H), H ** -0.5))
            w13[e], s13[e] = q.to(device), s.to(device)
            q, s = to.quant_fp8_block_wei(_randn(gen, (H, I), I ** -0.5))
            w2[e], s2[e] = q.to(device), s.to(device)
        out.update(w13=w13, w2=w2, w13_scale=s13, w2_scale=s2)
    elif cfg.recipe == "mxfp4":
        def codes(shape):
            return torch.randint(0, 256, shape, generator=gen, dtype=torch.int32).to(torch.uint8)
        def exps(shape):
            return torch.randint(117, 124, shape, generator=gen, dtype=torch.int32).to(torch.uint8)
        out.update(w13=codes((E, 2 * I, H // 2)).to(device), w2=codes((E, H, I // 2)).to(device),
                   w13_scale=exps((E, 2 * I, H // 32)).to(device),
                   w2_scale=exps((E, H, I // 32)).to(device))
    else:
        raise ValueError(cfg.recipe)
    if cfg.has_bias:
        out["w13_bias"] = _randn(gen, (E, 2 * I), 0.02).to(torch.bfloat16).to(device)
        out["w2_bias"] = _randn(gen, (E, H), 0.02).to(torch.bfloat16).to(device)
    else:
        out["w13_bias"] = None
        out["w2_bias"] = None
    return out


def make_inputs(cfg: MoeConfig, T: int, seed: int = 0):
    """-> x bf16 [T,H], router logits fp32 [T,E], routing bias fp32 [E] or None."""
    gen = torch.Generator().manual_seed(seed * 1000 + 2)
    x = _randn(gen, (T, cfg.H)).to(torch.bfloat16)
    logits = _randn(gen, (T, cfg.E))
    if cfg.logit_offset_std > 0:
        logits = logits + _randn(gen, (cfg.E,), cfg.logit_offset_std).unsqueeze(0)
    bias = None
    if cfg.routing == "grouped_sigmoid":
        bias = _randn(gen, (cfg.E,), 0.1)
    return x, logits, bias


def route_cpu(cfg: MoeConfig, logits, bias):
    """Routing with the torch restatements -> (weights f32 [T,K], ids i32 [T,K])."""
    if cfg.routing == "softmax":
        return to.topk_softmax(logits, cfg.K, cfg.renormalize)
    scores = torch.sigmoid(logits)
    w, ids = to.grouped_topk(scores, scores + bias.unsqueeze(0), cfg.n_group, cfg.topk_group,
                             cfg.K, cfg.renormalize, cfg.routed_scaling_factor)
    return w.float(), ids


def dequant_weights(cfg: MoeConfig, w):
    """Logical-layout weights -> fp32 [E,N,K] (for the CPU oracle)."""
    if cfg.recipe == "bf16":
        return w["w13"].float(), w["w2"].float()
    if cfg.recipe == "fp8block":
        d13 = torch.stack([to.dequant_fp8_block_wei(w["w13"][e].cpu(), w["w13_scale"][e].cpu())
                           for e in range(w["w13"].shape[0])])
        d2 = torch.stack([to.dequant_fp8_block_wei(w["w2"][e].cpu(), w["w2_scale"][e].cpu())
                          for e in range(w["w2"].shape[0])])
        return d13, d2
    d13 = to.dequant_mxfp4(w["w13"].cpu(), w["w13_scale"].cpu()).to(torch.bfloat16).float()
    d2 = to.dequant_mxfp4(w["w2"].cpu(), w["w2_scale"].cpu()).to(torch.bfloat16).float()
    return d13, d2


def to_op_layout(cfg: MoeConfig, w):
    """Logical [E,N,K] weights -> the tensors ``XpuFusedMoe`` takes
    (bf16: [E,K,N]; block fp8: [E,N,K] kept; mxfp4: float4_e2m1fn_x2 view)."""
    if cfg.recipe == "bf16":
        return (w["w13"].transpose(-1, -2).contiguous(), None,
                w["w2"].transpose(-1, -2).contiguous(), None)
    if cfg.recipe == "fp8block":
        return w["w13"], w["w13_scale"], w["w2"], w["w2_scale"]
    return (w["w13"].view(torch.float4_e2m1fn_x2), w["w13_scale"],
            w["w2"].view(torch.float4_e2m1fn_x2), w["w2_scale"])
