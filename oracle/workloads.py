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

import torch

from . import torch_oracle as to


# One table of shapes for the bench and the tests: it lives beside the bench.
from bench_workloads import CONFIGS, MoeConfig, make_inputs, scaled  # noqa: E402,F401


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


class ExpertView:
    """[E, N, K] fp32 weights for the layer restatements (they index ``w[e]`` and read
    ``w.shape``) without holding E dequantised experts: expert e is produced on access by
    `fetch(e)`.  Bounds host memory when a layer has hundreds of large experts."""

    def __init__(self, num_experts, n, k, fetch):
        self.shape = (num_experts, n, k)
        self._fetch = fetch

    def __getitem__(self, e):
        return self._fetch(int(e))


def expert_views(cfg: MoeConfig, w13, s13, w2, s2):
    """Lazy fp32 views of op-layout weights that may live on a GPU (``to_op_layout`` /
    ``bench_workloads.make_device_weights`` layouts): -> (w13 [E,2I,H], w2 [E,H,I])."""
    E = w13.shape[0]
    if cfg.recipe == "bf16":      # op layout [E,K,N]
        f13 = lambda e: w13[e].cpu().float().T
        f2 = lambda e: w2[e].cpu().float().T
    elif cfg.recipe == "fp8block":
        f13 = lambda e: to.dequant_fp8_block_wei(w13[e].cpu(), s13[e].cpu())
        f2 = lambda e: to.dequant_fp8_block_wei(w2[e].cpu(), s2[e].cpu())
    else:
        f13 = lambda e: to.dequant_mxfp4(w13[e:e + 1].cpu().view(torch.uint8), s13[e:e + 1].cpu())[0].to(torch.bfloat16).float()
        f2 = lambda e: to.dequant_mxfp4(w2[e:e + 1].cpu().view(torch.uint8), s2[e:e + 1].cpu())[0].to(torch.bfloat16).float()
    return (ExpertView(E, 2 * cfg.I, cfg.H, f13), ExpertView(E, cfg.H, cfg.I, f2))


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
