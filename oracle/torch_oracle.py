"""TEST INFRASTRUCTURE - pure-torch CPU restatement of the fused-MoE path.

Each function names the part of vllm-xpu-kernels it follows.  The functions are
written to run on CPU tensors; nothing in the product imports this module.

Pinning: ``tests/test_oracle_golden.py`` checks these functions against vectors
produced by the reference's own pure-torch test references on CPU (the .pt
files in ``tests/golden``, written by ``tests/golden/make_golden.py``).  Pieces
the reference's tests never exercise as a whole - SwigluOAI with biases in the
layer, block fp8 with real activation quantisation, grouped top-k at 256
experts, top-k > 1 in the layer - are pinned only through their parts
("parity unpinned" as a whole).
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0

_FP4_LUT = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                         -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=torch.float32)


# --------------------------------------------------------------------------- routing
def stable_topk(arr, k):
    """tests/ops/topk_op.py:11-13: stable descending sort, lower index wins ties."""
    values, indices = torch.sort(arr, dim=-1, descending=True, stable=True)
    return values[..., :k], indices[..., :k]


def topk_softmax(gating, topk, renormalize, bias=None):
    """tests/ops/topk_op.py:16-36."""
    p = torch.softmax(gating, dim=-1, dtype=torch.float32)
    if bias is not None:
        _, ids = stable_topk(p + bias.unsqueeze(0), topk)
        w = p.gather(1, ids)
    else:
        w, ids = stable_topk(p, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.float(), ids.to(torch.int32)


def topk_sigmoid(gating, topk, renormalize, bias=None, routed_scaling_factor=1.0):
    """tests/ops/topk_op.py:39-61."""
    p = torch.sigmoid(gating).to(torch.float32)
    if bias is not None:
        _, ids = stable_topk(p + bias.unsqueeze(0), topk)
        w = p.gather(1, ids)
    else:
        w, ids = stable_topk(p, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return (w * routed_scaling_factor).float(), ids.to(torch.int32)


def grouped_topk(scores, scores_with_bias, n_group, topk_group, topk, renormalize,
                 routed_scaling_factor):
    """tests/ops/grouped_topk_op.py:11-67 with the output order made definite:
    descending biased score, ties to the lower expert id (what the kernel of
    csrc/moe/grouped_topk.cpp:36-45 emits)."""
    T, E = scores.shape
    sb = scores_with_bias.float()
    group_scores = sb.view(T, n_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
    # keep the topk_group best groups, ties to the lower group index
    _, gidx = torch.sort(group_scores, dim=-1, descending=True, stable=True)
    mask = torch.zeros_like(group_scores)
    mask.scatter_(1, gidx[:, :topk_group], 1)
    score_mask = mask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, -1)
    tmp = sb.masked_fill(~score_mask.bool(), float("-inf"))
    _, ids = stable_topk(tmp, topk)
    w = scores.float().gather(1, ids)
    if renormalize:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    w = w * routed_scaling_factor
    return w.to(scores.dtype), ids.to(torch.int32)


# --------------------------------------------------------------------------- align / permute
def moe_align_block_size(topk_ids, block_size, num_experts, sorted_len, expert_ids_len,
                         expert_map=None):
    """tests/test_moe_align_block_size.py:97-183 (stable order inside an expert;
    with a map the segments are ordered by mapped id, as the kernel of
    csrc/moe/moe_align_sum_kernels.cpp:186-256 orders them)."""
    flat = topk_ids.flatten().long()
    numel = flat.numel()
    if expert_map is not None:
        valid = (flat >= 0) & (flat < num_experts)
        b = torch.full_like(flat, -1)
        b[valid] = expert_map.long()[flat[valid]]
    else:
        b = torch.where((flat >= 0) & (flat < num_experts), flat, torch.full_like(flat, -1))
    sorted_ids = torch.full((sorted_len,), numel, dtype=torch.int32)
    expert_ids = torch.zeros(expert_ids_len, dtype=torch.int32)
    pos = 0
    for e in range(num_experts):
        slots = torch.nonzero(b == e).flatten().to(torch.int32)
        n = slots.numel()
        padded = (n + block_size - 1) // block_size * block_size
        sorted_ids[pos:pos + n] = slots[: max(0, min(n, sorted_len - pos))]
        expert_ids[pos // block_size:(pos + padded) // block_size] = e
        pos += padded
    return sorted_ids, expert_ids, torch.tensor([pos], dtype=torch.int32)


def remap_hidden_states(hidden, scales, topk_ids, expert_map, local_experts):
    """tests/fused_moe/test_remap_hidden_states.py:38-83 (sequential, stable fill).
    -> remapped, remapped_scales, rows_per_expert, row_map."""
    T, K = topk_ids.shape
    local = expert_map.long()[topk_ids.long()] if expert_map is not None else topk_ids.long()
    flat = local.flatten()
    valid = flat >= 0
    rows = torch.bincount(flat[valid], minlength=local_experts).to(torch.int32)
    base = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(rows.long(), 0)])
    row_map = torch.full((T * K,), -1, dtype=torch.int32)
    fill = torch.zeros(local_experts, dtype=torch.long)
    for i in range(T * K):
        e = int(flat[i])
        if e < 0:
            continue
        row_map[i] = int(base[e] + fill[e])
        fill[e] += 1
    remapped = torch.zeros((T * K, hidden.shape[1]), dtype=hidden.dtype)
    rs = None
    if scales is not None:
        rs = torch.zeros((T * K, scales.shape[1]), dtype=scales.dtype)
    tok = torch.arange(T * K) // K
    sel = row_map >= 0
    remapped.view(torch.uint8 if hidden.element_size() == 1 else hidden.dtype)[row_map[sel].long()] = \
        hidden.view(torch.uint8 if hidden.element_size() == 1 else hidden.dtype)[tok[sel]]
    if scales is not None:
        sv = torch.uint8 if scales.element_size() == 1 else scales.dtype
        rs.view(sv)[row_map[sel].long()] = scales.view(sv)[tok[sel]]
    return remapped, rs, rows, row_map.view(T, K)


def ep_dispatch_plan(topk_ids, ep_size, num_local_experts, capacity, expert_slot=None):
    """The bookkeeping of the expert-parallel dispatch, sequentially: a token goes once to every
    rank that owns one of its experts (expert g on rank g // num_local_experts, the split of
    csrc/moe/init_expert_map.cpp:45-52; with `expert_slot` [E], a permutation expert -> slot,
    the slot takes the place of g); its row index at rank d is the number of earlier tokens
    of this source that also go to d.  -> send_counts [ep] i32, send_pos [T, ep] i32
    (d * capacity + index, or -1), loc_ids [T, ep, K] i32 (expert id local to rank d, -1 for
    experts of other ranks)."""
    T, K = topk_ids.shape
    ids = topk_ids.long()
    if expert_slot is not None:
        ids = torch.where(ids >= 0, expert_slot.long()[ids.clamp(min=0)], ids)
    counts = torch.zeros(ep_size, dtype=torch.int32)
    pos = torch.full((T, ep_size), -1, dtype=torch.int32)
    loc = torch.full((T, ep_size, K), -1, dtype=torch.int32)
    for t in range(T):
        for d in range(ep_size):
            mine = (ids[t] >= 0) & (ids[t] // num_local_experts == d)
            if bool(mine.any()):
                pos[t, d] = d * capacity + int(counts[d])
                counts[d] += 1
                loc[t, d] = torch.where(mine, ids[t] - d * num_local_experts, -1).to(torch.int32)
    return counts, pos, loc


def init_expert_map(n_local, ep_rank, ep_size):
    """tests/fused_moe/test_remap_hidden_states.py:333-345."""
    m = torch.full((n_local * ep_size,), -1, dtype=torch.int32)
    m[ep_rank * n_local:(ep_rank + 1) * n_local] = torch.arange(n_local, dtype=torch.int32)
    return m


# --------------------------------------------------------------------------- reductions
def moe_gather(moe_output, topk_weights, row_map, out_dtype):
    """tests/test_moe_gather.py:27-44."""
    idx = row_map.long()
    sel = moe_output[idx.clamp(min=0)] * (idx != -1).unsqueeze(-1)
    out = torch.einsum('ijk,ij->ik', sel.float(), topk_weights.float())
    return out.to(out_dtype)


def moe_sum(inp, topk_ids=None, expert_map=None):
    """tests/test_moe_sum.py:34-36, 62-65: fp32 sum over k, masked slots skipped."""
    x = inp.float()
    if topk_ids is not None:
        ids = topk_ids.long()
        skip = ids < 0
        if expert_map is not None:
            skip = skip | (expert_map.long()[ids.clamp(min=0)] < 0)
        x = x * (~skip).unsqueeze(-1)
    return x.sum(dim=1).to(inp.dtype)


# --------------------------------------------------------------------------- activations
def silu_and_mul(x):
    """tests/ops/activation_op.py:21-24."""
    d = x.shape[-1] // 2
    return torch.nn.functional.silu(x[..., :d]) * x[..., d:]


def swigluoai_and_mul(x, alpha=1.702, limit=7.0):
    """tests/ops/swigluoai_and_mul_op.py:27-35."""
    gate, up = x[..., ::2], x[..., 1::2]
    gate = gate.clamp(min=None, max=limit)
    up = up.clamp(min=-limit, max=limit)
    return (up + 1) * (gate * torch.sigmoid(gate * alpha))


def gelu_and_mul(x, approximate="none"):
    """tests/ops/activation_op.py:86-90 (csrc/activation.cpp:53-75): T(gelu(x)) *_T y."""
    d = x.shape[-1] // 2
    return torch.nn.functional.gelu(x[..., :d].float(), approximate=approximate).to(x.dtype) * x[..., d:]


def swiglustep_and_mul(x, limit=7.0):
    """csrc/activation.cpp:299-312: min(silu(gate), limit) * clamp(up, +-limit) in fp32,
    gate = first half (tests/ops/swiglustep_and_mul_op.py:27-33)."""
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return ((g / (1.0 + torch.exp(-g))).clamp(max=limit) * u.clamp(min=-limit, max=limit)).to(x.dtype)


def relu2_no_mul(x):
    """csrc/activation.cpp:45-50: max(x, 0)^2 in fp32, no gating."""
    r = x.float().clamp(min=0)
    return (r * r).to(x.dtype)


# --------------------------------------------------------------------------- quantisation
def per_token_group_fp8_quant(x, group=128, eps=1e-10, ue8m0=False):
    """Order of csrc/quantization/fp8/fp8_quant.cpp:340-387: amax floor eps,
    scale floor 1/(448*512), multiply by the reciprocal, clamp, round to e4m3."""
    shape = x.shape
    xf = x.float().reshape(-1, group)
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp(min=eps)
    s = torch.maximum(amax / FP8_MAX, torch.tensor(1.0 / (FP8_MAX * 512.0)))
    if ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s.clamp(min=1e-10))))
    q = (xf * (1.0 / s)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(shape), s.reshape(*shape[:-1], shape[-1] // group)


def quant_mxfp8(x, terms=1):
    """MX-format activation quantisation used by the block-scaled MXFP4 GEMM (the
    OCP microscaling recipe; the reference op with the same one-plane math is
    per_token_group_fp8_quant with group 32 and scale_ue8m0,
    csrc/quantization/fp8/fp8_quant.cpp:340-387): per 32 values the smallest
    power-of-two scale with amax / scale <= 448 (floor 1e-10), e4m3 codes of
    x / scale.  With terms == 2 a second plane quantises the residual
    x - code * scale the same way.  Returns (codes e4m3 [terms, rows, cols],
    scale bytes uint8 [terms, rows, cols/32])."""
    rows, cols = x.shape
    v = x.float().reshape(rows, cols // 32, 32)
    qs, ss = [], []
    for _ in range(terms):
        amax = v.abs().amax(dim=-1)
        m, e = torch.frexp((amax / FP8_MAX).clamp(min=1e-10))   # = m * 2^e, m in [0.5, 1)
        exp = torch.where(m == 0.5, e - 1, e)                    # ceil(log2(.)), exactly
        sc = torch.exp2(exp.float()).unsqueeze(-1)
        q = (v * (1.0 / sc)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
        v = v - q.float() * sc
        qs.append(q.reshape(rows, cols))
        ss.append((exp + 127).to(torch.uint8))
    return torch.stack(qs), torch.stack(ss)


def dequant_mxfp8(q, scale_u8):
    """Sum of the planes of quant_mxfp8: q [terms, rows, cols], scale_u8 [terms, rows, cols/32]."""
    terms, rows, cols = q.shape
    sc = torch.exp2(scale_u8.float() - 127.0)
    return (q.float().reshape(terms, rows, cols // 32, 32) * sc.unsqueeze(-1)).sum(dim=0).reshape(rows, cols)


def dequant_mxfp8_wei(w, scale_u8):
    """vllm_xpu_kernels/moe_utils.py:76-78: w [K,N] e4m3, scale_u8 [K/32,N] e8m0 bytes,
    one per 32 K rows -> fp32 [K,N]."""
    return w.float() * torch.exp2(scale_u8.float() - 127.0).repeat_interleave(32, dim=0)


def quant_mxfp8_wei(w):
    """Synthetic-weight helper: w [K,N] -> (e4m3 [K,N], e8m0 bytes [K/32,N]) with the
    smallest power-of-two scale per 32 K rows that keeps amax / scale <= 448."""
    K, N = w.shape
    v = w.float().reshape(K // 32, 32, N)
    sc = _ceil_pow2(v.abs().amax(dim=1) / FP8_MAX, 2.0 ** -100)
    q = (v / sc.unsqueeze(1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).reshape(K, N)
    return q, (torch.log2(sc) + 127).to(torch.uint8)


def _ceil_pow2(v, eps):
    """exp2(ceil(log2(max(|v|, eps)))) computed exactly."""
    m, e = torch.frexp(v.abs().clamp(min=eps))
    return torch.exp2(torch.where(m == 0.5, e - 1, e).float())


_E2M1_MID = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def f32_to_e2m1(x):
    """csrc/quantization/fp4/mxfp4_quant.h:17-30: code = number of midpoints strictly
    below |x| (ties go down), sign in bit 3 (x < 0)."""
    code = (x.abs().unsqueeze(-1) > _E2M1_MID).sum(-1).to(torch.uint8)
    return code | ((x < 0).to(torch.uint8) << 3)


def _pack_e2m1(codes):
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def _silu_mul_f32(x):
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (g / (1.0 + torch.exp(-g))) * u


def silu_and_mul_per_block_quant(x, group, out_dtype=torch.float8_e4m3fn, scale_ub=None, ue8m0=False):
    """csrc/quantization/fused_kernels/fused_silu_mul_block_quant.cpp:62-116: fp32
    silu(g)*u, per-group amax, scale = max(amax/448, 1/(448*512)) (int8:
    max(amax/127, FLT_EPSILON)), optional cap and power-of-two rounding, x / scale."""
    r = _silu_mul_f32(x)
    T, H = r.shape
    v = r.reshape(T, H // group, group)
    amax = v.abs().amax(-1)
    if out_dtype == torch.int8:
        sc = (amax / 127.0).clamp(min=torch.finfo(torch.float32).eps)
        q = torch.round(v / sc.unsqueeze(-1)).clamp(-128, 127).to(torch.int8)
    else:
        floor_s = 1.0 / (FP8_MAX * 512.0)
        sc = (amax / FP8_MAX).clamp(min=floor_s)
        if scale_ub is not None:
            sc = torch.minimum(sc, scale_ub.float()).clamp(min=floor_s)
        if ue8m0:
            sc = _ceil_pow2(sc, 1e-10)
        q = (v / sc.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(T, H), sc


def per_token_group_quant_mxfp4(x, eps=1e-10):
    """csrc/quantization/fp4/mxfp4_quant.h:186-240: scale = ceil_pow2(max(amax/6, eps))
    per 32 values, codes of clamp(x * (1/scale), -6, 6), low nibble = even element."""
    T, H = x.shape
    v = x.float().reshape(T, H // 32, 32)
    sc = _ceil_pow2(v.abs().amax(-1) / 6.0, eps)
    codes = f32_to_e2m1((v * (1.0 / sc).unsqueeze(-1)).clamp(-6.0, 6.0)).reshape(T, H)
    return _pack_e2m1(codes), sc


def silu_and_mul_mxfp4_quant(x, eps=1e-10):
    """csrc/quantization/fused_kernels/fused_silu_mul_mxfp4_quant.cpp:62-118."""
    return per_token_group_quant_mxfp4(_silu_mul_f32(x), eps)


def silu_and_mul_quant(x, scale):
    """csrc/activation.cpp:216-226: float(T(silu(x)) *_T y) * (1/scale), clamp, e4m3."""
    d = x.shape[-1] // 2
    g = x[..., :d].float()
    s = (g / (1.0 + torch.exp(-g))).to(x.dtype)
    prod = (s.float() * x[..., d:].float()).to(x.dtype)
    inv = 1.0 / scale.float()
    return (prod.float() * inv).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def dequant_fp8_block_act(q, s):
    """vllm_xpu_kernels/moe_utils.py:143-148."""
    shape = q.shape
    return (q.float().reshape(shape[0], -1, 128) * s.unsqueeze(-1)).reshape(shape)


def dequant_fp8_block_wei(w, s):
    """vllm_xpu_kernels/moe_utils.py:134-141: w [N,K] e4m3, s [N/128,K/128]."""
    N, K = w.shape
    x = w.float().view(N // 128, 128, K // 128, 128) * s.unsqueeze(1).unsqueeze(-1)
    return x.reshape(N, K)


def quant_fp8_block_wei(w):
    """Synthetic-weight helper: e4m3 + amax/448 scale per 128x128 block."""
    N, K = w.shape
    x = w.float().view(N // 128, 128, K // 128, 128)
    amax = x.abs().amax(dim=(1, 3), keepdim=True).clamp(min=1e-12)
    s = amax / FP8_MAX
    q = (x / s).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(N, K), s.reshape(N // 128, K // 128)


def dequant_mxfp4(packed, scale_u8):
    """vllm_xpu_kernels/moe_utils.py:29-68 and tests/fused_moe/test_fused_moe.py:79-116:
    low nibble = even k, value LUT, scale 2^(byte-127) per 32 elements."""
    u8 = packed.view(torch.uint8)
    lo = _FP4_LUT[(u8 & 0xF).long()]
    hi = _FP4_LUT[(u8 >> 4).long()]
    vals = torch.stack((lo, hi), dim=-1).reshape(*u8.shape[:-1], u8.shape[-1] * 2)
    sc = torch.exp2(scale_u8.view(torch.uint8).float() - 127.0)
    return (vals.reshape(-1, 32) * sc.reshape(-1, 1)).reshape(vals.shape)


def dequant_int4(packed_u4, scales, group_size):
    """tests/fused_moe/test_fused_moe.py:63-76 of the reference: uint4 pairs (low nibble =
    even k) with zero point 8, value = (q - 8) * scale[n, k // group] rounded to the
    scales' dtype.  packed_u4 [..., N, K/2] uint8, scales [..., N, K/group]."""
    u8 = packed_u4.view(torch.uint8)
    lo = (u8 & 0xF).to(torch.int32) - 8
    hi = (u8 >> 4).to(torch.int32) - 8
    q = torch.stack((lo, hi), dim=-1).reshape(*u8.shape[:-1], u8.shape[-1] * 2).float()
    sc = scales.float().repeat_interleave(group_size, dim=-1)
    return (q * sc).to(scales.dtype)


# --------------------------------------------------------------------------- grouped GEMM
def grouped_gemm(a, w_deq, bias, rows_per_expert, out_dtype, bias_after_rounding=False):
    """Per-expert fp32 matmul over the ragged segments (semantics of
    csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2.hpp:125-251): a [M,K] fp32,
    w_deq [E,N,K] fp32 (already dequantised), bias [E,N] or None.  The kernels add the
    bias to the fp32 accumulator; bias_after_rounding restates the reference's eager
    simulation instead, which rounds the product to out_dtype first and adds the bias in
    that type (vllm_xpu_kernels/moe_utils.py:345-351)."""
    M = a.shape[0]
    N = w_deq.shape[1]
    out = torch.zeros(M, N, dtype=torch.float32)
    off = 0
    for e, r in enumerate(rows_per_expert.tolist()):
        if r == 0:
            continue
        o = a[off:off + r].float() @ w_deq[e].float().T
        if bias is not None:
            o = (o.to(out_dtype) + bias[e].to(out_dtype)).float() if bias_after_rounding else o + bias[e].float()
        out[off:off + r] = o
        off += r
    return out.to(out_dtype)


# --------------------------------------------------------------------------- whole layer
def fused_moe_bf16(x, w13, w13_bias, w2, w2_bias, topk_weights, topk_ids, num_experts,
                   ep_rank=0, ep_size=1, gemm1_clamp_limit=None):
    """tests/fused_moe/test_fused_moe.py:119-176.  w13 [E_total,2I,H], w2
    [E_total,H,I] (logical [N,K] layout); gate = rows [0,I), up = rows [I,2I);
    SiLU; fp32 math on the 16-bit inputs, expert output rounded to x.dtype,
    multiplied by the routing weight and summed per token in x.dtype."""
    K = topk_ids.shape[1]
    flat_ids = topk_ids.reshape(-1).long()
    flat_w = topk_weights.reshape(-1, 1)
    lo, hi = num_experts * ep_rank, num_experts * (ep_rank + 1)
    out = torch.zeros_like(x)
    idxs = flat_ids.argsort(stable=True)
    counts = torch.bincount(flat_ids, minlength=int(flat_ids.max()) + 1 if flat_ids.numel() else 0)
    ends = counts.cumsum(0)
    token_idxs = idxs // K
    for e, end in enumerate(ends.tolist()):
        start = 0 if e == 0 else int(ends[e - 1])
        if start == end or e < lo or e >= hi:
            continue
        tok = token_idxs[start:end]
        xe = x[tok].float()
        I = w13.shape[1] // 2
        w1, w3 = w13[e, :I].float(), w13[e, I:].float()
        g = xe @ w1.T
        u = xe @ w3.T
        if w13_bias is not None:
            g = g + w13_bias[e, :I].float()
            u = u + w13_bias[e, I:].float()
        if gemm1_clamp_limit is not None and gemm1_clamp_limit > 0:
            g = g.clamp(max=gemm1_clamp_limit)
            u = u.clamp(min=-gemm1_clamp_limit, max=gemm1_clamp_limit)
        o = (torch.nn.functional.silu(g) * u) @ w2[e].float().T
        if w2_bias is not None:
            o = o + w2_bias[e].float()
        o = o.to(x.dtype)
        o = (o.float() * flat_w[idxs[start:end]].float()).to(x.dtype)
        out.index_add_(0, tok, o)
    return out


def fused_moe_staged(x, w13_deq, w13_bias, w2_deq, w2_bias, topk_weights, topk_ids, num_experts,
                     activation="silu", act_quant=False, expert_map=None, alpha=1.702, limit=7.0,
                     gemm1_clamp_limit=None, bias_after_rounding=False):
    """The layer as the reference's kernel path stages it
    (vllm_xpu_kernels/fused_moe_interface.py:328-419 with the qdq semantics of
    vllm_xpu_kernels/moe_utils.py:236-403): permute -> GEMM1 (fp32 accumulate,
    rounded to x.dtype) -> gated activation -> [per-1x128 e4m3 quant-dequant of
    the activations when act_quant; per-32 MX quant-dequant with one or two
    planes when act_quant is "mxfp8" / "mxfp8x2"] -> GEMM2 -> weighted gather in fp32.
    w13_deq [E,2I,H] / w2_deq [E,H,I] are the dequantised weights in fp32."""
    T, H = x.shape
    dt = x.dtype
    remapped, _, rows, row_map = remap_hidden_states(x, None, topk_ids, expert_map, num_experts)
    a1 = remapped.float()
    if act_quant in ("mxfp8", "mxfp8x2"):
        a1 = dequant_mxfp8(*quant_mxfp8(remapped, 2 if act_quant == "mxfp8x2" else 1))
    elif act_quant:
        q, s = per_token_group_fp8_quant(remapped)
        a1 = dequant_fp8_block_act(q, s)
    g1 = grouped_gemm(a1, w13_deq, w13_bias, rows, dt, bias_after_rounding)
    if gemm1_clamp_limit is not None and gemm1_clamp_limit > 0:
        I = g1.shape[1] // 2
        g1[:, :I] = g1[:, :I].clamp(max=gemm1_clamp_limit)
        g1[:, I:] = g1[:, I:].clamp(min=-gemm1_clamp_limit, max=gemm1_clamp_limit)
    if activation == "silu":
        d = g1.shape[1] // 2
        act = (torch.nn.functional.silu(g1[:, :d].float()).to(dt).float() * g1[:, d:].float()).to(dt)
    elif activation == "gelu":
        act = gelu_and_mul(g1)
    elif activation == "gelu_tanh":
        act = gelu_and_mul(g1, "tanh")
    elif activation == "swiglustep":
        act = swiglustep_and_mul(g1, 7.0)
    elif activation == "relu2_no_mul":
        act = relu2_no_mul(g1)
    else:
        act = swigluoai_and_mul(g1.float(), alpha, limit).to(dt)
    a2 = act.float()
    if act_quant in ("mxfp8", "mxfp8x2"):
        a2 = dequant_mxfp8(*quant_mxfp8(act, 2 if act_quant == "mxfp8x2" else 1))
    elif act_quant:
        q, s = per_token_group_fp8_quant(act)
        a2 = dequant_fp8_block_act(q, s)
    g2 = grouped_gemm(a2, w2_deq, w2_bias, rows, dt, bias_after_rounding)
    return moe_gather(g2, topk_weights, row_map, dt)
