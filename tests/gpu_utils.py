"""Helpers for the GPU parity tests: thin callers of the torch ops (which go
through the C ABI) that allocate outputs the way the reference's Python
wrappers do (tests/ops/*.py of vllm-xpu-kernels)."""
import torch

DEV = "cuda"


def topk_softmax(gating, topk, renormalize, bias=None, index_dtype=torch.int32):
    T = gating.shape[0]
    w = torch.empty(T, topk, dtype=torch.float32, device=DEV)
    ids = torch.empty(T, topk, dtype=index_dtype, device=DEV)
    src = torch.empty(T, topk, dtype=torch.int32, device=DEV)
    torch.ops._moe_C.topk_softmax(w, ids, src, gating, renormalize, bias)
    return w, ids, src


def topk_sigmoid(gating, topk, renormalize, bias=None, rsf=1.0, index_dtype=torch.int32):
    T = gating.shape[0]
    w = torch.empty(T, topk, dtype=torch.float32, device=DEV)
    ids = torch.empty(T, topk, dtype=index_dtype, device=DEV)
    src = torch.empty(T, topk, dtype=torch.int32, device=DEV)
    torch.ops._moe_C.topk_sigmoid(w, ids, src, gating, renormalize, bias, rsf)
    return w, ids, src


def align_sizes(numel, num_experts, block_size, pad_sorted_ids=False):
    n = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        n = (n + block_size - 1) // block_size * block_size
    if numel < num_experts:
        n = min(numel * block_size, n)
    return n, (n + block_size - 1) // block_size


def moe_align_block_size(topk_ids, block_size, num_experts, expert_map=None, pad_sorted_ids=False):
    n, nb = align_sizes(topk_ids.numel(), num_experts, block_size, pad_sorted_ids)
    s = torch.empty(n, dtype=torch.int32, device=DEV)
    e = torch.empty(nb, dtype=torch.int32, device=DEV)
    p = torch.empty(1, dtype=torch.int32, device=DEV)
    torch.ops._moe_C.moe_align_block_size(topk_ids, num_experts, block_size, s, e, p, expert_map)
    return s, e, p


def remap(hidden, scales, topk_ids, expert_map, total_experts, local_experts):
    T, K = topk_ids.shape
    remapped = torch.zeros(T * K, hidden.shape[1], dtype=hidden.dtype, device=DEV)
    rs = torch.zeros(T * K, scales.shape[1], dtype=scales.dtype, device=DEV) if scales is not None else None
    rows = torch.empty(local_experts, dtype=torch.int32, device=DEV)
    row_map = torch.empty(T, K, dtype=torch.int32, device=DEV)
    torch.ops._moe_C.remap_hidden_states(hidden, scales, remapped, rs, expert_map, rows, row_map,
                                         topk_ids, total_experts, local_experts)
    return remapped, rs, rows, row_map


def grouped_gemm(a, a_scale, w, w_scale, bias, rows, N, K, layout=0, epilogue=0, impl=0,
                 out_dtype=torch.bfloat16, clamp=0.0, rows_out=None, weight_sets=None):
    M = a.shape[0] if rows_out is None else rows_out
    E = rows.numel() if weight_sets is None else weight_sets   # fewer weight sets than row segments
    n_out = N // 2 if epilogue else N
    d = torch.full((M, n_out), float("nan"), dtype=out_dtype, device=DEV)
    torch.ops._xpu_C.b200_grouped_gemm(a, a_scale, w, w_scale, bias, d, rows, N, K, E, layout,
                                       epilogue, 1.702, 7.0, clamp, impl, 0)
    return d


def random_rows(E, total, gen, zero_frac=0.25):
    """A ragged split of `total` rows over E experts with some empty experts."""
    w = torch.rand(E, generator=gen)
    w[torch.rand(E, generator=gen) < zero_frac] = 0
    if float(w.sum()) == 0:
        w[0] = 1
    r = torch.floor(w / w.sum() * total).long()
    r[int(torch.argmax(w))] += total - int(r.sum())
    return r.to(torch.int32)


def quant_mxfp8(x, terms=1):
    """x [rows, cols] bf16/f16 -> (e4m3 codes [terms * rows, cols], int32 scale words
    [terms, ceil(cols/128), rows]) as the block-scaled GEMM takes them."""
    rows, cols = x.shape
    q = torch.empty(terms * rows, cols, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.full((terms, (cols + 127) // 128, rows), -1, dtype=torch.int32, device=DEV)
    torch.ops._C.b200_quant_mxfp8(x, q, s)
    return q, s


def mx_scale_bytes(s, cols):
    """int32 scale words [terms, nkb, rows] -> uint8 [terms, rows, 4 * nkb] (group order)."""
    terms, nkb, rows = s.shape
    return s.cpu().view(torch.uint8).reshape(terms, nkb, rows, 4).permute(0, 2, 1, 3).reshape(terms, rows, 4 * nkb)
