"""TEST INFRASTRUCTURE - ctypes front end of ``moe_oracle.c`` (the plain-C
restatement of routing, alignment and permutation bookkeeping).

``build()`` compiles the C file with the Makefile beside it; the wrappers take
and return torch CPU tensors.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB = None
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def build() -> Path:
    subprocess.run(["make", "-s", "-C", str(_HERE)], check=True, capture_output=True)
    return _HERE / "_build" / "libmoe_oracle.so"


def lib():
    global _LIB
    if _LIB is None:
        path = _HERE / "_build" / "libmoe_oracle.so"
        if not path.exists():
            build()
        _LIB = ctypes.CDLL(str(path))
        _LIB.orc_expf_export.restype = ctypes.c_float
        _LIB.orc_expf_export.argtypes = [ctypes.c_float]
    return _LIB


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def topk_gating(gating: torch.Tensor, topk: int, renormalize: bool, bias=None, softmax=True,
                routed_scaling_factor: float = 1.0):
    """-> (weights f32 [T,K], ids i32 [T,K], token_expert_indices i32 [T,K])"""
    T, E = gating.shape
    g = gating.float().contiguous()
    w = torch.empty(T, topk, dtype=torch.float32)
    idx = torch.empty(T, topk, dtype=torch.int32)
    src = torch.empty(T, topk, dtype=torch.int32)
    b = bias.float().contiguous() if bias is not None else None
    lib().orc_topk_gating(_p(g), _DT[gating.dtype], ctypes.c_int64(T), E, topk, int(softmax),
                          int(renormalize), _p(b), ctypes.c_double(routed_scaling_factor),
                          _p(w), _p(idx), _p(src))
    return w, idx, src


def topk_softplus_sqrt(gating: torch.Tensor, topk: int, renormalize: bool, routed_scaling_factor: float = 1.0,
                       bias=None, input_ids=None, tid2eid=None):
    """-> (weights f32 [T,K], ids i32 [T,K], token_expert_indices i32 [T,K])"""
    T, E = gating.shape
    g = gating.float().contiguous()
    w = torch.empty(T, topk, dtype=torch.float32)
    idx = torch.empty(T, topk, dtype=torch.int32)
    src = torch.empty(T, topk, dtype=torch.int32)
    b = bias.float().contiguous() if bias is not None else None
    ids = input_ids.long().contiguous() if input_ids is not None else None
    tab = tid2eid.long().contiguous() if tid2eid is not None else None
    lib().orc_topk_softplus_sqrt(_p(g), ctypes.c_int64(T), E, topk, int(renormalize),
                                 ctypes.c_double(routed_scaling_factor), _p(b), _p(ids), _p(tab),
                                 _p(w), _p(idx), _p(src))
    return w, idx, src


def grouped_topk(scores, scores_with_bias, n_group, topk_group, topk, renormalize,
                 routed_scaling_factor):
    """-> (values in scores.dtype [T,K], ids i32 [T,K]); descending biased score."""
    T, E = scores.shape
    s = scores.float().contiguous()
    sb = scores_with_bias.float().contiguous()
    val = torch.empty(T, topk, dtype=torch.float32)
    idx = torch.empty(T, topk, dtype=torch.int32)
    lib().orc_grouped_topk(_p(s), _p(sb), _DT[scores.dtype], ctypes.c_int64(T), E, n_group,
                           topk_group, topk, int(renormalize),
                           ctypes.c_double(routed_scaling_factor), _p(val), _p(idx))
    return val.to(scores.dtype), idx


def moe_align_block_size(topk_ids, num_experts, block_size, sorted_len, expert_ids_len,
                         expert_map=None):
    ids = topk_ids.reshape(-1).to(torch.int64).contiguous()
    sorted_ids = torch.empty(sorted_len, dtype=torch.int32)
    expert_ids = torch.empty(expert_ids_len, dtype=torch.int32)
    post = torch.empty(1, dtype=torch.int32)
    m = expert_map.to(torch.int32).contiguous() if expert_map is not None else None
    lib().orc_moe_align(_p(ids), ctypes.c_int64(ids.numel()), num_experts, block_size, _p(m),
                        _p(sorted_ids), ctypes.c_int64(sorted_len), _p(expert_ids),
                        ctypes.c_int64(expert_ids_len), _p(post))
    return sorted_ids, expert_ids, post


def remap_bookkeeping(topk_ids, expert_map, total_experts, local_experts):
    """-> (rows_per_expert i32 [E_local], row_map i32 [T,K])"""
    ids = topk_ids.reshape(-1).to(torch.int64).contiguous()
    rows = torch.empty(local_experts, dtype=torch.int32)
    row_map = torch.empty(ids.numel(), dtype=torch.int32)
    m = expert_map.to(torch.int32).contiguous() if expert_map is not None else None
    lib().orc_remap_bookkeeping(_p(ids), ctypes.c_int64(ids.numel()), _p(m), total_experts,
                                local_experts, _p(rows), _p(row_map))
    return rows, row_map.reshape(topk_ids.shape)


def init_expert_map(n_local, ep_rank, ep_size):
    m = torch.empty(n_local * ep_size, dtype=torch.int32)
    lib().orc_init_expert_map(_p(m), n_local, ep_rank, ep_size)
    return m


def expf(x: float) -> float:
    return lib().orc_expf_export(ctypes.c_float(x))


def batched_moe_align_block_size(max_tokens_per_batch: int, block_size: int, counts: torch.Tensor):
    """-> (sorted_ids i32, block_ids i32, num_tokens_post_pad i32 [1])"""
    B = counts.numel()
    n = (max_tokens_per_batch + block_size - 1) // block_size * block_size * B
    sorted_ids = torch.empty(n, dtype=torch.int32)
    block_ids = torch.empty(n // block_size, dtype=torch.int32)
    post = torch.empty(1, dtype=torch.int32)
    c = counts.int().contiguous()
    lib().orc_batched_align(_p(c), B, max_tokens_per_batch, block_size, _p(sorted_ids), _p(block_ids), _p(post))
    return sorted_ids, block_ids, post
