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


def moe_lora_align_block_size(topk_ids, token_lora_mapping, num_experts, block_size, max_loras,
                              max_num_tokens_padded, max_num_m_blocks, sorted_token_ids, expert_ids,
                              num_tokens_post_pad, adapter_enabled, lora_ids, expert_map=None):
    """Writes the three int32 CPU output tensors in place, like the op."""
    ids = topk_ids.reshape(-1).to(torch.int64).contiguous()
    m = expert_map.to(torch.int32).contiguous() if expert_map is not None else None
    for t in (sorted_token_ids, expert_ids, num_tokens_post_pad):
        assert t.dtype == torch.int32 and t.is_contiguous() and t.device.type == "cpu"
    tl = token_lora_mapping.int().contiguous()
    ae = adapter_enabled.int().contiguous()
    li = lora_ids.int().contiguous()
    lib().orc_moe_lora_align(_p(ids), ctypes.c_int64(ids.numel()), int(topk_ids.shape[1]), _p(tl),
                             num_experts, block_size, max_loras, max_num_tokens_padded,
                             max_num_m_blocks, _p(m), _p(ae), _p(li), _p(sorted_token_ids),
                             _p(expert_ids), _p(num_tokens_post_pad))


PROLOGUE_REGIONS = ("permuted_row_to_unpermuted_row", "permuted_token_selected_experts",
                    "unpermuted_row_to_permuted_row", "blocked_expert_counts",
                    "blocked_expert_counts_cumsum", "blocked_row_to_unpermuted_row",
                    "expert_first_token_offset", "permuted_token_final_scales",
                    "overlapped_gemm1_gemm2_inputs", "permuted_act_scales")


def prologue_layout(num_rows, topk, experts, hidden, block_k, elem_bytes, scale_bytes):
    """-> ({region name: byte offset}, total bytes) of the packed prologue workspace."""
    off = (ctypes.c_int64 * 10)()
    total = ctypes.c_int64()
    lib().orc_prologue_layout(ctypes.c_int64(num_rows), topk, experts, ctypes.c_int64(hidden), block_k,
                              elem_bytes, scale_bytes, off, ctypes.byref(total))
    return dict(zip(PROLOGUE_REGIONS, list(off))), total.value


def fused_moe_prologue(x, scales, topk_ids, topk_weights, workspace, hidden_size, block_k, ep_rank,
                       num_experts_on_rank):
    """Fills the uint8 CPU `workspace` in place; x / scales are taken as raw storage."""
    xb = x.contiguous().view(torch.uint8)
    sb = scales.contiguous().view(torch.uint8) if scales is not None else None
    ids = topk_ids.long().contiguous()
    w = topk_weights.float().contiguous()
    assert workspace.dtype == torch.uint8 and workspace.is_contiguous()
    lib().orc_fused_moe_prologue(_p(xb), x.element_size(), _p(sb), scales.element_size() if scales is not None else 0,
                                 _p(ids), _p(w), _p(workspace), ctypes.c_int64(x.shape[0]),
                                 ctypes.c_int64(hidden_size), block_k, int(topk_ids.shape[1]), ep_rank,
                                 num_experts_on_rank)


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
