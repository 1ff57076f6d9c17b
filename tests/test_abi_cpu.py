"""CPU: the C-ABI library loads and exports every symbol include/b200moe.h
declares; argument validation that needs no device; the torch op schemas."""
import ctypes
import re

import pytest
import torch

from conftest import PKG_DIR, ROOT


def _declared_symbols():
    text = (ROOT / "include" / "b200moe.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    path = PKG_DIR / "vllm_xpu_kernels" / "libb200moe.so"
    assert path.exists(), "libb200moe.so is not built (run __graft_entry__.build())"
    return ctypes.CDLL(str(path))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200moe.h but not exported"


def test_status_strings_and_version(lib):
    lib.b200moe_status_string.restype = ctypes.c_char_p
    lib.b200moe_last_error.restype = ctypes.c_char_p
    assert lib.b200moe_abi_version() == 7
    assert lib.b200moe_status_string(0) == b"ok"
    assert b"bad argument" in lib.b200moe_status_string(-1)


def test_argument_checks_reject_before_any_launch(lib):
    lib.b200moe_last_error.restype = ctypes.c_char_p
    # n_group > 32
    rc = lib.b200moe_grouped_topk(None, None, None, None, 0, ctypes.c_int64(4), 64, 64, 2, 2, 1,
                                  ctypes.c_double(1.0), None)
    assert rc == -1 and b"n_group should be smaller than or equal to 32" in lib.b200moe_last_error()
    rc = lib.b200moe_grouped_topk(None, None, None, None, 0, ctypes.c_int64(4), 30, 4, 2, 2, 1,
                                  ctypes.c_double(1.0), None)
    assert rc == -1 and b"divisible by n_group" in lib.b200moe_last_error()
    # align: too many experts
    rc = lib.b200moe_moe_align_block_size(None, 5, ctypes.c_int64(0), 1000, 16, None,
                                          ctypes.c_int64(0), None, ctypes.c_int64(0), None, None,
                                          None, ctypes.c_size_t(0), None)
    assert rc == -1 and b"padded_num_experts must be less than 1024" in lib.b200moe_last_error()
    # workspace sizing: single-block path needs none
    lib.b200moe_sort_workspace_bytes.restype = ctypes.c_size_t
    assert lib.b200moe_sort_workspace_bytes(ctypes.c_int64(2048), 256) == 0
    need = lib.b200moe_sort_workspace_bytes(ctypes.c_int64(131072), 128)
    assert need >= (128 * 512 + 129) * 4


def test_torch_schemas_match_the_reference(native):
    S = torch.ops._moe_C
    sch = S.topk_softmax.default._schema
    assert [a.name for a in sch.arguments] == ["topk_weights", "topk_indices", "token_expert_indices",
                                               "gating_output", "renormalize", "bias"]
    assert [a.is_write for a in sch.arguments] == [True, True, True, False, False, False]
    assert "routed_scaling_factor" in str(S.topk_sigmoid.default._schema)
    assert str(S.grouped_topk.default._schema).endswith("-> (Tensor, Tensor)")
    assert "maybe_expert_map" in str(S.moe_align_block_size.default._schema)
    assert "unpermuted_row_to_permuted_row" in str(S.remap_hidden_states.default._schema)
    assert "int num_experts" in str(S.moe_gather.default._schema)
    assert "Tensor? topk_ids, Tensor? expert_map" in str(S.moe_sum.default._schema)
    assert "int ep_rank, int ep_size" in str(S.init_expert_map.default._schema)
    g = str(torch.ops._xpu_C.cutlass_grouped_gemm_interface.default._schema)
    assert "Tensor ptr_A, Tensor? ptr_A_scale, Tensor ptr_B, Tensor? ptr_B_scale, Tensor? ptr_bias" in g
    assert "float alpha=1.702, float limit=7." in str(torch.ops._C.swigluoai_and_mul.default._schema)
    assert "bool dummy_is_tma_aligned" in str(torch.ops._C.per_token_group_fp8_quant.default._schema)
    assert [a.name for a in torch.ops._C.silu_and_mul.default._schema.arguments] == ["result", "input"]


def test_no_cpu_kernel_is_registered(native):
    # The ops exist for the CUDA dispatch key only: CPU tensors must not run.
    out = torch.empty(2, 4)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops._C.silu_and_mul(out, torch.randn(2, 8))


def _ref_prologue_layout(num_rows, topk, experts, hidden, block_k, elem, scale):
    """The workspace arithmetic of the reference's own test
    (tests/fused_moe/test_moe_prologue.py:42-49, 166-212 of vllm-xpu-kernels)."""
    def tokens_per_block(n, e):
        for t in (32, 64, 128, 256, 512, 1024):
            if (n + t - 1) // t * e <= t:
                return t
        return 1024
    n = num_rows * topk
    blocks = (num_rows + tokens_per_block(num_rows, experts) - 1) // tokens_per_block(num_rows, experts)
    sizes = [n * 4, n * 4, n * 4, experts * blocks * 4, experts * blocks * 4, experts * num_rows * 4,
             (experts + 1) * 8, n * 4, n * hidden * elem, (n * hidden // block_k) * scale]
    off, out = 0, []
    for sz in sizes:
        out.append(off)
        off += (sz + 255) // 256 * 256
    return out, off


@pytest.mark.parametrize("num_rows,topk,experts,hidden,block_k,elem,scale",
                         [(1, 1, 16, 8192, 1, 2, 0), (16, 2, 16, 8192, 128, 1, 4), (8192, 2, 16, 8192, 32, 1, 1),
                          (300, 8, 256, 7168, 128, 1, 4), (4, 1, 2, 4096, 16, 1, 1), (100000, 8, 32, 2880, 32, 1, 1)])
def test_prologue_workspace_layout_matches_the_reference(lib, num_rows, topk, experts, hidden, block_k, elem, scale):
    """The packed workspace of fused_moe_prologue: same ten offsets and total as the reference's test
    computes, from the C ABI (a host-only call) and from the C oracle."""
    from oracle import c_oracle as co
    want_off, want_total = _ref_prologue_layout(num_rows, topk, experts, hidden, block_k, elem, scale)
    off = (ctypes.c_size_t * 10)()
    total = ctypes.c_size_t()
    rc = lib.b200moe_fused_moe_prologue_layout(ctypes.c_int64(num_rows), topk, experts, ctypes.c_int64(hidden),
                                                block_k, elem, scale, off, ctypes.byref(total))
    assert rc == 0 and list(off) == want_off and total.value == want_total
    layout, ototal = co.prologue_layout(num_rows, topk, experts, hidden, block_k, elem, scale)
    assert [layout[k] for k in co.PROLOGUE_REGIONS] == want_off and ototal == want_total
    lib.b200moe_fused_moe_prologue_scratch_bytes.restype = ctypes.c_size_t
    lib.b200moe_sort_workspace_bytes.restype = ctypes.c_size_t
    need = lib.b200moe_fused_moe_prologue_scratch_bytes(ctypes.c_int64(num_rows), topk, experts)
    assert need >= (num_rows * topk + experts) * 4 + lib.b200moe_sort_workspace_bytes(ctypes.c_int64(num_rows * topk), experts)


def test_expert_parallel_owner_map_and_workspace_size(lib):
    """The owner of an expert (contiguous even split, as csrc/moe/init_expert_map.cpp:45-52 of the
    reference encodes it), the argument checks of the peer-memory dispatch, and the scratch size
    the Python layer computes for it."""
    import sys
    sys.path.insert(0, str(PKG_DIR))
    from vllm_xpu_kernels.ep_moe import owner_map
    assert owner_map(256, 8, "cpu").tolist() == [e // 32 for e in range(256)]
    lib.b200moe_ep_dispatch_workspace_bytes.restype = ctypes.c_size_t
    lib.b200moe_last_error.restype = ctypes.c_char_p
    for cap, ep in [(8192, 8), (64, 2), (300, 16), (1, 1)]:
        need = lib.b200moe_ep_dispatch_workspace_bytes(ctypes.c_int64(cap), ep)
        chunks = (cap * ep + 255) // 256
        assert need <= (ep * chunks + ep + 1) * 4 + 256       # what EpPeerFusedMoe allocates
    assert lib.b200moe_ep_dispatch(None, None, 2, None, 5, None, ctypes.c_int64(0), None, None, None,
                                   ctypes.c_size_t(0), None) == -1
    assert b"null peer table" in lib.b200moe_last_error()
