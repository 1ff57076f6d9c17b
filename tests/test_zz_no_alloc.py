"""GPU: the allocation-free align entry point, called straight through the C
ABI, must give exactly what the workspace-taking entry point gives - on two
calls in a row, because both share one scratch array that keeps the previous
call's contents.

Who needs it: hosts that bind this library over a foreign-function interface
and get only input / output buffers from their framework (no allocator of
their own), and serving loops that may not call cudaMalloc while serving.
This file sorts last on purpose, so a run that stops at the first failure has
already run every other test.
"""
import ctypes

import pytest
import torch

from conftest import PKG_DIR

pytestmark = pytest.mark.gpu


def _lib():
    lib = ctypes.CDLL(str(PKG_DIR / "vllm_xpu_kernels" / "libb200moe.so"))
    lib.b200moe_sort_workspace_bytes.restype = ctypes.c_size_t
    lib.b200moe_noalloc_scratch_capacity.restype = ctypes.c_size_t
    lib.b200moe_last_error.restype = ctypes.c_char_p
    return lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _align(lib, ids, E, bs, noalloc, expert_map=None):
    dev = ids.device
    numel = ids.numel()
    n = numel + E * (bs - 1)
    nb = (n + bs - 1) // bs
    s = torch.full((n,), -7, dtype=torch.int32, device=dev)
    e = torch.full((nb,), -7, dtype=torch.int32, device=dev)
    p = torch.full((1,), -7, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    I32 = {torch.int32: 5, torch.int64: 6}[ids.dtype]
    emap = _ptr(expert_map) if expert_map is not None else None
    if noalloc:
        rc = lib.b200moe_moe_align_block_size_noalloc(
            _ptr(ids), I32, ctypes.c_int64(numel), E, bs, _ptr(s), ctypes.c_int64(n), _ptr(e),
            ctypes.c_int64(nb), _ptr(p), emap, stream)
    else:
        need = lib.b200moe_sort_workspace_bytes(ctypes.c_int64(numel), E)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
        rc = lib.b200moe_moe_align_block_size(
            _ptr(ids), I32, ctypes.c_int64(numel), E, bs, _ptr(s), ctypes.c_int64(n), _ptr(e),
            ctypes.c_int64(nb), _ptr(p), emap, _ptr(ws), ctypes.c_size_t(need), stream)
    assert rc == 0, lib.b200moe_last_error()
    torch.cuda.synchronize()
    return s, e, p


def test_noalloc_align_matches_workspace_align_twice_in_a_row():
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    # two different problems back to back: the second runs on the first one's leftovers
    cases = [(4096, 8, 128, 64), (3000, 6, 200, 16)]
    assert all(lib.b200moe_sort_workspace_bytes(ctypes.c_int64(m * k), E) > 0 for m, k, E, _ in cases), \
        "the cases must take the scratch-using multi-block path"
    for (m, topk, E, bs) in cases:
        ids = torch.randint(0, E, (m, topk), generator=g, dtype=torch.int32).to(dev)
        ref = _align(lib, ids, E, bs, noalloc=False)
        got = _align(lib, ids, E, bs, noalloc=True)
        for a, b in zip(ref, got):
            assert torch.equal(a, b)  # integer outputs: exact
    # a small problem (single-block path, no scratch at all) also goes through
    ids = torch.randint(0, 8, (16, 2), generator=g, dtype=torch.int32).to(dev)
    for a, b in zip(_align(lib, ids, 8, 4, False), _align(lib, ids, 8, 4, True)):
        assert torch.equal(a, b)


def test_noalloc_align_with_int64_ids_and_an_expert_map():
    # the same entry point with the other id width and with the id -> local expert map of an
    # expert-parallel rank (-1 = not on this rank: those slots are dropped)
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(1)
    m, topk, E, bs = 2500, 4, 64, 32
    ids = torch.randint(0, E, (m, topk), generator=g, dtype=torch.int64).to(dev)
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[16:32] = torch.arange(16, dtype=torch.int32)
    emap = emap.to(dev)
    for _ in range(2):
        for a, b in zip(_align(lib, ids, E, bs, False, emap), _align(lib, ids, E, bs, True, emap)):
            assert torch.equal(a, b)


def test_noalloc_align_refuses_requests_beyond_its_scratch():
    lib = _lib()
    cap = lib.b200moe_noalloc_scratch_capacity()
    numel, E = 1 << 20, 512
    assert lib.b200moe_sort_workspace_bytes(ctypes.c_int64(numel), E) > cap
    dev = torch.device("cuda", 0)
    dummy = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = lib.b200moe_moe_align_block_size_noalloc(
        _ptr(dummy), 5, ctypes.c_int64(numel), E, 16, _ptr(dummy), ctypes.c_int64(8), _ptr(dummy),
        ctypes.c_int64(8), _ptr(dummy), None, None)
    assert rc == -4
    assert b"built-in buffer holds" in lib.b200moe_last_error()
