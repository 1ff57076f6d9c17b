"""GPU parity: moe_align_block_size, remap_hidden_states (plain and fused with
the fp8 group quantisation) and init_expert_map against the oracle; exact."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV, align_sizes, moe_align_block_size, remap
from oracle import c_oracle as co
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu


def _ids(m, topk, E, gen):
    return torch.stack([torch.randperm(E, generator=gen)[:topk] for _ in range(m)]).to(torch.int32)


@pytest.mark.parametrize("m,topk,E,bs", [(1, 1, 32, 32), (3, 2, 32, 128), (256, 2, 160, 32), (64, 8, 256, 64),
                                         (2256, 2, 32, 128), (4096, 8, 256, 128), (300, 16, 257, 32),
                                         (16384, 8, 128, 64), (1, 32, 32, 32), (0, 2, 8, 16)])
@pytest.mark.parametrize("pad", [False, True])
def test_moe_align_exact(native, m, topk, E, bs, pad):
    g = torch.Generator().manual_seed(m + E)
    if m <= 512:
        ids = _ids(m, topk, E, g) if m else torch.empty(0, topk, dtype=torch.int32)
    else:
        ids = torch.randint(0, E, (m, topk), generator=g, dtype=torch.int32)
    s, e, p = moe_align_block_size(ids.to(DEV), bs, E, pad_sorted_ids=pad)
    n, nb = align_sizes(ids.numel(), E, bs, pad)
    os_, oe, op = co.moe_align_block_size(ids, E, bs, n, nb)
    assert torch.equal(p.cpu(), op)
    assert torch.equal(e.cpu(), oe)
    assert torch.equal(s.cpu(), os_)
    # properties the reference's test states (tests/test_moe_align_block_size.py:236-246)
    assert int(p) % bs == 0 and int(p) >= ids.numel()
    assert int((s.cpu() < ids.numel()).sum()) == ids.numel()


def test_moe_align_reference_vectors_map_determinism_dtypes(native):
    for c in load_golden("moe_align.pt"):
        emap = c["expert_map"].to(DEV) if c["expert_map"] is not None else None
        s, e, p = moe_align_block_size(c["topk_ids"].to(DEV), c["block_size"], c["num_experts"], emap)
        assert torch.equal(p.cpu(), c["num_tokens_post_pad"])
        assert torch.equal(e.cpu(), c["expert_ids"])
        assert torch.equal(s.cpu(), c["sorted_ids"])
    g = torch.Generator().manual_seed(42)
    ids = torch.randint(0, 32, (128, 2), generator=g, dtype=torch.int32).to(DEV)
    first = moe_align_block_size(ids, 64, 32)
    for _ in range(4):
        again = moe_align_block_size(ids, 64, 32)
        assert all(torch.equal(a, b) for a, b in zip(first, again))
    # int64 ids and ids >= num_experts (dropped)
    ids64 = torch.tensor([[0, 5], [9, 1], [1, 1]], dtype=torch.int64)
    s, e, p = moe_align_block_size(ids64.to(DEV), 4, 4)
    os_, oe, op = co.moe_align_block_size(ids64, 4, 4, s.numel(), e.numel())
    assert torch.equal(s.cpu(), os_) and torch.equal(e.cpu(), oe) and torch.equal(p.cpu(), op)
    with pytest.raises(RuntimeError, match="padded_num_experts must be less than 1024"):
        moe_align_block_size(ids, 16, 1000)


@pytest.mark.parametrize("T,H,E_tot,K,use_map", [(8, 32, 16, 2, False), (33, 64, 16, 4, True), (1, 7168, 256, 8, False),
                                                 (64, 2048, 128, 8, False), (700, 128, 64, 6, True),
                                                 (5000, 64, 256, 8, True), (4096, 128, 8, 2, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_remap_hidden_states_exact(native, T, H, E_tot, K, use_map, dtype):
    g = torch.Generator().manual_seed(T + H)
    hidden = torch.randn(T, H, generator=g).to(dtype)
    if T <= 700:
        ids = torch.stack([torch.randperm(E_tot, generator=g)[:K] for _ in range(T)]).to(torch.int64)
    else:
        ids = torch.randint(0, E_tot, (T, K), generator=g, dtype=torch.int64)
    if use_map:
        E_loc = E_tot // 4
        emap = torch.full((E_tot,), -1, dtype=torch.int32)
        emap[E_loc:2 * E_loc] = torch.arange(E_loc, dtype=torch.int32)
    else:
        E_loc, emap = E_tot, None
    remapped, _, rows, row_map = remap(hidden.to(DEV), None, ids.to(DEV), emap.to(DEV) if use_map else None,
                                       E_tot, E_loc)
    orows, omap = co.remap_bookkeeping(ids, emap, E_tot, E_loc)
    assert torch.equal(rows.cpu(), orows)
    assert torch.equal(row_map.cpu(), omap)
    # every routed slot's row holds its token (the reference's check un-permutes the same way)
    sel = omap.reshape(-1) >= 0
    tok = (torch.arange(T * K) // K)[sel]
    assert torch.equal(remapped.cpu()[omap.reshape(-1)[sel].long()], hidden[tok])


def test_remap_reference_vectors_scales_and_fp8(native):
    for c in load_golden("remap.pt"):
        emap = c["expert_map"].to(DEV) if c["expert_map"] is not None else None
        remapped, _, rows, row_map = remap(c["hidden"].to(DEV), None, c["topk_ids"].to(DEV), emap,
                                           c["total_experts"], c["local_experts"])
        assert torch.equal(rows.cpu(), c["rows_per_expert"]) and torch.equal(row_map.cpu(), c["row_map"])
        n = int(rows.sum())
        assert torch.equal(remapped.cpu()[:n], c["remapped"][:n])
    # fp8 rows with fp32 block scales, int32 ids
    g = torch.Generator().manual_seed(5)
    q = torch.randn(40, 256, generator=g).to(torch.float8_e4m3fn)
    s = torch.rand(40, 2, generator=g)
    ids = torch.randint(0, 8, (40, 4), generator=g, dtype=torch.int32)
    remapped, rs, rows, row_map = remap(q.to(DEV), s.to(DEV), ids.to(DEV), None, 8, 8)
    oq, os_, orows, omap = to.remap_hidden_states(q, s, ids, None, 8)
    assert torch.equal(row_map.cpu(), omap) and torch.equal(rows.cpu(), orows)
    assert torch.equal(remapped.cpu().view(torch.uint8), oq.view(torch.uint8))
    assert torch.equal(rs.cpu(), os_)
    # e8m0 (1-byte) scales with an odd row length exercise the byte copy
    s8 = torch.randint(100, 140, (40, 5), generator=g, dtype=torch.int32).to(torch.uint8)
    _, rs8, _, _ = remap(q.to(DEV), s8.to(DEV), ids.to(DEV), None, 8, 8)
    _, os8, _, _ = to.remap_hidden_states(q, s8, ids, None, 8)
    assert torch.equal(rs8.cpu(), os8)


@pytest.mark.parametrize("T,H,E,K", [(16, 2048, 128, 8), (3, 7168, 32, 8), (600, 256, 16, 4)])
def test_remap_quant_fp8_exact(native, T, H, E, K):
    g = torch.Generator().manual_seed(T)
    x = (torch.randn(T, H, generator=g) * 3).to(torch.bfloat16)
    x[0, :128] = 0  # an all-zero group hits the scale floor
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    rq = torch.zeros(T * K, H, dtype=torch.float8_e4m3fn, device=DEV)
    rs = torch.zeros(T * K, H // 128, dtype=torch.float32, device=DEV)
    rows = torch.empty(E, dtype=torch.int32, device=DEV)
    row_map = torch.empty(T, K, dtype=torch.int32, device=DEV)
    torch.ops._moe_C.b200_remap_quant_fp8(x.to(DEV), rq, rs, None, rows, row_map, ids.to(DEV), E, E)
    q, s = to.per_token_group_fp8_quant(x, 128, 1e-10)
    oq, os_, orows, omap = to.remap_hidden_states(q, s, ids, None, E)
    assert torch.equal(row_map.cpu(), omap) and torch.equal(rows.cpu(), orows)
    assert torch.equal(rs.cpu(), os_)
    assert torch.equal(rq.cpu().view(torch.uint8), oq.view(torch.uint8))


def test_init_expert_map(native):
    for (n, r, s) in [(4, 0, 4), (4, 3, 4), (32, 5, 8), (300, 1, 3)]:
        m = torch.empty(n * s, dtype=torch.int32, device=DEV)
        torch.ops._moe_C.init_expert_map(m, n, r, s)
        assert torch.equal(m.cpu(), co.init_expert_map(n, r, s))
    with pytest.raises(RuntimeError, match="expert_map must be int32"):
        torch.ops._moe_C.init_expert_map(torch.empty(8, dtype=torch.int64, device=DEV), 4, 0, 2)


@pytest.mark.parametrize("max_tokens", [13, 16, 512])
@pytest.mark.parametrize("num_batches", [1, 8, 64, 1000])
@pytest.mark.parametrize("block", [8, 16, 64])
@pytest.mark.parametrize("empty", [False, True])
def test_batched_moe_align_block_size_exact(native, max_tokens, num_batches, block, empty):
    """Parameters of tests/test_moe_align_block_size.py:336-339 of the reference (plus a
    1000-batch case); exact against the C oracle and the recorded reference values."""
    g = torch.Generator().manual_seed(max_tokens + num_batches + block)
    counts = torch.randint(0, max_tokens + 1, (num_batches,), generator=g, dtype=torch.int32)
    if empty:
        counts[torch.randperm(num_batches, generator=g)[:num_batches // 2]] = 0
    n = (max_tokens + block - 1) // block * block * num_batches
    s = torch.empty(n, dtype=torch.int32, device=DEV)
    b = torch.empty(n // block, dtype=torch.int32, device=DEV)
    p = torch.empty(1, dtype=torch.int32, device=DEV)
    torch.ops._moe_C.batched_moe_align_block_size(max_tokens, block, counts.to(DEV), s, b, p)
    os_, ob, op = co.batched_moe_align_block_size(max_tokens, block, counts)
    assert torch.equal(s.cpu(), os_) and torch.equal(b.cpu(), ob) and torch.equal(p.cpu(), op)


def test_batched_moe_align_reference_vectors(native):
    for c in load_golden("batched_align.pt"):
        s = torch.empty_like(c["sorted_ids"], device=DEV)
        b = torch.empty_like(c["block_ids"], device=DEV)
        p = torch.empty(1, dtype=torch.int32, device=DEV)
        torch.ops._moe_C.batched_moe_align_block_size(c["max_tokens"], c["block"], c["counts"].to(DEV), s, b, p)
        assert torch.equal(s.cpu(), c["sorted_ids"]) and torch.equal(b.cpu(), c["block_ids"])
        assert torch.equal(p.cpu(), c["num_post_pad"])
