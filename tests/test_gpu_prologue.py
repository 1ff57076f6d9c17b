"""GPU parity: legacy fused_moe_prologue against the reference's vectors and the oracle
(byte-exact in every region the op defines), at the reference test's shapes
(tests/fused_moe/test_moe_prologue.py:12-20, 100-265 of vllm-xpu-kernels)."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV
from oracle import c_oracle as co
from prologue_cases import check_against_reference_vectors, regions, workspace_for

pytestmark = pytest.mark.gpu


def _run_gpu(c, ep_rank=0, ep_size=1, fill=0):
    layout, total = workspace_for(c)
    ws = torch.full((total,), fill, dtype=torch.uint8, device=DEV)
    x, sc = c["hidden_states"], c["scales"]
    torch.ops._moe_C.fused_moe_prologue(x.to(DEV), sc.to(DEV) if sc is not None else None, c["topk_ids"].to(DEV),
                                        c["topk_weights"].to(DEV), ws, x.shape[1], 4 * x.shape[1], c["block_k"],
                                        ep_rank, ep_size, c["num_experts"])
    return ws.cpu(), layout, total


def test_prologue_reference_vectors(native):
    for c in load_golden("prologue.pt"):
        ws, layout, _ = _run_gpu(c)
        check_against_reference_vectors(c, regions(c, ws, layout))


def _random_case(m, hidden, E_total, topk, elem, scale, block_k, seed):
    g = torch.Generator().manual_seed(seed)
    if elem == 2:
        x = torch.randn(m, hidden, generator=g).bfloat16()
    else:
        x = torch.randint(0, 256, (m, hidden), generator=g, dtype=torch.uint8)
    sc = None
    if scale == 4:
        sc = torch.randn(m, hidden // block_k, generator=g)
    elif scale == 1:
        sc = torch.randint(1, 256, (m, hidden // block_k), generator=g, dtype=torch.uint8)
    w, ids = torch.topk(torch.randn(m, E_total, generator=g), k=topk, dim=-1, sorted=False)
    return dict(hidden_states=x, scales=sc, topk=topk, block_k=block_k, topk_ids=ids, topk_weights=w)


@pytest.mark.parametrize("m,hidden,topk", [(1, 5120, 1), (4, 5120, 2), (16, 5120, 2), (8192, 5120, 2), (3000, 264, 8)])
@pytest.mark.parametrize("elem,scale,block_k", [(2, 0, 1), (1, 4, 128), (1, 1, 32), (1, 1, 16)])
@pytest.mark.parametrize("ep", [(0, 1), (1, 2)])
def test_prologue_exact(native, m, hidden, topk, elem, scale, block_k, ep):
    ep_rank, ep_size = ep
    if hidden % block_k:
        hidden = hidden // 128 * 128
    c = _random_case(m, hidden, 16, topk, elem, scale, block_k, m + hidden + topk)
    c["num_experts"] = 16 // ep_size
    ws, layout, total = _run_gpu(c, ep_rank, ep_size, fill=0xEE)
    ref = torch.full((total,), 0xEE, dtype=torch.uint8)
    co.fused_moe_prologue(c["hidden_states"], c["scales"], c["topk_ids"], c["topk_weights"], ref,
                          c["hidden_states"].shape[1], block_k, ep_rank, c["num_experts"])
    # identical everywhere except the three scratch regions of the reference's sort, which
    # neither side writes (both keep the fill byte there)
    assert torch.equal(ws, ref)


def test_prologue_duplicates_and_errors(native):
    ids = torch.tensor([[3, 9], [9, 9], [15, 8], [0, 1]])
    w = torch.arange(8, dtype=torch.float32).view(4, 2)
    x = torch.arange(4 * 16, dtype=torch.float32).view(4, 16).bfloat16()
    c = dict(hidden_states=x, scales=None, topk=2, num_experts=8, block_k=1, topk_ids=ids, topk_weights=w)
    ws, layout, total = _run_gpu(c, 1, 2, fill=0xEE)
    ref = torch.full((total,), 0xEE, dtype=torch.uint8)
    co.fused_moe_prologue(x, None, ids, w, ref, 16, 1, 1, 8)
    assert torch.equal(ws, ref)
    small = torch.zeros(16, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="workspace of"):
        torch.ops._moe_C.fused_moe_prologue(x.to(DEV), None, ids.to(DEV), w.to(DEV), small, 16, 64, 1, 0, 1, 16)
    with pytest.raises(RuntimeError, match="int64"):
        torch.ops._moe_C.fused_moe_prologue(x.to(DEV), None, ids.int().to(DEV), w.to(DEV), small, 16, 64, 1, 0, 1, 16)


def test_prologue_empty_and_nothing_local(native):
    """No rows at all, and rows whose experts all live on another rank: offsets are zero, nothing
    else is written."""
    x = torch.zeros(0, 64, dtype=torch.bfloat16)
    c = dict(hidden_states=x, scales=None, topk=2, num_experts=4, block_k=1,
             topk_ids=torch.zeros(0, 2, dtype=torch.int64), topk_weights=torch.zeros(0, 2))
    ws, layout, total = _run_gpu(c, fill=0xEE)
    r = regions(c, ws, layout)
    assert r["first"].tolist() == [0] * 5
    ids = torch.tensor([[0, 1], [2, 3], [1, 0]])
    x = torch.randn(3, 64).bfloat16()
    c = dict(hidden_states=x, scales=None, topk=2, num_experts=4, block_k=1, topk_ids=ids,
             topk_weights=torch.rand(3, 2))
    ws, layout, total = _run_gpu(c, ep_rank=1, ep_size=2, fill=0xEE)     # rank 1 owns experts 4..7
    ref = torch.full((total,), 0xEE, dtype=torch.uint8)
    co.fused_moe_prologue(x, None, ids, c["topk_weights"], ref, 64, 1, 1, 4)
    assert torch.equal(ws, ref)
    assert regions(c, ws, layout)["first"].tolist() == [0] * 5
