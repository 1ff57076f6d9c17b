"""GPU parity: router kernels against the plain-C oracle (bit-exact ids,
weights and source indices) and against the reference-made golden vectors."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV, topk_sigmoid, topk_softmax
from oracle import c_oracle as co

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,E,K", [(64, 8, 2), (1, 8, 2), (33, 128, 8), (2048, 128, 4), (17, 60, 6),
                                   (1000, 256, 8), (5, 512, 4), (3, 1000, 8), (7, 1, 1), (9, 3, 2)])
@pytest.mark.parametrize("renorm", [True, False])
@pytest.mark.parametrize("with_bias", [False, True])
def test_topk_softmax_bit_exact(native, T, E, K, renorm, with_bias):
    g = torch.Generator().manual_seed(T * 131 + E)
    gating = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.1 if with_bias else None
    w, ids, src = topk_softmax(gating.to(DEV), K, renorm, bias.to(DEV) if with_bias else None)
    ow, oi, osrc = co.topk_gating(gating, K, renorm, bias, True)
    assert torch.equal(ids.cpu(), oi)
    assert torch.equal(src.cpu(), osrc)
    assert torch.equal(w.cpu(), ow), f"max diff {(w.cpu() - ow).abs().max()}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64, torch.uint32])
def test_topk_sigmoid_bit_exact(native, dtype, index_dtype):
    g = torch.Generator().manual_seed(11)
    gating = torch.randn(77, 256, generator=g).to(dtype)
    bias = torch.randn(256, generator=g) * 0.1
    w, ids, src = topk_sigmoid(gating.to(DEV), 8, True, bias.to(DEV), 2.5, index_dtype)
    ow, oi, _ = co.topk_gating(gating, 8, True, bias, False, 2.5)
    assert torch.equal(ids.cpu().to(torch.int64), oi.to(torch.int64))
    assert torch.equal(w.cpu(), ow)
    # softmax with 16-bit logits too
    w, ids, _ = topk_softmax(gating.to(DEV), 4, False, None, index_dtype)
    ow, oi, _ = co.topk_gating(gating, 4, False, None, True)
    assert torch.equal(ids.cpu().to(torch.int64), oi.to(torch.int64)) and torch.equal(w.cpu(), ow)


def test_topk_against_reference_vectors(native):
    for c in load_golden("routing_topk.pt"):
        b = c["bias"].to(DEV) if c["bias"] is not None else None
        w, ids, _ = topk_softmax(c["gating"].to(DEV), c["topk"], c["renormalize"], b)
        assert torch.equal(ids.cpu(), c["softmax_ids"])
        torch.testing.assert_close(w.cpu(), c["softmax_w"], rtol=2e-6, atol=1e-7)
        w, ids, _ = topk_sigmoid(c["gating"].to(DEV), c["topk"], c["renormalize"], b,
                                 c["routed_scaling_factor"])
        assert torch.equal(ids.cpu(), c["sigmoid_ids"])
        torch.testing.assert_close(w.cpu(), c["sigmoid_w"], rtol=2e-6, atol=1e-7)


def test_topk_ties_go_to_the_lower_index_and_empty_input(native):
    gating = torch.zeros(4, 16, device=DEV)
    w, ids, _ = topk_softmax(gating, 3, True)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 4
    assert torch.allclose(w.cpu(), torch.full((4, 3), 1 / 3))
    w, ids, _ = topk_softmax(torch.empty(0, 16, device=DEV), 3, True)
    assert w.shape == (0, 3)
    with pytest.raises(RuntimeError, match="int32, uint32 or int64"):
        topk_softmax(gating, 3, True, index_dtype=torch.int16)


@pytest.mark.parametrize("T,E,ng,tg,K,rsf", [(64, 256, 8, 4, 8, 2.5), (1, 256, 8, 4, 8, 2.5),
                                              (33, 16, 8, 2, 2, 1.0), (1024, 256, 8, 4, 8, 2.5),
                                              (19, 64, 4, 2, 6, 1.0), (5, 384, 1, 1, 8, 1.0),
                                              (6, 96, 32, 5, 3, 1.5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("renorm", [True, False])
def test_grouped_topk_bit_exact(native, T, E, ng, tg, K, rsf, dtype, renorm):
    g = torch.Generator().manual_seed(E * 7 + T)
    scores = torch.sigmoid(torch.randn(T, E, generator=g)).to(dtype)
    swb = (scores.float() + torch.randn(E, generator=g) * 0.1).to(dtype)
    v, i = torch.ops._moe_C.grouped_topk(scores.to(DEV), swb.to(DEV), ng, tg, K, renorm, rsf)
    ov, oi = co.grouped_topk(scores, swb, ng, tg, K, renorm, rsf)
    assert i.dtype == torch.int32 and v.dtype == dtype
    assert torch.equal(i.cpu(), oi)
    assert torch.equal(v.cpu(), ov)


def test_grouped_topk_reference_vectors_ties_and_errors(native):
    for c in load_golden("routing_grouped.pt"):
        scores = torch.softmax(c["gating"], -1) if c["scoring"] == "softmax" else c["gating"].sigmoid()
        swb = scores + c["bias"].unsqueeze(0)
        v, i = torch.ops._moe_C.grouped_topk(scores.to(DEV), swb.to(DEV), c["n_group"], c["topk_group"],
                                             c["topk"], c["renormalize"], c["routed_scaling_factor"])
        assert [sorted(r) for r in i.cpu().tolist()] == [sorted(r) for r in c["ids"].tolist()]
        o1, o2 = i.cpu().long().argsort(-1), c["ids"].long().argsort(-1)
        torch.testing.assert_close(v.cpu().gather(1, o1), c["weights"].gather(1, o2), rtol=2e-6, atol=1e-7)
    # all scores equal: groups 0..tg-1 survive, experts in index order
    s = torch.full((2, 64), 0.5, device=DEV)
    v, i = torch.ops._moe_C.grouped_topk(s, s, 8, 2, 4, True, 1.0)
    assert i.cpu().tolist() == [[0, 1, 2, 3]] * 2
    # no finite score at all: experts 0..K-1, weight 1/K
    bad = torch.full((1, 64), float("-inf"), device=DEV)
    v, i = torch.ops._moe_C.grouped_topk(bad, bad, 8, 2, 4, True, 1.0)
    assert i.cpu().tolist() == [[0, 1, 2, 3]] and torch.allclose(v.cpu(), torch.full((1, 4), 0.25))
    with pytest.raises(RuntimeError, match="divisible by n_group"):
        torch.ops._moe_C.grouped_topk(s, s, 7, 2, 4, True, 1.0)
    with pytest.raises(RuntimeError, match="n_group should be smaller than or equal to 32"):
        torch.ops._moe_C.grouped_topk(s, s, 64, 2, 4, True, 1.0)


def _softplus_sqrt(gating, K, renorm, rsf, bias=None, input_ids=None, table=None, index_dtype=torch.int32):
    T = gating.shape[0]
    w = torch.empty(T, K, dtype=torch.float32, device=DEV)
    ids = torch.empty(T, K, dtype=index_dtype, device=DEV)
    src = torch.empty(T, K, dtype=torch.int32, device=DEV)
    mv = lambda t: t.to(DEV) if t is not None else None
    torch.ops._moe_C.topk_softplus_sqrt(w, ids, src, gating.to(DEV), renorm, rsf, mv(bias), mv(input_ids), mv(table))
    return w.cpu(), ids.cpu(), src.cpu()


@pytest.mark.parametrize("T", [1, 33, 128, 1024])
@pytest.mark.parametrize("E", [128, 256, 384, 512, 60])
@pytest.mark.parametrize("K", [6, 8, 16])
@pytest.mark.parametrize("renorm,rsf", [(True, 1.0), (False, 1.5)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_topk_softplus_sqrt_bit_exact(native, T, E, K, renorm, rsf, dtype):
    """Parameters of tests/test_topk_softplus_sqrt.py:243-256 of the reference; ids,
    weights and source indices equal to the C oracle bit for bit."""
    g = torch.Generator().manual_seed(T + E + K)
    gating = (torch.randn(T, E, generator=g) * 3).to(dtype)
    bias = torch.randn(E, generator=g)
    for b in (bias, None):
        w, ids, src = _softplus_sqrt(gating, K, renorm, rsf, b)
        ow, oi, osrc = co.topk_softplus_sqrt(gating, K, renorm, rsf, b)
        assert torch.equal(ids, oi) and torch.equal(src, osrc)
        assert torch.equal(w, ow), f"max diff {(w - ow).abs().max()}"


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_topk_softplus_sqrt_hash_and_reference_vectors(native, index_dtype):
    g = torch.Generator().manual_seed(5)
    T, E, K = 100, 256, 8
    gating = torch.randn(T, E, generator=g)
    gating[0, :4] = torch.tensor([float("inf"), float("nan"), 25.0, -50.0])
    table = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(64)]).to(index_dtype)
    table[0, :4] = torch.tensor([0, 1, 2, 3])
    input_ids = torch.randint(0, 64, (T,), generator=g).to(index_dtype)
    input_ids[0] = 0
    w, ids, src = _softplus_sqrt(gating, K, True, 2.5, None, input_ids, table, index_dtype)
    ow, oi, osrc = co.topk_softplus_sqrt(gating, K, True, 2.5, None, input_ids, table)
    assert torch.equal(ids.long(), oi.long()) and torch.equal(src, osrc) and torch.equal(w, ow)
    assert torch.equal(ids.long(), table[input_ids.long()].long())
    with pytest.raises(RuntimeError, match="input_ids is required for hash MoE"):
        _softplus_sqrt(gating, K, True, 1.0, None, None, table, index_dtype)
    if index_dtype == torch.int32:
        for c in load_golden("routing_softplus_sqrt.pt"):
            w, ids, _ = _softplus_sqrt(c["gating"], c["topk"], c["renormalize"], c["routed_scaling_factor"],
                                       c["bias"], c["input_ids"], c["tid2eid"])
            s_ref, i_ref = c["ids"].sort(dim=-1)
            s_our, i_our = ids.sort(dim=-1)
            assert torch.equal(s_ref, s_our)
            torch.testing.assert_close(c["weights"].gather(1, i_ref), w.gather(1, i_our), atol=2e-2, rtol=1e-2)
