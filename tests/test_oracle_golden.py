"""CPU: the oracle (torch restatement and plain-C restatement) against the
golden vectors produced by the reference's own pure-torch test references."""
import torch

from conftest import load_golden
from oracle import c_oracle as co
from oracle import torch_oracle as to


def _rows_as_sets(ids):
    return [sorted(r) for r in ids.tolist()]


def test_topk_softmax_sigmoid_against_reference_vectors():
    for c in load_golden("routing_topk.pt"):
        w, ids = to.topk_softmax(c["gating"], c["topk"], c["renormalize"], c["bias"])
        assert torch.equal(ids, c["softmax_ids"])
        assert torch.equal(w, c["softmax_w"])
        w, ids = to.topk_sigmoid(c["gating"], c["topk"], c["renormalize"], c["bias"],
                                 c["routed_scaling_factor"])
        assert torch.equal(ids, c["sigmoid_ids"])
        assert torch.equal(w, c["sigmoid_w"])
        # plain-C restatement: ids exact, weights to float rounding (its exp and its
        # summation order are its own; the reference's bar is atol 2e-2)
        cw, cids, src = co.topk_gating(c["gating"], c["topk"], c["renormalize"], c["bias"], True)
        assert torch.equal(cids, c["softmax_ids"])
        torch.testing.assert_close(cw, c["softmax_w"], rtol=2e-6, atol=1e-7)
        T = c["gating"].shape[0]
        expect_src = torch.arange(c["topk"]).unsqueeze(0) * T + torch.arange(T).unsqueeze(1)
        assert torch.equal(src, expect_src.to(torch.int32))
        cw, cids, _ = co.topk_gating(c["gating"], c["topk"], c["renormalize"], c["bias"], False,
                                     c["routed_scaling_factor"])
        assert torch.equal(cids, c["sigmoid_ids"])
        torch.testing.assert_close(cw, c["sigmoid_w"], rtol=2e-6, atol=1e-7)


def test_grouped_topk_against_reference_vectors():
    for c in load_golden("routing_grouped.pt"):
        scores = torch.softmax(c["gating"], -1) if c["scoring"] == "softmax" else c["gating"].sigmoid()
        swb = scores + c["bias"].unsqueeze(0)
        for fn in (to.grouped_topk, co.grouped_topk):
            w, ids = fn(scores, swb, c["n_group"], c["topk_group"], c["topk"], c["renormalize"],
                        c["routed_scaling_factor"])
            # the reference uses torch.topk(sorted=False): compare each row as a set,
            # and the weights after sorting both sides by expert id
            assert _rows_as_sets(ids) == _rows_as_sets(c["ids"])
            o1, o2 = ids.long().argsort(-1), c["ids"].long().argsort(-1)
            torch.testing.assert_close(w.float().gather(1, o1), c["weights"].gather(1, o2),
                                       rtol=2e-6, atol=1e-7)
            # definite order: descending biased score
            picked = swb.gather(1, ids.long())
            assert bool((picked[:, :-1] >= picked[:, 1:]).all())


def test_grouped_topk_c_equals_torch_restatement():
    g = torch.Generator().manual_seed(3)
    scores = torch.rand(40, 256, generator=g)
    swb = scores + torch.randn(256, generator=g) * 0.1
    w1, i1 = to.grouped_topk(scores, swb, 8, 4, 8, True, 2.5)
    w2, i2 = co.grouped_topk(scores, swb, 8, 4, 8, True, 2.5)
    assert torch.equal(i1, i2)
    torch.testing.assert_close(w1, w2, rtol=2e-6, atol=1e-7)
    # a row without any finite score falls back to experts 0..K-1 with weight 1/K
    bad = torch.full((1, 256), float("-inf"))
    w, i = co.grouped_topk(bad, bad, 8, 4, 8, True, 2.5)
    assert i.tolist() == [list(range(8))] and torch.allclose(w, torch.full((1, 8), 0.125))


def test_moe_align_against_reference_vectors():
    for c in load_golden("moe_align.pt"):
        n_sorted, n_blocks = c["sorted_ids"].numel(), c["expert_ids"].numel()
        for fn in (
            lambda: to.moe_align_block_size(c["topk_ids"], c["block_size"], c["num_experts"],
                                            n_sorted, n_blocks, c["expert_map"]),
            lambda: co.moe_align_block_size(c["topk_ids"], c["num_experts"], c["block_size"],
                                            n_sorted, n_blocks, c["expert_map"]),
        ):
            s, e, post = fn()
            assert torch.equal(post, c["num_tokens_post_pad"])
            assert torch.equal(e, c["expert_ids"])
            assert torch.equal(s, c["sorted_ids"])  # the golden is stable too


def test_remap_against_reference_vectors():
    for c in load_golden("remap.pt"):
        remapped, _, rows, row_map = to.remap_hidden_states(c["hidden"], None, c["topk_ids"],
                                                            c["expert_map"], c["local_experts"])
        assert torch.equal(rows, c["rows_per_expert"])
        assert torch.equal(row_map, c["row_map"])
        n = int(rows.sum())
        assert torch.equal(remapped[:n], c["remapped"][:n])
        crows, cmap = co.remap_bookkeeping(c["topk_ids"], c["expert_map"], c["total_experts"],
                                           c["local_experts"])
        assert torch.equal(crows, c["rows_per_expert"]) and torch.equal(cmap, c["row_map"])


def test_init_expert_map_semantics():
    for (n, r, s) in [(4, 0, 4), (4, 3, 4), (32, 5, 8)]:
        a, b = to.init_expert_map(n, r, s), co.init_expert_map(n, r, s)
        assert torch.equal(a, b)
        assert a[r * n:(r + 1) * n].tolist() == list(range(n)) and int((a >= 0).sum()) == n


def test_gather_activation_quant_dequant_against_reference_vectors():
    for c in load_golden("moe_gather.pt"):
        out = to.moe_gather(c["moe_output"], c["topk_weights"], c["row_map"], torch.bfloat16)
        assert torch.equal(out, c["output"])
    a = load_golden("activations.pt")
    assert torch.equal(to.silu_and_mul(a["x_bf16"]), a["silu_bf16"])
    assert torch.equal(to.swigluoai_and_mul(a["x_bf16"]), a["swiglu_bf16"])
    assert torch.equal(to.silu_and_mul(a["x_f32"]), a["silu_f32"])
    assert torch.equal(to.swigluoai_and_mul(a["x_f32"]), a["swiglu_f32"])
    q = load_golden("fp8_group_quant.pt")
    oq, os_ = to.per_token_group_fp8_quant(q["x"], 128, 1e-10)
    # the reference's golden divides by the scale, the kernel multiplies by its
    # reciprocal: scales agree exactly, codes may differ by one e4m3 step
    assert torch.equal(os_, q["s"])
    diff = (oq.float() - q["q"].float()).abs()
    assert float((diff > 0).float().mean()) < 0.02
    assert bool((diff <= q["q"].float().abs() * 0.13 + 2 ** -9).all())
    d = load_golden("dequant.pt")
    assert torch.equal(to.dequant_mxfp4(d["mxfp4_packed"], d["mxfp4_scale"]), d["mxfp4_deq"])
    assert torch.equal(to.dequant_fp8_block_wei(d["fp8_w"], d["fp8_scale"]), d["fp8_deq"])


def test_layer_bf16_against_reference_vectors():
    for c in load_golden("layer_bf16.pt"):
        out = to.fused_moe_bf16(c["x"], c["w13"], c["w13_bias"], c["w2"], c["w2_bias"],
                                c["topk_weights"], c["topk_ids"], c["num_experts"],
                                c.get("ep_rank", 0), c.get("ep_size", 1), c["clamp"])
        torch.testing.assert_close(out, c["output"], rtol=0, atol=0)
        # the staged form (what the kernel path computes) agrees within the
        # reference's own bf16 tolerance
        if c.get("ep_size", 1) == 1:
            staged = to.fused_moe_staged(c["x"], c["w13"].float(), c["w13_bias"], c["w2"].float(),
                                         c["w2_bias"], c["topk_weights"], c["topk_ids"],
                                         c["num_experts"], gemm1_clamp_limit=c["clamp"])
            torch.testing.assert_close(staged, c["output"], rtol=2e-2, atol=2e-2)


def _deq_mxfp4(packed, scales):
    return to.dequant_mxfp4(packed, (torch.log2(scales) + 127).round().to(torch.uint8))


def _close_mxfp4(packed, sc, ref_packed, ref_sc):
    """The reference test's bar (atol = rtol = 0.2 on dequantised values) holds except
    next to a rounding midpoint, where the reference's helper (round to few
    mantissa bits, then round to even) and the op (compare with the midpoints)
    may pick neighbouring codes: those must be rare and one code step apart."""
    a, b = _deq_mxfp4(packed, sc), _deq_mxfp4(ref_packed, ref_sc)
    bad = (a - b).abs() > 0.2 + 0.2 * b.abs()
    assert float(bad.float().mean()) < 0.03
    step = 2.0 * sc.repeat_interleave(32, dim=1)
    assert bool(((a - b).abs() <= step).all())


def test_fused_quant_ops_against_reference_vectors():
    """The oracle's restatements of the four activation + quantisation ops against
    the reference tests' own pure-torch references, at the reference tests' bars
    (tests/test_fused_silu_mul_block_quant.py:122-131, test_fused_silu_mul_mxfp4_quant.py,
    test_mxfp4_quant.py:86-110, test_fused_quant_activation.py:66-70)."""
    fq = load_golden("fused_quant.pt")
    for c in fq["per_block"]:
        q, sc = to.silu_and_mul_per_block_quant(c["x"], c["group"], c["q"].dtype)
        torch.testing.assert_close(sc, c["scales"], rtol=1e-2, atol=1e-5)   # reference ref rounds silu*up to 16 bit
        rep = lambda s: s.repeat_interleave(c["group"], dim=1)
        # the reference's reference rounds silu*up to 16 bits before quantising, the op does not:
        # values on a rounding boundary may land one code apart (one e4m3 step = 12.5 %, one int8 step = scale)
        torch.testing.assert_close(q.float() * rep(sc), c["q"].float() * rep(c["scales"]), rtol=0.13,
                                   atol=max(5e-2, float(sc.max())))
    for c in fq["silu_mxfp4"]:
        packed, sc = to.silu_and_mul_mxfp4_quant(c["x"])
        torch.testing.assert_close(sc, c["scales"], rtol=1e-5, atol=1e-5)
        _close_mxfp4(packed, sc, c["packed"], c["scales"])
    for c in fq["mxfp4"]:
        packed, sc = to.per_token_group_quant_mxfp4(c["x"])
        ref_sc = torch.exp2(c["scale_e8m0"].float() - 127.0)
        torch.testing.assert_close(sc, ref_sc, rtol=1e-5, atol=1e-5)
        _close_mxfp4(packed, sc, c["packed"], ref_sc)
    for c in fq["static"]:
        q = to.silu_and_mul_quant(c["x"], c["scale"])
        torch.testing.assert_close(q.float(), c["q"].float())


def test_other_activations_against_reference_vectors():
    """gelu / gelu_tanh / swiglustep restatements against the reference's native
    forward functions (tests/ops/activation_op.py:86-90, swiglustep_and_mul_op.py:27-33)."""
    for c in load_golden("activations2.pt").values():
        x = c["x"]
        tol = dict(rtol=2e-2, atol=1e-3) if x.dtype == torch.bfloat16 else dict(rtol=2e-3, atol=1e-3)
        torch.testing.assert_close(to.gelu_and_mul(x), c["gelu"], **tol)
        torch.testing.assert_close(to.gelu_and_mul(x, "tanh"), c["gelu_tanh"], **tol)
        torch.testing.assert_close(to.swiglustep_and_mul(x), c["swiglustep"], **tol)


def test_topk_softplus_sqrt_against_reference_vectors():
    """tests/test_topk_softplus_sqrt.py:283-289 of the reference: ids equal as sorted
    sets, weights within atol 2e-2 / rtol 1e-2 after the same sort."""
    for c in load_golden("routing_softplus_sqrt.pt"):
        w, ids, src = co.topk_softplus_sqrt(c["gating"], c["topk"], c["renormalize"], c["routed_scaling_factor"],
                                            c["bias"], c["input_ids"], c["tid2eid"])
        s_ref, i_ref = c["ids"].sort(dim=-1)
        s_our, i_our = ids.sort(dim=-1)
        assert torch.equal(s_ref, s_our)
        torch.testing.assert_close(c["weights"].gather(1, i_ref), w.gather(1, i_our), atol=2e-2, rtol=1e-2)
        T, K = ids.shape
        assert torch.equal(src, (torch.arange(K).view(1, K) * T + torch.arange(T).view(T, 1)).int())


def test_batched_align_against_reference_vectors():
    """Expected values recorded from the reference's own test
    (tests/test_moe_align_block_size.py:340-417), compared exactly."""
    for c in load_golden("batched_align.pt"):
        s, b, p = co.batched_moe_align_block_size(c["max_tokens"], c["block"], c["counts"])
        assert torch.equal(s, c["sorted_ids"]) and torch.equal(b, c["block_ids"]) and torch.equal(p, c["num_post_pad"])


def test_prologue_against_reference_vectors():
    """Legacy fused_moe_prologue: the restatement reproduces what the reference's pure-torch
    ref_prologue gives (tests/fused_moe/test_moe_prologue.py:52-97), byte for byte."""
    from prologue_cases import check_against_reference_vectors, regions, workspace_for
    for c in load_golden("prologue.pt"):
        layout, total = workspace_for(c)
        ws = torch.zeros(total, dtype=torch.uint8)
        x = c["hidden_states"]
        co.fused_moe_prologue(x, c["scales"], c["topk_ids"], c["topk_weights"], ws, x.shape[1], c["block_k"], 0,
                              c["num_experts"])
        check_against_reference_vectors(c, regions(c, ws, layout))
    # expert parallel: rank 1 of 2 keeps experts 8..15 as local 0..7; a repeated expert counts once
    ids = torch.tensor([[3, 9], [9, 9], [15, 8], [0, 1]])
    w = torch.arange(8, dtype=torch.float32).view(4, 2)
    x = torch.arange(4 * 16, dtype=torch.float32).view(4, 16).bfloat16()
    c = dict(hidden_states=x, scales=None, topk=2, num_experts=8, block_k=1, topk_ids=ids, topk_weights=w)
    layout, total = workspace_for(c)
    ws = torch.full((total,), 0xEE, dtype=torch.uint8)
    co.fused_moe_prologue(x, None, ids, w, ws, 16, 1, 1, 8)
    r = regions(c, ws, layout)
    assert r["first"].tolist() == [0, 1, 3, 3, 3, 3, 3, 3, 4]
    assert r["p2u"][:4].tolist() == [1 * 4 + 2, 1 * 4 + 0, 0 * 4 + 1, 0 * 4 + 2]
    assert r["pexp"][:4].tolist() == [0, 1, 1, 7]
    assert r["pscale"][:4].tolist() == [5.0, 1.0, 2.0, 4.0]
    assert torch.equal(r["rows"][:4], x[[2, 0, 1, 2]])


def test_layer_mxfp8_against_reference_vectors():
    """The staged oracle with the mxfp8 recipe (MXFP8 activations, [E,K,N] e4m3 weights with one
    e8m0 scale per 32 K rows) against outputs of the reference's ref_fused_moe("mxfp8")
    (vllm_xpu_kernels/moe_utils.py:236-403).  The simulation rounds the GEMM result to the
    16-bit type before it adds the bias, the kernels add it in fp32; both forms are checked."""
    for c in load_golden("layer_mxfp8.pt"):
        E = c["num_experts"]
        w13, w2 = c["w13"].view(torch.float8_e4m3fn), c["w2"].view(torch.float8_e4m3fn)
        w13d = torch.stack([to.dequant_mxfp8_wei(w13[e], c["w13_scales"][e]).t() for e in range(E)])
        w2d = torch.stack([to.dequant_mxfp8_wei(w2[e], c["w2_scales"][e]).t() for e in range(E)])
        top = float(c["out"].float().abs().max())
        # restated exactly as the simulation does it: agreement to the last bit or two
        sim = to.fused_moe_staged(c["x"], w13d, c["w13_bias"], w2d, c["w2_bias"], c["topk_weights"], c["topk_ids"], E,
                                  activation="silu", act_quant="mxfp8", bias_after_rounding=True)
        assert (sim.float() - c["out"].float()).abs().max() <= 2 ** -7 * top
        # as the kernels do it (bias added in fp32): the reference's own layer tolerance
        out = to.fused_moe_staged(c["x"], w13d, c["w13_bias"], w2d, c["w2_bias"], c["topk_weights"], c["topk_ids"], E,
                                  activation="silu", act_quant="mxfp8")
        torch.testing.assert_close(out.float(), c["out"].float(), rtol=2e-2, atol=4e-2 * top)
