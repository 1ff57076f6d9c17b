"""Generates the golden vectors in this folder from the reference's own
pure-torch test references, run on CPU.

Usage:  python tests/golden/make_golden.py /path/to/vllm-xpu-kernels

The reference's test helpers import its compiled extensions at module level;
those imports are satisfied here with empty stand-in modules, which is enough
because only the pure-torch reference functions are called.  Each .pt file
holds the seeded inputs and the reference's outputs for one op, so that the
checks in tests/test_oracle_golden.py need neither the reference nor this
script at run time.
"""
from __future__ import annotations

import sys
import types
from pathlib import Path

import torch

OUT = Path(__file__).resolve().parent


def _stub(name):
    m = types.ModuleType(name)
    sys.modules[name] = m
    return m


def load_reference(root: str):
    sys.path.insert(0, root)
    import importlib
    pkg = importlib.import_module("vllm_xpu_kernels")  # plain package, no native code
    for sub in ("_C", "_moe_C", "_xpu_C"):
        setattr(pkg, sub, _stub(f"vllm_xpu_kernels.{sub}"))
    import tests.ops.topk_op as topk_op
    import tests.ops.grouped_topk_op as grouped_op
    import tests.test_moe_align_block_size as align_t
    import tests.fused_moe.test_remap_hidden_states as remap_t
    import tests.test_moe_gather as gather_t
    import tests.fused_moe.test_fused_moe as layer_t
    import tests.ops.activation_op as act_op
    import tests.ops.swigluoai_and_mul_op as swi_op
    import tests.test_fp8_quant as fp8_t
    import vllm_xpu_kernels.moe_utils as mu
    import tests.test_fused_silu_mul_block_quant as sbq_t
    import tests.test_fused_silu_mul_mxfp4_quant as smx_t
    import tests.test_fused_quant_activation as sq_t
    import tests.ops.mx_utils as mx_utils
    import tests.ops.swiglustep_and_mul_op as step_op
    import tests.test_topk_softplus_sqrt as sps_t
    import tests.fused_moe.test_moe_prologue as pro_t
    return dict(pro=pro_t, sps=sps_t, step=step_op, sbq=sbq_t, smx=smx_t, sq=sq_t, mxu=mx_utils, topk=topk_op, grouped=grouped_op, align=align_t, remap=remap_t, gather=gather_t,
                layer=layer_t, act=act_op, swi=swi_op, fp8=fp8_t, mu=mu)


def install_cpu_ops():
    """CPU implementations of the few registered ops the reference's eager simulation
    ref_fused_moe (vllm_xpu_kernels/moe_utils.py:236-403) calls around its own torch code.
    They are this repository's restatements of those ops, each checked separately against
    reference-made vectors; everything recipe-specific (MX quantise / dequantise, the matmuls,
    their order and dtypes) stays the reference's own Python."""
    sys.path.insert(0, str(OUT.parents[1]))
    from oracle import torch_oracle as to
    moe = torch.library.Library("_moe_C", "DEF")
    moe.define("remap_hidden_states(Tensor hidden_states, Tensor? hidden_states_scales, "
               "Tensor(a!) remapped_hidden_states, Tensor? remapped_hidden_states_scales, Tensor? expert_map, "
               "Tensor(b!) rows_per_expert, Tensor(c!) unpermuted_row_to_permuted_row, Tensor topk_ids, "
               "int total_experts_num, int local_experts_num) -> ()")
    moe.define("moe_gather(Tensor(a!) output, Tensor moe_output, Tensor topk_weights, "
               "Tensor unpermuted_row_to_permuted_row, int num_experts) -> ()")
    c = torch.library.Library("_C", "DEF")
    c.define("per_token_group_fp8_quant(Tensor input, Tensor(a!) output_q, Tensor(b!) output_s, int group_size, "
             "float eps, float fp8_min, float fp8_max, bool scale_ue8m0, bool a, bool b) -> ()")
    c.define("silu_and_mul(Tensor(a!) out, Tensor input) -> ()")

    def remap(hidden_states, hidden_states_scales, remapped_hidden_states, remapped_hidden_states_scales,
              expert_map, rows_per_expert, unpermuted_row_to_permuted_row, topk_ids, total_experts_num,
              local_experts_num):
        r, _, rows, row_map = to.remap_hidden_states(hidden_states, None, topk_ids, expert_map, local_experts_num)
        remapped_hidden_states.copy_(r)
        rows_per_expert.copy_(rows)
        unpermuted_row_to_permuted_row.copy_(row_map)

    def gather(output, moe_output, topk_weights, unpermuted_row_to_permuted_row, num_experts):
        output.copy_(to.moe_gather(moe_output, topk_weights, unpermuted_row_to_permuted_row, output.dtype))

    def group_quant(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, a, b):
        q, sc = to.per_token_group_fp8_quant(input, group_size, eps, scale_ue8m0)
        output_q.copy_(q)
        output_s.copy_(sc)

    def silu(out, input):
        out.copy_(to.silu_and_mul(input))

    moe.impl("remap_hidden_states", remap, "CPU")
    moe.impl("moe_gather", gather, "CPU")
    c.impl("per_token_group_fp8_quant", group_quant, "CPU")
    c.impl("silu_and_mul", silu, "CPU")
    return moe, c, to


def capture_batched_align(align_t, max_tokens, num_experts, block, empty):
    """The reference's expected outputs for batched_moe_align_block_size live in a
    function nested in its test (tests/test_moe_align_block_size.py:340-417); run
    that test on CPU with the op replaced by a recorder and keep what it compares."""
    rec = {}
    real_to, real_close = torch.Tensor.to, torch.testing.assert_close

    def fake_to(self, *a, **k):
        if a and a[0] == "xpu":
            return self
        return real_to(self, *a, **k)

    def fake_op(mt, bs, counts):
        rec["counts"] = counts.clone()
        n = (mt + bs - 1) // bs * bs * counts.numel()
        return (torch.zeros(n, dtype=torch.int32), torch.zeros(n // bs, dtype=torch.int32),
                torch.zeros(1, dtype=torch.int32))

    def fake_close(expected, actual, **k):
        rec.setdefault("expected", []).append(expected.clone())

    torch.Tensor.to, torch.testing.assert_close = fake_to, fake_close
    old_op = align_t.batched_moe_align_block_size
    align_t.batched_moe_align_block_size = fake_op
    try:
        align_t.test_batched_moe_align_block_size.__wrapped__(max_tokens, num_experts, block, empty) \
            if hasattr(align_t.test_batched_moe_align_block_size, "__wrapped__") \
            else align_t.test_batched_moe_align_block_size(max_tokens, num_experts, block, empty)
    finally:
        torch.Tensor.to, torch.testing.assert_close = real_to, real_close
        align_t.batched_moe_align_block_size = old_op
    s_ids, b_ids, post = rec["expected"]
    return dict(max_tokens=max_tokens, block=block, counts=rec["counts"], sorted_ids=s_ids, block_ids=b_ids,
                num_post_pad=post)


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/vllm-xpu-kernels")
    root = sys.argv[1]
    ref = load_reference(root)
    g = torch.Generator().manual_seed(0)

    # ---- routing: softmax / sigmoid top-k -------------------------------------------
    cases = []
    for (T, E, K, renorm, with_bias) in [(33, 8, 2, True, False), (17, 128, 8, True, False),
                                         (9, 128, 4, False, True), (5, 60, 6, True, True),
                                         (64, 256, 8, True, False)]:
        gating = torch.randn(T, E, generator=g)
        bias = torch.randn(E, generator=g) * 0.1 if with_bias else None
        hidden = torch.zeros(T, 4)
        w, ids = ref["topk"].topk_softmax(hidden, gating, K, renorm, bias)
        ws, ids_s = ref["topk"].topk_sigmoid(hidden, gating, K, renorm, bias, None, 2.5)
        cases.append(dict(gating=gating, bias=bias, topk=K, renormalize=renorm,
                          softmax_w=w, softmax_ids=ids, sigmoid_w=ws, sigmoid_ids=ids_s,
                          routed_scaling_factor=2.5))
    torch.save(cases, OUT / "routing_topk.pt")

    # ---- routing: grouped top-k (ids are compared as sets: torch.topk(sorted=False)) ---
    cases = []
    for (T, E, ng, tg, K, scoring, renorm, rsf) in [(33, 16, 8, 2, 2, "softmax", True, 1.0),
                                                    (33, 16, 8, 2, 2, "sigmoid", False, 2.5),
                                                    (64, 256, 8, 4, 8, "sigmoid", True, 2.5),
                                                    (7, 64, 4, 2, 6, "sigmoid", True, 1.0)]:
        gating = torch.randn(T, E, generator=g)
        bias = torch.randn(E, generator=g) * (0.1 if E == 256 else 1.0)
        w, ids = ref["grouped"].grouped_topk(torch.zeros(T, 4), gating, K, renorm, ng, tg, scoring,
                                             rsf, bias)
        cases.append(dict(gating=gating, bias=bias, topk=K, n_group=ng, topk_group=tg,
                          scoring=scoring, renormalize=renorm, routed_scaling_factor=rsf,
                          weights=w, ids=ids))
    torch.save(cases, OUT / "routing_grouped.pt")

    # ---- moe_align_block_size ---------------------------------------------------------
    cases = []
    for (m, topk, E, bs, use_map) in [(1, 1, 32, 32, False), (3, 2, 32, 128, False),
                                      (256, 2, 160, 32, False), (300, 16, 257, 128, False),
                                      (16, 2, 8, 64, True), (32, 4, 8, 64, True)]:
        topk_ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(m)]).to(torch.int32)
        emap = None
        if use_map:
            emap = torch.full((E,), -1, dtype=torch.int32)
            for i, e in enumerate(range(0, E, 2)):
                emap[e] = i
        s, eids, post = ref["align"].torch_moe_align_block_size(topk_ids, bs, E, emap)
        cases.append(dict(topk_ids=topk_ids, num_experts=E, block_size=bs, expert_map=emap,
                          sorted_ids=s, expert_ids=eids, num_tokens_post_pad=post))
    torch.save(cases, OUT / "moe_align.pt")

    # ---- remap_hidden_states ----------------------------------------------------------
    cases = []
    for (T, H, E_tot, K, use_map) in [(8, 32, 16, 2, False), (33, 64, 16, 4, True), (64, 32, 32, 8, True)]:
        hidden = torch.randn(T, H, generator=g).to(torch.bfloat16)
        topk_ids = torch.stack([torch.randperm(E_tot, generator=g)[:K] for _ in range(T)]).to(torch.int64)
        if use_map:
            E_loc = E_tot // 4
            emap = torch.full((E_tot,), -1, dtype=torch.int32)
            emap[E_loc:2 * E_loc] = torch.arange(E_loc, dtype=torch.int32)
        else:
            E_loc, emap = E_tot, None
        remapped = torch.zeros(T * K, H, dtype=torch.bfloat16)
        rows = torch.zeros(E_loc, dtype=torch.int32)
        row_map = torch.zeros(T, K, dtype=torch.int32)
        ref["remap"].ref_remap_hidden_states(hidden, None, remapped, None, emap, rows, row_map,
                                             topk_ids, E_tot, E_loc)
        cases.append(dict(hidden=hidden, topk_ids=topk_ids, expert_map=emap, total_experts=E_tot,
                          local_experts=E_loc, remapped=remapped, rows_per_expert=rows, row_map=row_map))
    torch.save(cases, OUT / "remap.pt")

    # (init_expert_map has no CPU-runnable reference: its test helper allocates on the
    #  reference's device.  It is checked against the semantic statement instead.)

    # ---- moe_gather -----------------------------------------------------------------------
    cases = []
    for (T, H, K) in [(8, 128, 2), (5, 64, 8)]:
        moe_out = torch.randn(T * K, H, generator=g).to(torch.bfloat16)
        w = torch.rand(T, K, generator=g)
        perm = torch.randperm(T * K, generator=g).to(torch.int32).view(T, K)
        perm[0, 0] = -1
        out = torch.empty(T, H, dtype=torch.bfloat16)
        ref["gather"].ref_moe_gather(out, moe_out, w, perm, 16)
        cases.append(dict(moe_output=moe_out, topk_weights=w, row_map=perm, output=out))
    torch.save(cases, OUT / "moe_gather.pt")

    # ---- activations --------------------------------------------------------------------------
    x = (torch.randn(7, 256, generator=g) * 3).to(torch.bfloat16)
    xf = torch.randn(5, 128, generator=g) * 4
    torch.save(dict(x_bf16=x, silu_bf16=ref["act"].SiluAndMul.forward_native(None, x),
                    swiglu_bf16=ref["swi"].SwigluOAIAndMul().forward_native(x),
                    x_f32=xf, silu_f32=ref["act"].SiluAndMul.forward_native(None, xf),
                    swiglu_f32=ref["swi"].SwigluOAIAndMul().forward_native(xf)),
               OUT / "activations.pt")

    # ---- fp8 per-1x128 group quant (reference divides; tolerance applies, see its test) ----------
    x = torch.randn(6, 512, generator=g)
    q, s = ref["fp8"].ref_per_block_quant(x, 1, 128)
    torch.save(dict(x=x, q=q, s=s), OUT / "fp8_group_quant.pt")

    # ---- weight dequantisers ---------------------------------------------------------------------
    mu = ref["mu"]
    packed = torch.randint(0, 256, (4, 64), generator=g, dtype=torch.int32).to(torch.uint8)
    sc = torch.randint(117, 124, (4, 4), generator=g, dtype=torch.int32).to(torch.uint8)
    deq4 = mu.dequant_mxfp4(packed.view(torch.float4_e2m1fn_x2), sc.view(torch.float8_e8m0fnu))
    w8 = (torch.randn(128, 256, generator=g)).to(torch.float8_e4m3fn)
    s8 = torch.rand(1, 2, generator=g) + 0.5
    torch.save(dict(mxfp4_packed=packed, mxfp4_scale=sc, mxfp4_deq=deq4,
                    fp8_w=w8, fp8_scale=s8, fp8_deq=mu.dequant_fp8_block_wei(w8, s8)),
               OUT / "dequant.pt")

    # ---- whole layer, bf16 (tests/fused_moe/test_fused_moe.py:119-176) -----------------------------
    cases = []
    for (T, H, I, E, K, has_bias, clamp) in [(16, 128, 64, 4, 1, False, None), (12, 128, 64, 4, 2, True, None),
                                              (8, 64, 64, 8, 2, True, 0.5)]:
        a = (torch.randn(T, H, generator=g) / 4).to(torch.bfloat16)
        w13 = (torch.randn(E, 2 * I, H, generator=g) / 8).to(torch.bfloat16)
        w2 = (torch.randn(E, H, I, generator=g) / 8).to(torch.bfloat16)
        b13 = (torch.randn(E, 2 * I, generator=g) / 8).to(torch.bfloat16) if has_bias else None
        b2 = (torch.randn(E, H, generator=g) / 8).to(torch.bfloat16) if has_bias else None
        scores = torch.randn(T, E, generator=g)
        tw, tid = torch.topk(scores, k=K, dim=-1, sorted=False)
        out = ref["layer"].ref_fused_moe(a, w13, b13, w2, b2, tw.reshape(-1, 1), tid.reshape(-1), K,
                                         "silu", E, gemm1_clamp_limit=clamp)
        cases.append(dict(x=a, w13=w13, w2=w2, w13_bias=b13, w2_bias=b2, topk_weights=tw,
                          topk_ids=tid, num_experts=E, clamp=clamp, output=out))
    # expert-parallel variant: rank 1 of 2
    a = (torch.randn(10, 64, generator=g) / 4).to(torch.bfloat16)
    w13 = (torch.randn(8, 128, 64, generator=g) / 8).to(torch.bfloat16)
    w2 = (torch.randn(8, 64, 64, generator=g) / 8).to(torch.bfloat16)
    tw, tid = torch.topk(torch.randn(10, 8, generator=g), k=2, dim=-1, sorted=False)
    out = ref["layer"].ref_fused_moe(a, w13, None, w2, None, tw.reshape(-1, 1), tid.reshape(-1), 2, "silu",
                                     4, ep_rank=1, ep_size=2)
    cases.append(dict(x=a, w13=w13, w2=w2, w13_bias=None, w2_bias=None, topk_weights=tw, topk_ids=tid,
                      num_experts=4, ep_rank=1, ep_size=2, clamp=None, output=out))
    torch.save(cases, OUT / "layer_bf16.pt")

    # ---- fused activation + quantisation ops (own generator: earlier files stay as they are) --------
    g2 = torch.Generator().manual_seed(1)
    fq = dict(per_block=[], silu_mxfp4=[], mxfp4=[], static=[])
    for (T, hidden, group, dt, qdt) in [(3, 256, 128, torch.bfloat16, torch.float8_e4m3fn),
                                        (5, 384, 64, torch.float16, torch.float8_e4m3fn),
                                        (4, 256, 128, torch.bfloat16, torch.int8)]:
        x = (torch.randn(T, 2 * hidden, generator=g2) * 2).to(dt)
        q, sc = ref["sbq"].ref_silu_and_mul_per_block_quant(x, qdt, group)
        fq["per_block"].append(dict(x=x, group=group, q=q, scales=sc))
    for (T, hidden, dt) in [(3, 128, torch.bfloat16), (7, 256, torch.float16)]:
        x = (torch.randn(T, 2 * hidden, generator=g2) * 2).to(dt)
        packed, sc, silu_out = ref["smx"]._ref_silu_and_mul_mxfp4_quant(x)
        fq["silu_mxfp4"].append(dict(x=x, packed=packed, scales=sc, silu_out=silu_out))
    for (T, hidden, dt) in [(4, 128, torch.bfloat16), (2, 320, torch.float32)]:
        x = (torch.rand(T, hidden, generator=g2) + 1e-6).to(dt)
        sc, packed = ref["mxu"].to_mxfp(x, block_size=32, format="mxfp4")
        fq["mxfp4"].append(dict(x=x, packed=packed.view(torch.uint8), scale_e8m0=sc.view(torch.uint8)))
    for (T, d, dt) in [(3, 64, torch.bfloat16), (5, 24, torch.float16)]:
        x = torch.randn(T, 2 * d, generator=g2).to(dt)
        scale = torch.tensor([0.5])
        fq["static"].append(dict(x=x, scale=scale, q=ref["sq"].ref_silu_and_mul_quant(x, scale, torch.float8_e4m3fn)))
    torch.save(fq, OUT / "fused_quant.pt")

    # ---- the other gated activations ---------------------------------------------------------------
    g3 = torch.Generator().manual_seed(2)
    x = (torch.randn(6, 2 * 96, generator=g3) * 3).to(torch.bfloat16)
    xh = (torch.randn(5, 2 * 40, generator=g3) * 3).to(torch.float16)
    acts = {}
    for name, t in (("bf16", x), ("f16", xh)):
        acts[name] = dict(x=t,
                          gelu=ref["act"].GeluAndMul.forward_native(ref["act"].GeluAndMul("none"), t),
                          gelu_tanh=ref["act"].GeluAndMul.forward_native(ref["act"].GeluAndMul("tanh"), t),
                          swiglustep=ref["step"].SwigluStepAndMul.forward_native(ref["step"].SwigluStepAndMul(7.0), t))
    torch.save(acts, OUT / "activations2.pt")

    # ---- sqrt(softplus) routing (tests/test_topk_softplus_sqrt.py:19-47) ------------------------------
    g4 = torch.Generator().manual_seed(3)
    cases = []
    for (T, E, K, renorm, rsf, dt, use_hash) in [(33, 256, 8, True, 1.5, torch.float32, False),
                                                 (17, 384, 6, False, 1.0, torch.bfloat16, False),
                                                 (9, 128, 16, True, 2.5, torch.float16, False),
                                                 (21, 256, 8, True, 2.5, torch.float32, True)]:
        gating = torch.randn(T, E, generator=g4).to(dt)
        bias = torch.randn(E, generator=g4)
        ids = table = None
        if use_hash:
            table = torch.stack([torch.randperm(E, generator=g4)[:K] for _ in range(64)]).to(torch.int32)
            ids = torch.randint(0, 64, (T,), generator=g4, dtype=torch.int32)
            bias = None
        w, i = ref["sps"]._torch_topk_softplus_sqrt(gating, K, renorm, rsf, bias, ids, table)
        cases.append(dict(gating=gating, bias=bias, topk=K, renormalize=renorm, routed_scaling_factor=rsf,
                          input_ids=ids, tid2eid=table, weights=w, ids=i))
    torch.save(cases, OUT / "routing_softplus_sqrt.pt")

    # ---- batched align (expected values recorded from the reference's own test) -----------------------
    torch.manual_seed(4)
    cases = [capture_batched_align(ref["align"], mt, ne, bs, empty)
             for (mt, ne, bs, empty) in [(13, 8, 8, False), (16, 16, 16, True), (512, 64, 32, False), (13, 32, 64, True)]]
    torch.save(cases, OUT / "batched_align.pt")
    # ---- legacy prologue (tests/fused_moe/test_moe_prologue.py:52-97, 104-152) ------------------------
    cases = []
    for (m, k, e, topk, recipe) in [(1, 256, 16, 1, "bf16"), (4, 256, 16, 2, "fp16"), (16, 512, 16, 2, "mxfp8"),
                                    (300, 256, 16, 2, "fp8block"), (300, 256, 16, 1, "mxfp4"),
                                    (700, 128, 16, 2, "bf16"), (64, 256, 8, 2, "mxfp4")]:
        torch.manual_seed(7)
        data_dtype, scale_dtype = ref["pro"].RECIPE_TO_DTYPE[recipe]
        scales, block_k = None, 1
        if data_dtype in (torch.bfloat16, torch.float16):
            hidden = torch.randn(m, k, dtype=data_dtype) / 16
            ref_a = hidden.clone()
        elif data_dtype is torch.float8_e4m3fn:
            f32 = torch.randn(m, k)
            hidden, ref_a = f32.to(torch.float8_e4m3fn), f32
            if recipe == "fp8block":
                block_k = 128
                scales = torch.randn(m, k // block_k)
            else:
                block_k = 32
                scales = torch.randint(1, 256, (m, k // block_k), dtype=torch.uint8).view(torch.float8_e8m0fnu)
        else:
            block_k = 16
            ref_a = torch.randint(0, 256, (m, k // 2)).to(torch.bfloat16)   # byte values, as the test's cast makes them
            hidden = ref_a.to(torch.uint8).view(torch.float4_e2m1fn_x2)
            scales = torch.randint(1, 256, (m, k // 2 // block_k), dtype=torch.uint8).view(torch.float8_e8m0fnu)
        scores = torch.randn(m, e)
        topk_weights, topk_ids = torch.topk(scores, k=topk, dim=-1, sorted=False)
        # ref_prologue orders rows with Tensor.argsort(); the op's order inside an expert is
        # ascending token by construction (fused_moe_prologue.hpp:153-210, 423-462), which that
        # call only reproduces when the sort is stable - not the case for the CPU default.
        plain_argsort = torch.Tensor.argsort
        torch.Tensor.argsort = lambda self, *a, **kw: plain_argsort(self, *a, **{**kw, "stable": True})
        try:
            off, xin, xsc = ref["pro"].ref_prologue(ref_a, scales, topk_ids.view(-1), topk, e, recipe)
        finally:
            torch.Tensor.argsort = plain_argsort
        cases.append(dict(recipe=recipe, num_experts=e, topk=topk, block_k=block_k,
                          hidden_states=hidden.view(torch.uint8) if hidden.element_size() == 1 else hidden,
                          scales=None if scales is None else (scales.view(torch.uint8) if scales.element_size() == 1 else scales),
                          topk_ids=topk_ids, topk_weights=topk_weights, expert_offset=off,
                          expand_input=xin.view(torch.uint8) if xin.element_size() == 1 else xin,
                          expand_scales=None if xsc is None else (xsc.view(torch.uint8) if xsc.element_size() == 1 else xsc)))
    torch.save(cases, OUT / "prologue.pt")

    # ---- mxfp8 recipe: the reference's eager simulation is its only implementation ---------------------
    # (vllm_xpu_kernels/fused_moe_interface.py:27-31 routes mxfp8 weights to ref_fused_moe)
    _libs = install_cpu_ops()
    to = _libs[2]
    cases = []
    for (m, H, I, E, topk, dtype, bias) in [(1, 128, 128, 4, 2, torch.bfloat16, False),
                                            (33, 256, 160, 8, 2, torch.bfloat16, True),
                                            (40, 160, 128, 8, 4, torch.float16, False)]:
        torch.manual_seed(11 + m)
        x = (torch.randn(m, H) / 2).to(dtype)
        w13_q, w13_s, w2_q, w2_s = [], [], [], []
        for _ in range(E):
            q, sc = to.quant_mxfp8_wei(torch.randn(H, 2 * I) / H ** 0.5)
            w13_q.append(q); w13_s.append(sc)
            q, sc = to.quant_mxfp8_wei(torch.randn(I, H) / I ** 0.5)
            w2_q.append(q); w2_s.append(sc)
        w13, w13_s, w2, w2_s = torch.stack(w13_q), torch.stack(w13_s), torch.stack(w2_q), torch.stack(w2_s)
        b13 = (torch.randn(E, 2 * I) / 10).to(dtype) if bias else None
        b2 = (torch.randn(E, H) / 10).to(dtype) if bias else None
        tw, ti = torch.topk(torch.softmax(torch.randn(m, E), dim=-1), topk, dim=-1)
        out = torch.empty_like(x)
        ref["mu"].ref_fused_moe("mxfp8", out, x, w13, w13_s, b13, w2, w2_s, b2, tw, ti.int(), topk, "silu", E)
        cases.append(dict(x=x, w13=w13.view(torch.uint8), w13_scales=w13_s, w13_bias=b13, w2=w2.view(torch.uint8),
                          w2_scales=w2_s, w2_bias=b2, topk_weights=tw, topk_ids=ti.int(), num_experts=E, out=out))
    torch.save(cases, OUT / "layer_mxfp8.pt")
    print("wrote", sorted(p.name for p in OUT.glob("*.pt")))


if __name__ == "__main__":
    main()
