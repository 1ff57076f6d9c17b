"""GPU parity: the grouped GEMM.  The plain-CUDA checking kernel (impl=2) and
the tcgen05 tensor-core kernel (impl=1) are each compared with the CPU oracle
on ragged expert segments; tolerances are the reference's (bf16 2e-2) and the
benchmark's (fp8 5e-2, mxfp4 1e-1)."""
import pytest
import torch

from gpu_utils import DEV, grouped_gemm, random_rows
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu

CHECK, TC = 2, 1


def _bf16_case(E, M, N, K, gen, has_bias, zero_frac=0.25):
    rows = random_rows(E, M, gen, zero_frac)
    a = (torch.randn(M, K, generator=gen)).to(torch.bfloat16)
    w = (torch.randn(E, N, K, generator=gen) * K ** -0.5).to(torch.bfloat16)
    bias = (torch.randn(E, N, generator=gen) * 0.1).to(torch.bfloat16) if has_bias else None
    return rows, a, w, bias


def _close(out, ref, rows, tol):
    n = int(rows.sum())
    torch.testing.assert_close(out.cpu()[:n].float(), ref[:n].float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("impl", [CHECK, TC])
@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("E,M,N,K", [(4, 37, 256, 128), (8, 64, 2816, 512), (8, 5, 384, 256), (3, 700, 128, 192),
                                     (16, 2100, 512, 320), (2, 1, 128, 64), (5, 300, 200, 136)])
@pytest.mark.parametrize("has_bias", [False, True])
def test_grouped_gemm_bf16(native, impl, layout, E, M, N, K, has_bias):
    g = torch.Generator().manual_seed(E * M + N)
    rows, a, w, bias = _bf16_case(E, M, N, K, g, has_bias)
    ref = to.grouped_gemm(a.float(), w.float(), bias, rows, torch.bfloat16)
    wd = w.to(DEV) if layout == "nk" else w.transpose(1, 2).contiguous().to(DEV)
    out = grouped_gemm(a.to(DEV), None, wd, None, bias.to(DEV) if has_bias else None, rows.to(DEV), N, K,
                       layout=1 if layout == "nk" else 2, impl=impl)
    _close(out, ref, rows, 2e-2)
    # rows past the routed ones are never written
    n = int(rows.sum())
    assert bool(torch.isnan(out[n:].float()).all())


@pytest.mark.parametrize("impl", [CHECK, TC])
def test_grouped_gemm_fp16(native, impl):
    g = torch.Generator().manual_seed(9)
    rows, a, w, bias = _bf16_case(4, 100, 256, 256, g, True)
    a, w, bias = a.half(), w.half(), bias.half()
    ref = to.grouped_gemm(a.float(), w.float(), bias, rows, torch.float16)
    out = grouped_gemm(a.to(DEV), None, w.transpose(1, 2).contiguous().to(DEV), None, bias.to(DEV), rows.to(DEV),
                       256, 256, layout=2, impl=impl, out_dtype=torch.float16)
    _close(out, ref, rows, 1e-2)


def _fp8_case(E, M, N, K, gen):
    rows = random_rows(E, M, gen)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    wq, ws = zip(*[to.quant_fp8_block_wei(torch.randn(N, K, generator=gen) * K ** -0.5) for _ in range(E)])
    return rows, x, torch.stack(wq), torch.stack(ws)


@pytest.mark.parametrize("impl", [CHECK, TC])
@pytest.mark.parametrize("layout", ["nk", "kn"])
@pytest.mark.parametrize("E,M,N,K", [(4, 40, 256, 256), (8, 9, 1536, 2048), (6, 900, 384, 512), (32, 64, 256, 128)])
def test_grouped_gemm_fp8_block_w8a8(native, impl, layout, E, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    rows, x, wq, ws = _fp8_case(E, M, N, K, g)
    aq, a_s = to.per_token_group_fp8_quant(x, 128, 1e-10)
    wdeq = torch.stack([to.dequant_fp8_block_wei(wq[e], ws[e]) for e in range(E)])
    ref = to.grouped_gemm(to.dequant_fp8_block_act(aq, a_s), wdeq, None, rows, torch.bfloat16)
    wd = wq.to(DEV) if layout == "nk" else wq.transpose(1, 2).contiguous().to(DEV)
    out = grouped_gemm(aq.to(DEV), a_s.to(DEV), wd, ws.to(DEV), None, rows.to(DEV), N, K,
                       layout=1 if layout == "nk" else 2, impl=impl)
    _close(out, ref, rows, 2e-2)  # same quantised operands on both sides: only fp32 order differs


@pytest.mark.parametrize("layout", ["nk", "kn"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("E,M,N,K", [(3, 700, 640, 1024), (2, 300, 128, 384), (5, 1000, 256, 128), (4, 520, 1152, 640)])
def test_grouped_gemm_fp8_block_prefill_tiles(native, layout, dtype, E, M, N, K):
    """Segments of 12 rows per expert or more take the token-major kernels (256-feature tiles
    from N = 256, else 128): odd and even numbers of 128-feature blocks, bias, both output
    types, ragged and empty segments."""
    g = torch.Generator().manual_seed(M + N + K + 1)
    rows, x, wq, ws = _fp8_case(E, M, N, K, g)
    x = torch.cat([x, torch.randn(70, K, generator=g).to(torch.bfloat16)])   # rows no segment owns
    bias = (torch.randn(E, N, generator=g) * 0.1).to(dtype)
    aq, a_s = to.per_token_group_fp8_quant(x, 128, 1e-10)
    wdeq = torch.stack([to.dequant_fp8_block_wei(wq[e], ws[e]) for e in range(E)])
    ref = to.grouped_gemm(to.dequant_fp8_block_act(aq, a_s), wdeq, bias, rows, dtype)
    wd = wq.to(DEV) if layout == "nk" else wq.transpose(1, 2).contiguous().to(DEV)
    out = grouped_gemm(aq.to(DEV), a_s.to(DEV), wd, ws.to(DEV), bias.to(DEV), rows.to(DEV), N, K,
                       layout=1 if layout == "nk" else 2, impl=TC, out_dtype=dtype)
    _close(out, ref, rows, 2e-2)
    n = int(rows.sum())
    assert bool(torch.isnan(out[n:].float()).all())   # rows past the last segment are not written


def test_grouped_gemm_fp8_block_w8a16_and_per_tensor(native):
    g = torch.Generator().manual_seed(77)
    rows, x, wq, ws = _fp8_case(4, 50, 256, 256, g)
    wdeq = torch.stack([to.dequant_fp8_block_wei(wq[e], ws[e]) for e in range(4)]).to(torch.bfloat16)
    ref = to.grouped_gemm(x.float(), wdeq.float(), None, rows, torch.bfloat16)
    out = grouped_gemm(x.to(DEV), None, wq.to(DEV), ws.to(DEV), None, rows.to(DEV), 256, 256, layout=1, impl=0)
    _close(out, ref, rows, 2e-2)
    # per-tensor fp8 [E,K,N] with one scale per expert
    sc = torch.tensor([0.5, 2.0, 1.0, 0.25])
    ref = to.grouped_gemm(x.float(), wq.float() * sc.view(4, 1, 1), None, rows, torch.bfloat16)
    out = grouped_gemm(x.to(DEV), None, wq.transpose(1, 2).contiguous().to(DEV), sc.to(DEV), None,
                       rows.to(DEV), 256, 256, impl=0)
    _close(out, ref, rows, 2e-2)


@pytest.mark.parametrize("impl", [CHECK, TC])
def test_fp8_block_identity_known_answer_is_exact(native, impl):
    """Identity activations x every finite e4m3 code x block scales {0.5, 2}
    reproduce code * scale exactly (tests/fused_moe/test_grouped_gemm.py:275-307)."""
    codes = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn)
    finite = codes[torch.isfinite(codes.float())]
    K = N = 256
    w = finite[torch.arange(N * K) % finite.numel()].view(1, N, K).contiguous()
    ws = torch.tensor([[[0.5, 2.0], [2.0, 0.5]]])
    eye = torch.eye(K)
    rows = torch.tensor([K], dtype=torch.int32)
    expect = (to.dequant_fp8_block_wei(w[0], ws[0]).T).to(torch.bfloat16)
    if impl == CHECK:
        out = grouped_gemm(eye.to(torch.bfloat16).to(DEV), None, w.to(DEV), ws.to(DEV), None, rows.to(DEV),
                           N, K, layout=1, impl=impl)
    else:
        a_s = torch.ones(K, K // 128)
        out = grouped_gemm(eye.to(torch.float8_e4m3fn).to(DEV), a_s.to(DEV), w.to(DEV), ws.to(DEV), None,
                           rows.to(DEV), N, K, layout=1, impl=impl)
    torch.testing.assert_close(out.cpu(), expect, rtol=0, atol=0)


@pytest.mark.parametrize("impl", [CHECK, TC])
@pytest.mark.parametrize("E,M,N,K", [(4, 30, 256, 128), (8, 130, 5760 // 8, 2880 // 5), (6, 900, 360, 2880),
                                     (16, 40, 2880, 704)])
@pytest.mark.parametrize("has_bias", [False, True])
def test_grouped_gemm_mxfp4(native, impl, E, M, N, K, has_bias):
    g = torch.Generator().manual_seed(N + K)
    rows = random_rows(E, M, g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    packed = torch.randint(0, 256, (E, N, K // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    sc = torch.randint(117, 124, (E, N, K // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    bias = (torch.randn(E, N, generator=g) * 0.02).to(torch.bfloat16) if has_bias else None
    wdeq = to.dequant_mxfp4(packed, sc).to(torch.bfloat16).float()
    ref = to.grouped_gemm(x.float(), wdeq, bias, rows, torch.bfloat16)
    out = grouped_gemm(x.to(DEV), None, packed.to(DEV).view(torch.float4_e2m1fn_x2), sc.to(DEV),
                       bias.to(DEV) if has_bias else None, rows.to(DEV), N, K, impl=impl)
    n = int(rows.sum())
    torch.testing.assert_close(out.cpu()[:n].float(), ref[:n].float(), rtol=2e-2, atol=2e-2)
    if not has_bias:
        # float16 activations and scale bytes above 128 take the converter's general path
        sc2 = torch.randint(126, 133, (E, N, K // 32), generator=g, dtype=torch.int32).to(torch.uint8)
        for dt, scl in ((torch.float16, sc), (torch.bfloat16, sc2)):
            wd = to.dequant_mxfp4(packed, scl).to(dt).float()
            r2 = to.grouped_gemm(x.to(dt).float(), wd, None, rows, dt)
            o2 = grouped_gemm(x.to(dt).to(DEV), None, packed.to(DEV).view(torch.float4_e2m1fn_x2), scl.to(DEV),
                              None, rows.to(DEV), N, K, impl=impl, out_dtype=dt)
            torch.testing.assert_close(o2.cpu()[:n].float(), r2[:n].float(), rtol=2e-2, atol=2e-2 * float(r2.abs().max()))
    if has_bias:  # SwigluOAI fused into the epilogue (interleaved gate / up columns)
        # the tensor-core epilogue writes 16-byte pieces: other widths go to the checking kernel
        fused = grouped_gemm(x.to(DEV), None, packed.to(DEV).view(torch.float4_e2m1fn_x2), sc.to(DEV),
                             bias.to(DEV), rows.to(DEV), N, K, epilogue=2,
                             impl=impl if (N // 2) % 8 == 0 else 0)
        full = to.grouped_gemm(x.float(), wdeq, bias, rows, torch.float32)
        expect = to.swigluoai_and_mul(full)
        torch.testing.assert_close(fused.cpu()[:n].float(), expect[:n], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("epi", [1, 2])
def test_gated_epilogue_matches_unfused(native, epi):
    g = torch.Generator().manual_seed(epi)
    rows, a, w, bias = _bf16_case(4, 60, 512, 256, g, True)
    wd = w.transpose(1, 2).contiguous().to(DEV)
    full = grouped_gemm(a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), 512, 256, layout=2, impl=CHECK)
    fused = grouped_gemm(a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), 512, 256, layout=2, epilogue=epi,
                         impl=0)
    n = int(rows.sum())
    expect = to.silu_and_mul(full.cpu().float()) if epi == 1 else to.swigluoai_and_mul(full.cpu().float())
    torch.testing.assert_close(fused.cpu()[:n].float(), expect[:n], rtol=2e-2, atol=2e-2)


def test_tensor_core_kernel_matches_checking_kernel_on_mixtral_tile_shapes(native):
    """One expert segment per tile size (decode, mid, prefill) and a feature
    count that is not a multiple of the 128-wide tile."""
    g = torch.Generator().manual_seed(1)
    for (E, M, N, K) in [(8, 16, 1024, 4096), (8, 500, 1024, 1024), (4, 1500, 1152, 512), (2, 3000, 192, 256)]:
        rows, a, w, bias = _bf16_case(E, M, N, K, g, True, zero_frac=0.1)
        wd = w.transpose(1, 2).contiguous().to(DEV)
        ref = grouped_gemm(a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), N, K, layout=2, impl=CHECK)
        out = grouped_gemm(a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), N, K, layout=2, impl=TC)
        n = int(rows.sum())
        torch.testing.assert_close(out[:n].float(), ref[:n].float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("rows_list,N,K,epi,dtype", [
    ([300, 0, 1400, 513, 1000], 768, 384, 0, torch.bfloat16),    # ragged segments, an empty expert
    ([900, 700], 192, 256, 0, torch.bfloat16),                   # an odd number of 128-feature tiles
    ([900, 700], 640, 320, 2, torch.bfloat16),                   # SwigluOAI epilogue
    ([1100, 800], 384, 320, 0, torch.float16),
    ([300, 0, 1400, 513, 1000], 768, 384, 1, torch.bfloat16),    # SiLU-and-mul: gate in one CTA, up in the other
    ([900, 700], 512, 320, 1, torch.float16),
])
def test_16bit_prefill_cta_pair_kernel_matches_the_single_cta_kernel(native, layout, rows_list, N, K, epi, dtype):
    """16-bit prefill GEMMs run on clusters of two CTAs that share a 256-token tile (tcgen05.mma
    cta_group::2; impl=4 forces that form, impl=3 the single-CTA kernels).  With the SiLU epilogue
    the two CTAs hold gate and up and exchange chunks through shared memory.  Both forms against
    each other (same products, same fp32 accumulation) and against the checking kernel."""
    E, M = len(rows_list), sum(rows_list)
    g = torch.Generator().manual_seed(N + K)
    rows = torch.tensor(rows_list, dtype=torch.int32)
    a = (torch.randn(M + 40, K, generator=g) * 0.5).to(dtype)   # 40 rows that belong to no expert
    w = (torch.randn(E, N, K, generator=g) * 0.1).to(dtype)
    bias = torch.randn(E, N, generator=g).to(dtype)
    wd = (w.transpose(1, 2).contiguous() if layout == "kn" else w).to(DEV)
    lay = 2 if layout == "kn" else 1
    args = (a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), N, K)
    pair = grouped_gemm(*args, layout=lay, epilogue=epi, impl=4, out_dtype=dtype)
    single = grouped_gemm(*args, layout=lay, epilogue=epi, impl=3, out_dtype=dtype)
    check = grouped_gemm(*args, layout=lay, epilogue=epi, impl=CHECK, out_dtype=dtype)
    assert torch.equal(pair[:M], single[:M])
    torch.testing.assert_close(pair[:M].float(), check[:M].float(), rtol=1e-2, atol=1e-2)
    assert bool(torch.isnan(pair[M:].float()).all())            # rows past the segments are not written


def test_grouped_gemm_argument_checks(native):
    a = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(2, 64, 36, dtype=torch.bfloat16, device=DEV)
    d = torch.zeros(4, 36, dtype=torch.bfloat16, device=DEV)
    rows = torch.tensor([2, 2], dtype=torch.int32, device=DEV)
    f = torch.ops._xpu_C.cutlass_grouped_gemm_interface
    with pytest.raises(RuntimeError, match="N must be divisible by 8"):
        f(a, None, w, None, None, d, rows, 36, 64, 2)
    w = torch.zeros(2, 64, 32, dtype=torch.bfloat16, device=DEV)
    d = torch.zeros(4, 32, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="ptr_B.size\\(0\\) must match num_experts"):
        f(a, None, w, None, None, d, rows, 32, 64, 3)
    with pytest.raises(RuntimeError, match="w16a16 grouped gemm must not have scales"):
        f(a, None, w, torch.ones(2, device=DEV), None, d, rows, 32, 64, 2)
    with pytest.raises(RuntimeError, match="ptr_A.size\\(0\\) must match ptr_D.size\\(0\\)"):
        f(a, None, w, None, None, torch.zeros(5, 32, dtype=torch.bfloat16, device=DEV), rows, 32, 64, 2)
    w8 = torch.zeros(2, 128, 128, dtype=torch.float8_e4m3fn, device=DEV)
    with pytest.raises(RuntimeError, match="block scales must have shape"):
        f(torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV), None, w8, torch.ones(2, 2, 1, device=DEV), None,
          torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV), rows, 128, 128, 2)
    out = f(a, None, w, None, None, d, rows, 32, 64, 2)
    assert out.data_ptr() == d.data_ptr()


@pytest.mark.parametrize("E,M,N,K,group", [(4, 37, 256, 256, 128), (8, 130, 320, 512, 64), (3, 5, 128, 1024, 256),
                                           (6, 64, 72, 128, 32), (2, 900, 384, 2048, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("impl", [CHECK, TC])
def test_grouped_gemm_int4(native, E, M, N, K, group, dtype, has_bias, impl):
    """w4a16 with group scales: two's-complement nibbles at the op boundary (what the
    reference's layer hands its kernel after implement_zp)."""
    g = torch.Generator().manual_seed(N + K)
    rows = random_rows(E, M, g)
    x = (torch.randn(M, K, generator=g) / 4).to(dtype)
    u4 = torch.randint(0, 256, (E, N, K // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    sc = (torch.exp2(torch.randint(-6, -3, (E, N, K // group), generator=g).float()) *
          (1 + torch.rand(E, N, K // group, generator=g) * 0.5)).to(dtype)
    bias = (torch.randn(E, N, generator=g) * 0.05).to(dtype) if has_bias else None
    wdeq = to.dequant_int4(u4, sc, group).float()
    ref = to.grouped_gemm(x.float(), wdeq, bias, rows, dtype)
    s4 = (u4 ^ 0x88).view(torch.int8)
    out = grouped_gemm(x.to(DEV), None, s4.to(DEV), sc.to(DEV), bias.to(DEV) if has_bias else None, rows.to(DEV),
                       N, K, out_dtype=dtype, impl=impl)
    n = int(rows.sum())
    torch.testing.assert_close(out.cpu()[:n].float(), ref[:n].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("impl", [CHECK, TC])
@pytest.mark.parametrize("recipe", ["bf16", "fp8"])
@pytest.mark.parametrize("E,src,M,N,K", [(4, 3, 90, 256, 256), (3, 2, 1500, 384, 512), (8, 4, 40, 128, 384)])
def test_grouped_gemm_row_segments_share_weight_sets(native, impl, recipe, E, src, M, N, K):
    """rows_per_expert with src * E segments: segment s multiplies with weight set s % E - the rows
    of an expert-parallel exchange in arrival order (source-major, expert-minor)."""
    g = torch.Generator().manual_seed(E * M + N)
    rows = random_rows(E * src, M, g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    if recipe == "bf16":
        w = (torch.randn(E, N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
        ref = to.grouped_gemm(x.float(), w.float().repeat(src, 1, 1), bias.repeat(src, 1), rows, torch.bfloat16)
        out = grouped_gemm(x.to(DEV), None, w.to(DEV), None, bias.to(DEV), rows.to(DEV), N, K, layout=1, impl=impl,
                           weight_sets=E)
    else:
        wq, ws = zip(*[to.quant_fp8_block_wei(torch.randn(N, K, generator=g) * K ** -0.5) for _ in range(E)])
        wq, ws = torch.stack(wq), torch.stack(ws)
        aq, a_s = to.per_token_group_fp8_quant(x, 128, 1e-10)
        wdeq = torch.stack([to.dequant_fp8_block_wei(wq[e], ws[e]) for e in range(E)])
        ref = to.grouped_gemm(to.dequant_fp8_block_act(aq, a_s), wdeq.repeat(src, 1, 1), bias.repeat(src, 1), rows,
                              torch.bfloat16)
        out = grouped_gemm(aq.to(DEV), a_s.to(DEV), wq.to(DEV), ws.to(DEV), bias.to(DEV), rows.to(DEV), N, K,
                           layout=1, impl=impl, weight_sets=E)
    _close(out, ref, rows, 2e-2)


def test_fp8_token_major_kernel_against_checking_kernel_at_deepseek_shape(native):
    """Full-size K and N of the DeepSeek-V3 w13 GEMM (K=7168, N=4096), ragged segments from empty
    to several tiles: the token-major tensor-core kernel and the plain-CUDA checking kernel see
    the same fp8 operands and scales, so only the fp32 summation order differs."""
    E, N, K = 6, 4096, 7168
    g = torch.Generator(device=DEV).manual_seed(11)
    rows = torch.tensor([700, 0, 129, 1, 300, 128], dtype=torch.int32)
    M = int(rows.sum())
    a = (torch.randn(M, K, generator=g, device=DEV)).to(torch.float8_e4m3fn)
    a_s = torch.rand(M, K // 128, generator=g, device=DEV) * 0.02 + 0.005
    w = (torch.randn(E, N, K, generator=g, device=DEV)).to(torch.float8_e4m3fn)
    w_s = torch.rand(E, N // 128, K // 128, generator=g, device=DEV) * 0.02 + 0.005
    bias = (torch.randn(E, N, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    tc = grouped_gemm(a, a_s, w, w_s, bias, rows.to(DEV), N, K, layout=1, impl=TC)
    chk = grouped_gemm(a, a_s, w, w_s, bias, rows.to(DEV), N, K, layout=1, impl=CHECK)
    top = float(chk.float().abs().max())
    assert torch.isfinite(tc.float()).all() and top > 0
    assert float((tc.float() - chk.float()).abs().max()) <= 2 ** -7 * top


@pytest.mark.parametrize("layout", ["nk", "kn"])
@pytest.mark.parametrize("dtype,has_bias,clamp", [(torch.bfloat16, False, 0.0), (torch.float16, True, 0.0),
                                                 (torch.bfloat16, True, 0.4)])
@pytest.mark.parametrize("E,M,N,K", [(3, 700, 512, 1024), (5, 1000, 256, 128), (4, 130, 1280, 384), (8, 40, 768, 256)])
def test_fp8_gemm_with_silu_and_quantisation_in_the_epilogue(native, layout, dtype, has_bias, clamp, E, M, N, K):
    """gemm1 of a block-scaled fp8 layer with SiLU-and-mul and the 1x128 e4m3 quantisation of
    gemm2's input inside the tensor-core epilogue: codes and scales must equal, value for
    value, what the unfused GEMM followed by silu_and_mul_per_block_quant
    (csrc/quantization/fused_kernels/fused_silu_mul_block_quant.cpp:14-128 of the reference)
    produces - the epilogue rounds gate and up to the 16-bit type first, as the unfused output
    is.  Ragged and empty segments, rows no segment owns, both weight layouts."""
    g = torch.Generator().manual_seed(M + N + K + 3)
    rows, x, wq, ws = _fp8_case(E, M, N, K, g)
    x = torch.cat([x, torch.randn(33, K, generator=g).to(torch.bfloat16)])
    bias = (torch.randn(E, N, generator=g) * 0.1).to(dtype).to(DEV) if has_bias else None
    aq, a_s = to.per_token_group_fp8_quant(x, 128, 1e-10)
    wd = wq.to(DEV) if layout == "nk" else wq.transpose(1, 2).contiguous().to(DEV)
    lay = 1 if layout == "nk" else 2
    Mt, n = x.shape[0], int(rows.sum())
    full = grouped_gemm(aq.to(DEV), a_s.to(DEV), wd, ws.to(DEV), bias, rows.to(DEV), N, K, layout=lay, impl=TC,
                        out_dtype=dtype)
    if clamp > 0:
        full[:, :N // 2].clamp_(max=clamp)
        full[:, N // 2:].clamp_(min=-clamp, max=clamp)
    ref_q = torch.empty(Mt, N // 2, dtype=torch.float8_e4m3fn, device=DEV)
    ref_s = torch.empty(Mt, N // 256, dtype=torch.float32, device=DEV)
    torch.ops._C.silu_and_mul_per_block_quant(ref_q, full, ref_s, 128, None, False, False)
    q = torch.full((Mt, N // 2), 0x7f, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    s = torch.full((Mt, N // 256), -1.0, dtype=torch.float32, device=DEV)
    torch.ops._xpu_C.b200_grouped_gemm(aq.to(DEV), a_s.to(DEV), wd, ws.to(DEV), bias, q, rows.to(DEV), N, K, E, lay, 1,
                                       1.702, 7.0, clamp, 0, 0, 0, s, dtype == torch.float16)
    assert torch.equal(q.view(torch.uint8)[:n], ref_q.view(torch.uint8)[:n])
    assert torch.equal(s[:n], ref_s[:n])
    assert bool((q.view(torch.uint8)[n:] == 0x7f).all()) and bool((s[n:] == -1.0).all())   # rows past the segments


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("E,M,N,K,clamp,dtype", [(4, 20, 512, 256, 0.0, torch.bfloat16),      # 16-token tiles
                                                 (8, 300, 2816, 512, 0.0, torch.bfloat16),    # 64-token tiles, cfg1's N
                                                 (3, 330, 416, 192, 0.5, torch.bfloat16),     # 128-token tiles, I = 208
                                                 (2, 900, 768, 320, 0.0, torch.float16)])     # beyond 96 rows per expert
def test_16bit_gemm_with_silu_in_the_tensor_core_epilogue(native, layout, E, M, N, K, clamp, dtype):
    """gemm1 with SiLU-and-mul fused on 16-bit weights: gate tile j and up tile I/128 + j of the same
    tokens go into two accumulators and the epilogue writes silu(gate) * up as [M, N/2].  Against
    the checking kernel's fused form (fp32 throughout) and against the unfused GEMM followed by
    the torch statement of silu_and_mul."""
    g = torch.Generator().manual_seed(E + M + N)
    rows, a, w, bias = _bf16_case(E, M, N, K, g, True)
    a, w, bias = a.to(dtype), w.to(dtype), bias.to(dtype)
    wd = (w.transpose(1, 2).contiguous() if layout == "kn" else w).to(DEV)
    lay = 2 if layout == "kn" else 1
    args = (a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), N, K)
    fused = grouped_gemm(*args, layout=lay, epilogue=1, impl=TC, out_dtype=dtype, clamp=clamp)
    check = grouped_gemm(*args, layout=lay, epilogue=1, impl=CHECK, out_dtype=dtype, clamp=clamp)
    n = int(rows.sum())
    torch.testing.assert_close(fused[:n].float(), check[:n].float(), rtol=1e-2, atol=1e-2)
    assert bool(torch.isnan(fused[n:].float()).all())            # rows past the segments are not written
    full = grouped_gemm(*args, layout=lay, impl=TC, out_dtype=dtype).cpu().float()
    if clamp > 0:
        full[:, :N // 2].clamp_(max=clamp)
        full[:, N // 2:].clamp_(min=-clamp, max=clamp)
    torch.testing.assert_close(fused.cpu()[:n].float(), to.silu_and_mul(full)[:n].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("E,M,N,K,clamp,dtype", [(4, 20, 512, 256, 0.0, torch.bfloat16),      # 16-token tiles
                                                 (8, 300, 2816, 512, 0.0, torch.bfloat16),    # 64-token tiles
                                                 (3, 330, 416, 192, 0.5, torch.bfloat16),     # 128-token tiles, I = 208
                                                 (2, 900, 768, 320, 0.0, torch.float16)])     # 256-token tiles
def test_16bit_gemm_with_swigluoai_in_the_tensor_core_epilogue(native, layout, E, M, N, K, clamp, dtype):
    """gemm1 with SwigluOAI fused on 16-bit weights: gate (even feature) and up (odd feature) of an
    output sit on neighbouring accumulator lanes, the epilogue writes [M, N/2].  Against the checking
    kernel's fused form and against the unfused GEMM followed by the torch statement of the op."""
    g = torch.Generator().manual_seed(E + M + N + 1)
    rows, a, w, bias = _bf16_case(E, M, N, K, g, True)
    a, w, bias = a.to(dtype), w.to(dtype), bias.to(dtype)
    wd = (w.transpose(1, 2).contiguous() if layout == "kn" else w).to(DEV)
    lay = 2 if layout == "kn" else 1
    args = (a.to(DEV), None, wd, None, bias.to(DEV), rows.to(DEV), N, K)
    fused = grouped_gemm(*args, layout=lay, epilogue=2, impl=TC, out_dtype=dtype, clamp=clamp)
    check = grouped_gemm(*args, layout=lay, epilogue=2, impl=CHECK, out_dtype=dtype, clamp=clamp)
    n = int(rows.sum())
    torch.testing.assert_close(fused[:n].float(), check[:n].float(), rtol=1e-2, atol=1e-2)
    assert bool(torch.isnan(fused[n:].float()).all())            # rows past the segments are not written
    full = grouped_gemm(*args, layout=lay, impl=TC, out_dtype=dtype).cpu().float()
    if clamp > 0:
        full[:, 0::2].clamp_(max=clamp)
        full[:, 1::2].clamp_(min=-clamp, max=clamp)
    torch.testing.assert_close(fused.cpu()[:n].float(), to.swigluoai_and_mul(full)[:n].float(), rtol=2e-2, atol=2e-2)
