"""GPU parity: the block-scaled tensor-core grouped GEMM (MXFP4 weights x MXFP8
activations, one plane or two with the residual) and the MX activation
quantiser.  The quantiser is bit-exact against the oracle; the GEMM is compared
with an fp32 matmul of the dequantised operands (products and scales are exact,
so only the fp32 summation order and the bf16 rounding of the output differ:
2e-2); with two planes also against 16-bit activations at the bf16 tolerance,
with one plane at the benchmark's MXFP4 tolerance (1e-1, relative to the
largest output)."""
import pytest
import torch

from gpu_utils import DEV, grouped_gemm, mx_scale_bytes, quant_mxfp8, random_rows
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 32), (7, 2880), (300, 704), (64, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("terms", [1, 2])
def test_quant_mxfp8_bit_exact(native, rows, cols, dtype, terms):
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * torch.exp2(torch.randint(-12, 6, (rows, 1), generator=g).float()))
    x[0, :32] = 0
    x = x.to(dtype)
    q_ref, s_ref = to.quant_mxfp8(x, terms)
    q, s = quant_mxfp8(x.to(DEV), terms)
    sb = mx_scale_bytes(s, cols)
    assert torch.equal(sb[:, :, :cols // 32], s_ref)
    assert bool((sb[:, :, cols // 32:] == 0x7f).all())           # padding groups scale 2^0
    assert torch.equal(q.cpu().view(torch.uint8).reshape(terms, rows, cols), q_ref.view(torch.uint8))
    # two planes carry the 16-bit value almost exactly
    if terms == 2 and dtype == torch.bfloat16:
        back = to.dequant_mxfp8(q_ref, s_ref)
        err = (back - x.float()).abs().reshape(rows, -1, 32).amax(-1)
        amax = x.float().abs().reshape(rows, -1, 32).amax(-1)
        assert bool((err <= amax * 2.0 ** -7).all())


def _mx_case(E, M, N, K, g, has_bias):
    rows = random_rows(E, M, g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    packed = torch.randint(0, 256, (E, N, K // 2), generator=g, dtype=torch.int32).to(torch.uint8)
    sc = torch.randint(117, 124, (E, N, K // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    bias = (torch.randn(E, N, generator=g) * 0.02).to(torch.bfloat16) if has_bias else None
    return rows, x, packed, sc, bias


@pytest.mark.parametrize("E,M,N,K", [(4, 30, 256, 128), (4, 30, 256, 192), (8, 130, 5760 // 8, 2880 // 5),
                                     (6, 900, 360, 2880), (16, 40, 2880, 704), (2, 3, 128, 256),
                                     (3, 1300, 384, 1024), (5, 64, 200, 320)])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("terms", [1, 2])
def test_grouped_gemm_mxfp4_block_scaled(native, E, M, N, K, has_bias, terms):
    g = torch.Generator().manual_seed(N + K + M)
    rows, x, packed, sc, bias = _mx_case(E, M, N, K, g, has_bias)
    wdeq = to.dequant_mxfp4(packed, sc)
    xq, xs = quant_mxfp8(x.to(DEV), terms)
    xdq = to.dequant_mxfp8(xq.cpu().reshape(terms, M, K), mx_scale_bytes(xs, K)[:, :, :K // 32])
    ref = to.grouped_gemm(xdq, wdeq, bias, rows, torch.bfloat16)
    wd, sd = packed.to(DEV).view(torch.float4_e2m1fn_x2), sc.to(DEV)
    out = grouped_gemm(xq, xs, wd, sd, bias.to(DEV) if has_bias else None, rows.to(DEV), N, K, rows_out=M)
    n = int(rows.sum())
    torch.testing.assert_close(out.cpu()[:n].float(), ref[:n].float(), rtol=2e-2, atol=2e-2)
    assert bool(torch.isnan(out[n:].float()).all())
    ref16 = to.grouped_gemm(x.float(), wdeq, bias, rows, torch.bfloat16)
    if terms == 2:
        torch.testing.assert_close(out.cpu()[:n].float(), ref16[:n].float(), rtol=2e-2, atol=2e-2)
    else:
        torch.testing.assert_close(out.cpu()[:n].float(), ref16[:n].float(), rtol=1e-1,
                                   atol=1e-1 * float(ref16[:n].float().abs().max()))
    if has_bias and (N // 2) % 8 == 0:
        fused = grouped_gemm(xq, xs, wd, sd, bias.to(DEV), rows.to(DEV), N, K, epilogue=2, rows_out=M)
        full = to.grouped_gemm(xdq, wdeq, bias, rows, torch.float32)
        expect = to.swigluoai_and_mul(full)
        torch.testing.assert_close(fused.cpu()[:n].float(), expect[:n], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("E,M,N,K", [(4, 30, 256, 128), (4, 50, 256, 160), (8, 130, 720, 576), (3, 700, 2816, 2048),
                                     (2, 3, 128, 256), (5, 64, 208, 320)])
@pytest.mark.parametrize("w_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("terms", [1, 2])
def test_grouped_gemm_per_tensor_fp8_block_scaled(native, E, M, N, K, w_dtype, has_bias, terms):
    """Per-tensor-scaled fp8 weights [E,K,N] (the reference's w8a16 recipe) against
    MXFP8 activation planes on the block-scaled instruction: fp8 values are exact
    operands, the expert's scale multiplies the accumulator."""
    g = torch.Generator().manual_seed(N + K + M)
    rows = random_rows(E, M, g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, K, N, generator=g) * K ** -0.5 * 4).to(w_dtype)
    sc = torch.exp2(torch.randint(-3, 4, (E,), generator=g).float()) * 0.25
    bias = (torch.randn(E, N, generator=g) * 0.05).to(torch.bfloat16) if has_bias else None
    wdeq = w.float().transpose(1, 2) * sc.view(E, 1, 1)          # [E, N, K]
    xq, xs = quant_mxfp8(x.to(DEV), terms)
    xdq = to.dequant_mxfp8(xq.cpu().reshape(terms, M, K), mx_scale_bytes(xs, K)[:, :, :K // 32])
    ref = to.grouped_gemm(xdq, wdeq, bias, rows, torch.bfloat16)
    out = grouped_gemm(xq, xs, w.to(DEV), sc.to(DEV), bias.to(DEV) if has_bias else None, rows.to(DEV), N, K,
                       rows_out=M)
    n = int(rows.sum())
    torch.testing.assert_close(out.cpu()[:n].float(), ref[:n].float(), rtol=2e-2, atol=2e-2)
    assert bool(torch.isnan(out[n:].float()).all())
    if terms == 2:   # as good as 16-bit activations
        ref16 = to.grouped_gemm(x.float(), wdeq, bias, rows, torch.bfloat16)
        torch.testing.assert_close(out.cpu()[:n].float(), ref16[:n].float(), rtol=2e-2, atol=2e-2)
        # and the checking kernel with 16-bit activations agrees
        chk = grouped_gemm(x.to(DEV), None, w.to(DEV), sc.to(DEV), bias.to(DEV) if has_bias else None,
                           rows.to(DEV), N, K, impl=2)
        torch.testing.assert_close(out.cpu()[:n].float(), chk.cpu()[:n].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("E,M,N,K", [(4, 30, 256, 128), (4, 50, 256, 160), (8, 130, 720, 576), (3, 700, 2816, 2048),
                                     (2, 3, 128, 256), (5, 64, 208, 320), (2, 40, 144, 6144)])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("terms", [1, 2])
def test_grouped_gemm_mxfp8_weights_block_scaled(native, E, M, N, K, has_bias, terms):
    """MXFP8 weights ([E,K,N] e4m3, e8m0 scales [E,K/32,N]; the reference's "mxfp8" recipe,
    vllm_xpu_kernels/moe_utils.py:76-78) against MXFP8 activation planes: both operands'
    scales are applied inside the block-scaled instruction."""
    g = torch.Generator().manual_seed(N + K + M + 5)
    rows = random_rows(E, M, g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    wq, ws = zip(*[to.quant_mxfp8_wei(torch.randn(K, N, generator=g) * K ** -0.5 *
                                      torch.exp2(torch.randint(-6, 7, (1, N), generator=g).float())) for _ in range(E)])
    wq, ws = torch.stack(wq), torch.stack(ws)
    bias = (torch.randn(E, N, generator=g) * 0.05).to(torch.bfloat16) if has_bias else None
    wdeq = torch.stack([to.dequant_mxfp8_wei(wq[e], ws[e]).t() for e in range(E)])   # [E, N, K]
    xq, xs = quant_mxfp8(x.to(DEV), terms)
    xdq = to.dequant_mxfp8(xq.cpu().reshape(terms, M, K), mx_scale_bytes(xs, K)[:, :, :K // 32])
    ref = to.grouped_gemm(xdq, wdeq, bias, rows, torch.bfloat16)
    out = grouped_gemm(xq, xs, wq.to(DEV), ws.to(DEV), bias.to(DEV) if has_bias else None, rows.to(DEV), N, K,
                       rows_out=M)
    n = int(rows.sum())
    tol = 2e-2 * float(ref[:n].float().abs().max()) if n else 0
    torch.testing.assert_close(out.cpu()[:n].float(), ref[:n].float(), rtol=2e-2, atol=tol)
    assert bool(torch.isnan(out[n:].float()).all())
    # products and power-of-two scalings are exact: only the summation order differs
    assert (out.cpu()[:n].float() - ref[:n].float()).abs().max() <= 2 ** -7 * float(ref[:n].float().abs().max() if n else 0)
    if terms == 2:   # the checking kernel with 16-bit activations agrees
        chk = grouped_gemm(x.to(DEV), None, wq.to(DEV), ws.to(DEV), bias.to(DEV) if has_bias else None,
                           rows.to(DEV), N, K)
        torch.testing.assert_close(out.cpu()[:n].float(), chk.cpu()[:n].float(), rtol=2e-2, atol=tol)
