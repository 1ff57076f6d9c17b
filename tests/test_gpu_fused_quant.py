"""GPU parity of the activation + quantisation ops (silu_and_mul_per_block_quant,
silu_and_mul_mxfp4_quant, per_token_group_quant_mxfp4, silu_and_mul_quant)
against the oracle and the reference-made vectors.  Scales must agree to 1e-5
(the reference tests' bar); codes may differ only where exp differs by an ulp
across a rounding boundary, so dequantised values are compared at the
reference tests' tolerances plus the one-code allowance of the golden check."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu


def _per_block(x, group, qdt, transposed=False, ub=None, ue8m0=False):
    T, H = x.shape[0], x.shape[1] // 2
    out = torch.empty(T, H, dtype=qdt, device=DEV)
    if transposed:
        scales = torch.empty(H // group, T, dtype=torch.float32, device=DEV).t()
    else:
        scales = torch.empty(T, H // group, dtype=torch.float32, device=DEV)
    torch.ops._C.silu_and_mul_per_block_quant(out, x, scales, group, ub, transposed, ue8m0)
    return out, scales


@pytest.mark.parametrize("T,H", [(1, 64), (1, 5120), (16, 1024), (128, 1152), (512, 64), (0, 128)])
@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("qdt", [torch.float8_e4m3fn, torch.int8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_silu_and_mul_per_block_quant(native, T, H, group, transposed, qdt, dtype):
    if H % group:
        pytest.skip("hidden size not a multiple of the group")
    g = torch.Generator().manual_seed(T + H + group)
    x = (torch.randn(T, 2 * H, generator=g) * 1.5).to(dtype)
    q_ref, s_ref = to.silu_and_mul_per_block_quant(x, group, qdt)
    q, s = _per_block(x.to(DEV), group, qdt, transposed)
    assert q.shape == (T, H) and s.shape == (T, H // group)
    if T == 0:
        return
    torch.testing.assert_close(s.cpu().contiguous(), s_ref, rtol=1e-5, atol=1e-8)
    rep = lambda t: t.repeat_interleave(group, dim=1)
    same = q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)
    assert float(same.float().mean()) > 0.999          # an ulp of exp may move a value across a boundary
    torch.testing.assert_close(q.cpu().float() * rep(s.cpu()), q_ref.float() * rep(s_ref), rtol=0.13,
                               atol=float(s_ref.max()))


def test_silu_and_mul_per_block_quant_options_and_vectors(native):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(9, 512, generator=g) * 2).to(torch.bfloat16)
    ub = torch.tensor([0.004])
    for ue8m0 in (False, True):
        q_ref, s_ref = to.silu_and_mul_per_block_quant(x, 128, torch.float8_e4m3fn, scale_ub=ub, ue8m0=ue8m0)
        q, s = _per_block(x.to(DEV), 128, torch.float8_e4m3fn, False, ub.to(DEV), ue8m0)
        torch.testing.assert_close(s.cpu(), s_ref, rtol=1e-5, atol=1e-8)
        assert float((q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)).float().mean()) > 0.999
    for c in load_golden("fused_quant.pt")["per_block"]:
        q, s = _per_block(c["x"].to(DEV), c["group"], c["q"].dtype)
        torch.testing.assert_close(s.cpu(), c["scales"], rtol=1e-2, atol=1e-5)
        rep = lambda t: t.repeat_interleave(c["group"], dim=1)
        torch.testing.assert_close(q.cpu().float() * rep(s.cpu()), c["q"].float() * rep(c["scales"]), rtol=0.13,
                                   atol=max(5e-2, float(c["scales"].max())))
    with pytest.raises(RuntimeError, match="group_size must be 32, 64, or 128"):
        _per_block(x.to(DEV), 16, torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="scale_ub is only supported for FP8 output"):
        _per_block(x.to(DEV), 128, torch.int8, False, ub.to(DEV))


def _deq(packed, sc):
    return to.dequant_mxfp4(packed.cpu(), (torch.log2(sc.cpu()) + 127).round().to(torch.uint8))


@pytest.mark.parametrize("T", [1, 7, 83, 2048])
@pytest.mark.parametrize("H", [128, 1024, 5120])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_silu_and_mul_mxfp4_quant(native, T, H, dtype):
    g = torch.Generator().manual_seed(T + H)
    x = torch.randn(T, 2 * H, generator=g).to(dtype)
    p_ref, s_ref = to.silu_and_mul_mxfp4_quant(x)
    out = torch.empty(T, H // 2, dtype=torch.uint8, device=DEV)
    sc = torch.empty(T, H // 32, dtype=torch.float32, device=DEV)
    torch.ops._C.silu_and_mul_mxfp4_quant(out, x.to(DEV), sc, 32, 1e-10)
    assert torch.equal(sc.cpu(), s_ref)
    assert float((out.cpu() == p_ref).float().mean()) > 0.999
    torch.testing.assert_close(_deq(out, sc), _deq(p_ref, s_ref), rtol=0.0, atol=2.0 * float(s_ref.max()))


@pytest.mark.parametrize("T,H", [(1, 32), (7, 2880), (100, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("column_major", [False, True])
def test_per_token_group_quant_mxfp4_bit_exact(native, T, H, dtype, column_major):
    g = torch.Generator().manual_seed(T * H)
    x = ((torch.rand(T, H, generator=g) + 1e-6) * torch.exp2(torch.randint(-8, 8, (T, 1), generator=g).float())).to(dtype)
    x[0, :32] = 0
    p_ref, s_ref = to.per_token_group_quant_mxfp4(x)
    out = torch.empty(T, H // 2, dtype=torch.uint8, device=DEV)
    sc = (torch.empty(H // 32, T, dtype=torch.float32, device=DEV).t() if column_major
          else torch.empty(T, H // 32, dtype=torch.float32, device=DEV))
    torch.ops._C.per_token_group_quant_mxfp4(x.to(DEV), out, sc, 32, 1e-10)
    assert torch.equal(sc.cpu().contiguous(), s_ref)
    assert torch.equal(out.cpu(), p_ref)


def test_mxfp4_quant_reference_vectors(native):
    fq = load_golden("fused_quant.pt")
    for c in fq["mxfp4"]:
        x = c["x"]
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=torch.uint8, device=DEV)
        sc = torch.empty(x.shape[0], x.shape[1] // 32, dtype=torch.float32, device=DEV)
        torch.ops._C.per_token_group_quant_mxfp4(x.to(DEV), out, sc, 32, 1e-10)
        ref_sc = torch.exp2(c["scale_e8m0"].float() - 127.0)
        torch.testing.assert_close(sc.cpu(), ref_sc, rtol=1e-5, atol=1e-5)
        a, b = _deq(out, sc), _deq(c["packed"], ref_sc)
        assert float(((a - b).abs() > 0.2 + 0.2 * b.abs()).float().mean()) < 0.03
    for c in fq["silu_mxfp4"]:
        x = c["x"]
        H = x.shape[1] // 2
        out = torch.empty(x.shape[0], H // 2, dtype=torch.uint8, device=DEV)
        sc = torch.empty(x.shape[0], H // 32, dtype=torch.float32, device=DEV)
        torch.ops._C.silu_and_mul_mxfp4_quant(out, x.to(DEV), sc, 32, 1e-10)
        torch.testing.assert_close(sc.cpu(), c["scales"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("T", [1, 7, 83, 512])
@pytest.mark.parametrize("d", [16, 128, 4096, 20])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_silu_and_mul_quant(native, T, d, dtype):
    g = torch.Generator().manual_seed(T + d)
    x = torch.randn(T, 2 * d, generator=g).to(dtype)
    scale = torch.tensor([0.5])
    ref = to.silu_and_mul_quant(x, scale)
    out = torch.empty(T, d, dtype=torch.float8_e4m3fn, device=DEV)
    torch.ops._C.silu_and_mul_quant(out, x.to(DEV), scale.to(DEV))
    assert float((out.cpu().view(torch.uint8) == ref.view(torch.uint8)).float().mean()) > 0.999
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=0.13, atol=2e-3)
    for c in load_golden("fused_quant.pt")["static"]:
        o = torch.empty_like(c["q"], device=DEV)
        torch.ops._C.silu_and_mul_quant(o, c["x"].to(DEV), c["scale"].to(DEV))
        torch.testing.assert_close(o.cpu().float(), c["q"].float(), rtol=0.13, atol=2e-3)


def test_block_quant_over_the_rows_in_use_only():
    """b200_silu_and_mul_block_quant_rows: the layer's form of silu_and_mul_per_block_quant for row
    buffers sized for a worst case - the rows the segments use get exactly the full op's result,
    the rows past them are neither read nor written."""
    rows, hidden = 300, 512
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, 2 * hidden, generator=g).to(torch.bfloat16).to(DEV)
    seg = torch.tensor([40, 0, 91, 7], dtype=torch.int32, device=DEV)       # 138 rows in use
    used = int(seg.sum())
    ref_q = torch.empty(rows, hidden, dtype=torch.float8_e4m3fn, device=DEV)
    ref_s = torch.empty(rows, hidden // 128, dtype=torch.float32, device=DEV)
    torch.ops._C.silu_and_mul_per_block_quant(ref_q, x, ref_s, 128, None, False, False)
    q = torch.full((rows, hidden), 0x55, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    s = torch.full((rows, hidden // 128), -3.0, dtype=torch.float32, device=DEV)
    torch.ops._C.b200_silu_and_mul_block_quant_rows(q, x, s, seg)
    assert torch.equal(q.view(torch.uint8)[:used], ref_q.view(torch.uint8)[:used])
    assert torch.equal(s[:used], ref_s[:used])
    assert bool((q.view(torch.uint8)[used:] == 0x55).all()) and bool((s[used:] == -3.0).all())
