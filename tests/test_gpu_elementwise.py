"""GPU parity: gated activations, dynamic per-group fp8 quantisation, moe_gather
and moe_sum against the torch oracle, with the reference's tolerances."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-3, atol=1e-3), torch.float16: dict(rtol=2e-3, atol=1e-3),
       torch.bfloat16: dict(rtol=1.6e-2, atol=1e-3)}  # one bf16 ulp; tests/test_activation.py:70-73


@pytest.mark.parametrize("rows,d", [(7, 128), (1, 14336), (83, 1408), (2048, 768), (5, 13), (0, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_silu_and_swigluoai(native, rows, d, dtype):
    g = torch.Generator().manual_seed(rows + d)
    x = (torch.randn(rows, 2 * d, generator=g) * 3).to(dtype)
    out = torch.empty(rows, d, dtype=dtype, device=DEV)
    torch.ops._C.silu_and_mul(out, x.to(DEV))
    torch.testing.assert_close(out.cpu(), to.silu_and_mul(x), **TOL[dtype])
    out2 = torch.empty(rows, d, dtype=dtype, device=DEV)
    torch.ops._C.swigluoai_and_mul(out2, x.to(DEV), 1.702, 7.0)
    torch.testing.assert_close(out2.cpu(), to.swigluoai_and_mul(x.float()).to(dtype), **TOL[dtype])
    out3 = torch.empty(rows, d, dtype=dtype, device=DEV)
    torch.ops._C.swigluoai_and_mul(out3, x.to(DEV))  # schema defaults
    assert torch.equal(out2, out3)


def test_activation_reference_vectors(native):
    a = load_golden("activations.pt")
    for key, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        x = a[f"x_{key}"]
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=dt, device=DEV)
        torch.ops._C.silu_and_mul(out, x.to(DEV))
        torch.testing.assert_close(out.cpu(), a[f"silu_{key}"], **TOL[dt])
        torch.ops._C.swigluoai_and_mul(out, x.to(DEV), 1.702, 7.0)
        torch.testing.assert_close(out.cpu(), a[f"swiglu_{key}"], **TOL[dt])


@pytest.mark.parametrize("rows,cols,group", [(6, 512, 128), (1, 7168, 128), (300, 2048, 128), (17, 768, 128),
                                             (9, 256, 32), (4, 192, 64), (5, 96, 24)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_per_token_group_fp8_quant_exact(native, rows, cols, group, dtype, ue8m0):
    g = torch.Generator().manual_seed(rows * cols)
    x = (torch.randn(rows, cols, generator=g) * 2).to(dtype)
    x[0, :group] = 0
    q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.empty(rows, cols // group, dtype=torch.float32, device=DEV)
    torch.ops._C.per_token_group_fp8_quant(x.to(DEV), q, s, group, 1e-10, -448.0, 448.0, ue8m0, False, False)
    oq, os_ = to.per_token_group_fp8_quant(x, group, 1e-10, ue8m0)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
    # column-major scales (stride(0) < stride(1)), as the reference detects them
    st = torch.empty(cols // group, rows, dtype=torch.float32, device=DEV).t()
    torch.ops._C.per_token_group_fp8_quant(x.to(DEV), q, st, group, 1e-10, -448.0, 448.0, ue8m0, False, False)
    assert torch.equal(st.cpu(), os_)


def test_fp8_quant_reference_vector(native):
    c = load_golden("fp8_group_quant.pt")
    q = torch.empty(c["x"].shape, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.empty(c["s"].shape, dtype=torch.float32, device=DEV)
    torch.ops._C.per_token_group_fp8_quant(c["x"].to(DEV), q, s, 128, 1e-10, -448.0, 448.0, False, False, False)
    # bars of tests/test_fp8_quant.py:341-348: scales 1 %, values 0.15
    torch.testing.assert_close(s.cpu(), c["s"], rtol=1e-2, atol=0)
    torch.testing.assert_close(q.cpu().float(), c["q"].float(), rtol=0.15, atol=0.15)


@pytest.mark.parametrize("T,H,K", [(8, 128, 2), (1, 7168, 8), (1024, 2048, 8), (33, 100, 6), (5, 64, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_moe_gather(native, T, H, K, dtype):
    g = torch.Generator().manual_seed(T + K)
    moe_out = torch.randn(T * K, H, generator=g).to(dtype)
    w = torch.rand(T, K, generator=g)
    rm = torch.randperm(T * K, generator=g).to(torch.int32).view(T, K)
    rm[0, 0] = -1
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    torch.ops._moe_C.moe_gather(out, moe_out.to(DEV), w.to(DEV), rm.to(DEV), 16)
    torch.testing.assert_close(out.cpu(), to.moe_gather(moe_out, w, rm, dtype), rtol=1e-2, atol=1e-2)
    with pytest.raises(RuntimeError, match="topk_weights must be float32"):
        torch.ops._moe_C.moe_gather(out, moe_out.to(DEV), w.to(DEV).half(), rm.to(DEV), 16)


def test_moe_gather_reference_vectors(native):
    for c in load_golden("moe_gather.pt"):
        out = torch.empty_like(c["output"], device=DEV)
        torch.ops._moe_C.moe_gather(out, c["moe_output"].to(DEV), c["topk_weights"].to(DEV),
                                    c["row_map"].to(DEV), 16)
        torch.testing.assert_close(out.cpu(), c["output"], rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("T,K,H", [(1, 2, 64), (33, 8, 2048), (512, 4, 100), (7, 9, 32), (5, 5, 24)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_moe_sum(native, T, K, H, dtype):
    g = torch.Generator().manual_seed(T * K)
    x = torch.randn(T, K, H, generator=g).to(dtype)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    torch.ops._moe_C.moe_sum(x.to(DEV), out, None, None)
    torch.testing.assert_close(out.cpu(), to.moe_sum(x), rtol=1e-2, atol=2e-2)
    ids = torch.randint(-1, 8, (T, K), generator=g, dtype=torch.int32)
    emap = torch.tensor([0, -1, 1, -1, 2, 3, -1, 4], dtype=torch.int32)
    torch.ops._moe_C.moe_sum(x.to(DEV), out, ids.to(DEV), None)
    torch.testing.assert_close(out.cpu(), to.moe_sum(x, ids), rtol=1e-2, atol=2e-2)
    torch.ops._moe_C.moe_sum(x.to(DEV), out, ids.to(DEV).long(), emap.to(DEV))
    torch.testing.assert_close(out.cpu(), to.moe_sum(x, ids, emap), rtol=1e-2, atol=2e-2)


def test_moe_sum_input_validation(native):
    # messages of csrc/moe/moe_align_sum_kernels.cpp:1237-1279 (tests/test_moe_sum.py:104-133)
    x = torch.randn(4, 2, 8, device=DEV)
    out = torch.empty(4, 8, device=DEV)
    with pytest.raises(RuntimeError, match="same dtype"):
        torch.ops._moe_C.moe_sum(x, out.half(), None, None)
    with pytest.raises(RuntimeError, match="expects contiguous"):
        torch.ops._moe_C.moe_sum(x.transpose(0, 1), out, None, None)
    with pytest.raises(RuntimeError, match="input shape must be"):
        torch.ops._moe_C.moe_sum(x, torch.empty(3, 8, device=DEV), None, None)
    with pytest.raises(RuntimeError, match="expert_map requires topk_ids"):
        torch.ops._moe_C.moe_sum(x, out, None, torch.zeros(4, dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError, match=r"topk_ids must have shape"):
        torch.ops._moe_C.moe_sum(x, out, torch.zeros(4, 3, dtype=torch.int32, device=DEV), None)
    with pytest.raises(RuntimeError, match="expert_map must be int32"):
        torch.ops._moe_C.moe_sum(x, out, torch.zeros(4, 2, dtype=torch.int32, device=DEV),
                                 torch.zeros(4, dtype=torch.int64, device=DEV))
