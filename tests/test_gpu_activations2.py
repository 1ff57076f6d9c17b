"""GPU parity of gelu_and_mul, gelu_tanh_and_mul, swiglustep_and_mul and
relu2_no_mul (tolerances of the reference's tests/test_activation.py and
tests/test_swiglustep_and_mul.py: bf16 rtol 1.6e-2 / 2e-2, fp16 and fp32 tighter)
and of the layer with each of them."""
import pytest
import torch

from conftest import load_golden
from gpu_utils import DEV
from oracle import torch_oracle as to
from oracle import workloads as wl

pytestmark = pytest.mark.gpu

TOL = {torch.float16: dict(rtol=2e-3, atol=1e-3), torch.bfloat16: dict(rtol=2e-2, atol=1e-3),
       torch.float32: dict(rtol=1e-5, atol=1e-5)}


def _run(op, x, d_out, *extra):
    out = torch.empty(*x.shape[:-1], d_out, dtype=x.dtype, device=DEV)
    op(out, x.to(DEV), *extra)
    return out.cpu()


@pytest.mark.parametrize("T", [1, 7, 83, 2048])
@pytest.mark.parametrize("d", [32, 512, 13824, 20])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_gated_activations(native, T, d, dtype):
    if T * d > 4_000_000 and dtype == torch.float32:
        pytest.skip("covered by the 16-bit cases")
    g = torch.Generator().manual_seed(T + d)
    x = (torch.randn(T, 2 * d, generator=g) * 3).to(dtype)
    C = torch.ops._C
    torch.testing.assert_close(_run(C.gelu_and_mul, x, d), to.gelu_and_mul(x), **TOL[dtype])
    torch.testing.assert_close(_run(C.gelu_tanh_and_mul, x, d), to.gelu_and_mul(x, "tanh"), **TOL[dtype])
    torch.testing.assert_close(_run(C.swiglustep_and_mul, x, d, 7.0), to.swiglustep_and_mul(x, 7.0), **TOL[dtype])
    torch.testing.assert_close(_run(C.swiglustep_and_mul, x, d, 1.5), to.swiglustep_and_mul(x, 1.5), **TOL[dtype])
    torch.testing.assert_close(_run(C.relu2_no_mul, x, 2 * d), to.relu2_no_mul(x), **TOL[dtype])


def test_gated_activations_reference_vectors(native):
    C = torch.ops._C
    for c in load_golden("activations2.pt").values():
        x = c["x"]
        d = x.shape[-1] // 2
        tol = TOL[x.dtype]
        torch.testing.assert_close(_run(C.gelu_and_mul, x, d), c["gelu"], **tol)
        torch.testing.assert_close(_run(C.gelu_tanh_and_mul, x, d), c["gelu_tanh"], **tol)
        torch.testing.assert_close(_run(C.swiglustep_and_mul, x, d, 7.0), c["swiglustep"], **tol)
    x3 = torch.randn(2, 3, 64).to(torch.bfloat16)   # leading dimensions are flattened
    torch.testing.assert_close(_run(C.gelu_and_mul, x3, 32), to.gelu_and_mul(x3), **TOL[torch.bfloat16])


@pytest.mark.parametrize("activation", ["gelu", "gelu_tanh", "swiglustep", "relu2_no_mul"])
def test_layer_other_activations(native, activation):
    """XpuFusedMoe with the remaining activations of the reference's list
    (fused_moe_interface.py:119-133); relu2_no_mul keeps both halves of gemm1's
    output, so w2 takes 2*I inputs (:226, :393, :414)."""
    cfg = wl.scaled(wl.CONFIGS["cfg1_small_bf16"], H=256, I=128, E=4)
    w = wl.make_weights(cfg, seed=5)
    x, logits, _ = wl.make_inputs(cfg, 24, seed=5)
    tw, ids = wl.route_cpu(cfg, logits, None)
    w13, w2 = w["w13"], w["w2"]                   # [E, 2I, H], [E, H, I]
    if activation == "relu2_no_mul":
        g = torch.Generator().manual_seed(9)
        w2 = (torch.randn(cfg.E, cfg.H, 2 * cfg.I, generator=g) * (2 * cfg.I) ** -0.5).to(torch.bfloat16)
    ref = to.fused_moe_staged(x, w13.float(), None, w2.float(), None, tw, ids, cfg.E, activation=activation)
    layer = native.XpuFusedMoe(w13.transpose(1, 2).contiguous().to(DEV), None, None,
                               w2.transpose(1, 2).contiguous().to(DEV), None, None, cfg.K, activation, cfg.E)
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=DEV)
    layer.apply(out, x.to(DEV), tw.to(DEV), ids.to(DEV))
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
