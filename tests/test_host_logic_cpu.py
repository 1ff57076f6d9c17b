"""CPU: host-side logic of the Python surface (recipe detection, sizes, error
behaviour) - the parts of vllm_xpu_kernels/fused_moe_interface.py:33-69,
:239-254 of the reference that need no device."""
import pytest
import torch


def test_recipe_detection(native):
    f = native
    w = torch.empty(2, 8, 8, dtype=torch.bfloat16)
    assert f._get_weights_dtype(w, None) == (False, False, False, False, False)
    w8 = torch.empty(2, 256, 128, dtype=torch.float8_e4m3fn)
    assert f._get_weights_dtype(w8, torch.empty(2))[0] is True
    blk = f._get_weights_dtype(w8, torch.empty(2, 2, 1, dtype=torch.float32))
    assert blk == (False, False, False, False, True)
    mx8 = f._get_weights_dtype(w8, torch.empty(2, 256, 4, dtype=torch.uint8))
    assert mx8[3] is True and mx8[0] is False
    w4 = torch.empty(2, 64, 16, dtype=torch.uint8).view(torch.float4_e2m1fn_x2)
    assert f._get_weights_dtype(w4, torch.empty(2, 64, 1, dtype=torch.uint8))[2] is True
    assert f._get_recipe(False, False, False, False, True) == "fp8block"
    assert f._get_recipe(False, False, True, False, False) == "mxfp4"
    assert f._get_recipe(False, False, False, False, False) == "bf16"


@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_block_fp8_inter_size_uses_scales(native, layout):
    # the reference's own CPU-checkable test (tests/fused_moe/test_fused_moe.py:37-60)
    w_nk = torch.empty(2, 512, 256, dtype=torch.float8_e4m3fn)
    w = w_nk.transpose(-1, -2).contiguous() if layout == "kn" else w_nk
    scales = torch.empty(2, 4, 2, dtype=torch.float32)
    assert native._get_inter_size(w, scales, False, False, True) == 256


def test_inter_size_other_recipes(native):
    assert native._get_inter_size(torch.empty(2, 64, 96), None, False, False, False) == 48
    assert native._get_inter_size(torch.empty(2, 96, 32), None, False, True, False) == 48


def test_unknown_activation_raises_value_error(native):
    w13 = torch.empty(2, 16, 32, dtype=torch.bfloat16)
    w2 = torch.empty(2, 16, 16, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="Unsupported FusedMoe activation"):
        native.XpuFusedMoe(w13, None, None, w2, None, None, 1, "tanh", 2)
    with pytest.raises(ValueError, match="Unsupported FusedMoe activation"):
        native.fused_moe_activation(None, None, "relu")


def test_compute_num_tokens_per_block(native):
    assert native.compute_num_tokens_per_block(1, 8) == 32
    assert native.compute_num_tokens_per_block(4096, 8) == 256
    assert native.ceilDiv(7, 2) == 4


def test_xpu_fused_moe_checks_output_shape(native):
    x = torch.empty(4, 32, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="output shape must be the same"):
        native.xpu_fused_moe(x, None, None, None, None, None, None, None, None, 1, "silu", 2,
                             output=torch.empty(3, 32, dtype=torch.bfloat16))
