# SPDX-License-Identifier: Apache-2.0
"""Quantisation helpers of the fused-MoE layer.

Mirrors the helper surface of ``vllm_xpu_kernels/moe_utils.py`` in
vllm-xpu-kernels that the layer itself uses (``quant_fp8_block_act`` :150-166,
``quant_act_xpu`` :405-411) plus the pure-tensor dequantisers (:29-68,
:134-148).  The eager qdq simulation ``ref_fused_moe`` of the reference is not
part of this build: only the CUDA kernels run.
"""
import torch

finfo = torch.finfo(torch.float8_e4m3fn)
FP8_E4M3_MIN = finfo.min
FP8_E4M3_MAX = finfo.max

_FP4_E2M1_LUT = torch.tensor(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=torch.float32,
)


def _fp4_e2m1fn_x2_to_float_lut(packed: torch.Tensor) -> torch.Tensor:
    """``[..., N]`` packed e2m1 pairs -> ``[..., 2N]`` fp32 (low nibble first)."""
    lut = _FP4_E2M1_LUT.to(packed.device)
    u8 = packed.view(torch.uint8)
    lo = lut[(u8 & 0xF).long()]
    hi = lut[(u8 >> 4).long()]
    return torch.stack((lo, hi), dim=-1).reshape(*u8.shape[:-1], u8.shape[-1] * 2)


def _as_e8m0(s):
    if s.dtype == torch.uint8:
        return s.view(torch.float8_e8m0fnu)
    return s


def dequant_mxfp4(x_lp, x_scale):
    ori_shape = x_lp.shape
    x = _fp4_e2m1fn_x2_to_float_lut(x_lp).reshape(-1, 32) * (
        _as_e8m0(x_scale).reshape(-1, 1).to(torch.float32))
    return x.reshape(ori_shape[:-1] + (ori_shape[-1] * 2, ))


def dequant_fp8_block_wei(x_lp, x_scale):
    M, K = x_lp.shape
    x = x_lp.view(M // 128, 128, K // 128, 128).to(torch.float32)
    x = x * x_scale.unsqueeze(1).unsqueeze(-1)
    return x.reshape(M, K)


def dequant_fp8_block_act(x_lp, x_scale):
    shape = x_lp.shape
    x = x_lp.reshape(shape[0], shape[-1] // 128, 128).to(torch.float32)
    return (x * x_scale.unsqueeze(-1)).reshape(shape)


def quant_fp8_block_act(x: torch.Tensor):
    """Dynamic per-1x128 e4m3 quantisation through the CUDA op."""
    x_q = torch.empty(x.shape, device=x.device, dtype=torch.float8_e4m3fn)
    shape = x.shape[:-1] + (x.shape[-1] // 128, )
    x_s = torch.empty(shape, device=x.device, dtype=torch.float32)
    torch.ops._C.per_token_group_fp8_quant(x, x_q, x_s, 128, 1e-10,
                                           FP8_E4M3_MIN, FP8_E4M3_MAX, False,
                                           False, False)
    return x_q, x_s


def quant_act_xpu(x, recipe):
    if recipe == "fp8block":
        return quant_fp8_block_act(x)
    raise NotImplementedError(f"Unsupported recipe for quant_act_xpu: {recipe}")
