# SPDX-License-Identifier: Apache-2.0
"""Fused Mixture-of-Experts layer: the Python entry point.

Mirrors ``vllm_xpu_kernels/fused_moe_interface.py`` of vllm-xpu-kernels
(``XpuFusedMoe`` :165-419, ``xpu_fused_moe`` :421-619): same class and function
names, argument order, defaults and weight-layout contract, so a caller of the
reference can switch without edits.  The work is done by the CUDA kernels
registered as ``torch.ops._moe_C / _C / _xpu_C`` (hand-written for sm_100a);
there is no CPU or eager-torch fallback: if the native libraries are missing,
``FUSEDMOE_AVAILABLE`` is False and every call raises.

Weight layouts (as in the reference, :47-69 and
csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:200-223):

* bf16 / fp16 and per-tensor fp8:  ``[E, K, N]`` (the transposed checkpoint);
* block fp8 (fp32 scales ``[E, N/128, K/128]``): ``[E, N, K]`` or ``[E, K, N]``;
* MXFP4 (``float4_e2m1fn_x2``): ``[E, N, K/2]`` with e8m0 scales ``[E, N, K/32]``.
"""
import os
from typing import Optional

import torch

try:
    from . import _C  # noqa: F401
    from . import _moe_C  # noqa: F401
    from . import _xpu_C  # noqa: F401
    FUSEDMOE_UNAVAILABLE_REASON = None
    FUSEDMOE_AVAILABLE = True
except ImportError as e:  # native libraries not built
    FUSEDMOE_UNAVAILABLE_REASON = str(e)
    FUSEDMOE_AVAILABLE = False

from .moe_utils import quant_act_xpu

REF_FUSED_MOE_ENV = "VLLM_XPU_FUSED_MOE_USE_REF"
USE_MXFP4_FP8_ENV = "VLLM_XPU_FUSED_MOE_USE_MXFP4_FP8"
FP8_BLOCK_SIZE = 128
FP8_FUSED_MIN_ROWS = 512   # routed rows per expert from which gemm1 of an fp8 layer fuses SiLU + quantisation

# Epilogue codes of torch.ops._xpu_C.b200_grouped_gemm (b200moe_epilogue).
_EPI_NONE, _EPI_SILU, _EPI_SWIGLUOAI = 0, 1, 2


def _require_native():
    if not FUSEDMOE_AVAILABLE:
        raise RuntimeError(
            "vllm_xpu_kernels: the native CUDA libraries are not built "
            f"({FUSEDMOE_UNAVAILABLE_REASON}); run build.py - there is no fallback path")


def _is_env_enabled(env_name: str, default: str = "0") -> bool:
    value = os.environ.get(env_name, default).strip().upper()
    return value in ("1", "ON", "TRUE", "YES", "Y")


def _get_recipe(is_fp8, is_mxfp8, is_mxfp4, is_int4, is_block_fp8):
    if is_mxfp8:
        return "mxfp8"
    elif is_block_fp8:
        return "fp8block"
    elif is_mxfp4:
        return "mxfp4_fp8" if _is_env_enabled(USE_MXFP4_FP8_ENV) else "mxfp4"
    elif is_int4:
        return "int4"
    elif is_fp8:
        return "fp8"
    else:
        return "bf16"


def _get_weights_dtype(weight, scales):
    weight_dtype = weight.dtype
    is_fp8 = weight_dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
    is_int4 = weight_dtype == torch.uint8
    is_mxfp4 = weight_dtype == torch.float4_e2m1fn_x2
    is_mxfp8 = (is_fp8 and scales is not None and scales.dtype == torch.uint8)
    is_block_fp8 = (is_fp8 and scales is not None
                    and scales.dtype == torch.float32 and scales.ndim == 3)
    is_fp8 = is_fp8 and not is_mxfp8 and not is_block_fp8
    return is_fp8, is_int4, is_mxfp4, is_mxfp8, is_block_fp8


def _get_inter_size(w13, w13_scales, is_int4, is_mxfp4, is_block_fp8):
    if is_block_fp8:
        return w13_scales.shape[-2] * FP8_BLOCK_SIZE // 2
    if is_int4 or is_mxfp4:
        return w13.shape[-2] // 2
    return w13.shape[-1] // 2


def cutlass_grouped_gemm_xe2(input_A, input_B, scales, bias, output,
                             num_rows_per_expert, n, k, num_experts):
    """Same helper as the reference (:92-104): one grouped GEMM call."""
    _require_native()
    torch.ops._xpu_C.cutlass_grouped_gemm_interface(
        ptr_A=input_A, ptr_A_scale=None, ptr_B=input_B, ptr_B_scale=scales,
        ptr_bias=bias, ptr_D=output, rows_per_expert=num_rows_per_expert,
        N=n, K=k, num_experts=num_experts)


def cutlass_grouped_gemm(input_A, input_A_scale, input_B, input_B_scale, bias,
                         output, expert_token_count, n, k, num_experts):
    """Reference helper (:72-89) taking the row counts as a host list."""
    _require_native()
    num_rows_per_expert = torch.tensor(expert_token_count, dtype=torch.int32,
                                       device=input_A.device)
    torch.ops._xpu_C.cutlass_grouped_gemm_interface(
        ptr_A=input_A, ptr_A_scale=input_A_scale, ptr_B=input_B,
        ptr_B_scale=input_B_scale, ptr_bias=bias, ptr_D=output,
        rows_per_expert=num_rows_per_expert, N=n, K=k, num_experts=num_experts)


def ceilDiv(a, b):
    return (a + b - 1) // b


def compute_num_tokens_per_block(num_tokens, num_experts_per_node):
    for num_tokens_per_block in [32, 64, 128, 256, 512, 1024]:
        num_blocks_per_seq = ceilDiv(num_tokens, num_tokens_per_block)
        if num_blocks_per_seq * num_experts_per_node <= num_tokens_per_block:
            return num_tokens_per_block
    return 1024


# Intermediates of a layer call (permuted rows, the two GEMM outputs, scales, index maps) live
# in one grow-only pool per device, shared by all layer objects: layers of a model run one after
# the other on a stream, so the next call may overwrite what the previous one left.  A caller
# that runs layer calls concurrently on several streams of one device must pass
# ``persistent_workspace=False`` (fresh torch allocations per call, as the reference does).
_WORKSPACE = {}


def _pooled(name, shape, dtype, device):
    n = 1
    for d in shape:
        n *= int(d)
    key = (device, name, dtype)
    buf = _WORKSPACE.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1), dtype=dtype, device=device)
        _WORKSPACE[key] = buf
    return buf[:n].view(shape)


def _signed_nibbles(w):
    """uint8 pairs of uint4 (zero point 8) -> int8 pairs of two's-complement int4, cached on
    the source tensor while its contents are unchanged."""
    cached = getattr(w, "_b200_signed_nibbles", None)
    if cached is not None and cached[0] == w._version:
        return cached[1]
    conv = (w ^ 0x88).view(torch.int8)
    w._b200_signed_nibbles = (w._version, conv)
    return conv


def _activation_kind(activation):
    """Maps the reference's activation names (:119-133, :239-254) to an op."""
    if activation in ("silu", "gelu", "gelu_tanh", "relu2_no_mul", "swiglustep"):
        return activation
    if activation == "swigluoai" or ("SWIGLUOAI" in str(activation)):
        return "swigluoai"
    raise ValueError(f"Unsupported FusedMoe activation: {activation}.")


def _activation_op(kind):
    """The op ``act(out, gemm1_output)`` of an activation kind."""
    C = torch.ops._C
    return {
        "silu": C.silu_and_mul,
        "gelu": C.gelu_and_mul,
        "gelu_tanh": C.gelu_tanh_and_mul,
        "swigluoai": lambda out, x: C.swigluoai_and_mul(out, x, 1.702, 7.0),
        "relu2_no_mul": C.relu2_no_mul,
        "swiglustep": lambda out, x: C.swiglustep_and_mul(out, x, 7.0),
    }[kind]


def fused_moe_activation(act_output, gemm1_output, activation):
    _activation_op(_activation_kind(activation))(act_output, gemm1_output)


class XpuFusedMoe:
    """The fused-MoE layer object (reference :165-419).

    ``fuse_activation`` (not in the reference; keyword only) applies the gated
    activation inside the first grouped GEMM's epilogue instead of a separate
    pass over ``[T*K, 2I]``.  ``None`` (default) picks it where the tensor-core
    kernel of the recipe has that epilogue and it pays: MXFP4 and 16-bit
    weights with SwigluOAI always; 16-bit weights with SiLU always when the
    intermediate size is a multiple of 128 (else up to 96 routed rows per
    expert); block-scaled fp8 with SiLU (where the epilogue also
    quantises gemm2's input to e4m3 per 1x128 group, with the same values as
    the two-kernel form) from ``FP8_FUSED_MIN_ROWS`` routed rows per expert on.
    ``True`` forces it wherever a kernel has it, ``False`` never fuses.

    ``persistent_workspace`` (not in the reference; keyword only, default
    True): intermediates come from one grow-only pool per device shared by all
    layer objects instead of fresh allocations per call; a layer object (and
    the pool) must then be used from one stream at a time.

    ``mxfp4_activations`` (not in the reference; keyword only) chooses what the
    MXFP4 (and per-tensor fp8, and MXFP8, whose default is one plane as its recipe
    defines) grouped GEMMs multiply the quantised weights with:
    ``"mxfp8x2"`` (default where the shapes allow it: hidden and intermediate
    sizes multiples of 64) quantises the activations to two MXFP8 planes (e4m3
    codes with one power-of-two scale per 32 values, plus the residual
    quantised the same way) and runs the block-scaled tensor-core instruction
    on both: 16-bit-like activation accuracy with nothing dequantised by CUDA
    cores; ``"mxfp8"`` uses one plane (about 3 % activation rounding error, like
    the reference's ``VLLM_XPU_FUSED_MOE_USE_MXFP4_FP8`` recipe, which also
    selects it); ``"bf16"`` keeps 16-bit activations exactly as the reference's
    device kernel does (w4a16) and dequantises the weights on the way into the
    tensor cores.
    """

    def __init__(
        self,
        w13,
        w13_scales,
        w13_bias,
        w2,
        w2_scales,
        w2_bias,
        n_experts_per_token,
        activation,
        num_experts,
        ep_rank=0,
        ep_size=1,
        expert_map=None,
        gemm1_clamp_limit: Optional[float] = None,
        *,
        fuse_activation: Optional[bool] = None,
        mxfp4_activations: Optional[str] = None,
        persistent_workspace: bool = True,
    ):
        assert w13.is_contiguous() and w2.is_contiguous()
        _require_native()

        (is_fp8, is_int4, is_mxfp4, is_mxfp8,
         is_block_fp8) = _get_weights_dtype(w13, w13_scales)
        if w13.dtype == torch.float8_e5m2 and is_block_fp8:
            raise NotImplementedError("block-scaled float8_e5m2 weights are not built for sm_100a yet")
        if _is_env_enabled(REF_FUSED_MOE_ENV):
            raise NotImplementedError(
                f"{REF_FUSED_MOE_ENV} selects the reference's eager qdq simulation, "
                "which this build does not ship: only the CUDA kernels run")

        self.inter_size = _get_inter_size(w13, w13_scales, is_int4, is_mxfp4, is_block_fp8)
        if is_int4 and not getattr(w13, "xpu_fused_moe", False):
            # uint4 with the default zero point 8 -> two's-complement int4 (reference
            # implement_zp, :135-162: u4 - 8 re-encoded per nibble, i.e. bit 3 flipped).
            # The caller's tensors are left as they are; the converted copy rides on them,
            # so the functional form (a new layer object per call) converts once, as the
            # reference does by marking its in-place conversion with `xpu_fused_moe`.
            w13, w2 = _signed_nibbles(w13), _signed_nibbles(w2)
        self.w13 = w13
        self.w2 = w2
        if not (is_fp8 or is_mxfp4 or is_mxfp8 or is_block_fp8 or is_int4):
            self.gemm1_wei_scales = None
            self.gemm2_wei_scales = None
        else:
            self.gemm1_wei_scales = w13_scales
            self.gemm2_wei_scales = w2_scales
        self.w13_bias = w13_bias
        self.w2_bias = w2_bias

        self.n_experts_per_token = n_experts_per_token
        self.activation = activation
        self._act_kind = _activation_kind(activation)
        # relu2_no_mul keeps both halves of gemm1's output (reference :226)
        self.inter_size_scale = 2 if self._act_kind == "relu2_no_mul" else 1
        self.num_experts = num_experts
        self.ep_rank = ep_rank
        self.ep_size = ep_size
        self.is_fp8 = is_fp8
        self.is_int4 = is_int4
        self.is_mxfp4 = is_mxfp4
        self.is_mxfp8 = is_mxfp8
        self.is_block_fp8 = is_block_fp8
        self.gemm1_clamp_limit = gemm1_clamp_limit
        self.recipe = _get_recipe(is_fp8, is_mxfp8, is_mxfp4, is_int4, is_block_fp8)
        self._use_ref = False
        # block-scaled fp8 with SiLU: the token-major tensor-core kernel can apply the activation and the
        # 1x128 e4m3 quantisation of gemm2's input in its epilogue (same values as the two-kernel form).
        # The epilogue runs on the warps that also promote the K blocks' partial sums, the kernel's
        # bottleneck, so it pays only where a weight tile is reused by many token tiles; measured on
        # B200 (gemm1 of the DeepSeek-V3 shape, 65536 rows): 2048 rows per expert 2.61 ms fused against
        # 2.62 + 0.21 ms, 256 rows per expert 2.80 against 2.51 + 0.20 ms.  Taken per call from
        # FP8_FUSED_MIN_ROWS routed rows per expert on; fuse_activation=True / False force it.
        self._fp8_fused_ok = (is_block_fp8 and self._act_kind == "silu" and self.inter_size % FP8_BLOCK_SIZE == 0
                              and fuse_activation is not False)
        self._fp8_fused_min_rows = 12 if fuse_activation else FP8_FUSED_MIN_ROWS
        # 16-bit weights with SiLU: the tensor-core kernel pairs gate and up tiles in two
        # accumulators, which tensor memory holds for token tiles up to 128; for long expert
        # segments and K >= 4096 a CTA pair splits gate and up between its CTAs on 256-token
        # tiles.  With whole 128-feature tiles (I % 128 == 0) the fused form is taken at every
        # size; otherwise up to 96 routed rows per expert, where 128-token tiles are picked anyway
        # (fuse_activation=True forces it at every size).
        is_16bit = not (is_fp8 or is_mxfp4 or is_mxfp8 or is_block_fp8 or is_int4)
        # SwigluOAI keeps gate and up of a feature on neighbouring accumulator lanes: one accumulator,
        # every tile size, so it is fused at every size.
        self._w16_fused_ok = (is_16bit and self._act_kind in ("silu", "swigluoai") and self.inter_size % 16 == 0
                              and fuse_activation is not False)
        self._w16_fused_max_rows = None if (fuse_activation or self._act_kind == "swigluoai"
                                            or self.inter_size % 128 == 0) else 96
        if fuse_activation is None:
            # fused where the tensor-core kernel of this recipe has the epilogue
            fuse_activation = self.is_mxfp4 and self._act_kind == "swigluoai"
        if is_block_fp8:
            fuse_activation = False     # (the fp8 form is chosen per call, see _experts)
        self.fuse_activation = fuse_activation
        if mxfp4_activations is None:
            # the mxfp8 recipe is defined with MXFP8 activations (reference moe_utils.py:198-200)
            mxfp4_activations = "mxfp8" if self.recipe in ("mxfp4_fp8", "mxfp8") else "mxfp8x2"
        if mxfp4_activations not in ("mxfp8x2", "mxfp8", "bf16"):
            raise ValueError("mxfp4_activations must be 'mxfp8x2', 'mxfp8' or 'bf16', "
                             f"got {mxfp4_activations!r}")
        self.mx_planes = 2 if mxfp4_activations == "mxfp8x2" else 1
        # MXFP4 and per-tensor fp8 weights both run on the block-scaled tensor-core
        # instruction against MXFP8 activation planes where the shapes allow it
        # ([E,N,K/2] resp. [E,K,N] weights; K of both GEMMs a multiple of 64, N of 16)
        if is_mxfp4:
            hidden, gran = w2.shape[-2], 64
        elif is_fp8 or is_mxfp8:
            hidden, gran = w2.shape[-1], 32
        else:
            hidden, gran = 0, 1
        k2 = self.inter_size * self.inter_size_scale
        self.mx_acts = bool((is_mxfp4 or is_fp8 or is_mxfp8) and mxfp4_activations != "bf16"
                            and hidden % gran == 0 and k2 % gran == 0 and hidden >= 128 and k2 >= 128
                            and hidden % 16 == 0 and self.inter_size % 8 == 0)
        if self.mx_acts and self._act_kind == "silu" and fuse_activation:
            raise ValueError("the block-scaled MXFP4 GEMM has no fused SiLU epilogue")
        if fuse_activation and self._act_kind not in ("silu", "swigluoai"):
            raise ValueError(f"no fused epilogue for the {self._act_kind} activation")
        self.act_func = _activation_op(self._act_kind)

        self.expert_map = expert_map
        if self.expert_map is None and self.ep_size > 1:
            self.expert_map = torch.empty((self.num_experts * self.ep_size),
                                          dtype=torch.int32, device=w13.device)
            torch.ops._moe_C.init_expert_map(self.expert_map, self.num_experts,
                                             self.ep_rank, self.ep_size)
        if self.expert_map is not None:
            self.total_experts_num = self.expert_map.shape[0]
        else:
            self.total_experts_num = self.num_experts * self.ep_size
        self.local_experts_num = self.num_experts
        # >0: cap on the CTAs of the persistent GEMM kernels (set by callers that
        # overlap a collective with this layer and need free SMs for it)
        self.gemm_max_ctas = 0
        # >0: rows expected in use when the row buffers are sized for a worst case (set by the
        # expert-parallel layer, whose receive regions are mostly empty): tile sizes only
        self.rows_hint = 0
        self.persistent_workspace = persistent_workspace
        # optional callable(name), called after every stage of a call (routing is what precedes the
        # first mark): lets a harness put CUDA events between the stages, as the reference's
        # benchmark does (benchmark/src/fused_moe_interface_.py:12-40)
        self.stage_hook = None

    def _mark(self, name):
        if self.stage_hook is not None:
            self.stage_hook(name)

    def _buf(self, name, shape, dtype, device):
        if self.persistent_workspace:
            return _pooled(name, shape, dtype, device)
        return torch.empty(shape, dtype=dtype, device=device)

    def apply(self, output, hidden_states, topk_weights, topk_ids,
              expert_map=None, a1q_scale=None):
        self._apply_kernel(output, hidden_states, topk_weights, topk_ids,
                           expert_map, a1q_scale)

    def _quant_mx(self, x):
        """[rows, cols] 16-bit -> (e4m3 codes [planes * rows, cols], int32 scale words
        [planes, ceil(cols / 128), rows]); planes = 2 adds the residual plane."""
        rows, cols = x.shape
        planes = self.mx_planes
        q = self._buf(f"mxq{cols}", (planes * rows, cols), torch.float8_e4m3fn, x.device)
        s = self._buf(f"mxs{cols}", (planes, (cols + 127) // 128, rows), torch.int32, x.device)
        torch.ops._C.b200_quant_mxfp8(x, q, s)
        return q, s

    # The stages below are the reference's eight steps (:328-419); what differs
    # is inside the ops and, for block fp8, that activations really are
    # quantised to e4m3 per 1x128 group and multiplied on the fp8 tensor cores.
    def _apply_kernel(self, output, hidden_states, topk_weights, topk_ids,
                      expert_map=None, a1q_scale=None, gather=True, out_dtype=None):
        """With ``gather=False`` the last stage is left to the caller: returns the expert-major
        rows ``[T*K, hidden]`` after gemm2 and the row map ``[T, K]`` (valid until the next
        layer call on this device)."""
        self._mark("routing")
        num_rows, hidden_size = hidden_states.shape
        K = self.n_experts_per_token
        num_moe_inputs = K * num_rows
        dev = hidden_states.device
        E = self.num_experts
        I = self.inter_size
        if expert_map is None and self.ep_size > 1:
            expert_map = self.expert_map
        if out_dtype is None:
            out_dtype = output.dtype if output is not None else hidden_states.dtype
        if (a1q_scale is not None and hidden_states.dtype != out_dtype and not self.is_block_fp8):
            # The reference forwards caller-quantised activations and their scales to gemm1 for
            # every recipe; here only the block-scaled fp8 kernels take them (1x128 fp32 scales).
            raise NotImplementedError(
                f"a1q_scale with pre-quantised hidden_states is built for block-scaled fp8 weights only "
                f"(recipe of this layer: {self.recipe}); pass 16-bit hidden_states instead")

        rows_per_expert = self._buf("rows_per_expert", (E,), torch.int32, dev)
        row_map = self._buf("row_map", (num_rows, K), torch.int32, dev)

        quant_acts = self.is_block_fp8
        if quant_acts and a1q_scale is None:
            # permute + dynamic 1x128 e4m3 quantisation in one pass
            remapped = self._buf("remapped", (num_moe_inputs, hidden_size), torch.float8_e4m3fn, dev)
            remapped_scales = self._buf("remapped_scales", (num_moe_inputs, hidden_size // FP8_BLOCK_SIZE),
                                        torch.float32, dev)
            torch.ops._moe_C.b200_remap_quant_fp8(
                hidden_states, remapped, remapped_scales, expert_map, rows_per_expert,
                row_map, topk_ids, self.total_experts_num, self.local_experts_num)
        else:
            if a1q_scale is not None:
                remapped_scales = self._buf("remapped_scales", (num_moe_inputs, a1q_scale.shape[1]),
                                            a1q_scale.dtype, dev)
            else:
                remapped_scales = None
            remapped = self._buf("remapped", (num_moe_inputs, hidden_size), hidden_states.dtype, dev)
            torch.ops._moe_C.remap_hidden_states(
                hidden_states=hidden_states, hidden_states_scales=a1q_scale,
                remapped_hidden_states=remapped,
                remapped_hidden_states_scales=remapped_scales, expert_map=expert_map,
                rows_per_expert=rows_per_expert,
                unpermuted_row_to_permuted_row=row_map, topk_ids=topk_ids,
                total_experts_num=self.total_experts_num,
                local_experts_num=self.local_experts_num)

        self._mark("permute")
        a_scale1 = remapped_scales if quant_acts else None
        gemm2_output = self._buf("gemm2_output", (num_moe_inputs, hidden_size), out_dtype, dev)
        self._experts(gemm2_output, remapped, a_scale1, rows_per_expert)
        if not gather:
            return gemm2_output, row_map
        torch.ops._moe_C.moe_gather(output, gemm2_output, topk_weights, row_map, E)
        self._mark("gather")

    def apply_sorted(self, output_rows, rows, rows_per_segment, a1q_scale=None):
        """The experts alone (gemm1 -> activation -> gemm2) on rows that are already grouped:
        ``rows_per_segment`` (int32, a multiple of ``num_experts`` entries) gives consecutive row
        segments, segment ``s`` belongs to expert ``s % num_experts``; ``output_rows[i]`` is the
        result for ``rows[i]``.  No permutation and no top-k reduction happen here: this is what
        an expert-parallel exchange needs for rows that arrive grouped by source rank and, inside
        a source, by local expert.  16-bit weights, or block-scaled fp8 weights with fp8 ``rows``
        and their 1x128 scales in ``a1q_scale``.  (Not in the reference.)"""
        if self.is_block_fp8:
            if rows.dtype != torch.float8_e4m3fn or a1q_scale is None:
                raise ValueError("apply_sorted with block-scaled fp8 weights takes fp8 rows and a1q_scale")
        elif self.is_fp8 or self.is_mxfp4 or self.is_mxfp8 or self.is_int4:
            raise NotImplementedError("apply_sorted: 16-bit or block-scaled fp8 weights only")
        if rows.shape[0] == 0:
            return
        self._experts(output_rows, rows, a1q_scale if self.is_block_fp8 else None, rows_per_segment)

    def fuses_activation(self, num_moe_inputs):
        """Which form gemm1 takes for a call with `num_moe_inputs` routed rows: "fp8" (SiLU and the
        1x128 quantisation in the epilogue), "epilogue" (the gated activation in the epilogue), or
        None (a separate activation kernel)."""
        rows_expected = self.rows_hint if self.rows_hint > 0 else num_moe_inputs
        E = self.num_experts
        if self._fp8_fused_ok and rows_expected >= self._fp8_fused_min_rows * E:
            return "fp8"
        if self.fuse_activation or (self._w16_fused_ok and (
                self._w16_fused_max_rows is None or rows_expected <= self._w16_fused_max_rows * E)):
            return "epilogue"
        return None

    def _experts(self, gemm2_output, remapped, a_scale1, rows_per_expert):
        """gemm1 (+ activation) and gemm2 on permuted rows; writes gemm2_output [rows, hidden]."""
        num_moe_inputs, hidden_size = remapped.shape
        dev = remapped.device
        E = self.num_experts
        I = self.inter_size
        quant_acts = self.is_block_fp8
        output = gemm2_output
        if self.mx_acts:
            remapped, a_scale1 = self._quant_mx(remapped)
        clamp = float(self.gemm1_clamp_limit) if (self.gemm1_clamp_limit is not None
                                                   and self.gemm1_clamp_limit > 0) else 0.0

        # ---- gemm1 (+ activation) ----
        fused = self.fuses_activation(num_moe_inputs)
        if fused == "fp8":
            act_output = None
            act_q = self._buf("act_q", (num_moe_inputs, I), torch.float8_e4m3fn, dev)
            gemm2_act_scale = self._buf("act_q_scale", (num_moe_inputs, I // FP8_BLOCK_SIZE), torch.float32, dev)
            torch.ops._xpu_C.b200_grouped_gemm(
                remapped, a_scale1, self.w13, self.gemm1_wei_scales, self.w13_bias, act_q,
                rows_per_expert, 2 * I, hidden_size, E, 0, _EPI_SILU, 1.702, 7.0, clamp, 0,
                self.gemm_max_ctas, self.rows_hint, gemm2_act_scale, output.dtype == torch.float16)
            self._mark("gemm1")
        elif fused == "epilogue":
            act_output = self._buf("act_output", (num_moe_inputs, I), output.dtype, dev)
            torch.ops._xpu_C.b200_grouped_gemm(
                remapped, a_scale1, self.w13, self.gemm1_wei_scales, self.w13_bias, act_output,
                rows_per_expert, 2 * I, hidden_size, E, 0,
                _EPI_SILU if self._act_kind == "silu" else _EPI_SWIGLUOAI, 1.702, 7.0, clamp, 0,
                self.gemm_max_ctas, self.rows_hint)
            self._mark("gemm1")
        else:
            gemm1_output = self._buf("gemm1_output", (num_moe_inputs, 2 * I), output.dtype, dev)
            torch.ops._xpu_C.b200_grouped_gemm(
                remapped, a_scale1, self.w13, self.gemm1_wei_scales, self.w13_bias, gemm1_output,
                rows_per_expert, 2 * I, hidden_size, E, 0, _EPI_NONE, 1.702, 7.0, 0.0, 0,
                self.gemm_max_ctas, self.rows_hint)
            self._mark("gemm1")
            if clamp > 0:
                gate = gemm1_output[:, :I]
                up = gemm1_output[:, I:]
                gate.clamp_(max=clamp)
                up.clamp_(min=-clamp, max=clamp)
            if quant_acts and self._act_kind == "silu" and I % FP8_BLOCK_SIZE == 0:
                # SiLU, multiply and the 1x128 e4m3 quantisation of gemm2's input in one pass
                act_output = None
                act_q = self._buf("act_q", (num_moe_inputs, I), torch.float8_e4m3fn, dev)
                gemm2_act_scale = self._buf("act_q_scale", (num_moe_inputs, I // FP8_BLOCK_SIZE), torch.float32, dev)
                # (only the rows the experts' segments use: the buffers may be sized for a worst case)
                torch.ops._C.b200_silu_and_mul_block_quant_rows(act_q, gemm1_output, gemm2_act_scale,
                                                                rows_per_expert)
            else:
                act_output = self._buf("act_output", (num_moe_inputs, I * self.inter_size_scale), output.dtype, dev)
                self.act_func(act_output, gemm1_output)

        self._mark("activation")
        # ---- gemm2 ----
        if quant_acts and act_output is None:
            pass   # already quantised together with the activation
        elif quant_acts:
            act_q, gemm2_act_scale = quant_act_xpu(act_output, self.recipe)
        elif self.mx_acts:
            act_q, gemm2_act_scale = self._quant_mx(act_output)
        else:
            act_q, gemm2_act_scale = act_output, None
        torch.ops._xpu_C.b200_grouped_gemm(
            act_q, gemm2_act_scale, self.w2, self.gemm2_wei_scales, self.w2_bias, gemm2_output,
            rows_per_expert, hidden_size, I * self.inter_size_scale, E, 0, _EPI_NONE, 1.702, 7.0, 0.0, 0,
            self.gemm_max_ctas, self.rows_hint)
        self._mark("gemm2")


def xpu_fused_moe(hidden_states,
                  w13,
                  w13_scales,
                  w13_bias,
                  w2,
                  w2_scales,
                  w2_bias,
                  topk_weights,
                  topk_ids,
                  n_experts_per_token,
                  activation,
                  num_experts,
                  ep_rank=0,
                  ep_size=1,
                  expert_map=None,
                  output=None,
                  is_fp8=False,
                  is_int4=False,
                  is_mxfp4=False,
                  is_mxfp8=False,
                  is_block_fp8=False,
                  gemm1_clamp_limit: Optional[float] = None):
    """Functional form (reference :421-619).  The recipe flags are accepted for
    signature compatibility; as in the class, the recipe is read off the weight
    and scale dtypes."""
    if output is None:
        output = torch.empty_like(hidden_states)
    else:
        assert output.shape == hidden_states.shape, \
            "output shape must be the same as hidden_states shape"
    layer = XpuFusedMoe(w13, w13_scales, w13_bias, w2, w2_scales, w2_bias,
                        n_experts_per_token, activation, num_experts, ep_rank,
                        ep_size, expert_map, gemm1_clamp_limit)
    layer.apply(output, hidden_states, topk_weights, topk_ids)
    return output
