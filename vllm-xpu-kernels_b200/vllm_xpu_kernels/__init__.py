"""B200 (sm_100a) fused-MoE kernels behind the ``vllm_xpu_kernels`` Python surface.

Importing the package does not load any native code; ``fused_moe_interface``
imports the three op-registration libraries (``_C``, ``_moe_C``, ``_xpu_C``)
and records whether they are present.
"""
__all__ = ["fused_moe_interface", "moe_utils"]
