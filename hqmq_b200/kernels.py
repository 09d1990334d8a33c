"""Kernel entry points under the reference's hardware-specific names (hqmq/kernels.py:6-36).

The reference ships one Triton kernel body under three names (Ada, Hopper, "Blackwell"); here
all three resolve to the single sm_100a CUDA kernel family.
"""
from .attention import blackwell_available, decode_dequant, encode_joint_fp8, hopper_available
from .attention import fused_hqmq_attention as fused_attention_ada
from .attention import fused_hqmq_attention as fused_attention_blackwell
from .attention import fused_hqmq_attention as fused_attention_hopper
from .attention import fused_hqmq_attention_dequant_sdpa as fused_attention_reference

__all__ = [
    "fused_attention_ada", "fused_attention_hopper", "fused_attention_blackwell", "fused_attention_reference",
    "decode_dequant", "encode_joint_fp8", "hopper_available", "blackwell_available",
]
