"""hqmq_b200: B200 (sm_100a) implementation of the HQMQ KV-cache hot path, behind the public
names of the reference package (hqmq/__init__.py:54-123 of kswain98/hqmq):

    import hqmq_b200 as hqmq
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(n_layers=32, n_heads=8, secondary_size=96, radius_bits=4), C=3.0)
    Kq = q.quantize_K(K, layer_idx=0)                       # fake-quant, as the reference
    cache = q.encode(K, layer_idx=0, kv=0)                  # compressed planes (new)
    O = hqmq.fused_attention(Q, K_idx, K_rq, K_rs, joint_K, V_idx, V_rq, V_rs, joint_V, r_qmax=15, causal=False)

All arithmetic runs in hand-written CUDA kernels loaded from libhqmq_b200.so; there is no Triton,
no backend dispatch and no CPU fallback (CPU tensors raise).
"""
from . import attention as kernels_ada          # noqa: F401  one kernel family serves all three names
from . import attention as kernels_hopper       # noqa: F401
from . import attention as kernels_blackwell    # noqa: F401
from .attention import fused_attention_packed, fused_attention_packed_noalloc, combine_partials, decode_dequant  # noqa: F401
from .attention import fused_hqmq_attention as fused_attention
from .attention import fused_hqmq_attention_dequant_sdpa as fused_attention_reference
from ._lib import HqmqError  # noqa: F401
from .packed import PackedKV  # noqa: F401
from .cache import PackedKVCache  # noqa: F401
from .quantizers import HQMQQuantizer as HQMQ
from .quantizers import KVQuantizer  # noqa: F401
from .quantizers import OutlierAwareGenericQuantizer, OutlierAwareHQMQQuantizer
from .quantizers import PaddedHQMQQuantizer as PaddedHQMQ


def with_outlier_extraction(quantizer, C: float = 3.0, *, generic: bool = False):
    """Wrap a quantizer with median-multiplier outlier extraction: chunks whose norm exceeds
    C * (per-call, per-head median) keep their original values (hqmq/__init__.py:71-91)."""
    if generic:
        return OutlierAwareGenericQuantizer(quantizer, chunk_dim=4, threshold_mode="median_mult", median_mult=C)
    return OutlierAwareHQMQQuantizer(quantizer, threshold_mode="median_mult", median_mult=C)


def device_info() -> dict:
    """GPU and kernel variant in use (hqmq/__init__.py:94-114).  Both the CPU-branch and the
    GPU-branch keys of the reference are always present."""
    import torch
    info = {"gpu": None, "variant": "cpu", "fp8_codebook": False, "compute_capability": None,
            "variant_auto_dispatched": "cpu", "fp8_codebook_supported": False}
    if not torch.cuda.is_available():
        return info
    cap = torch.cuda.get_device_capability()
    if cap[0] >= 10:
        variant, fp8 = "blackwell", True
    elif cap[0] >= 9:
        variant, fp8 = "hopper", True
    elif cap[0] >= 8:
        variant, fp8 = "ada", False
    else:
        variant, fp8 = "ada (older)", False
    info.update(gpu=torch.cuda.get_device_name(), compute_capability=f"{cap[0]}.{cap[1]}", variant=variant,
                variant_auto_dispatched=variant, fp8_codebook=fp8, fp8_codebook_supported=fp8)
    return info


__all__ = [
    "HQMQ", "PaddedHQMQ", "OutlierAwareHQMQQuantizer", "OutlierAwareGenericQuantizer",
    "fused_attention", "fused_attention_reference", "with_outlier_extraction", "device_info",
    "kernels_ada", "kernels_hopper", "kernels_blackwell",
    "PackedKV", "PackedKVCache", "fused_attention_packed", "combine_partials", "decode_dequant", "HqmqError",
]
__version__ = "0.1.0"
