"""The reference's ``QuantizedCache`` (src/model_utils.py:22-32) on this library's quantizers.

The reference subclasses HuggingFace's ``DynamicCache`` and passes every new K / V tensor through
``quantizer.quantize_K`` / ``quantize_V`` before the parent class stores it, so a model called with
``past_key_values=QuantizedCache(q)`` attends over fake-quantised tensors.  ``QuantizedCache`` here is the same
class with the same constructor and ``update`` signature; its quantize calls run the CUDA encoder and decoder of
this library (bit-identical outputs for fp32 inputs, the contract of ``quantize_K`` / ``quantize_V``).

``store="packed"`` keeps only the compressed planes (``PackedKVCache``) and hands the attention of the calling
model a dense reconstruction of the layer on every ``update`` -- the memory saving the reference's class
does not have, at the price of one dequantisation of the layer per step; a caller that can take the compressed
planes directly uses ``cache.packed.attend(query, layer_idx)`` instead and reads nothing dense at all.

``transformers`` is imported when this module is, not with the package: the kernels do not depend on it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
from transformers import DynamicCache

from .cache import PackedKVCache


class QuantizedCache(DynamicCache):
    """``DynamicCache`` that quantises K and V on every update (src/model_utils.py:22-32).

    ``quantizer``: anything with ``quantize_K(k, layer_idx)`` / ``quantize_V(v, layer_idx)`` of this package
    (``HQMQ``, ``with_outlier_extraction(...)``, ``PaddedHQMQ``).  ``store``: ``"dense"`` (the reference's behaviour:
    the parent class keeps the fake-quantised 16-bit tensors) or ``"packed"`` (compressed planes only; needs
    ``max_tokens``, the fixed capacity per layer, and a quantizer the packed cache accepts)."""

    def __init__(self, quantizer, store: str = "dense", max_tokens: Optional[int] = None,
                 sliding_window: Optional[Dict[int, int]] = None, outlier_capacity: float = 0.125):
        super().__init__()
        if store not in ("dense", "packed"):
            raise ValueError(f"store={store!r}: expected 'dense' or 'packed'")
        if store == "packed" and not max_tokens:
            raise ValueError("store='packed' keeps fixed-capacity planes: pass max_tokens")
        self.quantizer = quantizer
        self.store = store
        self.packed = (PackedKVCache(quantizer, max_tokens, sliding_window=sliding_window,
                                     outlier_capacity=outlier_capacity) if store == "packed" else None)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int, cache_kwargs=None):
        if self.packed is None:
            k_q = self.quantizer.quantize_K(key_states, layer_idx)
            v_q = self.quantizer.quantize_V(value_states, layer_idx)
            return super().update(k_q, v_q, layer_idx, cache_kwargs)
        self.packed.update(key_states, value_states, layer_idx)
        return self.packed.dense(layer_idx, dtype=key_states.dtype)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if self.packed is None:
            return super().get_seq_length(layer_idx)
        return self.packed.get_seq_length(layer_idx)

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0):
        """(kv_length, kv_offset) the calling model builds its attention mask for."""
        if self.packed is None:
            return super().get_mask_sizes(query_length, layer_idx)
        return self.packed.get_seq_length(layer_idx) + query_length, 0

    def compressed_bytes(self) -> int:
        """Bytes of the compressed planes behind the tokens cached so far (``store="packed"``)."""
        if self.packed is None:
            raise ValueError("store='dense' keeps 16-bit tensors, like the reference's cache")
        return self.packed.compressed_bytes()
