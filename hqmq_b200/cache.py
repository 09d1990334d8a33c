"""A KV cache that HOLDS the compressed representation, one pair of packed planes per layer.

The reference's cache (src/model_utils.py:22-32, ``QuantizedCache``) passes every new K / V tensor through
``quantize_K`` / ``quantize_V`` and then stores the dense fake-quantised result, so it saves no memory and
attention reads 16-bit tensors.  This class keeps the call pattern -- ``update(key_states, value_states,
layer_idx)`` once per layer and forward pass, a prompt first and then one token at a time -- but appends to
the native compressed planes (``PackedKV``) and answers attention straight from them.

Capacity is fixed when the cache is made (``max_tokens``), like the block pools of serving engines: nothing
is reallocated or copied while tokens are appended, so addresses stay stable for CUDA graphs.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .attention import fused_attention_packed
from .packed import PackedKV


class PackedKVCache:
    """Per-layer compressed K and V planes behind the reference cache's ``update`` call.

    ``quantizer``: an ``HQMQQuantizer`` or its outlier-aware wrapper (``with_outlier_extraction``); with the
    wrapper every ``update`` takes its own Med3x median per head, exactly like the reference's wrapper does
    per ``quantize_K`` call.  ``sliding_window``: optional ``{layer_idx: window}`` for layers that attend to
    the last ``window`` tokens only.  ``outlier_capacity``: share of a (batch, head)'s chunks the full-precision
    side buffer can hold (Med3x flags a few percent; 1.0 can never overflow but costs as much memory as a dense
    16-bit cache); ``check()`` tells whether it was exceeded."""

    def __init__(self, quantizer, max_tokens: int, sliding_window: Optional[Dict[int, int]] = None,
                 outlier_capacity: float = 0.125):
        self.quantizer = quantizer
        self.max_tokens = int(max_tokens)
        self.outlier_capacity = float(outlier_capacity)
        self.sliding_window = dict(sliding_window or {})
        self._layers: Dict[int, Tuple[PackedKV, PackedKV]] = {}

    # the quantizer without its wrapper, and the multiplier the wrapper adds (None = no outlier extraction)
    @property
    def _inner(self):
        return getattr(self.quantizer, "inner", self.quantizer)

    @property
    def _with_outliers(self) -> bool:
        return hasattr(self.quantizer, "median_mult")

    def _new_pair(self, k: torch.Tensor) -> Tuple[PackedKV, PackedKV]:
        B, H, _, d = k.shape
        sd = k.dtype if k.dtype in (torch.float16, torch.bfloat16) else torch.float32
        cap = max(1024, int(self.outlier_capacity * self.max_tokens * (d // 4))) if self._with_outliers else None
        mk = lambda kv: self._inner.new_cache(B, self.max_tokens, d, k.device, scale_dtype=sd,
                                              with_outliers=self._with_outliers, out_dtype=k.dtype, out_cap=cap,
                                              ofrag=self._with_outliers and kv == 0)
        return mk(0), mk(1)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs=None) -> Tuple[PackedKV, PackedKV]:
        """Append (B, H_kv, T_new, d) keys and values of one layer; returns the layer's packed pair."""
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have the same shape")
        pair = self._layers.get(layer_idx)
        if pair is None:
            pair = self._layers[layer_idx] = self._new_pair(key_states)
        self.quantizer.encode_pair(key_states, value_states, layer_idx, pair[0], pair[1])
        return pair

    def check(self) -> None:
        """Synchronise and raise if some side buffer was too small for the outliers it was given (rows, flags
        and counts are complete then, but payload entries beyond the capacity were dropped)."""
        from ._lib import HqmqError
        for layer, pair in self._layers.items():
            for name, pk in zip("KV", pair):
                if pk.with_outliers and int(pk.out_count.max()) > pk.out_cap:
                    raise HqmqError(f"hqmq_b200: outlier side buffer of layer {layer} {name} overflowed "
                                    f"({int(pk.out_count.max())} > {pk.out_cap} chunks per (b, h)); raise outlier_capacity")

    def get_seq_length(self, layer_idx: int = 0) -> int:
        pair = self._layers.get(layer_idx)
        return pair[0].T if pair else 0

    def __len__(self) -> int:
        return len(self._layers)

    def attend(self, query_states: torch.Tensor, layer_idx: int, softmax_scale: Optional[float] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of (B, H_q, T_q, d) queries over everything cached for the layer (its last ``window`` tokens
        for a sliding-window layer), read in place from the compressed planes.  The queries are the last ``T_q``
        positions of the cache (call ``update`` first): one decode token sees everything, a prompt chunk is masked
        causally, bottom-right aligned."""
        Kp, Vp = self._layers[layer_idx]
        dev = query_states.device
        tk, tv = self._inner.tables(layer_idx, 0, dev), self._inner.tables(layer_idx, 1, dev)
        return fused_attention_packed(query_states, Kp, Vp, tk["table16"], tv["table16"],
                                      causal="bottom_right" if query_states.shape[2] > 1 else False,
                                      softmax_scale=softmax_scale, window=self.sliding_window.get(layer_idx), out=out)

    def dense(self, layer_idx: int, dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense (B, H_kv, T, d) reconstruction of a layer (outliers restored): what the reference's cache
        would hold, for callers that still need 16-bit tensors."""
        Kp, Vp = self._layers[layer_idx]
        dt = dtype or Kp.out_dtype or torch.float32
        return (self.quantizer.decode(Kp, layer_idx, 0, dtype=dt), self.quantizer.decode(Vp, layer_idx, 1, dtype=dt))

    def compressed_bytes(self) -> int:
        """Algorithmic bytes held for the tokens cached so far (the figure the roofline uses)."""
        return sum(k.algorithmic_bytes() + v.algorithmic_bytes() for k, v in self._layers.values())
