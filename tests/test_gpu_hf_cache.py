"""The reference's QuantizedCache (src/model_utils.py:22-32) behind a HuggingFace model: a tiny randomly
initialised Llama decodes with ``past_key_values=QuantizedCache(quantizer)``."""
import pytest
import torch

import hqmq_b200 as hqmq

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _model():
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=256,
                      attn_implementation="eager")
    return LlamaForCausalLM(cfg).eval().cuda()


class _Recorder(transformers.DynamicCache):
    """Plain cache that remembers what the model handed to ``update``."""
    def __init__(self):
        super().__init__()
        self.seen = []

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.seen.append((layer_idx, key_states.clone(), value_states.clone()))
        return super().update(key_states, value_states, layer_idx, cache_kwargs)


def test_dense_store_is_the_reference_cache():
    """Layer 0 of a prompt sees keys that do not depend on the cache, so what the cache stores for it must be
    quantize_K / quantize_V of exactly those tensors; later steps append one token each."""
    from hqmq_b200.hf_cache import QuantizedCache
    model = _model()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(n_layers=2, n_heads=2, secondary_size=24, radius_bits=3, device="cuda"), 3.0)
    ids = torch.randint(0, 128, (2, 12), device="cuda")
    rec = _Recorder()
    cache = QuantizedCache(q)
    with torch.no_grad():
        model(ids, past_key_values=rec, use_cache=True)
        out = model(ids, past_key_values=cache, use_cache=True)
        k0, v0 = rec.seen[0][1], rec.seen[0][2]
        assert torch.equal(cache.layers[0].keys, q.quantize_K(k0, 0))
        assert torch.equal(cache.layers[0].values, q.quantize_V(v0, 0))
        nxt = out.logits[:, -1:].argmax(-1)
        for _ in range(3):
            out = model(nxt, past_key_values=cache, use_cache=True)
            nxt = out.logits[:, -1:].argmax(-1)
    assert cache.get_seq_length() == 15 and cache.layers[1].keys.shape == (2, 2, 15, 32)
    assert torch.isfinite(out.logits).all()


def test_packed_store_holds_compressed_planes_only():
    """store="packed": the model gets a dense reconstruction per step, the cache keeps the compressed planes, and
    the logits stay close to the dense store's (same quantiser, 16-bit instead of fp32 token scales)."""
    from hqmq_b200.hf_cache import QuantizedCache
    model = _model().half()
    mk = lambda: hqmq.with_outlier_extraction(hqmq.HQMQ(n_layers=2, n_heads=2, secondary_size=96, radius_bits=4, device="cuda"), 3.0)
    ids = torch.randint(0, 128, (2, 20), device="cuda")
    dense, packed = QuantizedCache(mk()), QuantizedCache(mk(), store="packed", max_tokens=64)
    with torch.no_grad():
        a = model(ids, past_key_values=dense, use_cache=True).logits
        b = model(ids, past_key_values=packed, use_cache=True).logits
        na, nb = a[:, -1:].argmax(-1), b[:, -1:].argmax(-1)
        for _ in range(4):
            a = model(na, past_key_values=dense, use_cache=True).logits
            b = model(na, past_key_values=packed, use_cache=True).logits
            na = a[:, -1:].argmax(-1)
    assert packed.get_seq_length() == dense.get_seq_length() == 24
    assert len(packed.layers) == 0                       # nothing dense is kept
    assert 0 < packed.compressed_bytes() < 2 * 2 * 2 * 24 * 32 * 2    # fewer bytes than the 16-bit tensors of both layers
    rel = ((a.float() - b.float()).norm() / a.float().norm()).item()
    assert rel < 2e-2, rel
