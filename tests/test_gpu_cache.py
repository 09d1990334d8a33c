"""PackedKVCache: the reference cache's call pattern (a prompt, then one token per step and layer) on compressed
planes.  Attention over the cache must match the oracle run on the oracle's own encoding of the same calls, and
the dense view must equal what the reference's cache would hold (its fake-quantised tensors)."""
import math

import pytest
import torch

import hqmq_b200 as hqmq
from hqmq_b200.cache import PackedKVCache
from oracle import hqmq_oracle as orc
from tests.util import make_kv

pytestmark = pytest.mark.gpu


def _rel_l2(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def test_prompt_then_token_appends_over_two_layers_with_a_sliding_window():
    S, br, Cm, d, Hq, Hkv, B = 24, 3, 3.0, 64, 8, 2, 2
    n_layers, prompt, steps, window = 2, 40, 5, 16
    quant = hqmq.with_outlier_extraction(hqmq.HQMQ(n_layers, Hkv, S, br, device="cuda"), Cm)
    cache = PackedKVCache(quant, max_tokens=64, sliding_window={1: window}, outlier_capacity=1.0)
    calls = {l: [] for l in range(n_layers)}
    for step in range(1 + steps):
        T_new = prompt if step == 0 else 1
        for l in range(n_layers):
            k = make_kv("spiky", (B, Hkv, T_new, d), seed=100 + 10 * step + l, dtype=torch.float16)
            v = make_kv("randn", (B, Hkv, T_new, d), seed=500 + 10 * step + l, dtype=torch.float16)
            cache.update(k.cuda(), v.cuda(), l)
            calls[l].append((k, v))
    cache.check()
    assert len(cache) == n_layers and cache.get_seq_length(1) == prompt + steps
    raw = orc.secondary_raw(n_layers, Hkv, S, 42)
    for l in range(n_layers):
        # the oracle encodes call by call (its own median per call), like the reference's wrapper would
        dense = {0: [], 1: []}
        for k, v in calls[l]:
            for kv, x in ((0, k), (1, v)):
                joint = orc.joint_codebook(raw[l, :, kv])
                e = orc.encode(x.float(), joint, br, Cm)
                dec = orc.decode_packed(e["idx"], e["rq"], e["r_max"].to(torch.float16).float(), joint, (1 << br) - 1)
                xc = x.float().view(*x.shape[:3], d // 4, 4)
                dense[kv].append(torch.where(e["flags"][..., None], xc, dec.view_as(xc)).reshape(x.shape))
        Kd, Vd = torch.cat(dense[0], 2), torch.cat(dense[1], 2)
        got_K, got_V = cache.dense(l, dtype=torch.float32)
        assert torch.allclose(got_K.cpu(), Kd, atol=2e-3, rtol=1e-3) and torch.allclose(got_V.cpu(), Vd, atol=2e-3, rtol=1e-3)
        Q = torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(7 + l)) / math.sqrt(d)
        O = cache.attend(Q.cuda().half(), l, out=torch.empty(B, Hq, 1, d, device="cuda"))
        w = window if l == 1 else Kd.shape[2]
        G = Hq // Hkv
        Kw, Vw = Kd[:, :, -w:].repeat_interleave(G, 1), Vd[:, :, -w:].repeat_interleave(G, 1)
        ref = torch.softmax(Q.half().float() @ Kw.transpose(-1, -2) / math.sqrt(d), -1) @ Vw
        assert float((O.cpu() - ref).abs().max()) < 2e-3 and _rel_l2(O.cpu(), ref) < 1e-3, l
    assert cache.compressed_bytes() > 0
