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


def test_packed_cache_file_round_trip(tmp_path):
    """The on-disk format: the native planes cut to the tokens held, so the body is the algorithmic byte count
    (plus one counter per (batch, head)); a loaded cache decodes and attends exactly like the one that was saved."""
    import math
    S, br, C, d, Hq, Hkv, T, B = 96, 4, 3.0, 128, 8, 2, 1500, 2
    K = make_kv("hot", (B, Hkv, T, d), seed=91, dtype=torch.bfloat16)
    V = make_kv("spiky", (B, Hkv, T, d), seed=92, dtype=torch.bfloat16)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), C)
    Kp, Vp = q.encode(K.cuda(), 0, 0), q.encode(V.cuda(), 0, 1)
    tk, tv = q.inner.tables(0, 0, "cuda"), q.inner.tables(0, 1, "cuda")
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(93)) / math.sqrt(d)).bfloat16().cuda()
    loaded = []
    for name, pk, kv in (("k.hqmq", Kp, 0), ("v.hqmq", Vp, 1)):
        path = tmp_path / name
        n = pk.save(str(path), meta={"C": C, "seed": 42, "layer": 0, "kv": kv})
        blob = path.read_bytes()
        hdr_len = 12 + int.from_bytes(blob[8:12], "little")
        assert n == len(blob) == hdr_len + pk.algorithmic_bytes() + 4 * B * Hkv
        back, meta = hqmq.PackedKV.load(str(path), "cuda", T_cap=T + 64)
        assert meta == {"C": C, "seed": 42, "layer": 0, "kv": kv} and back.T == T
        for g, w in zip(back.to_reference(), pk.to_reference()):
            assert torch.equal(g, w)
        assert torch.equal(q.decode(back, 0, kv, dtype=torch.float32), q.decode(pk, 0, kv, dtype=torch.float32))
        loaded.append(back)
    # the loaded K cache has no fragment records: same result through the flag / payload path, within the tolerance
    O1 = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
    O2 = torch.empty_like(O1)
    hqmq.fused_attention_packed(Q, Kp, Vp, tk["table16"], tv["table16"], out=O1)
    hqmq.fused_attention_packed(Q, loaded[0], loaded[1], tk["table16"], tv["table16"], out=O2)
    assert (O1 - O2).abs().max().item() < 2e-3
    # and it can be appended to
    more = make_kv("hot", (B, Hkv, 16, d), seed=94, dtype=torch.bfloat16).cuda()
    q.encode(more, 0, 0, out=loaded[0])
    assert loaded[0].T == T + 16
    with pytest.raises(ValueError):
        hqmq.PackedKV.load(_truncated(tmp_path / "k.hqmq"), "cuda")


def _truncated(path):
    import io
    return io.BytesIO(path.read_bytes()[:-10])


def test_padded_head_dim_matches_the_oracle():
    """PaddedHQMQ (head dims that are not a multiple of 4: zero-pad, quantise, truncate; src/quantizers/hqmq_padded.py:51-71)
    through the CUDA encoder and dequant: bit-identical to the oracle's fake-quant of the padded tensor, truncated."""
    from oracle import hqmq_oracle as orc
    S, br, Hkv, T, B, d = 24, 3, 2, 70, 2, 45
    x = torch.randn(B, Hkv, T, d, generator=torch.Generator().manual_seed(95))
    pq = hqmq.PaddedHQMQ(n_layers=1, n_heads=Hkv, d_head=d, secondary_size=S, radius_bits=br, device="cuda")
    assert (pq.d_head_padded, pq.pad_count) == (48, 3)
    got = pq.quantize_K(x.cuda(), 0).cpu()
    assert got.shape == x.shape
    joint = orc.joint_codebook(orc.secondary_raw(1, Hkv, S, 42)[0, :, 0])
    xp = torch.nn.functional.pad(x, (0, 3))
    enc = orc.encode(xp, joint, br, None)
    want = orc.fake_quant(xp, joint, br, None, enc=enc)[..., :d]
    near_tie = (enc["gap"] < 1e-6).unsqueeze(-1).expand(B, Hkv, T, 12, 4).reshape(B, Hkv, T, 48)[..., :d]
    assert torch.equal(got[~near_tie], want[~near_tie])


def test_update_with_another_geometry_than_the_cache_is_refused():
    """The library takes batch, heads and chunks per token from the destination planes, so a call whose x has
    another batch (sequences that finished), head count or head dim must fail before anything is launched."""
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, 2, 24, 3, device="cuda"), 3.0)
    dst = q.inner.new_cache(4, 64, 32, "cuda", with_outliers=True)
    x = torch.randn(4, 2, 8, 32, device="cuda")
    q.encode(x, 0, 0, out=dst)
    assert dst.T == 8
    for bad in (torch.randn(3, 2, 8, 32, device="cuda"),       # smaller batch
                torch.randn(4, 2, 8, 64, device="cuda"),       # other head dim
                torch.randn(4, 1, 8, 32, device="cuda")):      # other head count
        with pytest.raises((ValueError, hqmq.HqmqError)):
            q.encode(bad, 0, 0, out=dst)
    assert dst.T == 8
    other = hqmq.HQMQ(1, 2, 96, 4, device="cuda")
    with pytest.raises(ValueError):
        other.encode(x, 0, 0, out=dst)                          # another codebook than the planes were made for


@pytest.mark.parametrize("outliers", [True, False])
def test_pair_append_equals_two_single_appends(outliers):
    """K and V of a layer appended in one launch (hqmq_encode_pair: codes, offset scan and side planes of both tensors)
    leave every plane byte-identical to one tensor appended after the other by single-tensor calls: a prompt and longer
    chunks (large calls: run one after the other inside the library), one to five tokens at a time across block
    boundaries, a chunk of three blocks."""
    B, H, d, S, br = 3, 2, 64, 96, 4
    inner = hqmq.HQMQ(1, H, S, br, device="cuda")
    q = hqmq.with_outlier_extraction(inner, 3.0) if outliers else inner
    mk = lambda kv: inner.new_cache(B, 1024, d, "cuda", scale_dtype=torch.bfloat16, with_outliers=outliers,
                                    out_dtype=torch.bfloat16, ofrag=outliers and kv == 0)
    pair, single = (mk(0), mk(1)), (mk(0), mk(1))
    g = torch.Generator().manual_seed(11)
    for step, T in enumerate([40, 1, 1, 3, 1, 5, 1, 33, 1, 170, 2, 600, 1]):
        k = torch.randn(B, H, T, d, generator=g)
        k[:, :, :, 7] *= 9.0
        v = torch.randn(B, H, T, d, generator=g)
        k, v = k.bfloat16().cuda(), v.bfloat16().cuda()
        q.encode_pair(k, v, 0, pair[0], pair[1])
        q.encode(k, 0, 0, out=single[0])
        q.encode(v, 0, 1, out=single[1])
    torch.cuda.synchronize()
    for a, b in zip(pair, single):
        assert a.T == b.T == 859
        names = ["codes", "rs"] + (["flags", "out_vals", "out_off", "out_count"] if outliers else [])
        names += ["ofrag", "ofrag_off"] if a.with_ofrag else []
        for name in names:
            assert torch.equal(getattr(a, name), getattr(b, name)), name


@pytest.mark.parametrize("T_prompt,T_chunk,window", [(300, 5, None), (1500, 37, None), (200, 9, 64), (3, 3, None)])
def test_prompt_chunk_attends_causally_over_the_cache(T_prompt, T_chunk, window):
    """A chunk of T_q prompt tokens is appended and then attends over the cache that now holds it: query i sees
    the keys up to its own position (bottom-right aligned mask), within the layer's window if it has one.  Against
    the oracle called once per query position over the keys that position may see."""
    B, Hkv, Hq, d, S, br = 2, 2, 8, 64, 96, 4
    inner = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    q = hqmq.with_outlier_extraction(inner, 3.0)
    cache = PackedKVCache(q, max_tokens=2048, sliding_window={0: window} if window else None)
    K = make_kv("hot", (B, Hkv, T_prompt, d), seed=61, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T_prompt, d), seed=62, dtype=torch.bfloat16)
    first = T_prompt - T_chunk
    if first:
        cache.update(K[:, :, :first].cuda(), V[:, :, :first].cuda(), 0)
    Kp, Vp = cache.update(K[:, :, first:].cuda(), V[:, :, first:].cuda(), 0)
    Q = (torch.randn(B, Hq, T_chunk, d, generator=torch.Generator().manual_seed(63)) / math.sqrt(d)).bfloat16()
    O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
    cache.attend(Q.cuda(), 0, out=O)
    ki, kr, ks, kf = (t.cpu() for t in Kp.to_reference())
    vi, vr, vs, vf = (t.cpu() for t in Vp.to_reference())
    tk, tv = inner.tables(0, 0, "cuda"), inner.tables(0, 1, "cuda")
    for i in range(T_chunk):
        n = first + i + 1                      # keys query i may see
        ref = orc.fused_attention(Q[:, :, i:i + 1], ki[:, :, :n], kr[:, :, :n], ks[:, :, :n], tk["joint"].cpu(),
                                  vi[:, :, :n], vr[:, :, :n], vs[:, :, :n], tv["joint"].cpu(), (1 << br) - 1, causal=False,
                                  K_flags=kf[:, :, :n], K_orig=K[:, :, :n], V_flags=vf[:, :, :n], V_orig=V[:, :, :n],
                                  window=window)
        err = (O[:, :, i:i + 1].cpu() - ref).abs().max().item()
        assert err < 2e-3, f"query {i}: max-abs {err:.2e}"
