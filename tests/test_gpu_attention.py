"""Dequant and fused decode attention on the GPU, through the C ABI, against the fp32 oracle.
Tolerances are the ones the path's contract states: 2e-3 max-abs and 1e-3 relative L2."""
import math

import pytest
import torch

import hqmq_b200 as hqmq
from hqmq_b200 import kernels
from oracle import hqmq_oracle as orc
from tests.util import load_npz, make_kv, rel_l2

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-3, 1e-3


def _random_packed(B, Hkv, T, d, S, qmax, seed, zero_rq=True):
    g = torch.Generator().manual_seed(seed)
    K = 24 * S
    idx = torch.randint(0, K, (B, Hkv, T, d // 4), dtype=torch.int32, generator=g)
    rq = torch.randint(0 if zero_rq else 1, qmax + 1, (B, Hkv, T, d // 4), dtype=torch.int32, generator=g)
    rs = torch.rand(B, Hkv, T, generator=g) + 0.5
    joint = torch.randn(Hkv, K, 4, generator=g)
    joint = joint / joint.norm(dim=-1, keepdim=True).clamp(min=1e-6)
    return idx, rq, rs, joint


def _check(O, ref, what=""):
    err = (O.float().cpu() - ref).abs().max().item()
    r2 = rel_l2(O.float().cpu(), ref)
    assert err < MAX_ABS and r2 < REL_L2, f"{what}: max-abs {err:.2e}, rel-L2 {r2:.2e}"


@pytest.mark.parametrize("name", ["ref_gpu_test", "decode_g4", "decode_g7", "decode_d64", "causal_tq1"])
def test_attention_matches_reference_fixtures(name):
    z = load_npz("golden_attention.npz")
    B, Hq, Hkv, Tq, Tkv, d, S, qmax, causal = (int(v) for v in z[name + ".meta"])
    t = {k: torch.from_numpy(z[f"{name}.{k}"]) for k in ("Q", "kidx", "krq", "krs", "jk", "vidx", "vrq", "vrs", "jv", "O", "Kd")}
    kidx, vidx = (t["kidx"].to(torch.int32) & 0xFFFF).cuda(), (t["vidx"].to(torch.int32) & 0xFFFF).cuda()
    O = hqmq.fused_attention(t["Q"].cuda(), kidx, t["krq"].cuda(), t["krs"].cuda(), t["jk"].cuda(), vidx,
                             t["vrq"].cuda(), t["vrs"].cuda(), t["jv"].cuda(), r_qmax=qmax, causal=bool(causal))
    err = (O.cpu() - t["O"]).abs().max().item()
    assert err < 1e-3, f"{name}: {err}"           # the reference's own Triton-vs-oracle bound (tests/test_gpu.py:49)
    Kd = kernels.decode_dequant(kidx, t["krq"].cuda(), t["krs"].cuda(), t["jk"].cuda(), qmax)
    assert torch.equal(Kd.cpu(), t["Kd"]), "fp32 dequant is not bit-identical to the reference decode"


@pytest.mark.parametrize("B,Hq,Hkv,T,d,S,qmax", [
    (1, 32, 8, 1000, 128, 24, 7), (2, 32, 8, 777, 128, 96, 15), (1, 28, 4, 513, 128, 192, 63),
    (2, 64, 8, 300, 64, 96, 15), (1, 4, 4, 65, 32, 24, 7), (1, 16, 1, 40, 16, 24, 7), (1, 6, 2, 50, 48, 24, 7)])
@pytest.mark.parametrize("qdtype", [torch.float32, torch.bfloat16])
def test_decode_attention_reference_layout(B, Hq, Hkv, T, d, S, qmax, qdtype):
    idx, rq, rs, jk = _random_packed(B, Hkv, T, d, S, qmax, seed=T)
    vidx, vrq, vrs, jv = _random_packed(B, Hkv, T, d, S, qmax, seed=T + 1)
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(7)) / math.sqrt(d) * 3).to(qdtype)
    ref = orc.fused_attention(Q, idx, rq, rs, jk, vidx, vrq, vrs, jv, qmax, causal=False)
    O = hqmq.fused_attention(Q.cuda(), idx.cuda(), rq.to(torch.int8 if qmax < 128 else torch.int16).cuda(), rs.cuda(),
                             jk.cuda(), vidx.cuda(), vrq.cuda(), vrs.cuda(), jv.cuda(), r_qmax=qmax, causal=False)
    assert O.dtype == qdtype and O.shape == Q.shape
    if qdtype == torch.float32:
        _check(O, ref, "ref layout")
    else:
        # rounding the result to bf16 alone costs ~1.5e-3 relative L2, so the tolerance is checked on
        # an fp32 output of the same call and the bf16 output must be that result rounded once
        O32 = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
        hqmq.fused_attention(Q.cuda(), idx.cuda(), rq.cuda(), rs.cuda(), jk.cuda(), vidx.cuda(), vrq.cuda(), vrs.cuda(),
                             jv.cuda(), r_qmax=qmax, causal=False, out=O32)
        _check(O32, ref, "ref layout, fp32 out")
        assert torch.equal(O32.to(qdtype), O)


@pytest.mark.parametrize("S,br,d,Hq,Hkv,T", [(24, 3, 128, 32, 8, 700), (96, 4, 128, 32, 8, 1029), (192, 6, 128, 28, 4, 515),
                                             (96, 4, 64, 64, 8, 333), (24, 3, 64, 16, 2, 100), (96, 4, 32, 8, 2, 90)])
def test_decode_attention_native_layout_and_splits(S, br, d, Hq, Hkv, T):
    B, qmax = 2, (1 << br) - 1
    idx, rq, rs, _ = _random_packed(B, Hkv, T, d, S, qmax, seed=S + T)
    vidx, vrq, vrs, _ = _random_packed(B, Hkv, T, d, S, qmax, seed=S + T + 1)
    q = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    tk, tv = q.tables(0, 0, "cuda"), q.tables(0, 1, "cuda")
    rs16, vrs16 = rs.bfloat16(), vrs.bfloat16()
    Kp = hqmq.PackedKV.from_reference(idx.cuda(), rq.cuda(), rs16.cuda(), S, br, scale_dtype=torch.bfloat16)
    Vp = hqmq.PackedKV.from_reference(vidx.cuda(), vrq.cuda(), vrs16.cuda(), S, br, scale_dtype=torch.bfloat16)
    # pack -> unpack round trip is the identity
    i2, r2, s2, _ = Kp.to_reference()
    assert torch.equal(i2.cpu(), idx) and torch.equal(r2.cpu(), rq) and torch.equal(s2.cpu(), rs16.float())
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(3)) / math.sqrt(d) * 3).bfloat16()
    ref = orc.fused_attention(Q, idx, rq, rs16, tk["joint"].cpu(), vidx, vrq, vrs16, tv["joint"].cpu(), qmax, causal=False)
    outs = []
    for splits in (None, 1, 3):
        O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
        hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], kv_splits=splits, out=O)
        _check(O, ref, f"native splits={splits}")
        outs.append(O)
    assert torch.equal(hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"]), outs[0].bfloat16())
    # the oracle's own dense decode equals the CUDA dequant of the native planes
    dense = q.decode(Kp, 0, 0, dtype=torch.float32).cpu()
    assert torch.equal(dense, orc.decode_packed(idx, rq, rs16.float(), tk["joint"].cpu(), qmax))


def test_window_and_partials_combine():
    S, br, d, Hq, Hkv, T, B = 96, 4, 128, 16, 4, 900, 1
    qmax = 15
    idx, rq, rs, _ = _random_packed(B, Hkv, T, d, S, qmax, seed=1)
    vidx, vrq, vrs, _ = _random_packed(B, Hkv, T, d, S, qmax, seed=2)
    q = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    tk, tv = q.tables(0, 0, "cuda"), q.tables(0, 1, "cuda")
    rs16, vrs16 = rs.half(), vrs.half()
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(3)) / math.sqrt(d) * 3).half()
    Kp = hqmq.PackedKV.from_reference(idx.cuda(), rq.cuda(), rs16.cuda(), S, br, scale_dtype=torch.float16)
    Vp = hqmq.PackedKV.from_reference(vidx.cuda(), vrq.cuda(), vrs16.cuda(), S, br, scale_dtype=torch.float16)
    for window in (128, 100, 17):
        ref = orc.fused_attention(Q, idx, rq, rs16, tk["joint"].cpu(), vidx, vrq, vrs16, tv["joint"].cpu(), qmax,
                                  causal=False, window=window)
        O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
        hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], window=window, out=O)
        _check(O, ref, f"window={window}")
    # sequence shards: two caches holding the halves, partials merged afterwards
    ref = orc.fused_attention(Q, idx, rq, rs16, tk["joint"].cpu(), vidx, vrq, vrs16, tv["joint"].cpu(), qmax, causal=False)
    parts = []
    for lo, hi in ((0, 400), (400, 900)):
        Ks = hqmq.PackedKV.from_reference(idx[:, :, lo:hi].cuda(), rq[:, :, lo:hi].cuda(), rs16[:, :, lo:hi].cuda(), S, br, scale_dtype=torch.float16)
        Vs = hqmq.PackedKV.from_reference(vidx[:, :, lo:hi].cuda(), vrq[:, :, lo:hi].cuda(), vrs16[:, :, lo:hi].cuda(), S, br, scale_dtype=torch.float16)
        p = torch.empty(B, Hq, 1, d + 2, device="cuda")
        hqmq.fused_attention_packed(Q.cuda(), Ks, Vs, tk["table16"], tv["table16"], partials=p)
        parts.append(p)
    O = hqmq.combine_partials(torch.stack(parts))
    _check(O, ref, "sequence shards")


def test_encode_then_attend_end_to_end():
    """The two halves connected: encode K/V on the GPU, attend over the native cache, compare with the
    oracle attending over the oracle's own encoding (Med3x outliers merged)."""
    S, br, C, d, Hq, Hkv, T, B = 96, 4, 3.0, 128, 16, 4, 600, 2
    K = make_kv("hot", (B, Hkv, T, d), seed=41, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T, d), seed=42, dtype=torch.bfloat16)
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(43)) / math.sqrt(d)).bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), C)
    Kp, Vp = q.encode(K.cuda(), 0, 0), q.encode(V.cuda(), 0, 1)
    tk, tv = q.inner.tables(0, 0, "cuda"), q.inner.tables(0, 1, "cuda")
    O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
    hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], out=O)
    ki, kr, ks, kf = (t.cpu() if t is not None else None for t in Kp.to_reference())
    vi, vr, vs, vf = (t.cpu() if t is not None else None for t in Vp.to_reference())
    ref = orc.fused_attention(Q, ki, kr, ks, tk["joint"].cpu(), vi, vr, vs, tv["joint"].cpu(), 15, causal=False,
                              K_flags=kf, K_orig=K, V_flags=vf, V_orig=V)
    assert kf.float().mean() > 0.02        # the hot channels really are flagged
    _check(O, ref, "encode -> attend with outliers")


def test_bad_arguments_raise():
    from hqmq_b200 import _lib
    idx, rq, rs, jk = _random_packed(1, 2, 20, 32, 24, 7, seed=0)
    Q = torch.randn(1, 3, 1, 32).cuda()
    with pytest.raises(AssertionError):
        hqmq.fused_attention(Q, idx.cuda(), rq.cuda(), rs.cuda(), jk.cuda(), idx.cuda(), rq.cuda(), rs.cuda(), jk.cuda(), r_qmax=7)
    q = hqmq.HQMQ(1, 2, device="cuda")
    with pytest.raises(ValueError):
        q.quantize_K(torch.randn(1, 2, 4, 18).cuda(), 0)


def test_empty_cache_and_empty_append():
    """Edge cases: attention over a cache that holds no token gives zeros (no key carries weight) instead of
    failing, and an append of zero tokens leaves the cache as it was."""
    S, br, d, Hq, Hkv, B = 24, 3, 64, 4, 2, 2
    q = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    Kp = q.new_cache(B, 64, d, "cuda")
    Vp = q.new_cache(B, 64, d, "cuda")
    tk, tv = q.tables(0, 0, "cuda"), q.tables(0, 1, "cuda")
    Q = torch.randn(B, Hq, 1, d, device="cuda").half()
    O = torch.full(Q.shape, 7.0, dtype=torch.float32, device="cuda")
    hqmq.fused_attention_packed(Q, Kp, Vp, tk["table16"], tv["table16"], out=O)
    assert torch.equal(O, torch.zeros_like(O))
    x = make_kv("randn", (B, Hkv, 20, d), seed=3, dtype=torch.float16).cuda()
    q.encode(x, 0, 0, out=Kp)
    before = (Kp.codes.clone(), Kp.rs.clone(), Kp.T)
    q.encode(x[:, :, :0], 0, 0, out=Kp)
    assert Kp.T == before[2] and torch.equal(Kp.codes, before[0]) and torch.equal(Kp.rs, before[1])


def test_large_codebook_generic_kernels():
    """A codebook far larger than the benchmark ones (S = 512: 12288 codewords, 14 index bits, fields that are
    not a multiple of 8 bits): the encoder's exhaustive / table search and the generic attention kernel."""
    S, br, C, d, Hq, Hkv, T, B = 512, 2, 3.0, 32, 4, 2, 40, 1
    K = make_kv("spiky", (B, Hkv, T, d), seed=71)
    V = make_kv("randn", (B, Hkv, T, d), seed=72)
    Q = torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(73)) / math.sqrt(d)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), C)
    Kp, Vp = q.encode(K.cuda(), 0, 0, scale_dtype=torch.float16), q.encode(V.cuda(), 0, 1, scale_dtype=torch.float16)
    tk, tv = q.inner.tables(0, 0, "cuda"), q.inner.tables(0, 1, "cuda")
    joint = orc.joint_codebook(orc.secondary_raw(1, Hkv, S, 42)[0, :, 0])
    enc = orc.encode(K, joint, br, C)
    ki, kr, ks, kf = (t.cpu() for t in Kp.to_reference())
    vi, vr, vs, vf = (t.cpu() for t in Vp.to_reference())
    assert torch.equal(kf, enc["flags"]) and torch.equal(kr, torch.where(enc["flags"], 0, enc["rq"]))
    assert int(((ki != enc["idx"]) & (enc["gap"] >= 1e-6)).sum()) == 0
    O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
    hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], out=O)
    ref = orc.fused_attention(Q, ki, kr, ks, tk["joint"].cpu(), vi, vr, vs, tv["joint"].cpu(), (1 << br) - 1,
                              causal=False, K_flags=kf, K_orig=K, V_flags=vf, V_orig=V)
    _check(O, ref, "S=512")
