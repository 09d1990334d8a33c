"""The oracle against the fixtures generated from the reference (tests/golden/make_golden.py)."""
import numpy as np
import torch

from oracle import hqmq_oracle as orc
from tests.util import load_npz

ENC_CASES = ["s24_r3", "s24_r3_med3", "s96_r4_med3", "s192_r6_med3", "s96_r4_d64"]
ATT_CASES = ["ref_gpu_test", "decode_g4", "decode_g7", "decode_d64", "causal_tq1"]


def test_24cell_geometry():
    pts = orc.make_24cell()
    assert pts.shape == (24, 4)
    assert torch.allclose(pts.norm(dim=-1), torch.ones(24), atol=1e-6)
    cos = pts @ pts.T
    cos.fill_diagonal_(-2)
    assert abs(cos.max().item() - 0.5) < 1e-4
    # closure under the Hamilton product
    S = {tuple(round(float(v), 5) for v in p) for p in pts}
    for i in range(24):
        for j in range(24):
            prod = orc.quat_mul(pts[i:i + 1], pts[j:j + 1])[0]
            assert tuple(round(float(v), 5) for v in prod) in S


def test_encoder_matches_reference_fixtures():
    z = load_npz("golden_encode.npz")
    for name in ENC_CASES:
        S, br, C, B, H, T, d = z[name + ".meta"]
        S, br = int(S), int(br)
        C = None if C < 0 else float(C)
        for kv in (0, 1):
            key = f"{name}.kv{kv}"
            x = torch.from_numpy(z[key + ".x"])
            joint = orc.joint_codebook(torch.from_numpy(z[key + ".raw"]))
            enc = orc.encode(x, joint, br, C)
            fq = orc.fake_quant(x, joint, br, C, enc=enc)
            ref = torch.from_numpy(z[key + ".ref_fake_quant"])
            # radius codes, scales, flags and medians are exact everywhere; an index may differ only
            # where the host BLAS orders the 4-term dot product differently on a near-tie
            assert np.array_equal(enc["rq"].numpy().astype(np.uint8), z[key + ".rq"]), key
            assert np.array_equal(enc["r_max"].numpy(), z[key + ".r_max"]), key
            mism = enc["idx"].numpy().astype(np.uint16) != z[key + ".idx"]
            assert not (mism & (z[key + ".gap"] >= 1e-6)).any(), key
            if C is not None:
                assert np.array_equal(np.packbits(enc["flags"].numpy().reshape(-1)), z[key + ".flags"]), key
                assert np.array_equal(enc["med"].numpy(), z[key + ".med"]), key
            if not mism.any():
                assert torch.equal(fq, ref), key


def test_attention_matches_reference_fixtures():
    z = load_npz("golden_attention.npz")
    for name in ATT_CASES:
        B, Hq, Hkv, Tq, Tkv, d, S, qmax, causal = (int(v) for v in z[name + ".meta"])
        t = {k: torch.from_numpy(z[f"{name}.{k}"]) for k in ("Q", "kidx", "krq", "krs", "jk", "vidx", "vrq", "vrs", "jv", "O", "Kd")}
        kidx, vidx = t["kidx"].to(torch.int32) & 0xFFFF, t["vidx"].to(torch.int32) & 0xFFFF
        Kd = orc.decode_packed(kidx, t["krq"].to(torch.int32), t["krs"], t["jk"], qmax)
        assert torch.equal(Kd, t["Kd"]), name
        O = orc.fused_attention(t["Q"], kidx, t["krq"].to(torch.int32), t["krs"], t["jk"], vidx,
                                t["vrq"].to(torch.int32), t["vrs"], t["jv"], qmax, causal=bool(causal))
        assert torch.allclose(O, t["O"], atol=2e-6, rtol=1e-5), name


def test_causal_single_query_sees_key_zero_only():
    # top-left aligned mask: with T_q = 1 the query attends to key 0 only
    z = load_npz("golden_attention.npz")
    name = "causal_tq1"
    B, Hq, Hkv, Tq, Tkv, d, S, qmax, causal = (int(v) for v in z[name + ".meta"])
    vidx = torch.from_numpy(z[name + ".vidx"]).to(torch.int32) & 0xFFFF
    Vd = orc.decode_packed(vidx, torch.from_numpy(z[name + ".vrq"]).to(torch.int32), torch.from_numpy(z[name + ".vrs"]),
                           torch.from_numpy(z[name + ".jv"]), qmax)
    O = torch.from_numpy(z[name + ".O"])
    assert torch.allclose(O[:, :, 0], Vd[:, :, 0].repeat_interleave(Hq // Hkv, dim=1), atol=1e-6)


def test_median_matches_torch_quantile():
    g = torch.Generator().manual_seed(3)
    for n in (1, 2, 7, 64, 1001, 4096):
        flat = torch.rand(3, n, generator=g) * 5
        assert torch.equal(orc.median_quantile(flat), torch.quantile(flat, 0.5, dim=-1)), n


def test_combine_partials_equals_unsplit_softmax():
    g = torch.Generator().manual_seed(5)
    s = torch.randn(4, 96, generator=g) * 3
    v = torch.randn(96, 8, generator=g)
    full = torch.softmax(s, -1) @ v
    ms, ls, os_ = [], [], []
    for lo, hi in ((0, 10), (10, 64), (64, 96)):
        m = s[:, lo:hi].amax(-1)
        p = torch.exp(s[:, lo:hi] - m[:, None])
        ms.append(m); ls.append(p.sum(-1)); os_.append(p @ v[lo:hi])
    out = orc.combine_partials(torch.stack(ms), torch.stack(ls), torch.stack(os_))
    assert torch.allclose(out, full, atol=1e-5)


def test_fraction_threshold_matches_reference_fixtures():
    """The wrapper's threshold_mode="fraction" (src/quantizers/outlier_aware.py:64-66) against the reference's output."""
    z = load_npz("golden_fraction.npz")
    for name in ("frac1_s96_r4", "frac5_s24_r3", "frac10_s96_r4"):
        S, br, frac, B, H, T, d = z[name + ".meta"]
        x = torch.from_numpy(z[name + ".x"])
        joint = orc.joint_codebook(torch.from_numpy(z[name + ".raw"]))
        enc = orc.encode(x, joint, int(br), 1.0, quantile=1.0 - float(frac))
        assert np.array_equal(enc["thr"].numpy(), z[name + ".thr"]), name
        assert np.array_equal(np.packbits(enc["flags"].numpy().reshape(-1)), z[name + ".flags"]), name
        mism = enc["idx"].numpy().astype(np.uint16) != z[name + ".idx"]
        if not mism.any():
            assert torch.equal(orc.fake_quant(x, joint, int(br), 1.0, enc=enc), torch.from_numpy(z[name + ".ref_fake_quant"]))


def test_quantile_restatement_equals_torch_quantile():
    """Ranks in fp32, fused interpolation: bit-equal to torch.quantile for whole and fractional ranks, from two
    elements up to the most torch.quantile accepts (2^24 elements, where the fp32 rank has no fraction bits left)."""
    g = torch.Generator().manual_seed(5)
    for N in (2, 7, 100, 4099, 65537, 1000003):
        flat = torch.randn(3, N, generator=g).abs()
        for q in (0.5, 0.9, 0.95, 0.99, 0.999, 0.37):
            assert torch.equal(orc.quantile_torch(flat, q), torch.quantile(flat, q, dim=-1)), (N, q)
    flat = torch.rand(1, (1 << 24) - 3, generator=g)
    for q in (0.99, 0.9, 0.731):
        assert torch.equal(orc.quantile_torch(flat, q), torch.quantile(flat, q, dim=-1)), q
