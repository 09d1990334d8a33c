"""Generate the golden fixtures in this directory from the reference implementation.

Run in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own ``hqmq`` package (unmodified, CPU), and for every case
(a) asserts that ``oracle/hqmq_oracle.py`` reproduces the reference bit for bit, and
(b) stores the inputs, the reference outputs and the oracle's exposed intermediates
(indices, radius codes, flags) in ``golden_*.npz``.  The fixtures are what travels; the
reference does not need to exist where the tests run.
"""
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import hqmq_oracle as orc  # noqa: E402

ENC_CASES = [
    # name, S, b_r, C, (B,H,T,d), kind
    ("s24_r3", 24, 3, None, (1, 2, 16, 128), "randn"),
    ("s24_r3_med3", 24, 3, 3.0, (2, 2, 24, 128), "spiky"),
    ("s96_r4_med3", 96, 4, 3.0, (2, 2, 16, 128), "hot"),
    ("s192_r6_med3", 192, 6, 3.0, (1, 2, 16, 128), "student"),
    ("s96_r4_d64", 96, 4, 3.0, (3, 2, 7, 64), "hot"),
]

FRACTION_CASES = [
    # name, S, b_r, outlier_fraction, (B,H,T,d), kind   (sizes with fractional and with whole ranks)
    ("frac1_s96_r4", 96, 4, 0.01, (2, 2, 24, 128), "hot"),
    ("frac5_s24_r3", 24, 3, 0.05, (1, 2, 33, 64), "spiky"),
    ("frac10_s96_r4", 96, 4, 0.10, (3, 2, 7, 64), "randn"),
]


def make_input(kind, shape, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    B, H, T, d = shape
    if kind == "hot":
        for h in range(H):
            ch = torch.randperm(d, generator=g)[:4]
            x[:, h, :, ch] *= 8.0
    elif kind == "spiky":
        m = torch.rand(B, H, T, d // 4, generator=g) < 0.02
        x = (x.view(B, H, T, d // 4, 4) * torch.where(m, 20.0, 1.0).unsqueeze(-1)).view(shape)
    elif kind == "student":
        for h in range(H):
            ch = torch.randperm(d, generator=g)[:2]
            z = torch.randn(B, T, 2, generator=g)
            chi = (torch.randn(B, T, 2, generator=g) ** 2 + torch.randn(B, T, 2, generator=g) ** 2) / 2
            x[:, h, :, ch] = 100.0 * z / chi.sqrt()
    return x


def main(ref_root):
    sys.path.insert(0, ref_root)
    warnings.filterwarnings("ignore")
    import hqmq  # the reference
    from src.quantizers.hqmq_attention import _decode_kv_torch

    # ---- 24-cell and codebooks -------------------------------------------------------
    from src.quantizers.spherical import _make_24cell_codebook
    assert torch.equal(_make_24cell_codebook(), orc.make_24cell())

    out = {}
    for i, (name, S, br, C, shape, kind) in enumerate(ENC_CASES):
        B, H, T, d = shape
        q = hqmq.HQMQ(n_layers=2, n_heads=H, secondary_size=S, radius_bits=br, device="cpu", seed=42)
        raw = orc.secondary_raw(2, H, S, 42)
        assert torch.equal(raw, q.secondary_raw.detach())
        x = make_input(kind, shape, 1000 + i)
        for kv, layer in ((0, 0), (1, 1)):
            joint_ref = q._get_codebook(layer, kv, x).detach()
            joint = orc.joint_codebook(raw[layer, :, kv])
            assert torch.equal(joint, joint_ref), name
            qq = hqmq.with_outlier_extraction(q, C) if C is not None else q
            with torch.no_grad():
                ref = (qq.quantize_K if kv == 0 else qq.quantize_V)(x, layer)
            enc = orc.encode(x, joint, br, C)
            mine = orc.fake_quant(x, joint, br, C, enc=enc)
            assert torch.equal(ref, mine), f"{name} kv={kv}: oracle != reference"
            if C is not None:
                # reference norm / quantile vs the spelled-out versions
                nrm = x.view(B, H, T, d // 4, 4).norm(dim=-1)
                assert torch.equal(nrm, enc["norms"]), name
                flat = nrm.permute(1, 0, 2, 3).reshape(H, -1)
                assert torch.equal(torch.quantile(flat, 0.5, dim=-1), enc["med"]), name
            key = f"{name}.kv{kv}"
            out[key + ".x"] = x.numpy()
            out[key + ".raw"] = raw[layer, :, kv].numpy()
            out[key + ".ref_fake_quant"] = ref.numpy()
            out[key + ".idx"] = enc["idx"].numpy().astype(np.uint16)
            out[key + ".rq"] = enc["rq"].numpy().astype(np.uint8)
            out[key + ".r_max"] = enc["r_max"].numpy()
            out[key + ".gap"] = enc["gap"].numpy()
            if C is not None:
                out[key + ".flags"] = np.packbits(enc["flags"].numpy().reshape(-1))
                out[key + ".med"] = enc["med"].numpy()
        out[name + ".meta"] = np.array([S, br, -1.0 if C is None else C, B, H, T, d], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "golden_encode.npz"), **out)

    # ---- the wrapper's other threshold: the per-head quantile 1 - outlier_fraction ("fraction" mode) -------------
    from src.quantizers.outlier_aware import OutlierAwareHQMQQuantizer
    fr = {}
    for i, (name, S, br, frac, shape, kind) in enumerate(FRACTION_CASES):
        B, H, T, d = shape
        q = hqmq.HQMQ(n_layers=1, n_heads=H, secondary_size=S, radius_bits=br, device="cpu", seed=42)
        raw = orc.secondary_raw(1, H, S, 42)
        x = make_input(kind, shape, 3000 + i)
        qq = OutlierAwareHQMQQuantizer(q, outlier_fraction=frac, threshold_mode="fraction")
        joint = orc.joint_codebook(raw[0, :, 0])
        with torch.no_grad():
            ref = qq.quantize_K(x, 0)
        quant = 1.0 - frac
        enc = orc.encode(x, joint, br, 1.0, quantile=quant)
        assert torch.equal(ref, orc.fake_quant(x, joint, br, 1.0, enc=enc)), f"{name}: oracle != reference"
        flat = enc["norms"].permute(1, 0, 2, 3).reshape(H, -1)
        assert torch.equal(torch.quantile(flat, quant, dim=-1), enc["med"]), name
        fr[name + ".x"] = x.numpy()
        fr[name + ".raw"] = raw[0, :, 0].numpy()
        fr[name + ".ref_fake_quant"] = ref.numpy()
        fr[name + ".thr"] = enc["thr"].numpy()
        fr[name + ".flags"] = np.packbits(enc["flags"].numpy().reshape(-1))
        fr[name + ".idx"] = enc["idx"].numpy().astype(np.uint16)
        fr[name + ".rq"] = enc["rq"].numpy().astype(np.uint8)
        fr[name + ".gap"] = enc["gap"].numpy()
        fr[name + ".meta"] = np.array([S, br, frac, B, H, T, d], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "golden_fraction.npz"), **fr)

    # ---- packed decode + attention --------------------------------------------------
    att = {}
    cases = [
        # name, B, Hq, Hkv, Tq, Tkv, d, S, qmax, causal, seed  (first = the reference's own GPU test case)
        ("ref_gpu_test", 1, 4, 1, 64, 64, 32, 24, 7, True, 0),
        ("decode_g4", 2, 8, 2, 1, 300, 128, 96, 15, False, 1),
        ("decode_g7", 1, 7, 1, 1, 257, 128, 192, 63, False, 2),
        ("decode_d64", 2, 16, 2, 1, 129, 64, 96, 15, False, 3),
        ("causal_tq1", 1, 4, 1, 1, 40, 32, 24, 7, True, 4),
    ]
    for name, B, Hq, Hkv, Tq, Tkv, d, S, qmax, causal, seed in cases:
        torch.manual_seed(seed)
        K = 24 * S
        Q = torch.randn(B, Hq, Tq, d) * 0.3
        kidx = torch.randint(0, K, (B, Hkv, Tkv, d // 4), dtype=torch.int32)
        krq = torch.randint(1, qmax + 1, (B, Hkv, Tkv, d // 4), dtype=torch.int32)
        krs = torch.rand(B, Hkv, Tkv) + 0.5
        jk = torch.randn(Hkv, K, 4)
        jk = jk / jk.norm(dim=-1, keepdim=True).clamp(min=1e-6)
        if name == "ref_gpu_test":
            vidx, vrq, vrs, jv = kidx, krq, krs, jk
        else:
            vidx = torch.randint(0, K, (B, Hkv, Tkv, d // 4), dtype=torch.int32)
            vrq = torch.randint(0, qmax + 1, (B, Hkv, Tkv, d // 4), dtype=torch.int32)
            vrs = torch.rand(B, Hkv, Tkv) + 0.5
            jv = torch.randn(Hkv, K, 4)
            jv = jv / jv.norm(dim=-1, keepdim=True).clamp(min=1e-6)
        O = hqmq.fused_attention_reference(Q, kidx, krq, krs, jk, vidx, vrq, vrs, jv, r_qmax=qmax, causal=causal)
        O2 = orc.fused_attention(Q, kidx, krq, krs, jk, vidx, vrq, vrs, jv, qmax, causal=causal)
        assert torch.equal(O, O2), name
        Kd = _decode_kv_torch(kidx, krq, krs, jk, qmax)
        assert torch.equal(Kd, orc.decode_packed(kidx, krq, krs, jk, qmax)), name
        for k, v in dict(Q=Q, kidx=kidx.to(torch.int16), krq=krq.to(torch.uint8), krs=krs, jk=jk,
                         vidx=vidx.to(torch.int16), vrq=vrq.to(torch.uint8), vrs=vrs, jv=jv, O=O, Kd=Kd).items():
            att[f"{name}.{k}"] = v.numpy()
        att[name + ".meta"] = np.array([B, Hq, Hkv, Tq, Tkv, d, S, qmax, int(causal)], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "golden_attention.npz"), **att)
    print("golden fixtures written; oracle bit-identical to the reference on every case")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of kswain98/hqmq>")
    main(sys.argv[1])
