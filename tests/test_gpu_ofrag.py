"""The optional fragment-record plane of a K cache (include/hqmq_b200.h, `ofrag`): the encoder's records
are checked value by value against a numpy restatement built from the same flags, scales and inputs, and
decode attention must give the same answer (within the path's tolerance of the fp32 oracle) with the
records, without them, and for blocks that own none (append boundaries, capacity overflow)."""
import math

import numpy as np
import pytest
import torch

import hqmq_b200 as hqmq
from hqmq_b200 import _lib
from oracle import hqmq_oracle as orc
from tests.util import make_kv, rel_l2

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-3, 1e-3
REC = _lib.OFRAG_BYTES


def _expected_records(x, flags, rs, qmax, t_lo, t_hi, cap):
    """Records and offsets for one (b, h): x (T, d) fp32, flags (T, n) bool, rs (T,) fp32 (the stored scale).
    Only blocks inside [t_lo, t_hi) get records; returns (off[n_blocks+1], list of 528-byte arrays)."""
    T = flags.shape[0]
    nblk = (T + 15) // 16
    off, recs, full = [0], [], False
    for blk in range(nblk):
        t0 = blk * 16
        mine = []
        if t0 >= t_lo and t0 + 16 <= t_hi:
            pos = np.flatnonzero(flags[t0:t0 + 16].any(axis=0))
            ng = (len(pos) + 3) // 4
            if 0 < ng <= 2:
                for g in range(ng):
                    rec = np.zeros(REC, dtype=np.uint8)
                    cs = list(pos[4 * g:4 * g + 4])
                    rec[0:4] = [int(c) for c in cs] + [0xFF] * (4 - len(cs))
                    body = np.zeros((32, 8), dtype=np.float16)
                    for lane in range(32):
                        r, j = lane // 4, lane % 4
                        if j >= len(cs):
                            continue
                        c = cs[j]
                        for nt in range(2):
                            t = t0 + nt * 8 + r
                            if flags[t, c]:
                                inv = np.float32(qmax) / np.float32(rs[t])
                                v = (x[t, 4 * c:4 * c + 4].astype(np.float32) * inv).astype(np.float16)
                                body[lane, 2 * nt:2 * nt + 2] = v[0:2]
                                body[lane, 4 + 2 * nt:6 + 2 * nt] = v[2:4]
                    rec[16:] = body.view(np.uint8).reshape(-1)
                    mine.append(rec)
        if full or len(recs) + len(mine) > cap:
            full, mine = True, []
        recs += mine
        off.append(len(recs))
    return np.array(off, dtype=np.int64), recs


def _planes(pk):
    nb = pk.T_cap // 16 + 1
    off = pk.ofrag_off.cpu().numpy().reshape(pk.B, pk.H, nb)
    recs = pk.ofrag[:pk.B * pk.H * pk.ofrag_cap * REC].cpu().numpy().reshape(pk.B, pk.H, pk.ofrag_cap, REC)
    return off, recs


@pytest.mark.parametrize("kind,T,cap", [("hot", 336, None), ("student", 200, None), ("spiky", 512, None),
                                        ("hot", 336, 5)])
def test_records_match_restatement(kind, T, cap):
    S, br, C, d, H, B = 96, 4, 3.0, 128, 2, 2
    qmax = (1 << br) - 1
    K = make_kv(kind, (B, H, T, d), seed=7, dtype=torch.bfloat16)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, H, S, br, device="cuda"), C)
    pk = q.inner.new_cache(B, T, d, "cuda", scale_dtype=torch.bfloat16, with_outliers=True,
                           out_dtype=torch.bfloat16, ofrag=True, ofrag_cap=cap)
    q.encode(K.cuda(), 0, 0, out=pk)
    _, _, rs, fl = (t.cpu() for t in pk.to_reference())
    off, recs = _planes(pk)
    total = 0
    for b in range(B):
        for h in range(H):
            eo, er = _expected_records(K[b, h].float().numpy(), fl[b, h].numpy(), rs[b, h].numpy(), qmax, 0, T,
                                       pk.ofrag_cap)
            nblk = len(eo) - 1
            assert np.array_equal(off[b, h, :nblk + 1], eo), f"offsets of (b={b}, h={h})"
            for i, rec in enumerate(er):
                assert np.array_equal(recs[b, h, i], rec), f"record {i} of (b={b}, h={h})"
            total += len(er)
    assert total > 0
    if cap is not None:
        assert (off <= cap).all() and total >= B * H * (cap - 1)      # the capacity really was hit


def _attend(Q, Kp, Vp, tk, tv, **kw):
    O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
    hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], out=O, **kw)
    return O.cpu()


@pytest.mark.parametrize("kind,T1,T2,cap", [("hot", 600, 0, None), ("hot", 250, 391, None), ("student", 333, 0, None),
                                            ("spiky", 1024, 0, None), ("hot", 640, 0, 7)])
def test_attention_with_and_without_records(kind, T1, T2, cap):
    """T2 > 0 appends a second call that starts inside a block."""
    S, br, C, d, Hq, Hkv, B = 96, 4, 3.0, 128, 16, 4, 2
    T = T1 + T2
    K = make_kv(kind, (B, Hkv, T, d), seed=51, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T, d), seed=52, dtype=torch.bfloat16)
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(53)) / math.sqrt(d)).bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), C)
    Kp = q.inner.new_cache(B, T, d, "cuda", scale_dtype=torch.bfloat16, with_outliers=True,
                           out_dtype=torch.bfloat16, ofrag=True, ofrag_cap=cap)
    q.encode(K[:, :, :T1].cuda(), 0, 0, out=Kp)
    if T2:
        q.encode(K[:, :, T1:].cuda(), 0, 0, out=Kp)
    Vp = q.inner.encode(V.cuda(), 0, 1)
    tk, tv = q.inner.tables(0, 0, "cuda"), q.inner.tables(0, 1, "cuda")
    ki, kr, ks, kf = (t.cpu() for t in Kp.to_reference())
    vi, vr, vs, _ = Vp.to_reference()
    ref = orc.fused_attention(Q, ki, kr, ks, tk["joint"].cpu(), vi.cpu(), vr.cpu(), vs.cpu(), tv["joint"].cpu(),
                              15, causal=False, K_flags=kf, K_orig=K)
    off, _ = _planes(Kp)
    n_rec = int(off[..., (T + 15) // 16].sum())
    assert n_rec > 0
    if T2:   # the block that the second call started in was completed by it: it owns records built from the side buffer
        blk = T1 // 16
        assert (off[..., blk + 1] > off[..., blk]).all() and kf[:, :, blk * 16:blk * 16 + 16].any()
        _, recs = _planes(Kp)
        for b in range(B):
            for h in range(Hkv):
                eo, er = _expected_records(K[b, h].float().numpy(), kf[b, h].numpy(), ks[b, h].numpy(), 15, 0, T, Kp.ofrag_cap)
                assert np.array_equal(off[b, h, :len(eo)], eo)
                for i, rec in enumerate(er):
                    assert np.array_equal(recs[b, h, i], rec), f"record {i} of (b={b}, h={h})"
    for window in (None, 100):
        if window is not None:
            ref_w = orc.fused_attention(Q, ki, kr, ks, tk["joint"].cpu(), vi.cpu(), vr.cpu(), vs.cpu(),
                                        tv["joint"].cpu(), 15, causal=False, window=window, K_flags=kf, K_orig=K)
        else:
            ref_w = ref
        O = _attend(Q, Kp, Vp, tk, tv, window=window)
        err, r2 = (O - ref_w).abs().max().item(), rel_l2(O, ref_w)
        # max-abs is stated for outputs of order one; where one key takes all the weight the output is a single
        # V row of magnitude ~3 (Student-t keys), so the bound scales with the largest reference value
        atol = MAX_ABS * max(1.0, float(ref_w.abs().max()))
        assert err < atol and r2 < REL_L2, f"with records, window={window}: {err:.2e} {r2:.2e}"
    # the same cache without its records: the generic outlier merge must agree too
    Kp.drop_ofrag()
    O2 = _attend(Q, Kp, Vp, tk, tv)
    err, r2 = (O2 - ref).abs().max().item(), rel_l2(O2, ref)
    assert err < MAX_ABS * max(1.0, float(ref.abs().max())) and r2 < REL_L2, f"without records: {err:.2e} {r2:.2e}"


def test_records_under_token_by_token_appends():
    """Serving pattern: a prefill call, then one token per call (each call with its own Med3x median).  Every
    block gets its records in the call that completes it, from flags and side buffer; the last, incomplete
    block has none and is merged from flags / side buffer by the attention kernel."""
    S, br, C, d, Hq, Hkv, B, T0, n_app = 96, 4, 3.0, 128, 8, 2, 2, 70, 45
    T = T0 + n_app
    K = make_kv("hot", (B, Hkv, T, d), seed=61, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T, d), seed=62, dtype=torch.bfloat16)
    Q = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(63)) / math.sqrt(d)).bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), C)
    Kp = q.inner.new_cache(B, T, d, "cuda", scale_dtype=torch.bfloat16, with_outliers=True,
                           out_dtype=torch.bfloat16, ofrag=True)
    q.encode(K[:, :, :T0].cuda(), 0, 0, out=Kp)
    for t in range(T0, T):
        q.encode(K[:, :, t:t + 1].cuda(), 0, 0, out=Kp)
    Vp = q.inner.encode(V.cuda(), 0, 1)
    tk, tv = q.inner.tables(0, 0, "cuda"), q.inner.tables(0, 1, "cuda")
    ki, kr, ks, kf = (t.cpu() for t in Kp.to_reference())
    vi, vr, vs, _ = Vp.to_reference()
    off, recs = _planes(Kp)
    for b in range(B):
        for h in range(Hkv):
            eo, er = _expected_records(K[b, h].float().numpy(), kf[b, h].numpy(), ks[b, h].numpy(), 15, 0, T, Kp.ofrag_cap)
            assert np.array_equal(off[b, h, :len(eo)], eo), f"offsets of (b={b}, h={h})"
            for i, rec in enumerate(er):
                assert np.array_equal(recs[b, h, i], rec), f"record {i} of (b={b}, h={h})"
            assert len(er) >= T // 16                 # every complete block has hot channels, hence records
    ref = orc.fused_attention(Q, ki, kr, ks, tk["joint"].cpu(), vi.cpu(), vr.cpu(), vs.cpu(), tv["joint"].cpu(),
                              15, causal=False, K_flags=kf, K_orig=K)
    O = _attend(Q, Kp, Vp, tk, tv)
    err, r2 = (O - ref).abs().max().item(), rel_l2(O, ref)
    assert err < MAX_ABS * max(1.0, float(ref.abs().max())) and r2 < REL_L2, f"{err:.2e} {r2:.2e}"
