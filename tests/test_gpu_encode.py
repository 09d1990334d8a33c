"""Encoder parity on the GPU, through the C ABI: indices, radius codes, per-token scales, Med3x
medians, flags and outlier payloads against the oracle and the reference-generated fixtures.
Integer outputs must be bit-exact; an index may differ only where the oracle's two best
similarities are closer than 1e-6 (tolerance of the path's parity contract)."""
import numpy as np
import pytest
import torch

import hqmq_b200 as hqmq
from oracle import hqmq_oracle as orc
from tests.util import classify_idx, load_npz, make_kv

pytestmark = pytest.mark.gpu
NEAR_TIE = 1e-6


def _encode_and_compare(x, S, br, C, layer=0, kv=0, n_layers=2, search=0, scale_dtype=torch.float32, quantile=None):
    B, H, T, d = x.shape
    q = hqmq.HQMQ(n_layers=n_layers, n_heads=H, secondary_size=S, radius_bits=br, device="cuda", seed=42)
    joint = orc.joint_codebook(orc.secondary_raw(n_layers, H, S, 42)[layer, :, kv])
    enc = orc.encode(x, joint, br, C, quantile=quantile)
    med = torch.zeros(H, device="cuda")
    pk = q.encode(x.cuda(), layer, kv, median_mult=C, scale_dtype=scale_dtype, search=search,
                  med_out=med if C is not None else None, quantile=quantile)
    idx, rq, rs, flags = pk.to_reference()
    torch.cuda.synchronize()
    # the packed row stores 0 as the radius code of a flagged chunk (its values are in the side buffer)
    want_rq = enc["rq"] if C is None else torch.where(enc["flags"], 0, enc["rq"])
    assert torch.equal(rq.cpu(), want_rq), "radius codes differ"
    if scale_dtype == torch.float32:
        assert torch.equal(rs.cpu(), enc["r_max"]), "per-token scales differ"
    else:
        assert torch.equal(rs.cpu(), enc["r_max"].to(scale_dtype).float())
    n_mis, n_bad = classify_idx(idx, enc, NEAR_TIE)
    assert n_bad == 0, f"{n_bad} index mismatches with oracle top-2 gap >= {NEAR_TIE}"
    assert n_mis <= max(2, int(2e-3 * idx.numel())), f"{n_mis} near-tie mismatches is implausibly many"
    if C is not None:
        assert torch.equal(med.cpu(), enc["med"]), "median differs"
        assert torch.equal(flags.cpu(), enc["flags"]), "outlier flags differ"
        # payload: original values of flagged chunks in (token, chunk) order per (b,h)
        n = d // 4
        xc = x.view(B, H, T, n, 4)
        cnt = pk.out_count.cpu().view(B, H)
        ov = pk.out_vals.cpu()[: B * H * pk.out_cap * 4].view(B, H, pk.out_cap, 4).float()
        for b in range(B):
            for h in range(H):
                want = xc[b, h][enc["flags"][b, h]].float()
                assert cnt[b, h] == want.shape[0]
                assert torch.equal(ov[b, h, : want.shape[0]], want), (b, h)
    return q, pk, enc, n_mis


@pytest.mark.parametrize("name", ["s24_r3", "s24_r3_med3", "s96_r4_med3", "s192_r6_med3", "s96_r4_d64"])
def test_encode_matches_reference_fixtures(name):
    z = load_npz("golden_encode.npz")
    S, br, C, B, H, T, d = z[name + ".meta"]
    S, br, C = int(S), int(br), (None if C < 0 else float(C))
    for kv, layer in ((0, 0), (1, 1)):
        key = f"{name}.kv{kv}"
        x = torch.from_numpy(z[key + ".x"])
        q, pk, enc, _ = _encode_and_compare(x, S, br, C, layer=layer, kv=kv)
        # against the stored reference-derived integers, not only the live oracle
        idx, rq, rs, flags = pk.to_reference()
        gold_rq = z[key + ".rq"].copy()
        if C is not None:
            gold_rq[np.unpackbits(z[key + ".flags"])[: gold_rq.size].reshape(gold_rq.shape).astype(bool)] = 0
        assert np.array_equal(rq.cpu().numpy().astype(np.uint8), gold_rq)
        mism = idx.cpu().numpy().astype(np.uint16) != z[key + ".idx"]
        assert not (mism & (z[key + ".gap"] >= NEAR_TIE)).any()
        # fake-quant output against the reference's own quantize_K / quantize_V output
        qq = hqmq.with_outlier_extraction(q, C) if C is not None else q
        fq = (qq.quantize_K if kv == 0 else qq.quantize_V)(x.cuda(), layer).cpu()
        ref = torch.from_numpy(z[key + ".ref_fake_quant"])
        if not mism.any():
            assert torch.equal(fq, ref), "fake-quant output is not bit-identical to the reference"
        else:
            bad = (fq != ref).view(int(B), int(H), int(T), -1, 4).any(-1)
            assert int(bad.sum()) <= int(mism.sum())


@pytest.mark.parametrize("S,br,kind,C", [(24, 3, "randn", None), (96, 4, "hot", 3.0), (192, 6, "student", 3.0),
                                         (24, 3, "spiky", 3.0)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_encode_16bit_inputs_upcast_contract(S, br, kind, C, dtype):
    x16 = make_kv(kind, (2, 2, 96, 128), seed=11, dtype=dtype)
    if dtype == torch.float16:
        x16 = x16.clamp(-6e4, 6e4)
    _encode_and_compare(x16.float(), S, br, C)                       # oracle sees the upcast
    # the 16-bit tensor itself gives the same integers
    H = 2
    q = hqmq.HQMQ(n_layers=2, n_heads=H, secondary_size=S, radius_bits=br, device="cuda")
    a = q.encode(x16.cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32).to_reference()
    b = q.encode(x16.float().cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32).to_reference()
    for u, v in zip(a, b):
        if u is not None:
            assert torch.equal(u, v)


@pytest.mark.parametrize("shape", [(1, 1, 1, 16), (1, 2, 3, 32), (2, 1, 33, 48), (1, 2, 129, 64), (3, 2, 31, 128)])
def test_encode_ragged_shapes(shape):
    x = make_kv("hot" if shape[3] >= 64 else "randn", shape, seed=5)
    _encode_and_compare(x, 24, 3, 3.0)
    _encode_and_compare(x, 96, 4, None)


def test_encode_zero_and_tiny_chunks():
    x = make_kv("randn", (1, 2, 8, 32), seed=9)
    x[0, 0, 0] = 0.0                 # whole token zero: radius clamps to 1e-8
    x[0, 1, 3, 4:8] = 0.0            # one zero chunk
    x[0, 1, 5] *= 1e-12
    _encode_and_compare(x, 24, 3, 3.0)


def test_encode_append_keeps_earlier_rows_and_offsets():
    S, br, C = 96, 4, 3.0
    x = make_kv("hot", (2, 2, 200, 64), seed=21)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, 2, S, br, device="cuda"), C)
    joint = orc.joint_codebook(orc.secondary_raw(1, 2, S, 42)[0, :, 0])
    cache = q.inner.new_cache(2, 256, 64, "cuda", scale_dtype=torch.float32, with_outliers=True,
                              out_dtype=torch.float32)
    cuts = [0, 70, 71, 128, 200]
    encs = []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        q.encode(x[:, :, lo:hi].cuda(), 0, 0, out=cache)
        encs.append(orc.encode(x[:, :, lo:hi], joint, br, C))      # each call has its own median
    idx, rq, rs, flags = cache.to_reference()
    want = {k: torch.cat([e[k] for e in encs], dim=2) for k in ("idx", "rq", "r_max", "flags", "gap")}
    assert torch.equal(rq.cpu(), torch.where(want["flags"], 0, want["rq"])) and torch.equal(rs.cpu(), want["r_max"])
    assert torch.equal(flags.cpu(), want["flags"])
    assert classify_idx(idx, want)[1] == 0
    # merged dequant == oracle fake-quant with originals restored
    dense = q.decode(cache, 0, 0, dtype=torch.float32, scale_first=True).cpu()
    for (lo, hi), e in zip(zip(cuts[:-1], cuts[1:]), encs):
        ref = orc.fake_quant(x[:, :, lo:hi], joint, br, C, enc=e)
        same_idx = (idx.cpu()[:, :, lo:hi] == e["idx"]).repeat_interleave(4, dim=-1).view_as(ref)
        assert torch.equal(dense[:, :, lo:hi][same_idx], ref[same_idx])
    assert abs(q._observed_outlier_rate - np.mean([float(e["flags"].float().mean()) for e in encs])) < 1e-6


@pytest.mark.parametrize("S,br", [(24, 3), (96, 4), (192, 6)])
@pytest.mark.parametrize("kind", ["randn", "hot", "spiky"])
def test_exhaustive_and_default_search_agree(S, br, kind):
    """The look-up-table search against the exhaustive closed-form scan on a million chunks per case (GPU against
    GPU); every chunk on which they disagree is then put to the oracle, and a disagreement is allowed only where
    the oracle's two best similarities differ by less than 1e-6 (a documented near-tie)."""
    B, H, T, d = 4, 8, 1024, 128
    x = make_kv(kind, (B, H, T, d), seed=500 + S, dtype=torch.bfloat16)
    q = hqmq.HQMQ(1, H, S, br, device="cuda")
    a = q.encode(x.cuda(), 0, 0, search=0).to_reference()[0].cpu()
    b = q.encode(x.cuda(), 0, 0, search=1).to_reference()[0].cpu()
    diff = a != b
    assert diff.float().mean().item() < 2e-3
    raw = orc.secondary_raw(1, H, S, 42)
    joint = orc.joint_codebook(raw[0, :, 0])
    xc = x.float().view(B, H, T, d // 4, 4)
    for h in range(H):
        m = diff[:, h]
        if not m.any():
            continue
        chunks = xc[:, h][m].reshape(1, 1, -1, 4)            # every disagreeing chunk as a one-chunk token
        enc = orc.encode(chunks, joint[h:h + 1], br, None)
        gap, want = enc["gap"].reshape(-1), enc["idx"].reshape(-1)
        for got in (a[:, h][m], b[:, h][m]):
            bad = (got.to(torch.int32) != want) & (gap >= 1e-6)
            assert int(bad.sum()) == 0, f"S={S} {kind} head {h}: {int(bad.sum())} indices differ from the oracle outside near-ties"


def test_full_size_properties_config2_slice():
    """One (b, h) column of the Llama-3-8B-shaped configuration at its full context (32768 tokens):
    size-independent properties instead of an element-wise oracle."""
    S, br, C = 96, 4, 3.0
    x = make_kv("hot", (1, 2, 32768, 128), seed=1002, dtype=torch.bfloat16).cuda()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, 2, S, br, device="cuda"), C)
    med = torch.zeros(2, device="cuda")
    pk = q.encode(x, 0, 0, scale_dtype=torch.float32, med_out=med)
    idx, rq, rs, flags = pk.to_reference()
    xf = x.float().view(1, 2, 32768, 32, 4)
    sq = xf * xf          # the contract's norm: separate IEEE multiplies and adds in this order, then one square root
    nrm = (((sq[..., 0] + sq[..., 1]) + sq[..., 2]) + sq[..., 3]).sqrt()
    # median property: at least half of the norms are <= med and at least half are >= med
    for h in range(2):
        v = nrm[0, h].reshape(-1)
        assert (v <= med[h]).float().mean() >= 0.5 and (v >= med[h]).float().mean() >= 0.5
        assert torch.equal(flags[0, h], nrm[0, h] > med[h] * C)
    assert int(rq.max()) == 15 and int(rq.min()) >= 0
    assert (torch.where(flags, 15, rq).max(dim=-1).values == 15).all()   # the token's largest chunk codes qmax (or is flagged)
    assert int(idx.max()) < 24 * S and int(idx.min()) >= 0
    assert pk.n_outliers() == int(flags.sum())
    # idempotence: re-encoding the fake-quantised tensor reproduces the same codes (outliers restored)
    dense = q.decode(pk, 0, 0, dtype=torch.float32, scale_first=True)
    cos = torch.nn.functional.cosine_similarity(dense.view(-1, 4), x.float().view(-1, 4), dim=-1)
    assert cos.mean() > 0.98


def test_side_buffer_overflow_is_reported_not_fatal():
    """A side buffer that is too small: rows, flags and counts stay complete, the status word of the call's
    workspace says so (hqmq_read_status), and nothing is written past the capacity."""
    S, br, C, d, H, B, T = 96, 4, 3.0, 128, 2, 1, 256
    K = make_kv("hot", (B, H, T, d), seed=9, dtype=torch.bfloat16).cuda()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, H, S, br, device="cuda"), C)
    full = q.encode(K, 0, 0)
    need = int(full.out_count.max())
    assert need > 64
    small = q.inner.new_cache(B, T, d, "cuda", scale_dtype=torch.bfloat16, with_outliers=True,
                              out_dtype=torch.bfloat16, out_cap=64)
    guard = small.out_vals.clone()
    with pytest.raises(hqmq.HqmqError, match="side buffer too small"):
        q.inner.encode(K, 0, 0, out=small, median_mult=C, check_status=True)
    assert torch.equal(small.flags[:B * H * T], full.flags[:B * H * T])
    assert torch.equal(small.out_count, full.out_count)
    n_per = small.out_cap * 4
    assert torch.equal(small.out_vals[:n_per], full.out_vals[:n_per])          # the entries that fit are the right ones
    assert torch.equal(small.out_vals[H * n_per:], guard[H * n_per:])            # nothing past the planes


@pytest.mark.parametrize("T", [256, 4096])
def test_med3x_chunks_next_to_the_threshold(T):
    """The 16-bit fast path decides most flags before the last ten bits of the median are known and settles
    the chunks within 2^-13 of the threshold afterwards (from a list, or by re-reading x when the list
    overflows: T = 4096).  Norms exactly at the threshold must stay unflagged (strict compare)."""
    B, H, d, S, br, C = 1, 2, 128, 96, 4, 3.0
    n = d // 4
    g = torch.Generator().manual_seed(5)
    kind = torch.rand(B, H, T, n, generator=g)
    near, far = (kind >= 0.6) & (kind < 0.8), kind >= 0.8
    x = torch.zeros(B, H, T, n, 4)
    x[..., 0] = 1.0                                                    # 60 % of the chunks: norm exactly 1 = the median
    eps = torch.randint(0, 5, (B, H, T, n), generator=g).float() * 0.01
    x[..., 0] = torch.where(near, torch.tensor(3.0), x[..., 0])        # norm sqrt(9 + eps^2): 3 or just above
    x[..., 1] = torch.where(near, eps, x[..., 1])
    x[..., 0] = torch.where(far, torch.rand(B, H, T, n, generator=g) * 8.0, x[..., 0])
    x = x.view(B, H, T, d).bfloat16()
    joint = orc.joint_codebook(orc.secondary_raw(1, H, S, 42)[0, :, 0])
    enc = orc.encode(x.float(), joint, br, C)
    assert torch.equal(enc["med"], torch.ones(H))
    norms = x.float().view(B, H, T, n, 4).norm(dim=-1)
    band = (norms > 3.0) & (norms < 3.0004)
    assert int(band.sum()) > (4096 if T == 4096 else 100) * H            # the list really overflows at T = 4096
    assert enc["flags"][band].all() and not enc["flags"][norms == 3.0].any() and (norms == 3.0).any()
    q = hqmq.HQMQ(n_layers=1, n_heads=H, secondary_size=S, radius_bits=br, device="cuda", seed=42)
    med = torch.zeros(H, device="cuda")
    pk = q.encode(x.cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32, med_out=med)
    idx, rq, rs, flags = pk.to_reference()
    assert torch.equal(med.cpu(), enc["med"])
    assert torch.equal(flags.cpu(), enc["flags"]), "outlier flags differ"
    assert torch.equal(rq.cpu(), torch.where(enc["flags"], 0, enc["rq"])), "radius codes differ"
    assert torch.equal(pk.out_count.cpu().view(B, H), enc["flags"].sum(dim=(2, 3)).int())
    xc = x.view(B, H, T, n, 4)
    ov = pk.out_vals.cpu()[: B * H * pk.out_cap * 4].view(B, H, pk.out_cap, 4)
    for h in range(H):
        want = xc[0, h][enc["flags"][0, h]]
        assert torch.equal(ov[0, h, : want.shape[0]], want)


@pytest.mark.parametrize("mislead", [False, True])
def test_med3x_sampled_prediction_and_its_fallback(mislead):
    """Long 16-bit calls histogram the second digit of the median inside the main pass, for the bins a sample
    (every 32nd token) predicts.  With `mislead` the sampled tokens are 100x larger than the rest, the
    prediction is wrong and the separate pass must take over; either way the integers match the oracle."""
    B, H, T, d, S, br, C = 1, 2, 2048, 128, 96, 4, 3.0
    x = make_kv("hot", (B, H, T, d), seed=21, dtype=torch.float32)
    if mislead:
        x[:, :, ::32] *= 100.0
    x = x.bfloat16()
    joint = orc.joint_codebook(orc.secondary_raw(1, H, S, 42)[0, :, 0])
    enc = orc.encode(x.float(), joint, br, C)
    q = hqmq.HQMQ(n_layers=1, n_heads=H, secondary_size=S, radius_bits=br, device="cuda", seed=42)
    med = torch.zeros(H, device="cuda")
    pk = q.encode(x.cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32, med_out=med)
    idx, rq, rs, flags = pk.to_reference()
    assert torch.equal(med.cpu(), enc["med"]), "median differs"
    assert torch.equal(flags.cpu(), enc["flags"]), "outlier flags differ"
    assert torch.equal(rq.cpu(), torch.where(enc["flags"], 0, enc["rq"])), "radius codes differ"
    assert torch.equal(rs.cpu(), enc["r_max"])
    n_mis, n_bad = classify_idx(idx, enc, NEAR_TIE)
    assert n_bad == 0


@pytest.mark.parametrize("shape,S,br", [((2, 2, 32, 128), 96, 4), ((16, 2, 1, 128), 96, 4), ((64, 2, 2, 64), 24, 3),
                                        ((3, 1, 7, 48), 192, 6), ((1, 1, 1, 4), 24, 3)])
@pytest.mark.parametrize("C", [None, 3.0])
def test_small_calls_one_kernel_per_head(shape, S, br, C):
    """Calls with at most 2048 chunks per head (decode-time appends) run main pass, median and flags in one
    kernel per head; same integers as the oracle, and the same as the 16-bit input gives."""
    B, H, T, d = shape
    x = make_kv("spiky" if d >= 16 else "randn", shape, seed=31)
    if d >= 16:
        x[:, :, :, :4] *= 6.0                           # one hot chunk per token: flagged by Med3x
    _encode_and_compare(x, S, br, C)
    x16 = x.bfloat16()
    q = hqmq.HQMQ(n_layers=2, n_heads=H, secondary_size=S, radius_bits=br, device="cuda")
    a = q.encode(x16.cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32).to_reference()
    b = q.encode(x16.float().cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32).to_reference()
    for u, v in zip(a, b):
        if u is not None:
            assert torch.equal(u, v)


@pytest.mark.parametrize("shape,dtype,S,br", [((4, 2, 160, 128), torch.bfloat16, 96, 4), ((3, 3, 96, 64), torch.float32, 24, 3)])
def test_split_batch_median_and_encode_match_the_whole_batch(shape, dtype, S, br):
    """A head whose batch entries sit on two GPUs: the per-level histograms of the two parts, summed (what the
    all_reduce between the levels does; here both parts live on one device and the sum is a tensor add), must
    select the median of the whole batch bit for bit, and encoding each part against that median must give the
    rows, flags and payload of the whole-batch call."""
    import ctypes as C
    from hqmq_b200 import _lib
    from hqmq_b200.dist import HIST_BINS
    B, H, T, d = shape
    Cm = 3.0
    x = make_kv("spiky", shape, seed=311, dtype=dtype).cuda()
    inner = hqmq.HQMQ(1, H, S, br, device="cuda")
    quant = hqmq.with_outlier_extraction(inner, Cm)
    med_ref = torch.zeros(H, device="cuda")
    whole = quant.encode(x, 0, 0, med_out=med_ref, scale_dtype=torch.float32)
    assert whole.n_outliers() > 0
    parts = [x[:1], x[1:]]                       # uneven on purpose
    L = _lib.lib()
    nbytes = L.hqmq_med3x_state_bytes(H)
    sd = torch.float32
    caches = [inner.new_cache(p.shape[0], T, d, "cuda", scale_dtype=sd, with_outliers=True, out_dtype=dtype, ofrag=True)
              for p in parts]
    args = [inner._enc_args(p, 0, 0, c, Cm) for p, c in zip(parts, caches)]
    states = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in parts]
    hists = [s[: H * 3 * 2 * HIST_BINS * 4].view(torch.int32).view(H, 3, 2, HIST_BINS) for s in states]
    meds = [torch.zeros(H, device="cuda") for _ in parts]
    n_total = B * T * (d // 4)
    for level in range(3):
        for a, s in zip(args, states):
            _lib.check(L.hqmq_med3x_hist(C.byref(a), level, s.data_ptr(), nbytes, _lib.stream_ptr()), "hist")
        total = hists[0][:, level] + hists[1][:, level]
        for h_ in hists:
            h_[:, level] = total
        for s, m in zip(states, meds):
            _lib.check(L.hqmq_med3x_select(H, level, n_total, Cm, s.data_ptr(), nbytes, m.data_ptr(), _lib.stream_ptr()), "select")
    torch.cuda.synchronize()
    assert torch.equal(meds[0], med_ref) and torch.equal(meds[1], med_ref)
    b0 = 0
    for p, c, m in zip(parts, caches, meds):
        got_med = torch.zeros(H, device="cuda")
        quant.encode(p, 0, 0, out=c, med_in=m, med_out=got_med)
        assert torch.equal(got_med, med_ref)
        nb = p.shape[0]
        for got, want in zip(c.to_reference(), whole.to_reference()):
            assert torch.equal(got, want[b0:b0 + nb])
        cw = whole.out_count.view(B, H)[b0:b0 + nb]
        assert torch.equal(c.out_count.view(nb, H), cw)
        ov_w = whole.out_vals[: B * H * whole.out_cap * 4].view(B, H, whole.out_cap, 4)[b0:b0 + nb]
        ov_c = c.out_vals[: nb * H * c.out_cap * 4].view(nb, H, c.out_cap, 4)
        for b in range(nb):
            for h in range(H):
                k = int(cw[b, h])
                assert torch.equal(ov_c[b, h, :k], ov_w[b, h, :k])
        b0 += nb


@pytest.mark.parametrize("name", ["frac1_s96_r4", "frac5_s24_r3", "frac10_s96_r4"])
def test_fraction_threshold_matches_reference_fixtures(name):
    """threshold_mode="fraction" of the reference wrapper (src/quantizers/outlier_aware.py:64-66): the per-head
    quantile 1 - outlier_fraction of the chunk norms is the threshold.  Flags, radius codes and the fake-quant
    output against what the reference itself produced (small calls: the one-kernel path)."""
    z = load_npz("golden_fraction.npz")
    S, br, frac, B, H, T, d = z[name + ".meta"]
    S, br, B, H, T = int(S), int(br), int(B), int(H), int(T)
    x = torch.from_numpy(z[name + ".x"])
    inner = hqmq.HQMQ(n_layers=1, n_heads=H, secondary_size=S, radius_bits=br, device="cuda", seed=42)
    qq = hqmq.OutlierAwareHQMQQuantizer(inner, outlier_fraction=float(frac), threshold_mode="fraction")
    pk = qq.encode(x.cuda(), 0, 0)
    idx, rq, rs, flags = pk.to_reference()
    gold_flags = np.unpackbits(z[name + ".flags"])[: rq.numel()].reshape(rq.shape).astype(bool)
    assert np.array_equal(flags.cpu().numpy(), gold_flags)
    gold_rq = z[name + ".rq"].copy()
    gold_rq[gold_flags] = 0
    assert np.array_equal(rq.cpu().numpy().astype(np.uint8), gold_rq)
    mism = idx.cpu().numpy().astype(np.uint16) != z[name + ".idx"]
    assert not (mism & (z[name + ".gap"] >= NEAR_TIE)).any()
    fq = qq.quantize_K(x.cuda(), 0).cpu()
    if not mism.any():
        assert torch.equal(fq, torch.from_numpy(z[name + ".ref_fake_quant"]))
    assert abs(qq._observed_outlier_rate - gold_flags.mean()) < 1e-6


@pytest.mark.parametrize("S,br,kind,q", [(96, 4, "hot", 0.97), (24, 3, "spiky", 0.995), (192, 6, "student", 0.9)])
def test_fraction_threshold_large_calls(S, br, kind, q):
    """The same statistic through the multi-pass path of large calls (sampled prediction, three-level select,
    threshold bounds and fix-up), against the oracle's torch.quantile restatement."""
    x = make_kv(kind, (2, 2, 3000, 128), seed=21, dtype=torch.bfloat16).float()
    _encode_and_compare(x, S, br, 1.0, quantile=q)
    _encode_and_compare(x[:, :, :1500, :64].contiguous(), S, br, 1.0, quantile=q)       # generic geometry


def _threshold_compare(x, S, br, C, quantile=None):
    """Scales, threshold statistic, flags and radius codes of a large call against the oracle (the codeword search
    does not depend on the threshold path and has its own tests; leaving it out keeps the oracle fast here)."""
    B, H, T, d = x.shape
    q = hqmq.HQMQ(n_layers=1, n_heads=H, secondary_size=S, radius_bits=br, device="cuda", seed=42)
    med = torch.zeros(H, device="cuda")
    pk = q.encode(x.cuda(), 0, 0, median_mult=C, scale_dtype=torch.float32, med_out=med, quantile=quantile)
    _, rq, rs, flags = pk.to_reference()
    qmax = (1 << br) - 1
    nrm = orc.chunk_norms(x.float())
    want_med, _, want_flags = orc.med3x_flags(nrm, C, quantile)
    radius = nrm.clamp(min=1e-8)
    r_max = radius.amax(dim=-1).clamp(min=1e-8)
    want_rq = (radius / (r_max / qmax).unsqueeze(-1)).round().clamp(0, qmax).to(torch.int32)
    assert torch.equal(med.cpu(), want_med), "threshold statistic differs"
    assert torch.equal(flags.cpu(), want_flags), f"{int((flags.cpu() != want_flags).sum())} flags differ"
    assert torch.equal(rs.cpu(), r_max)
    assert torch.equal(rq.cpu(), torch.where(want_flags, 0, want_rq)), "radius codes differ"
    return pk


@pytest.mark.parametrize("kind,S,br", [("hot", 96, 4), ("spiky", 24, 3), ("student", 192, 6), ("randn", 96, 4)])
def test_single_read_pass_of_large_calls(kind, S, br):
    """Calls with at least 65536 tokens per head decide the flags in the pass that reads x, around a threshold
    predicted from a sample, and take the exact order statistics from the norms listed near the prediction."""
    x = make_kv(kind, (16, 2, 4096, 128), seed=41, dtype=torch.bfloat16).float()
    pk = _threshold_compare(x, S, br, 3.0)
    _threshold_compare(x[:, :, :4095], S, br, 3.0)                  # odd count: one middle order statistic
    _threshold_compare(x, S, br, 1.0, quantile=0.7)
    if kind == "hot":
        assert pk.n_outliers() > 0.03 * x.numel() / 4


@pytest.mark.parametrize("kind", ["constant", "two_levels", "tiny", "drift"])
def test_single_read_pass_gives_way_when_its_prediction_cannot_hold(kind):
    """When the list cannot hold the norms around the prediction (every chunk has the same norm), when the statistic
    sits where the sample does not place it (the sampled tokens differ from the rest, or the distribution drifts
    along the sequence in step with the sampling), or when it is next to zero, the multi-pass kernels must take the
    call over and give the oracle's result all the same."""
    g = torch.Generator().manual_seed(31)
    B, H, T, d = 16, 2, 4096, 128
    sign = torch.where(torch.rand(B, H, T, d, generator=g) < 0.5, -1.0, 1.0)
    if kind == "constant":
        x = sign * 0.5                                    # every chunk norm is exactly 1
        x[:, :, ::97, 8:12] *= 10.0                       # and a few outliers
    elif kind == "two_levels":
        x = sign * 0.5
        x[:, :, 1::2] *= 1.5                              # half of the tokens at 1.5: the median falls between two spikes
        x[0, 0, :33] *= 1.5
    elif kind == "drift":
        x = torch.randn(B, H, T, d, generator=g)
        x[:, :, ::32] *= 1.2                              # exactly the sampled tokens are larger than the others
    else:
        x = sign * 1e-30                                  # norms far down among the small floats
        x[:, :, ::50, :4] = 3e-29
    _threshold_compare(x.bfloat16().float(), 96, 4, 3.0)
    _threshold_compare(x.bfloat16().float(), 24, 3, 1.0, quantile=0.5)


@pytest.mark.parametrize("S,br,kind", [(96, 4, "hot"), (24, 3, "spiky"), (192, 6, "student")])
def test_head_dim_64_through_the_token_pair_kernels(S, br, kind):
    """d_head 64 with contiguous tokens, an even token count and an even first row runs the kernels written for 32
    chunks per token on pairs of tokens (scale, flag word and row per half-warp): every plane against the oracle,
    for a call that starts a cache and for one appended behind an even number of tokens; an odd count or an odd
    first row takes the generic kernels and must agree too."""
    x = make_kv(kind, (2, 2, 2304, 64), seed=51, dtype=torch.bfloat16).float()
    q, pk, enc, _ = _encode_and_compare(x, S, br, 3.0)
    _encode_and_compare(x[:, :, :2303].contiguous(), S, br, 3.0)               # odd count: generic kernels
    # appended behind 16 tokens (even first row) and behind 17 (odd): rows, scales and flags of the appended part
    for first in (16, 17):
        qq = hqmq.with_outlier_extraction(hqmq.HQMQ(n_layers=2, n_heads=2, secondary_size=S, radius_bits=br, device="cuda", seed=42), 3.0)
        dst = qq.inner.new_cache(2, 4096, 64, "cuda", scale_dtype=torch.float32, with_outliers=True, out_dtype=torch.float32)
        qq.encode(x[:, :, :first].contiguous().cuda(), 0, 0, out=dst)
        qq.encode(x[:, :, first:first + 2048].contiguous().cuda(), 0, 0, out=dst)
        joint = orc.joint_codebook(orc.secondary_raw(2, 2, S, 42)[0, :, 0])
        want = orc.encode(x[:, :, first:first + 2048], joint, br, 3.0)
        idx, rq, rs, flags = dst.to_reference(first, 2048)
        assert torch.equal(flags.cpu(), want["flags"]) and torch.equal(rs.cpu(), want["r_max"])
        assert torch.equal(rq.cpu(), torch.where(want["flags"], 0, want["rq"]))
        n_mis, n_bad = classify_idx(idx, want, NEAR_TIE)
        assert n_bad == 0


@pytest.mark.parametrize("kind", ["hot", "spiky", "constant"])
def test_head_dim_64_single_read_pass(kind):
    """The same pairs through the single-read pass of large calls (and through its fallback for a constant-norm tensor)."""
    if kind == "constant":
        g = torch.Generator().manual_seed(33)
        x = torch.where(torch.rand(16, 2, 8192, 64, generator=g) < 0.5, -0.5, 0.5)
        x[:, :, ::97, 8:12] *= 10.0
    else:
        x = make_kv(kind, (16, 2, 8192, 64), seed=52, dtype=torch.bfloat16).float()
    _threshold_compare(x.bfloat16().float(), 96, 4, 3.0)
    _threshold_compare(x.bfloat16().float()[:, :, :8190], 24, 3, 1.0, quantile=0.5)
