"""Decode attention at the shapes the benchmark times, against the fp32 oracle (2e-3 max-abs / 1e-3 relative L2).

Each case encodes seeded K / V of the configuration's value distribution on the GPU, attends over the native
cache through the C ABI and compares with the oracle attending over the same codes with the original values of
the flagged chunks merged in (the oracle call is made one KV head at a time to bound host memory).  The work
decomposition is varied (default flat split, one CTA per unit, forced splits) because it decides how many tiles
a CTA walks and how far into the side buffers its offsets reach."""
import math

import pytest
import torch

import hqmq_b200 as hqmq
from oracle import hqmq_oracle as orc
from tests.util import make_kv, rel_l2

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-3, 1e-3


def _oracle_per_head(Q, Kp, Vp, K, V, tk, tv, qmax, window=None):
    ki, kr, ks, kf = (t.cpu() if t is not None else None for t in Kp.to_reference())
    vi, vr, vs, vf = (t.cpu() if t is not None else None for t in Vp.to_reference())
    Hkv = ki.shape[1]
    G = Q.shape[1] // Hkv
    jk, jv = tk["joint"].cpu(), tv["joint"].cpu()
    outs = []
    for h in range(Hkv):
        s = slice(h, h + 1)
        outs.append(orc.fused_attention(
            Q[:, h * G:(h + 1) * G], ki[:, s], kr[:, s], ks[:, s], jk[s], vi[:, s], vr[:, s], vs[:, s], jv[s], qmax,
            causal=False, K_flags=None if kf is None else kf[:, s], K_orig=K[:, s],
            V_flags=None if vf is None else vf[:, s], V_orig=V[:, s], window=window))
    return torch.cat(outs, dim=1), kf, vf


def _attend_and_check(q, Q, K, V, S, br, what, window=None, ofrag=None, splits=(None, 1, 7), min_k_flag=None,
                      relative_to_output=False):
    inner = q.inner if hasattr(q, "inner") else q
    Kp, Vp = q.encode(K.cuda(), 0, 0, ofrag=ofrag), q.encode(V.cuda(), 0, 1)
    tk, tv = inner.tables(0, 0, "cuda"), inner.tables(0, 1, "cuda")
    ref, kf, vf = _oracle_per_head(Q, Kp, Vp, K, V, tk, tv, (1 << br) - 1, window=window)
    if min_k_flag is not None:
        assert kf.float().mean().item() > min_k_flag, "the synthetic outliers were not flagged"
    # (the 2e-3 bound is stated for outputs of order one; where outlier channels of V make the outputs much larger,
    #  a case may ask for the bound relative to the largest output instead)
    max_abs = MAX_ABS * max(1.0, ref.abs().max().item()) if relative_to_output else MAX_ABS
    for sp in splits:
        O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
        hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], kv_splits=sp, window=window, out=O)
        err = (O.cpu() - ref).abs().max().item()
        r2 = rel_l2(O.cpu(), ref)
        assert err < max_abs and r2 < REL_L2, f"{what} splits={sp}: max-abs {err:.2e} (bound {max_abs:.1e}), rel-L2 {r2:.2e}"
    return Kp, Vp


def _queries(B, Hq, d, seed, dtype=torch.bfloat16):
    return (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(seed)) / math.sqrt(d)).to(dtype)


@pytest.mark.parametrize("ofrag", [True, False])
def test_config2_full_context_slice(ofrag):
    """Llama-3-8B shape at full context: one batch entry, 8 KV heads, 32768 tokens, s96_r4 + Med3x, K with 4
    hot channels x8 (about 6 % of its chunks flagged), with and without the fragment records."""
    S, br, d, Hq, Hkv, T, B = 96, 4, 128, 32, 8, 32768, 1
    K = make_kv("hot", (B, Hkv, T, d), seed=1002, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T, d), seed=2002, dtype=torch.bfloat16)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    _attend_and_check(q, _queries(B, Hq, d, 3002), K, V, S, br, f"config 2, ofrag={ofrag}", ofrag=ofrag, min_k_flag=0.03)


def test_config2_without_med3x():
    S, br, d, Hq, Hkv, T, B = 96, 4, 128, 32, 8, 8192, 2
    K = make_kv("hot", (B, Hkv, T, d), seed=1012, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T, d), seed=2012, dtype=torch.bfloat16)
    q = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    _attend_and_check(q, _queries(B, Hq, d, 3012), K, V, S, br, "config 2 without Med3x")


def test_config3_student_t_outliers():
    """Qwen2.5-7B shape: G = 7 (one padded head column), 19-bit fields that straddle words, heavy-tailed K."""
    S, br, d, Hq, Hkv, T, B = 192, 6, 128, 28, 4, 8192, 2
    K = make_kv("student", (B, Hkv, T, d), seed=1003, dtype=torch.bfloat16)
    V = make_kv("randn", (B, Hkv, T, d), seed=2003, dtype=torch.bfloat16)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    _attend_and_check(q, _queries(B, Hq, d, 3003), K, V, S, br, "config 3", min_k_flag=0.01)


def test_config4_long_single_sequence():
    """One sequence of 131072 tokens, s24_r3 + Med3x, 0.5 % of the chunks of K and of V scaled x20: a unit is
    spread over many CTAs and most tiles carry a few flagged chunks at random positions."""
    S, br, d, Hq, Hkv, T, B = 24, 3, 128, 32, 8, 131072, 1
    K = make_kv("spiky", (B, Hkv, T, d), seed=1004, dtype=torch.bfloat16)
    V = make_kv("spiky", (B, Hkv, T, d), seed=2004, dtype=torch.bfloat16)
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    Kp, Vp = _attend_and_check(q, _queries(B, Hq, d, 3004), K, V, S, br, "config 4", splits=(None, 1, 37), min_k_flag=0.003)
    assert Vp.to_reference()[3].float().mean().item() > 0.003


@pytest.mark.parametrize("window", [None, 128])
def test_config5_layer(window):
    """gpt-oss-20b-shaped layer: d_head 64, G = 8, 16384 tokens, one outlier channel per KV head in K and in V
    (every token carries a flagged chunk at the same position), full attention and a 128-token window."""
    S, br, d, Hq, Hkv, T, B = 96, 4, 64, 64, 8, 16384, 2
    g = torch.Generator().manual_seed(5005)
    K = make_kv("randn", (B, Hkv, T, d), seed=1005)
    V = make_kv("randn", (B, Hkv, T, d), seed=2005)
    for h in range(Hkv):
        K[:, h, :, int(torch.randint(0, d, (1,), generator=g))] *= 40.0
        V[:, h, :, int(torch.randint(0, d, (1,), generator=g))] *= 25.0
    K, V = K.bfloat16(), V.bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    _attend_and_check(q, _queries(B, Hq, d, 3005), K, V, S, br, f"config 5 window={window}", window=window,
                      splits=(None, 1) if window else (None, 1, 5), min_k_flag=0.02)


def test_side_buffer_overflow_is_memory_safe():
    """A side buffer that is too small: the encoder drops the entries beyond its capacity and says so; every
    reader treats a dropped entry as zeros and stays inside the buffer."""
    S, br, d, Hq, Hkv, T, B = 96, 4, 128, 8, 2, 2048, 2
    K = make_kv("hot", (B, Hkv, T, d), seed=77, dtype=torch.bfloat16)
    V = make_kv("spiky", (B, Hkv, T, d), seed=78, dtype=torch.bfloat16)
    inner = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    q = hqmq.with_outlier_extraction(inner, 3.0)
    cap = 1000                                            # K needs about 4000 entries per (b, h), V about 330
    Kp = inner.new_cache(B, T, d, "cuda", with_outliers=True, out_cap=cap, ofrag=False)
    Vp = inner.new_cache(B, T, d, "cuda", with_outliers=True, out_cap=100)
    q.encode(K.cuda(), 0, 0, out=Kp)
    q.encode(V.cuda(), 0, 1, out=Vp)
    assert int(Kp.out_count.max()) > cap and int(Vp.out_count.max()) > 100
    with pytest.raises(hqmq.HqmqError):
        q.encode(K.cuda(), 0, 0, out=inner.new_cache(B, T, d, "cuda", with_outliers=True, out_cap=cap), check_status=True)
    tk, tv = inner.tables(0, 0, "cuda"), inner.tables(0, 1, "cuda")
    # oracle: the flagged chunks whose entry index is beyond the capacity are zero
    ki, kr, ks, kf = (t.cpu() for t in Kp.to_reference())
    vi, vr, vs, vf = (t.cpu() for t in Vp.to_reference())

    def drop(x, flags, capacity):
        order = flags.reshape(B, Hkv, -1).cumsum(-1).reshape(flags.shape)      # 1-based entry index in (token, chunk) order
        keep = (order <= capacity).unsqueeze(-1)
        return (x.float().reshape(B, Hkv, T, d // 4, 4) * keep).reshape(B, Hkv, T, d)

    Q = _queries(B, Hq, d, 79)
    ref = orc.fused_attention(Q, ki, kr, ks, tk["joint"].cpu(), vi, vr, vs, tv["joint"].cpu(), 15, causal=False,
                              K_flags=kf, K_orig=drop(K, kf, cap), V_flags=vf, V_orig=drop(V, vf, 100))
    for sp in (None, 1):
        O = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
        hqmq.fused_attention_packed(Q.cuda(), Kp, Vp, tk["table16"], tv["table16"], kv_splits=sp, out=O)
        assert (O.cpu() - ref).abs().max().item() < MAX_ABS and rel_l2(O.cpu(), ref) < REL_L2
    dense = inner.decode(Kp, 0, 0, dtype=torch.float32).cpu()
    want = orc.merge_outliers(orc.decode_packed(ki, kr, ks, tk["joint"].cpu(), 15), kf, drop(K, kf, cap))
    assert torch.equal(dense, want)

def test_head_dim_64_value_outlier_columns():
    """d_head 64, V tiles whose flagged chunks fill chunk columns (added column by column through the tensor cores)
    next to the cases that must not take that path: one outlier channel that moves to another chunk half way through
    the context; two channels in different chunks; a channel
    plus scattered spikes (tiles with many columns fall back to the per-chunk correction); a channel in rows that are
    zero otherwise (every seventh token: the row's scale is the outlier's own norm, its codes decode to nothing)."""
    S, br, d, Hq, Hkv, T, B = 96, 4, 64, 16, 4, 16379, 4       # (the last tile is a partial one)
    g = torch.Generator().manual_seed(6006)
    K = make_kv("randn", (B, Hkv, T, d), seed=1006)
    V = make_kv("randn", (B, Hkv, T, d), seed=2006)
    V[:, 0, :8000, 13] *= 25.0                                   # the channel moves to another chunk half way
    V[:, 0, 8000:, 50] *= 25.0
    V[:, 1, :, 6] *= 25.0
    V[:, 1, :, 41] *= 40.0
    V[:, 2, :, 30] *= 25.0
    spikes = torch.rand(B, T, d // 4, generator=g) < 0.02
    V[:, 2] *= 1.0 + 19.0 * spikes.repeat_interleave(4, dim=-1).float()
    V[:, 3, :, 57] *= 30.0
    hot = V[:, 3, ::7, 57].clone()
    V[:, 3, ::7] = 0.0
    V[:, 3, ::7, 57] = hot
    K, V = K.bfloat16(), V.bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    Kp, Vp = _attend_and_check(q, _queries(B, Hq, d, 3006), K, V, S, br, "d_head 64 outlier columns", splits=(None, 1, 3))
    vi, vr, vs, vf = Vp.to_reference()
    assert vf[:, 0, :8000, 13 // 4].float().mean() > 0.7 and vf[:, 0, 8000:, 50 // 4].float().mean() > 0.7 and \
        vf[:, 1, :, 41 // 4].float().mean() > 0.7, \
        "the outlier channels were not flagged"
    assert vf[:, 3, ::7, 57 // 4].float().mean() > 0.5, "the lone outliers were not flagged"
def test_head_dim_64_many_units_per_cta():
    """d_head 64 with more than two units per CTA of the ring kernel (320 units of 65 tiles): the units of a CTA are
    taken from different KV heads there, so heads of very different outlier density -- a strong channel, a weak one,
    none -- are mixed in every CTA; the last tile of every unit is a partial one."""
    S, br, d, Hq, Hkv, T, B = 96, 4, 64, 16, 8, 1035, 40
    K = make_kv("randn", (B, Hkv, T, d), seed=1008)
    V = make_kv("randn", (B, Hkv, T, d), seed=2008)
    for h, scale in enumerate([40.0, 1.0, 6.0, 1.0, 25.0, 3.0, 1.0, 90.0]):
        K[:, h, :, (5 * h + 2) % d] *= scale
        V[:, h, :, (11 * h + 7) % d] *= scale
    K, V = K.bfloat16(), V.bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    _attend_and_check(q, _queries(B, Hq, d, 3008), K, V, S, br, "d_head 64, many units per CTA", splits=(None, 2),
                      min_k_flag=0.01, relative_to_output=True)


@pytest.mark.parametrize("d,S,br,window", [(64, 96, 4, 128), (64, 96, 4, None), (128, 24, 3, 128), (128, 96, 4, None)])
def test_many_units_short_ranges(d, S, br, window):
    """A large batch of short key ranges (a sliding-window layer of a serving batch): 384 units of at most 300 keys;
    outlier channels in K and V plus scattered spikes.  With so few keys the outputs reach the size of V's outlier
    channel (tens), so the max-abs bound is taken relative to the largest output.  The default decomposition lets the
    warps of a CTA walk through the units independently; forced splits use the in-CTA merge of the same kernel with less
    shared memory, and the default is called once more after them (the kernel's shared-memory limit must survive the
    smaller launch)."""
    Hq, Hkv, T, B = 32, 8, 300, 48
    g = torch.Generator().manual_seed(7007 + d)
    K = make_kv("randn", (B, Hkv, T, d), seed=1007)
    V = make_kv("randn", (B, Hkv, T, d), seed=2007)
    for h in range(Hkv):
        K[:, h, :, int(torch.randint(0, d, (1,), generator=g))] *= 30.0
        V[:, h, :, int(torch.randint(0, d, (1,), generator=g))] *= 25.0
    V *= 1.0 + 19.0 * (torch.rand(B, Hkv, T, d // 4, generator=g) < 0.01).repeat_interleave(4, dim=-1).float()
    K, V = K.bfloat16(), V.bfloat16()
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)
    _attend_and_check(q, _queries(B, Hq, d, 3007), K, V, S, br, f"many short ranges d={d} window={window}", window=window,
                      splits=(None, 1, 2, None), min_k_flag=0.01, relative_to_output=True)
    plain = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    _attend_and_check(plain, _queries(B, Hq, d, 3008), K, V, S, br, f"many short ranges, no outliers, d={d}", window=window,
                      splits=(None,), relative_to_output=True)


@pytest.mark.parametrize("T,B", [(640, 1), (20000, 4)])
def test_all_zero_value_rows_keep_their_softmax_weight(T, B):
    """A token whose V row is all zero gets scale 0 under fp16 scales (1e-8 is below fp16's range): it adds nothing
    to the output's numerator but its weight stays in the denominator.  Short range: the per-warp-ring kernel; long
    range with a large batch: the CTA-wide ring kernel."""
    S, br, d, Hq, Hkv = 24, 3, 128, 8, 2
    K = make_kv("randn", (B, Hkv, T, d), seed=1101, dtype=torch.float16)
    V = make_kv("randn", (B, Hkv, T, d), seed=2101, dtype=torch.float16)
    V[:, :, ::3] = 0.0                       # every third token
    V[:, 1, 5:200] = 0.0                     # and a long run in one head
    for q in (hqmq.HQMQ(1, Hkv, S, br, device="cuda"), hqmq.with_outlier_extraction(hqmq.HQMQ(1, Hkv, S, br, device="cuda"), 3.0)):
        Kp, Vp = _attend_and_check(q, _queries(B, Hq, d, 3101, dtype=torch.float16), K, V, S, br, "zero V rows", splits=(None, 3))
        assert (Vp.to_reference()[2][:, :, ::3] == 0).all()
