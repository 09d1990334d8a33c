"""CPU oracle for the HQMQ hot path (KV-cache encode, packed decode, decode attention).

TEST INFRASTRUCTURE ONLY.  This module restates, in plain PyTorch CPU ops on fp32, the
algorithm of the reference implementation (kswain98/hqmq) for the one path this
repository accelerates.  Nothing in the shipped package imports it: only the test-suite,
the smoke check and the CPU-baseline leg of the benchmark do, and only as the checker.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference itself and
(a) asserts that every function below is bit-identical to the reference on seeded inputs
and (b) writes the reference's outputs as fixtures; ``tests/test_oracle_golden.py`` then
re-checks this module against those fixtures wherever the tests run.

Each function cites the reference lines it follows (paths relative to the reference
repository root).  The reference computes in the dtype it is handed; the parity contract
for this path is "upcast the input to fp32, then bit-exact", so everything here takes
fp32 (``x.float()``) and every step is a single IEEE fp32 operation.
"""
from __future__ import annotations

import math
from itertools import product
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

CHUNK = 4


# --------------------------------------------------------------------------------------
# Codebooks
# --------------------------------------------------------------------------------------
def make_24cell() -> torch.Tensor:
    """The 24 Hurwitz units in the reference's order (src/quantizers/spherical.py:22-43):
    index 2*axis + (sign<0) for the 8 axis points, then 8 + sum_i (sign_i<0) << (3-i) for
    the 16 half-integer points."""
    rows = []
    for axis in range(4):
        for sign in (1.0, -1.0):
            v = [0.0, 0.0, 0.0, 0.0]
            v[axis] = sign
            rows.append(v)
    for signs in product((1.0, -1.0), repeat=4):
        rows.append([0.5 * s for s in signs])
    return torch.tensor(rows, dtype=torch.float32)


def quat_mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Hamilton product, (w, x, y, z) components, evaluated left to right exactly as
    src/quantizers/hqmq.py:33-41."""
    w1, x1, y1, z1 = a.unbind(-1)
    w2, x2, y2, z2 = b.unbind(-1)
    w = w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2
    x = w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2
    y = w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2
    z = w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2
    return torch.stack([w, x, y, z], dim=-1)


def secondary_raw(n_layers: int, n_heads: int, S: int, seed: int = 42) -> torch.Tensor:
    """Raw secondary codebook (n_layers, n_heads, 2, S, 4), init="random"
    (src/quantizers/hqmq.py:90-92,105)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n_layers, n_heads, 2, S, 4, generator=g)


def unit_secondary(raw_hs4: torch.Tensor) -> torch.Tensor:
    """Unit-normalised secondary quaternions (H, S, 4) (src/quantizers/hqmq.py:130-132):
    raw / raw.norm(dim=-1).clamp(min=1e-8), the norm spelled out as in chunk_norms()."""
    raw = raw_hs4.float()
    sq = raw * raw
    ssq = ((sq[..., 0] + sq[..., 1]) + sq[..., 2]) + sq[..., 3]
    nrm = torch.from_numpy(np.sqrt(ssq.contiguous().numpy())).unsqueeze(-1)
    return raw / nrm.clamp(min=1e-8)


def joint_codebook(raw_hs4: torch.Tensor) -> torch.Tensor:
    """Joint table q_p * q_s, shape (H, 24*S, 4), flattened as k = p*S + s
    (src/quantizers/hqmq.py:119-143), fp32."""
    sec = unit_secondary(raw_hs4.float())
    H, S, _ = sec.shape
    prim = make_24cell()
    p_exp = prim.view(1, 24, 1, 4).expand(H, 24, S, 4)
    s_exp = sec.view(H, 1, S, 4).expand(H, 24, S, 4)
    return quat_mul(p_exp, s_exp).reshape(H, 24 * S, 4)


# --------------------------------------------------------------------------------------
# Encoder
# --------------------------------------------------------------------------------------
def chunk_norms(x: torch.Tensor) -> torch.Tensor:
    """Euclidean norm of every 4-element chunk, (B,H,T,d) fp32 -> (B,H,T,d/4) fp32.

    The reference calls ``x_chunked.norm(dim=-1)`` (src/quantizers/hqmq.py:152,
    src/quantizers/outlier_aware.py:60).  On fp32 that is sqrt(((x0^2+x1^2)+x2^2)+x3^2)
    with separate multiplies and adds; it is spelled out here so the result does not
    depend on which vectorised reduction kernel a given CPU selects.  The square root is
    taken with numpy because ``torch.sqrt`` on CPU fp32 tensors is a vectorised
    approximation that is off by one ulp on ~0.7 % of inputs, whereas the reference's
    ``norm`` uses the correctly rounded scalar sqrt."""
    B, H, T, d = x.shape
    xc = x.reshape(B, H, T, d // CHUNK, CHUNK)
    sq = xc * xc
    ssq = ((sq[..., 0] + sq[..., 1]) + sq[..., 2]) + sq[..., 3]
    return torch.from_numpy(np.sqrt(ssq.contiguous().numpy()))


def median_quantile(flat: torch.Tensor) -> torch.Tensor:
    """``torch.quantile(flat, 0.5, dim=-1)`` for fp32 ``flat`` of shape (H, N)
    (src/quantizers/outlier_aware.py:68), restated as sort + the interpolation torch uses:
    pos = 0.5*(N-1), lo = floor(pos), hi = ceil(pos), w = pos - lo,
    result = a + w*(b-a) if w < 0.5 else b - (b-a)*(1-w)."""
    H, N = flat.shape
    srt, _ = torch.sort(flat, dim=-1)
    pos = 0.5 * (N - 1)
    lo, hi = int(math.floor(pos)), int(math.ceil(pos))
    w = torch.tensor(pos - lo, dtype=torch.float32)
    a, b = srt[:, lo], srt[:, hi]
    if float(w) < 0.5:
        return a + w * (b - a)
    return b - (b - a) * (torch.tensor(1.0) - w)


def quantile_torch(flat: torch.Tensor, q: float) -> torch.Tensor:
    """``torch.quantile(flat, q, dim=-1)`` for fp32 ``flat`` of shape (H, N) and any q in [0, 1]
    (src/quantizers/outlier_aware.py:64-66), restated with the arithmetic ATen uses: the rank is the fp32 product
    fl32(q) * fl32(N - 1), the neighbours are its truncation and its ceiling, the weight their fp32 difference, and
    the interpolation is one fused multiply-add: a + w*(b-a) for w < 0.5, else b - (b-a)*(1-w)."""
    H, N = flat.shape
    srt = np.sort(flat.numpy().astype(np.float32), axis=-1)
    rank = np.float32(np.float32(q) * np.float32(N - 1))
    lo, hi = int(rank), int(math.ceil(rank))
    w = np.float32(rank - np.float32(lo))
    a, b = srt[:, lo], srt[:, hi]
    diff = (b - a).astype(np.float32)
    # (the fp32 product w * diff is exact in float64, so one rounding of the float64 sum is the fused result
    #  up to double rounding, which the pin against torch.quantile has not met)
    if abs(float(w)) < 0.5:
        out = a.astype(np.float64) + np.float64(w) * diff.astype(np.float64)
    else:
        out = b.astype(np.float64) - diff.astype(np.float64) * np.float64(np.float32(1.0) - w)
    return torch.from_numpy(out.astype(np.float32))


def med3x_flags(norms: torch.Tensor, C: float, quantile: Optional[float] = None):
    """Per-KV-head threshold and strict outlier flag (src/quantizers/outlier_aware.py:63-72): C times the median
    (threshold_mode="median_mult"), or with ``quantile`` C times that quantile (threshold_mode="fraction" is
    quantile = 1 - outlier_fraction, C = 1).  norms (B,H,T,n) fp32 -> (statistic (H,), thr (H,), flags bool)."""
    B, H, T, n = norms.shape
    flat = norms.permute(1, 0, 2, 3).reshape(H, -1).float()
    med = median_quantile(flat) if quantile is None else quantile_torch(flat, quantile)
    thr = med * C
    flags = norms > thr.view(1, H, 1, 1)
    return med, thr, flags


def encode(x: torch.Tensor, joint: torch.Tensor, radius_bits: int,
           median_mult: Optional[float] = None, t_slice: int = 0, quantile: Optional[float] = None) -> dict:
    """Encoder with the intermediates exposed.

    Follows src/quantizers/hqmq.py:150-152 (norm, clamp), :157-158,164 (direction, einsum
    similarity against the joint table, argmax = first maximal index), :208-211 (per-token
    max over ALL chunks, scale = r_max/qmax, round-half-even, clamp) and, when
    ``median_mult`` is given, src/quantizers/outlier_aware.py:60-72.

    x (B,H,T,d) any float dtype (upcast to fp32); joint (H,24S,4) fp32.
    Returns idx int32, rq int32, r_max fp32 (B,H,T), norms fp32, gap fp32 (best minus
    second-best similarity, for classifying near-ties), and with Med3x: med, thr, flags.
    """
    x = x.float()
    joint = joint.float()
    B, H, T, d = x.shape
    if d % CHUNK:
        raise ValueError(f"d_head={d} not divisible by 4")
    n = d // CHUNK
    qmax = (1 << radius_bits) - 1
    nrm = chunk_norms(x)
    radius = nrm.clamp(min=1e-8)
    xc = x.reshape(B, H, T, n, CHUNK)
    idx = torch.empty(B, H, T, n, dtype=torch.int32)
    gap = torch.empty(B, H, T, n, dtype=torch.float32)
    K = joint.shape[1]
    if t_slice <= 0:
        t_slice = max(1, (1 << 27) // max(1, B * H * n * K))
    for t0 in range(0, T, t_slice):
        t1 = min(T, t0 + t_slice)
        direction = xc[:, :, t0:t1] / radius[:, :, t0:t1].unsqueeze(-1)
        sims = torch.einsum("bhtnc,hkc->bhtnk", direction, joint)
        top2 = sims.topk(2, dim=-1).values
        idx[:, :, t0:t1] = sims.argmax(dim=-1).to(torch.int32)
        gap[:, :, t0:t1] = top2[..., 0] - top2[..., 1]
    r_max = radius.amax(dim=-1).clamp(min=1e-8)
    scale = r_max / qmax
    rq = (radius / scale.unsqueeze(-1)).round().clamp(0, qmax).to(torch.int32)
    out = dict(idx=idx, rq=rq, r_max=r_max, norms=nrm, gap=gap)
    if median_mult is not None:
        med, thr, flags = med3x_flags(nrm, float(median_mult), quantile)
        out.update(med=med, thr=thr, flags=flags)
    return out


def fake_quant(x: torch.Tensor, joint: torch.Tensor, radius_bits: int,
               median_mult: Optional[float] = None, enc: Optional[dict] = None,
               quantile: Optional[float] = None) -> torch.Tensor:
    """What ``quantize_K`` / ``quantize_V`` return for fp32 input: codeword * (rq * scale)
    (src/quantizers/hqmq.py:166-169,210-211,216), and with Med3x the original chunk where
    flagged (src/quantizers/outlier_aware.py:86)."""
    x = x.float()
    B, H, T, d = x.shape
    n = d // CHUNK
    if enc is None:
        enc = encode(x, joint, radius_bits, median_mult, quantile=quantile)
    qmax = (1 << radius_bits) - 1
    cw = gather_codewords(enc["idx"], joint.float())
    scale = enc["r_max"] / qmax
    radius_q = enc["rq"].float() * scale.unsqueeze(-1)
    out = radius_q.unsqueeze(-1) * cw
    if median_mult is not None:
        out = torch.where(enc["flags"].unsqueeze(-1), x.reshape(B, H, T, n, CHUNK), out)
    return out.reshape(B, H, T, d)


# --------------------------------------------------------------------------------------
# Packed decode and attention
# --------------------------------------------------------------------------------------
def gather_codewords(idx: torch.Tensor, joint: torch.Tensor) -> torch.Tensor:
    """joint[h, idx[b,h,t,c], :] -> (B,H,T,n,4)."""
    B, H, T, n = idx.shape
    hh = torch.arange(H).view(1, H, 1, 1).expand(B, H, T, n)
    return joint[hh, idx.long()]


def decode_packed(idx: torch.Tensor, rq: torch.Tensor, rs: torch.Tensor, joint: torch.Tensor,
                  r_qmax: int) -> torch.Tensor:
    """Dense reconstruction of a packed tensor: codeword * ((rq * rs) / r_qmax) in the
    dtype of ``joint`` (src/quantizers/hqmq_attention.py:39-65)."""
    B, H, T, n = idx.shape
    cw = gather_codewords(idx, joint)
    radius = (rq.to(joint.dtype) * rs.unsqueeze(-1)) / r_qmax
    return (cw * radius.unsqueeze(-1)).reshape(B, H, T, n * CHUNK)


def merge_outliers(dense: torch.Tensor, flags: Optional[torch.Tensor],
                   x_orig: Optional[torch.Tensor]) -> torch.Tensor:
    """Replace flagged chunks by their original values
    (src/quantizers/outlier_aware.py:86 applied to the packed decode)."""
    if flags is None:
        return dense
    B, H, T, d = dense.shape
    n = d // CHUNK
    out = torch.where(flags.unsqueeze(-1), x_orig.to(dense.dtype).reshape(B, H, T, n, CHUNK),
                      dense.reshape(B, H, T, n, CHUNK))
    return out.reshape(B, H, T, d)


def attention_dense(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, causal: bool,
                    softmax_scale: Optional[float] = None, window: Optional[int] = None) -> torch.Tensor:
    """GQA attention over dense K/V exactly as src/quantizers/hqmq_attention.py:85-101:
    repeat_interleave the KV heads, scaled_dot_product_attention with a top-left aligned
    causal mask when ``causal``.  ``window`` keeps only the last ``window`` keys."""
    B, Hq, Tq, d = Q.shape
    Hkv = K.shape[1]
    assert Hq % Hkv == 0
    g = Hq // Hkv
    if window is not None and window < K.shape[2]:
        K = K[:, :, -window:]
        V = V[:, :, -window:]
    if g > 1:
        K = K.repeat_interleave(g, dim=1)
        V = V.repeat_interleave(g, dim=1)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    return F.scaled_dot_product_attention(Q, K, V, attn_mask=None, is_causal=causal,
                                          scale=softmax_scale)


def fused_attention(Q, K_idx, K_rq, K_rs, joint_K, V_idx, V_rq, V_rs, joint_V, r_qmax,
                    causal=True, softmax_scale=None, K_flags=None, K_orig=None,
                    V_flags=None, V_orig=None, window=None) -> torch.Tensor:
    """fp32 oracle of the fused attention call (src/quantizers/hqmq_attention.py:68-101),
    extended with the Med3x merge and an optional sliding window.  All float inputs are
    upcast to fp32 first."""
    Kd = decode_packed(K_idx, K_rq, K_rs.float(), joint_K.float(), r_qmax)
    Vd = decode_packed(V_idx, V_rq, V_rs.float(), joint_V.float(), r_qmax)
    Kd = merge_outliers(Kd, K_flags, None if K_orig is None else K_orig.float())
    Vd = merge_outliers(Vd, V_flags, None if V_orig is None else V_orig.float())
    return attention_dense(Q.float(), Kd, Vd, causal, softmax_scale, window)


def combine_partials(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor) -> torch.Tensor:
    """Merge split-KV partial results.  m, l: (n_split, ...) running max and sum of
    exponentials; o: (n_split, ..., d) un-normalised outputs.  Returns (..., d)."""
    m_star = m.amax(dim=0, keepdim=True)
    w = torch.exp(m - m_star)
    l_star = (l * w).sum(0)
    return (o * w.unsqueeze(-1)).sum(0) / l_star.unsqueeze(-1)
