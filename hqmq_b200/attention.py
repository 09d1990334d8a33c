"""Fused attention over a compressed KV cache: the host side of hqmq_attn_decode.

``fused_hqmq_attention`` keeps the signature and semantics of the reference's
``fused_hqmq_attention_triton`` (src/quantizers/hqmq_attention.py:425-518): the packed tuple
(idx, radius_q, radius_scale, joint) per K and V, GQA by ``h_kv = h_q // (H_q // H_kv)``,
``softmax_scale`` defaulting to 1/sqrt(d), and a top-left aligned causal mask (query i sees keys
0..i), so a single decode query over a whole cache must be called with ``causal=False``.
The Triton tuning knobs are accepted and ignored.  ``fused_attention_packed`` is the same
operation on the native bit-packed cache.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .packed import PackedKV


def _fill_q(a: _lib.AttnArgs, Q: torch.Tensor, O: Optional[torch.Tensor]):
    a.q_dtype, a.Q = _lib.dtype_enum(Q.dtype), Q.data_ptr()
    a.q_stride = (C.c_int64 * 3)(*Q.stride()[:3])
    a.o_dtype = a.q_dtype
    if O is not None:
        if O.stride(-1) != 1:
            raise _lib.HqmqError("hqmq_b200: the output tensor needs unit stride on the last dim")
        a.o_dtype = _lib.dtype_enum(O.dtype)
        a.O = O.data_ptr()
        a.o_stride = (C.c_int64 * 3)(*O.stride()[:3])


def _run(a: _lib.AttnArgs, device):
    L = _lib.lib()
    with _lib.device_guard(device):
        nbytes = L.hqmq_attn_workspace_bytes(C.byref(a))
        if nbytes == 0:
            # run the validation again to get the error code
            _lib.check(L.hqmq_attn_decode(C.byref(a), None, 0, _lib.stream_ptr()), "hqmq_attn_decode")
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _lib.check(L.hqmq_attn_decode(C.byref(a), ws.data_ptr(), nbytes, _lib.stream_ptr()), "hqmq_attn_decode")
    return ws, nbytes


def fused_hqmq_attention(
    Q: torch.Tensor,
    K_idx: torch.Tensor, K_radius_q: torch.Tensor, K_radius_scale: torch.Tensor, joint_K: torch.Tensor,
    V_idx: torch.Tensor, V_radius_q: torch.Tensor, V_radius_scale: torch.Tensor, joint_V: torch.Tensor,
    r_qmax: int,
    causal: bool = True,
    softmax_scale: Optional[float] = None,
    block_q: Optional[int] = None, block_kv: Optional[int] = None, optimized: bool = True,
    num_warps: Optional[int] = None, num_stages: Optional[int] = None, use_fp8_codebook: bool = False,
    window: Optional[int] = None, kv_splits: Optional[int] = None, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """O (B, H_q, T_q, d) = softmax(scale * Q K^T + mask) V with K, V decoded on the fly from the
    reference's packed tuple.  Indices address ``joint_*`` directly (reference order)."""
    _lib.require_cuda(Q, "fused_attention")
    _lib.check_device(Q.device)
    assert Q.dim() == 4 and K_idx.dim() == 4, "Q is (B,H_q,T_q,d); idx is (B,H_kv,T_kv,n_chunks)"
    B, H_q, T_q, d_h = Q.shape
    H_kv, T_kv, n_chunks = K_idx.shape[1], K_idx.shape[2], K_idx.shape[3]
    assert d_h == n_chunks * 4, f"d_h={d_h} != n_chunks*4={n_chunks * 4}"
    assert H_q % H_kv == 0, f"H_q={H_q} must be divisible by H_kv={H_kv}"
    assert joint_K.shape == joint_V.shape and joint_K.dtype == joint_V.dtype, "joint_K / joint_V must match"
    if Q.stride(-1) != 1:
        Q = Q.contiguous()
    joint_K, joint_V = joint_K.contiguous(), joint_V.contiguous()
    O = out if out is not None else torch.empty_like(Q)
    a = _lib.AttnArgs()
    a.struct_size = C.sizeof(_lib.AttnArgs)
    a.layout = 1
    _fill_q(a, Q, O)
    a.B, a.H_q, a.H_kv, a.T_q, a.T_kv, a.d = B, H_q, H_kv, T_q, T_kv, d_h
    a.r_qmax, a.causal = int(r_qmax), int(bool(causal))
    a.window = int(window) if window else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 0.0
    a.kv_splits = int(kv_splits) if kv_splits else 0
    a.K_ref = _lib.ref_packed(K_idx, K_radius_q, K_radius_scale)
    a.V_ref = _lib.ref_packed(V_idx, V_radius_q, V_radius_scale)
    a.joint_dtype, a.K_size = _lib.dtype_enum(joint_K.dtype), joint_K.shape[1]
    a.joint_K, a.joint_V = joint_K.data_ptr(), joint_V.data_ptr()
    _run(a, Q.device)
    return O


def fused_attention_packed(
    Q: torch.Tensor, K: PackedKV, V: PackedKV, table_K: torch.Tensor, table_V: torch.Tensor,
    causal: bool = False, softmax_scale: Optional[float] = None, window: Optional[int] = None,
    kv_splits: Optional[int] = None, out: Optional[torch.Tensor] = None,
    partials: Optional[torch.Tensor] = None, T_kv: Optional[int] = None,
) -> torch.Tensor:
    """Attention over native caches K, V (``table_*`` = the fp16 native-order tables of the
    quantizer).  With ``partials`` (B, H_q, T_q, d+2) fp32 given, the un-normalised result
    (o[d], m, l) is written there instead of O, for merging across sequence shards."""
    _lib.require_cuda(Q, "fused_attention_packed")
    # A decode loop repeats one call shape on one pair of caches: the argument struct and the workspace of such a call
    # are kept with the K cache (per stream: calls on one stream are ordered, calls on different streams get their
    # own workspace), and a repeat only patches the addresses and the key count.
    st = _lib.stream_ptr()
    T_now = K.T if T_kv is None else T_kv
    key = None
    if Q.stride(-1) == 1 and (out is not None or partials is not None):
        dst = partials if partials is not None else out
        key = (id(V), st, Q.dtype, tuple(Q.shape), Q.stride(), dst.dtype, dst.stride(), partials is not None, causal, window,
               softmax_scale, kv_splits, table_K.data_ptr(), table_V.data_ptr(), K.with_ofrag, V.with_ofrag)
        hit = K._attn_cache.get(key)
        if hit is not None:
            a, ws, _, t_sized, _ = hit
            a.Q, a.T_kv = Q.data_ptr(), T_now
            if partials is not None:
                a.partials = partials.data_ptr()
            else:
                a.O = out.data_ptr()
            L = _lib.lib()
            with _lib.device_guard(Q.device):
                if T_now != t_sized:
                    nbytes = L.hqmq_attn_workspace_bytes(C.byref(a))
                    if nbytes == 0:
                        _lib.check(L.hqmq_attn_decode(C.byref(a), None, 0, st), "hqmq_attn_decode")
                    if nbytes > ws.numel():
                        ws = torch.empty(nbytes, dtype=torch.uint8, device=Q.device)
                    K._attn_cache[key] = (a, ws, nbytes, T_now, hit[4])
                else:
                    nbytes = hit[2]
                _lib.check(L.hqmq_attn_decode(C.byref(a), ws.data_ptr(), nbytes, st), "hqmq_attn_decode")
            return partials if partials is not None else out
    _lib.check_device(Q.device)
    B, H_q, T_q, d_h = Q.shape
    if Q.stride(-1) != 1:
        Q = Q.contiguous()
    O = None
    if partials is None:
        O = out if out is not None else torch.empty_like(Q)
    a = _lib.AttnArgs()
    a.struct_size = C.sizeof(_lib.AttnArgs)
    a.layout = 0
    _fill_q(a, Q, O)
    a.B, a.H_q, a.H_kv, a.T_q, a.d = B, H_q, K.H, T_q, d_h
    a.T_kv = K.T if T_kv is None else T_kv
    a.r_qmax, a.causal = K.qmax, _causal_mode(causal)
    a.window = int(window) if window else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 0.0
    a.kv_splits = int(kv_splits) if kv_splits else 0
    a.K, a.V = K.c_struct(), V.c_struct()
    a.table_K, a.table_V = table_K.data_ptr(), table_V.data_ptr()
    if partials is not None:
        a.partials_only, a.partials = 1, partials.data_ptr()
    ws, nbytes = _run(a, Q.device)
    if key is not None:
        if len(K._attn_cache) > 64:
            K._attn_cache.clear()
        K._attn_cache[key] = (a, ws, nbytes, T_now, (V, table_K, table_V))      # (the last item keeps what the struct points to alive)
    return partials if partials is not None else O


def fused_attention_packed_noalloc(Q: torch.Tensor, K: PackedKV, V: PackedKV, table_K: torch.Tensor,
                                   table_V: torch.Tensor, out: torch.Tensor, causal: bool = False,
                                   softmax_scale: Optional[float] = None, window: Optional[int] = None) -> torch.Tensor:
    """``fused_attention_packed`` for callers that must not allocate device memory while they run (for
    example a server whose memory pool already owns the whole GPU).  ``out`` has to exist already; the
    kernel's scratch is a fixed ``_lib.ATTN_STATIC_SCRATCH_BYTES`` buffer inside the library, shared by all
    calls on the device, so calls must not overlap on the GPU.  Shapes whose scratch would be larger raise
    ``HqmqError``.  The first call on a device resolves the buffer's address: make it during set-up."""
    _lib.require_cuda(Q, "fused_attention_packed_noalloc")
    _lib.check_device(Q.device)
    if Q.stride(-1) != 1:
        raise _lib.HqmqError("hqmq_b200: Q needs unit stride on the last dim (no copy is made here)")
    B, H_q, T_q, d_h = Q.shape
    a = _lib.AttnArgs()
    a.struct_size = C.sizeof(_lib.AttnArgs)
    a.layout = 0
    _fill_q(a, Q, out)
    a.B, a.H_q, a.H_kv, a.T_q, a.d, a.T_kv = B, H_q, K.H, T_q, d_h, K.T
    a.r_qmax, a.causal = K.qmax, _causal_mode(causal)
    a.window = int(window) if window else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 0.0
    a.K, a.V = K.c_struct(), V.c_struct()
    a.table_K, a.table_V = table_K.data_ptr(), table_V.data_ptr()
    with _lib.device_guard(Q.device):
        _lib.check(_lib.lib().hqmq_attn_decode_static(C.byref(a), _lib.stream_ptr()), "hqmq_attn_decode_static")
    return out


def _causal_mode(causal) -> int:
    """False / True (the reference's top-left aligned mask) / "bottom_right" (the queries are the last T_q positions
    of the keys: a prompt chunk attending over a cache that already holds it)."""
    if causal == "bottom_right":
        return 2
    if isinstance(causal, str):
        raise ValueError(f"causal={causal!r}: expected False, True or 'bottom_right'")
    return int(bool(causal))


def combine_partials(parts: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Merge (n_parts, ..., d+2) fp32 partials (o[d], m, l; m in the exp2 domain) into (..., d)."""
    _lib.require_cuda(parts, "combine_partials")
    n_parts, d = parts.shape[0], parts.shape[-1] - 2
    lead = parts.shape[1:-1]
    rows = 1
    for s in lead:
        rows *= s
    p = parts.reshape(n_parts, rows, d + 2).contiguous()      # part-major, as an all_gather leaves it
    out = torch.empty(rows, d, dtype=out_dtype, device=parts.device)
    with torch.cuda.device(parts.device):
        _lib.check(_lib.lib().hqmq_combine_partials(p.data_ptr(), n_parts, rows, d, 1, _lib.dtype_enum(out_dtype),
                                                    out.data_ptr(), _lib.stream_ptr()), "hqmq_combine_partials")
    return out.view(*lead, d)


def decode_dequant(idx: torch.Tensor, radius_q: torch.Tensor, radius_scale: torch.Tensor, joint: torch.Tensor,
                   r_qmax: int) -> torch.Tensor:
    """Dense (B, H, T, d) reconstruction of the reference's packed tuple: codeword * ((rq * rs) / r_qmax)
    in the dtype of ``joint`` (src/quantizers/hqmq_kernel.py:102-132, hqmq_attention.py:39-65)."""
    _lib.require_cuda(idx, "decode_dequant")
    _lib.check_device(idx.device)
    B, H, T, n = idx.shape
    joint = joint.contiguous()
    out_dtype = joint.dtype if joint.dtype == radius_scale.dtype else torch.float32
    out = torch.empty(B, H, T, n * 4, dtype=out_dtype, device=idx.device)
    a = _lib.DequantArgs()
    a.struct_size = C.sizeof(_lib.DequantArgs)
    a.layout = 1
    a.src_ref = _lib.ref_packed(idx, radius_q, radius_scale)
    a.B, a.H, a.T, a.n_chunks = B, H, T, n
    a.r_qmax = int(r_qmax)
    a.joint_dtype, a.joint, a.K = _lib.dtype_enum(joint.dtype), joint.data_ptr(), joint.shape[1]
    a.out_dtype, a.out = _lib.dtype_enum(out_dtype), out.data_ptr()
    with torch.cuda.device(idx.device):
        _lib.check(_lib.lib().hqmq_dequant(C.byref(a), _lib.stream_ptr()), "hqmq_dequant")
    return out


def fused_hqmq_attention_dequant_sdpa(
    Q, K_idx, K_radius_q, K_radius_scale, joint_K, V_idx, V_radius_q, V_radius_scale, joint_V, r_qmax,
    causal: bool = True, softmax_scale: Optional[float] = None,
) -> torch.Tensor:
    """The reference's non-fused path (src/quantizers/hqmq_attention.py:68-101) on the GPU:
    dequantise the whole cache with the CUDA dequant kernel, then library SDPA."""
    import math
    import torch.nn.functional as F
    K = decode_dequant(K_idx, K_radius_q, K_radius_scale, joint_K, r_qmax)
    V = decode_dequant(V_idx, V_radius_q, V_radius_scale, joint_V, r_qmax)
    g = Q.shape[1] // K.shape[1]
    if g > 1:
        K, V = K.repeat_interleave(g, dim=1), V.repeat_interleave(g, dim=1)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(Q.shape[-1])
    return F.scaled_dot_product_attention(Q, K.to(Q.dtype), V.to(Q.dtype), attn_mask=None, is_causal=causal,
                                          scale=softmax_scale)


def encode_joint_fp8(joint: torch.Tensor) -> torch.Tensor:
    """Joint table cast to float8_e4m3fn (src/quantizers/hqmq_attention_hopper.py:43-53).  Kept for
    interface parity; the kernels here gather an fp16 table."""
    return joint.to(torch.float8_e4m3fn)


def hopper_available() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 9


def blackwell_available() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 10
