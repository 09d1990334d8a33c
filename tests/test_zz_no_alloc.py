"""The entry point for hosts that cannot allocate device memory (hqmq_attn_decode_static): a server whose
own pool already holds all of HBM, or a binding with no allocator, still gets decode attention because the
kernel's scratch is a fixed buffer inside the library.  Checked through the C ABI against the ordinary entry
point, twice in a row (the second call finds the first call's leftovers in the shared buffer)."""
import ctypes as C
import math

import pytest
import torch

import hqmq_b200 as hqmq
from hqmq_b200 import _lib

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-3, 1e-3      # the tolerances of the attention parity tests


def _case(B, Hq, Hkv, T, d, S, br, seed, outliers):
    g = torch.Generator().manual_seed(seed)
    q = hqmq.HQMQ(1, Hkv, S, br, device="cuda")
    quant = hqmq.with_outlier_extraction(q, 3.0) if outliers else q
    K = torch.randn(B, Hkv, T, d, generator=g)
    if outliers:
        K[:, :, :, 5] *= 8.0
    V = torch.randn(B, Hkv, T, d, generator=g)
    Kp, Vp = quant.encode(K.bfloat16().cuda(), 0, 0), quant.encode(V.bfloat16().cuda(), 0, 1)
    Q = (torch.randn(B, Hq, 1, d, generator=g) / math.sqrt(d)).bfloat16().cuda()
    return Q, Kp, Vp, q.tables(0, 0, "cuda")["table16"], q.tables(0, 1, "cuda")["table16"]


@pytest.mark.parametrize("outliers", [False, True])
def test_static_scratch_matches_workspace_entry_point(outliers):
    Q, Kp, Vp, tk, tv = _case(2, 16, 4, 1500, 128, 96, 4, seed=3, outliers=outliers)
    ref = torch.empty(Q.shape, dtype=torch.float32, device="cuda")
    hqmq.fused_attention_packed(Q, Kp, Vp, tk, tv, out=ref)
    for call in range(2):
        out = torch.full(Q.shape, float("nan"), dtype=torch.float32, device="cuda")
        hqmq.fused_attention_packed_noalloc(Q, Kp, Vp, tk, tv, out=out)
        torch.cuda.synchronize()
        err = (out - ref).abs().max().item()
        rel = ((out - ref).norm() / ref.norm()).item()
        assert err < MAX_ABS and rel < REL_L2, f"call {call}: max-abs {err:.2e}, rel-L2 {rel:.2e}"
        # the give-up word of the built-in buffer is readable without its address, and says "all rows valid"
        assert _lib.static_status(Q.device) == 0
    # a different shape afterwards reuses the same buffer with other contents in it
    Q2, K2, V2, tk2, tv2 = _case(1, 8, 2, 333, 64, 24, 3, seed=4, outliers=outliers)
    ref2 = torch.empty(Q2.shape, dtype=torch.float32, device="cuda")
    hqmq.fused_attention_packed(Q2, K2, V2, tk2, tv2, out=ref2)
    out2 = torch.empty_like(ref2)
    hqmq.fused_attention_packed_noalloc(Q2, K2, V2, tk2, tv2, out=out2)
    assert (out2 - ref2).abs().max().item() < MAX_ABS


def test_static_scratch_rejects_oversized_problems():
    L = _lib.lib()
    B, Hq, Hkv, T, d = 512, 64, 8, 64, 128
    q = hqmq.HQMQ(1, Hkv, 24, 3, device="cuda")
    Kp = q.new_cache(B, T, d, "cuda")
    Vp = q.new_cache(B, T, d, "cuda")
    Kp.T = Vp.T = T
    Q = torch.zeros(B, Hq, 1, d, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(Q)
    a = _lib.AttnArgs()
    a.struct_size = C.sizeof(_lib.AttnArgs)
    a.layout = 0
    a.q_dtype = a.o_dtype = _lib.dtype_enum(Q.dtype)
    a.Q, a.O = Q.data_ptr(), out.data_ptr()
    a.q_stride = (C.c_int64 * 3)(*Q.stride()[:3])
    a.o_stride = (C.c_int64 * 3)(*out.stride()[:3])
    a.B, a.H_q, a.H_kv, a.T_q, a.T_kv, a.d = B, Hq, Hkv, 1, T, d
    a.r_qmax = 7
    a.K, a.V = Kp.c_struct(), Vp.c_struct()
    tb = q.tables(0, 0, "cuda")["table16"]
    a.table_K = a.table_V = tb.data_ptr()
    need = L.hqmq_attn_workspace_bytes(C.byref(a))
    assert need > _lib.ATTN_STATIC_SCRATCH_BYTES
    rc = L.hqmq_attn_decode_static(C.byref(a), None)
    assert rc == -10 and b"built-in buffer" in L.hqmq_strerror(rc)
    with pytest.raises(_lib.HqmqError):
        hqmq.fused_attention_packed_noalloc(Q, Kp, Vp, tb, tb, out=out)
