"""ctypes binding of libhqmq_b200.so (the C ABI declared in include/hqmq_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhqmq_b200.so")

F32, F16, BF16, I32, I16, I8, U8, I64 = range(8)
ABI_VERSION = 4
OUT_BLOCK = 16
OFRAG_BYTES = 528
T_ALIGN = 64
ATTN_STATIC_SCRATCH_BYTES = 16 << 20

_TORCH_TO_ENUM = {
    torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32,
    torch.int16: I16, torch.int8: I8, torch.uint8: U8, torch.int64: I64,
}
_ENUM_TO_TORCH = {v: k for k, v in _TORCH_TO_ENUM.items()}


def dtype_enum(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_ENUM[dt]
    except KeyError:
        raise TypeError(f"hqmq_b200: unsupported dtype {dt}") from None


def torch_dtype(e: int) -> torch.dtype:
    return _ENUM_TO_TORCH[e]


class HqmqError(RuntimeError):
    pass


class Packed(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("B", C.c_int32), ("H", C.c_int32), ("T_cap", C.c_int32),
        ("n_chunks", C.c_int32), ("S", C.c_int32), ("radius_bits", C.c_int32), ("row_bytes", C.c_int32),
        ("scale_dtype", C.c_int32), ("out_dtype", C.c_int32), ("out_cap", C.c_int32), ("ofrag_cap", C.c_int32),
        ("codes", C.c_void_p), ("rs", C.c_void_p), ("flags", C.c_void_p), ("out_vals", C.c_void_p),
        ("out_off", C.c_void_p), ("out_count", C.c_void_p), ("ofrag", C.c_void_p), ("ofrag_off", C.c_void_p),
    ]


class RefPacked(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("idx_dtype", C.c_int32), ("rq_dtype", C.c_int32), ("rs_dtype", C.c_int32),
        ("idx", C.c_void_p), ("rq", C.c_void_p), ("rs", C.c_void_p),
        ("idx_stride", C.c_int64 * 3), ("rq_stride", C.c_int64 * 3), ("rs_stride", C.c_int64 * 2),
    ]


class EncodeArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("x_dtype", C.c_int32), ("x", C.c_void_p), ("x_stride", C.c_int64 * 3),
        ("T_new", C.c_int32), ("t_start", C.c_int32), ("qs", C.c_void_p), ("joint", C.c_void_p),
        ("median_mult", C.c_float), ("search", C.c_int32), ("dst", Packed), ("med_out", C.c_void_p),
        ("lut", C.c_void_p), ("lut_footprint", C.c_int32), ("quantile", C.c_float), ("med_in", C.c_void_p),
    ]


class DequantArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("layout", C.c_int32), ("src_native", Packed), ("src_ref", RefPacked),
        ("B", C.c_int32), ("H", C.c_int32), ("T", C.c_int32), ("n_chunks", C.c_int32), ("t0", C.c_int32),
        ("r_qmax", C.c_int32), ("scale_first", C.c_int32), ("joint_dtype", C.c_int32), ("joint", C.c_void_p),
        ("K", C.c_int32), ("joint_f32", C.c_void_p), ("out_dtype", C.c_int32), ("out", C.c_void_p),
        ("merge_outliers", C.c_int32),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("layout", C.c_int32), ("q_dtype", C.c_int32), ("o_dtype", C.c_int32),
        ("Q", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("O", C.c_void_p), ("o_stride", C.c_int64 * 3),
        ("B", C.c_int32), ("H_q", C.c_int32), ("H_kv", C.c_int32), ("T_q", C.c_int32), ("T_kv", C.c_int32),
        ("d", C.c_int32), ("r_qmax", C.c_int32), ("causal", C.c_int32), ("window", C.c_int32),
        ("softmax_scale", C.c_float), ("kv_splits", C.c_int32), ("partials_only", C.c_int32),
        ("K", Packed), ("V", Packed), ("table_K", C.c_void_p), ("table_V", C.c_void_p),
        ("K_ref", RefPacked), ("V_ref", RefPacked), ("joint_dtype", C.c_int32), ("K_size", C.c_int32),
        ("joint_K", C.c_void_p), ("joint_V", C.c_void_p), ("partials", C.c_void_p),
    ]


EXCHANGE_MAX_RANKS = 16


class Exchange(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("world", C.c_int32), ("rank", C.c_int32), ("reserved", C.c_int32),
        ("block_floats", C.c_int64), ("recv", C.c_void_p * EXCHANGE_MAX_RANKS), ("flags", C.c_void_p * EXCHANGE_MAX_RANKS),
    ]


_lib = None


def lib():
    """The loaded shared library.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise HqmqError(
            f"hqmq_b200: {LIB_PATH} is missing. Build it with `python -m hqmq_b200.build` "
            "(needs nvcc); there is no fallback implementation.")
    L = C.CDLL(LIB_PATH)
    L.hqmq_abi_version.restype = C.c_int
    L.hqmq_strerror.restype = C.c_char_p
    L.hqmq_strerror.argtypes = [C.c_int]
    L.hqmq_device_check.argtypes = [C.c_int]
    L.hqmq_idx_bits.argtypes = [C.c_int]
    L.hqmq_row_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
    L.hqmq_native_index_maps.argtypes = [C.c_void_p, C.c_void_p]
    L.hqmq_codebook_tables.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    L.hqmq_encode_lut_bytes.restype = C.c_size_t
    L.hqmq_encode_lut_bytes.argtypes = [C.c_int, C.c_int]
    L.hqmq_encode_lut_workspace_bytes.restype = C.c_size_t
    L.hqmq_encode_lut_workspace_bytes.argtypes = [C.c_int, C.c_int]
    L.hqmq_encode_lut_build.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                        C.c_void_p]
    L.hqmq_encode_lut_footprint.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_void_p]
    L.hqmq_encode_workspace_bytes.restype = C.c_size_t
    L.hqmq_encode_workspace_bytes.argtypes = [C.POINTER(EncodeArgs)]
    L.hqmq_encode.argtypes = [C.POINTER(EncodeArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    L.hqmq_med3x_state_bytes.restype = C.c_size_t
    L.hqmq_med3x_state_bytes.argtypes = [C.c_int]
    L.hqmq_med3x_hist.argtypes = [C.POINTER(EncodeArgs), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    L.hqmq_med3x_select.argtypes = [C.c_int, C.c_int, C.c_uint64, C.c_float, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    L.hqmq_unpack.argtypes = [C.POINTER(Packed), C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                              C.c_void_p]
    L.hqmq_pack.argtypes = [C.POINTER(RefPacked), C.c_int, C.POINTER(Packed), C.c_int, C.c_void_p]
    L.hqmq_dequant.argtypes = [C.POINTER(DequantArgs), C.c_void_p]
    L.hqmq_attn_workspace_bytes.restype = C.c_size_t
    L.hqmq_attn_workspace_bytes.argtypes = [C.POINTER(AttnArgs)]
    L.hqmq_attn_decode.argtypes = [C.POINTER(AttnArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    L.hqmq_attn_decode_static.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
    L.hqmq_encode_pair_workspace_bytes.argtypes = [C.POINTER(EncodeArgs), C.POINTER(EncodeArgs)]
    L.hqmq_encode_pair_workspace_bytes.restype = C.c_size_t
    L.hqmq_encode_pair.argtypes = [C.POINTER(EncodeArgs), C.POINTER(EncodeArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    L.hqmq_encode_pair.restype = C.c_int
    L.hqmq_exchange_step.argtypes = [C.POINTER(Exchange), C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_int64,
                                     C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    L.hqmq_exchange_step.restype = C.c_int
    L.hqmq_attn_static_status.argtypes = [C.POINTER(C.c_uint32), C.c_void_p]
    L.hqmq_exchange_recv_bytes.restype = C.c_size_t
    L.hqmq_exchange_recv_bytes.argtypes = [C.c_int, C.c_int64]
    L.hqmq_exchange_flag_bytes.restype = C.c_size_t
    L.hqmq_exchange_flag_bytes.argtypes = [C.c_int]
    L.hqmq_exchange_enable_peer.argtypes = [C.c_int]
    L.hqmq_exchange_verify.argtypes = [C.POINTER(Exchange)]
    L.hqmq_exchange_ipc_export.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    L.hqmq_exchange_ipc_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    L.hqmq_exchange_ipc_close.argtypes = [C.c_void_p]
    L.hqmq_exchange_push.argtypes = [C.POINTER(Exchange), C.c_void_p, C.c_uint32, C.c_void_p]
    L.hqmq_exchange_wait.argtypes = [C.POINTER(Exchange), C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    L.hqmq_read_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_void_p]
    L.hqmq_combine_partials.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    if L.hqmq_abi_version() != ABI_VERSION:
        raise HqmqError("hqmq_b200: library ABI version mismatch; rebuild with `python -m hqmq_b200.build --force`")
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise HqmqError(f"hqmq_b200: {what} failed: {lib().hqmq_strerror(rc).decode()} ({rc})")


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise HqmqError(f"hqmq_b200: {what} needs CUDA tensors (got device {t.device}); this package has no CPU path")


_checked_devices = set()


def check_device(device: torch.device) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _checked_devices:
        return
    check(lib().hqmq_device_check(idx), f"device check of cuda:{idx}")
    _checked_devices.add(idx)


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(device: torch.device):
    """torch.cuda.device(device), or nothing when that device is already current (saves the switch on the
    decode-time hot path)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """cudaStream_t of torch's current stream on the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def read_status(workspace: torch.Tensor) -> int:
    """First word of a workspace after synchronising the current stream (see hqmq_read_status)."""
    st = C.c_uint32(0)
    with torch.cuda.device(workspace.device):
        check(lib().hqmq_read_status(workspace.data_ptr(), C.byref(st), stream_ptr()), "hqmq_read_status")
    return int(st.value)


def static_status(device) -> int:
    """Give-up word of the last ``hqmq_attn_decode_static`` call on ``device`` (0: every output row is valid), read
    after synchronising the current stream (see hqmq_attn_static_status)."""
    st = C.c_uint32(0)
    with device_guard(torch.device(device)):
        check(lib().hqmq_attn_static_status(C.byref(st), stream_ptr()), "hqmq_attn_static_status")
    return st.value


def ref_packed(idx: torch.Tensor, rq: torch.Tensor, rs: torch.Tensor) -> RefPacked:
    """Descriptor of the reference's packed tuple; last dims must be contiguous."""
    if idx.stride(-1) != 1 or rq.stride(-1) != 1 or rs.stride(-1) != 1:
        raise HqmqError("hqmq_b200: idx / radius_q / radius_scale need unit stride on the last dim")
    r = RefPacked()
    r.struct_size = C.sizeof(RefPacked)
    r.idx_dtype, r.rq_dtype, r.rs_dtype = dtype_enum(idx.dtype), dtype_enum(rq.dtype), dtype_enum(rs.dtype)
    r.idx, r.rq, r.rs = idx.data_ptr(), rq.data_ptr(), rs.data_ptr()
    r.idx_stride = (C.c_int64 * 3)(*idx.stride()[:3])
    r.rq_stride = (C.c_int64 * 3)(*rq.stride()[:3])
    r.rs_stride = (C.c_int64 * 2)(*rs.stride()[:2])
    return r


def index_maps():
    a = (C.c_uint8 * 24)()
    b = (C.c_uint8 * 24)()
    check(lib().hqmq_native_index_maps(a, b), "hqmq_native_index_maps")
    return list(a), list(b)
