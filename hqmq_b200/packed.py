"""The native compressed representation of one K or V tensor and its device buffers.

The reference has no compressed in-memory format (its packed tuple is int32 indices, integer
radius codes and a per-token scale: src/quantizers/hqmq_attention.py:11-18).  ``PackedKV`` owns
the planes described in include/hqmq_b200.h and converts to and from the reference tuple.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib


def idx_bits(S: int) -> int:
    return max(0, math.ceil(math.log2(24 * S)))


def row_bytes(n_chunks: int, S: int, radius_bits: int) -> int:
    bits = n_chunks * (idx_bits(S) + radius_bits)
    return ((bits + 31) // 32) * 4


class PackedKV:
    """Bit-packed cache planes for one tensor of shape (B, H, T<=T_cap, 4*n_chunks)."""

    def __init__(self, B: int, H: int, T_cap: int, n_chunks: int, S: int, radius_bits: int, device,
                 scale_dtype: torch.dtype = torch.bfloat16, with_outliers: bool = False,
                 out_dtype: torch.dtype = torch.bfloat16, out_cap: Optional[int] = None,
                 ofrag: bool = False, ofrag_cap: Optional[int] = None):
        if n_chunks < 1 or n_chunks > 32:
            raise ValueError(f"n_chunks={n_chunks}: the native layout supports d_head <= 128")
        self.B, self.H, self.n_chunks, self.S, self.radius_bits = B, H, n_chunks, S, radius_bits
        self.T_cap = max(_lib.T_ALIGN, ((T_cap + _lib.T_ALIGN - 1) // _lib.T_ALIGN) * _lib.T_ALIGN)
        self.T = 0
        self.row_bytes = row_bytes(n_chunks, S, radius_bits)
        self.scale_dtype, self.out_dtype = scale_dtype, out_dtype
        dev = torch.device(device)
        rows = B * H * self.T_cap
        # 64 bytes of slack so that whole-word reads near the end of the last row stay in bounds
        self.codes = torch.zeros(rows * self.row_bytes + 64, dtype=torch.uint8, device=dev)
        self.rs = torch.zeros(rows + 8, dtype=scale_dtype, device=dev)
        self.with_outliers = with_outliers
        if with_outliers:
            self.out_cap = (int(out_cap) + 1) & ~1 if out_cap is not None else self.T_cap * n_chunks
            self.flags = torch.zeros(rows + 4, dtype=torch.int32, device=dev)
            self.out_vals = torch.zeros(B * H * self.out_cap * 4 + 8, dtype=out_dtype, device=dev)
            self.out_off = torch.zeros(B * H * (self.T_cap // _lib.OUT_BLOCK + 1), dtype=torch.int32, device=dev)
            self.out_count = torch.zeros(B * H, dtype=torch.int32, device=dev)
        else:
            self.out_cap = 0
            self.flags = self.out_vals = self.out_off = self.out_count = None
        # optional fragment records (see include/hqmq_b200.h): by default room for one record per block
        self.with_ofrag = bool(ofrag) and with_outliers
        if self.with_ofrag:
            self.ofrag_cap = int(ofrag_cap) if ofrag_cap is not None else self.T_cap // _lib.OUT_BLOCK
            self.ofrag = torch.zeros(B * H * self.ofrag_cap * _lib.OFRAG_BYTES + 16, dtype=torch.uint8, device=dev)
            self.ofrag_off = torch.zeros(B * H * (self.T_cap // _lib.OUT_BLOCK + 1), dtype=torch.int32, device=dev)
        else:
            self.ofrag_cap = 0
            self.ofrag = self.ofrag_off = None

    @property
    def device(self):
        return self.codes.device

    @property
    def qmax(self) -> int:
        return (1 << self.radius_bits) - 1

    def c_struct(self) -> _lib.Packed:
        p = _lib.Packed()
        p.struct_size = C.sizeof(_lib.Packed)
        p.B, p.H, p.T_cap, p.n_chunks = self.B, self.H, self.T_cap, self.n_chunks
        p.S, p.radius_bits, p.row_bytes = self.S, self.radius_bits, self.row_bytes
        p.scale_dtype = _lib.dtype_enum(self.scale_dtype)
        p.out_dtype = _lib.dtype_enum(self.out_dtype)
        p.out_cap = self.out_cap
        p.codes, p.rs = self.codes.data_ptr(), self.rs.data_ptr()
        if self.with_outliers:
            p.flags, p.out_vals = self.flags.data_ptr(), self.out_vals.data_ptr()
            p.out_off, p.out_count = self.out_off.data_ptr(), self.out_count.data_ptr()
        if self.with_ofrag:
            p.ofrag_cap = self.ofrag_cap
            p.ofrag, p.ofrag_off = self.ofrag.data_ptr(), self.ofrag_off.data_ptr()
        return p

    def drop_ofrag(self) -> None:
        """Forget the fragment records: attention then merges K outliers from flags / out_vals."""
        self.with_ofrag, self.ofrag_cap, self.ofrag, self.ofrag_off = False, 0, None, None

    # ---- accounting -------------------------------------------------------------------------
    def n_outliers(self) -> int:
        """Flagged chunks stored so far (reads a device counter: synchronises)."""
        return int(self.out_count.sum().item()) if self.with_outliers else 0

    def algorithmic_bytes(self, T: Optional[int] = None, n_out: Optional[int] = None) -> int:
        """Bytes a decode step must read for T tokens of this tensor: code rows, per-token scale,
        and with outlier extraction the flag words and 4 original values per flagged chunk."""
        T = self.T if T is None else T
        scale_b = 4 if self.scale_dtype == torch.float32 else 2
        per_tok = self.n_chunks * (idx_bits(self.S) + self.radius_bits) / 8 + scale_b
        total = self.B * self.H * T * per_tok
        if self.with_outliers:
            n_out = self.n_outliers() if n_out is None else n_out
            val_b = 4 if self.out_dtype == torch.float32 else 2
            total += self.B * self.H * T * self.n_chunks / 8 + n_out * 4 * val_b
        return int(total)

    # ---- conversion ----------------------------------------------------------------------------
    def to_reference(self, t0: int = 0, T: Optional[int] = None):
        """(idx int32, rq int32, rs fp32, flags bool or None) for tokens [t0, t0+T), indices in the
        reference's k = p*S + s order."""
        T = self.T - t0 if T is None else T
        dev = self.device
        shape = (self.B, self.H, T, self.n_chunks)
        idx = torch.empty(shape, dtype=torch.int32, device=dev)
        rq = torch.empty(shape, dtype=torch.int32, device=dev)
        rs = torch.empty(shape[:3], dtype=torch.float32, device=dev)
        flags = torch.empty(shape, dtype=torch.uint8, device=dev) if self.with_outliers else None
        p = self.c_struct()
        _lib.check(_lib.lib().hqmq_unpack(C.byref(p), t0, T, idx.data_ptr(), rq.data_ptr(), rs.data_ptr(),
                                          flags.data_ptr() if flags is not None else None, _lib.stream_ptr()),
                   "hqmq_unpack")
        return idx, rq, rs, (flags.bool() if flags is not None else None)

    @classmethod
    def from_reference(cls, idx: torch.Tensor, rq: torch.Tensor, rs: torch.Tensor, S: int, radius_bits: int,
                       scale_dtype: Optional[torch.dtype] = None, T_cap: Optional[int] = None) -> "PackedKV":
        """Pack the reference tuple (indices in reference order) into native planes."""
        _lib.require_cuda(idx, "PackedKV.from_reference")
        B, H, T, n = idx.shape
        if scale_dtype is None:
            scale_dtype = rs.dtype if rs.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
        out = cls(B, H, T_cap or T, n, S, radius_bits, idx.device, scale_dtype=scale_dtype)
        src = _lib.ref_packed(idx, rq, rs)
        p = out.c_struct()
        _lib.check(_lib.lib().hqmq_pack(C.byref(src), T, C.byref(p), 0, _lib.stream_ptr()), "hqmq_pack")
        out.T = T
        return out
