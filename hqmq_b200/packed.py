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
        self._enc_cache = {}      # argument structs of repeated small encode calls (see HQMQQuantizer.encode)
        self._attn_cache = {}        # argument structs and workspaces of repeated attention calls (hqmq_b200.attention)
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
        self._enc_cache.clear()
        self._attn_cache.clear()

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

    # ---- on-disk / wire format -----------------------------------------------------------------------
    # The reference keeps no compressed representation at all; its bit accounting (experiments/18_memory.py:22-35,
    # README.md:77-83: code bits + 16-bit scale per token, with outlier extraction one flag bit per chunk and the
    # original 16-bit values of every flagged chunk) is what a stored cache has to honour.  A file is
    #     magic "HQMQKV1\0" | uint32 header length | JSON header, padded with spaces to a multiple of 16 bytes |
    #     codes [B][H][T][row_bytes] | rs [B][H][T] | flags [B][H][T] (uint16 for d_head <= 64, else uint32) |
    #     out_count [B][H] uint32 | payload: the out_count[b][h] entries of every (b, h) in order, 4 values each
    # i.e. the native planes cut to the T tokens held, so the body is exactly algorithmic_bytes() plus the B*H
    # counters.  Derived data (block offsets, fragment records) is not stored: offsets are rebuilt on load; a loaded
    # cache has no fragment records (attention then merges its outliers from flags and payload).
    MAGIC = b"HQMQKV1\x00"

    def save(self, file, meta: Optional[dict] = None) -> int:
        """Write the T tokens held to ``file`` (a path or a binary file object).  ``meta``: what the planes do not
        know about themselves and a reader needs to rebuild the codebooks (for example {"C": 3.0, "seed": 42,
        "layer": 0, "kv": 0}); it is stored in the header as given.  Returns the number of bytes written."""
        import json
        B, H, T, n = self.B, self.H, self.T, self.n_chunks
        hdr = {"format": 1, "S": self.S, "radius_bits": self.radius_bits, "d_head": 4 * n, "H_kv": H, "B": B, "T": T,
               "row_bytes": self.row_bytes, "scale_dtype": str(self.scale_dtype).replace("torch.", ""),
               "outliers": bool(self.with_outliers), "out_dtype": str(self.out_dtype).replace("torch.", ""),
               "flag_bytes": (2 if n <= 16 else 4) if self.with_outliers else 0, "meta": meta or {}}
        hb = json.dumps(hdr, sort_keys=True).encode()
        hb += b" " * (-(len(self.MAGIC) + 4 + len(hb)) % 16)
        rows = self.codes[:B * H * self.T_cap * self.row_bytes].view(B, H, self.T_cap, self.row_bytes)[:, :, :T]
        rs = self.rs[:B * H * self.T_cap].view(B, H, self.T_cap)[:, :, :T].contiguous().cpu()
        parts = [self.MAGIC, len(hb).to_bytes(4, "little"), hb, rows.contiguous().cpu().numpy().tobytes(),
                 rs.view(torch.int16 if rs.element_size() == 2 else torch.int32).numpy().tobytes()]
        if self.with_outliers:
            fl = self.flags[:B * H * self.T_cap].view(B, H, self.T_cap)[:, :, :T].contiguous().cpu()
            parts.append((fl.to(torch.int16) if n <= 16 else fl).numpy().tobytes())
            cnt = self.out_count.cpu()
            parts.append(cnt.numpy().tobytes())
            vals = self.out_vals[:B * H * self.out_cap * 4].view(B * H, self.out_cap, 4).cpu()
            vbits = vals.view(torch.int16 if vals.element_size() == 2 else torch.int32)
            for bh in range(B * H):
                k = min(int(cnt[bh]), self.out_cap)
                parts.append(vbits[bh, :k].numpy().tobytes())
                if k < int(cnt[bh]):            # entries the side buffer had dropped read as zeros, like everywhere else
                    parts.append(bytes((int(cnt[bh]) - k) * 4 * vals.element_size()))
        blob = b"".join(parts)
        if hasattr(file, "write"):
            file.write(blob)
        else:
            with open(file, "wb") as f:
                f.write(blob)
        return len(blob)

    @classmethod
    def load(cls, file, device, T_cap: Optional[int] = None, out_cap: Optional[int] = None):
        """Read a cache written by ``save`` onto ``device``.  Returns (PackedKV, meta).  ``T_cap`` / ``out_cap``:
        capacities of the new planes (defaults: what the file holds), for a cache that will be appended to."""
        import json
        import numpy as np
        blob = file.read() if hasattr(file, "read") else open(file, "rb").read()
        if blob[:8] != cls.MAGIC:
            raise ValueError("not a packed HQMQ cache (bad magic)")
        hl = int.from_bytes(blob[8:12], "little")
        hdr = json.loads(blob[12:12 + hl].decode())
        if hdr.get("format") != 1:
            raise ValueError(f"unsupported packed-cache format {hdr.get('format')}")
        B, H, T, n = hdr["B"], hdr["H_kv"], hdr["T"], hdr["d_head"] // 4
        sdt, odt = getattr(torch, hdr["scale_dtype"]), getattr(torch, hdr["out_dtype"])
        pos = 12 + hl

        def take(nbytes, np_dtype):
            nonlocal pos
            if pos + nbytes > len(blob):
                raise ValueError("packed-cache file is truncated")
            a = np.frombuffer(blob, dtype=np_dtype, count=nbytes // np.dtype(np_dtype).itemsize, offset=pos)
            pos += nbytes
            return torch.from_numpy(a.copy())

        rows = take(B * H * T * hdr["row_bytes"], np.uint8).view(B, H, T, hdr["row_bytes"])
        sb = 4 if sdt == torch.float32 else 2
        rs = take(B * H * T * sb, np.int16 if sb == 2 else np.int32).view(sdt).view(B, H, T)
        cnt = fl = payload = None
        if hdr["outliers"]:
            fb = hdr["flag_bytes"]
            fl = take(B * H * T * fb, np.uint16 if fb == 2 else np.int32).to(torch.int32).view(B, H, T)
            cnt = take(B * H * 4, np.int32)
            vb = 4 if odt == torch.float32 else 2
            payload = take(int(cnt.sum()) * 4 * vb, np.int16 if vb == 2 else np.int32).view(odt).view(-1, 4)
        if pos != len(blob):
            raise ValueError("packed-cache file has trailing bytes")
        need_cap = int(cnt.max()) if cnt is not None and cnt.numel() else 0
        out = cls(B, H, max(T_cap or T, T, 1), n, hdr["S"], hdr["radius_bits"], device, scale_dtype=sdt,
                  with_outliers=hdr["outliers"], out_dtype=odt, out_cap=max(out_cap or 0, need_cap, 2) if hdr["outliers"] else None)
        if out.row_bytes != hdr["row_bytes"]:
            raise ValueError("row size in the file does not match the geometry in its header")
        dev = out.device
        out.codes[:B * H * out.T_cap * out.row_bytes].view(B, H, out.T_cap, out.row_bytes)[:, :, :T] = rows.to(dev)
        out.rs[:B * H * out.T_cap].view(B, H, out.T_cap)[:, :, :T] = rs.to(dev)
        if hdr["outliers"]:
            fl = fl.to(dev)
            out.flags[:B * H * out.T_cap].view(B, H, out.T_cap)[:, :, :T] = fl
            out.out_count.copy_(cnt.to(dev))
            vals = out.out_vals[:B * H * out.out_cap * 4].view(B * H, out.out_cap, 4)
            o = 0
            for bh in range(B * H):
                k = int(cnt[bh])
                vals[bh, :k] = payload[o:o + k].to(dev)
                o += k
            # entries before every 16-token block: popcount of the flag words, summed per block, scanned
            pc = torch.zeros_like(fl)
            for k in range(32):
                pc += (fl >> k) & 1
            nb = out.T_cap // _lib.OUT_BLOCK
            per_blk = torch.zeros(B * H, nb, dtype=torch.int64, device=dev)
            tb = (T + _lib.OUT_BLOCK - 1) // _lib.OUT_BLOCK
            padded = torch.zeros(B * H, tb * _lib.OUT_BLOCK, dtype=torch.int64, device=dev)
            padded[:, :T] = pc.view(B * H, T)
            per_blk[:, :tb] = padded.view(B * H, tb, _lib.OUT_BLOCK).sum(-1)
            off = torch.zeros(B * H, nb + 1, dtype=torch.int64, device=dev)
            off[:, 1:] = per_blk.cumsum(-1)
            out.out_off.copy_(off.to(torch.int32).view(-1))
        out.T = T
        return out, hdr.get("meta", {})
