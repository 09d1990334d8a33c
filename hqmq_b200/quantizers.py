"""Host-side mirror of the reference's quantizer plugin interface for the HQMQ path.

Same class names, constructor arguments, attributes and error behaviour as
src/quantizers/base.py:17-34 (KVQuantizer), src/quantizers/hqmq.py:44-278 (HQMQQuantizer),
src/quantizers/outlier_aware.py:28-114 (OutlierAwareHQMQQuantizer),
src/quantizers/outlier_generic.py (OutlierAwareGenericQuantizer) and
src/quantizers/hqmq_padded.py:19-86 (PaddedHQMQQuantizer).  The arithmetic runs in the CUDA
library; the reference only ever returns a dense fake-quantised tensor, so ``encode`` /
``decode`` (which expose the compressed representation) are additions.
"""
from __future__ import annotations

import ctypes as C
import math
from abc import ABC, abstractmethod
from itertools import product
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from .packed import PackedKV


class KVQuantizer(ABC):
    """Plugin interface: quantize_K / quantize_V take and return (B, n_kv_heads, T_new, d_head)."""

    @abstractmethod
    def quantize_K(self, k: torch.Tensor, layer_idx: int) -> torch.Tensor: ...

    @abstractmethod
    def quantize_V(self, v: torch.Tensor, layer_idx: int) -> torch.Tensor: ...

    @abstractmethod
    def bits_per_value(self) -> float: ...

    @property
    def name(self) -> str:
        return type(self).__name__


def hurwitz_units() -> torch.Tensor:
    """The 24-cell vertices in the reference's order: +-e_i (index 2*i + [sign<0]) then the 16
    points (+-1/2)^4 (index 8 + sum_i [sign_i<0] << (3-i))."""
    pts = []
    for i in range(4):
        for sgn in (1.0, -1.0):
            pts.append([sgn if j == i else 0.0 for j in range(4)])
    pts += [[0.5 * s for s in signs] for signs in product((1.0, -1.0), repeat=4)]
    return torch.tensor(pts, dtype=torch.float32)


def quat_mul(q1: torch.Tensor, q2: torch.Tensor) -> torch.Tensor:
    """Hamilton product of (..., 4) tensors in (w, x, y, z) order."""
    a, b, c, d = q1.unbind(-1)
    e, f, g, h = q2.unbind(-1)
    return torch.stack([a * e - b * f - c * g - d * h,
                        a * f + b * e + c * h - d * g,
                        a * g - b * h + c * e + d * f,
                        a * h + b * g - c * f + d * e], dim=-1)


def _norm4(v: torch.Tensor) -> torch.Tensor:
    # sqrt(((v0^2+v1^2)+v2^2)+v3^2) with a correctly rounded square root (computed in float64 and
    # rounded once), independent of which vectorised kernel the host CPU would pick for norm().
    sq = v * v
    ssq = ((sq[..., 0] + sq[..., 1]) + sq[..., 2]) + sq[..., 3]
    return ssq.double().sqrt().float()


class HQMQQuantizer(KVQuantizer):
    """Hurwitz quaternion multiplicative quantizer; direction of each 4-chunk = q_p * q_s."""

    def __init__(self, n_layers: int, n_heads: int, secondary_size: int = 24, radius_bits: int = 4,
                 jl_dim: int = 0, magnitude_mode: str = "unit", robust_radius_scale: bool = False,
                 log_radius: bool = False, device: str = "cuda", init: str = "random", seed: int = 42):
        self.chunk_dim = 4
        self.n_layers, self.n_heads = n_layers, n_heads
        self.secondary_size, self.radius_bits = secondary_size, radius_bits
        self.jl_dim, self.magnitude_mode = jl_dim, magnitude_mode
        self.robust_radius_scale, self.log_radius = robust_radius_scale, log_radius
        if magnitude_mode not in ("unit", "free"):
            raise ValueError(f"magnitude_mode={magnitude_mode}")
        self.training = False
        self.tau = 1.0
        self._primary = hurwitz_units()
        g = torch.Generator().manual_seed(seed)
        if init == "random":
            raw = torch.randn(n_layers, n_heads, 2, secondary_size, 4, generator=g)
        elif init == "hurwitz_perturbed":
            base = self._primary
            if secondary_size <= 24:
                base = base[:secondary_size]
            else:
                base = base.repeat((secondary_size + 23) // 24, 1)[:secondary_size]
            raw = base.view(1, 1, 1, secondary_size, 4).expand(n_layers, n_heads, 2, secondary_size, 4).clone()
            raw = raw + 0.1 * torch.randn_like(raw)
        else:
            raise ValueError(init)
        self.secondary_raw = nn.Parameter(raw.to(device=device, dtype=torch.float32))
        self._tables: dict = {}

    # ---- reference plumbing ---------------------------------------------------------------
    def trainable_parameters(self):
        return [self.secondary_raw]

    def set_training(self, training: bool, tau: Optional[float] = None):
        self.training = training
        if tau is not None:
            self.tau = tau

    def _refresh_rotations(self):
        self._tables.clear()

    def _unsupported(self) -> Optional[str]:
        if self.magnitude_mode != "unit":
            return "magnitude_mode='free'"
        if self.jl_dim:
            return "jl_dim > 0"
        if self.log_radius:
            return "log_radius"
        if self.robust_radius_scale:
            return "robust_radius_scale"
        if self.training:
            return "training (soft codebook)"
        if not 1 <= self.radius_bits <= 8:
            return f"radius_bits={self.radius_bits}"
        return None

    # ---- codebooks -------------------------------------------------------------------------------
    def _codebook_fp32(self, layer_idx: int, kv: int):
        """(unit secondaries (H,S,4), joint (H,24S,4)) in fp32, computed on the host with single IEEE
        operations (same operation order as src/quantizers/hqmq.py:119-143) so that the tables do
        not depend on a device's reduction order."""
        raw = self.secondary_raw.detach()[layer_idx, :, kv].to("cpu", torch.float32)
        sec = raw / _norm4(raw).unsqueeze(-1).clamp(min=1e-8)
        H, S, _ = sec.shape
        p = self._primary.view(1, 24, 1, 4).expand(H, 24, S, 4)
        s = sec.view(H, 1, S, 4).expand(H, 24, S, 4)
        return sec.contiguous(), quat_mul(p, s).reshape(H, 24 * S, 4).contiguous()

    def _get_codebook(self, layer_idx: int, kv: int, ref: torch.Tensor) -> torch.Tensor:
        """Joint table (H, 24*S, 4), k = p*S + s, on ref's device in ref's dtype."""
        return self.tables(layer_idx, kv, ref.device)["joint"].to(ref.dtype)

    def tables(self, layer_idx: int, kv: int, device) -> dict:
        """Device tables for one (layer, K|V): 'qs' (H,S,4) fp32, 'joint' (H,24S,4) fp32 in the
        reference's order, 'table16' (H,24S,4) fp16 in the native index order."""
        device = torch.device(device)
        key = (layer_idx, kv, device)
        t = self._tables.get(key)
        if t is None:
            qs, joint = self._codebook_fp32(layer_idx, kv)
            t = {"qs": qs.to(device), "joint": joint.to(device)}
            if device.type == "cuda":
                _lib.check_device(device)
                H, S = self.n_heads, self.secondary_size
                t16 = torch.empty(H, 24 * S, 4, dtype=torch.float16, device=device)
                with torch.cuda.device(device):
                    _lib.check(_lib.lib().hqmq_codebook_tables(t["joint"].data_ptr(), H, S, t16.data_ptr(),
                                                               _lib.stream_ptr()), "hqmq_codebook_tables")
                t["table16"] = t16
                # nearest-codeword look-up table for the encoder
                L = _lib.lib()
                lut = torch.empty(L.hqmq_encode_lut_bytes(H, S), dtype=torch.uint8, device=device)
                ws = torch.empty(L.hqmq_encode_lut_workspace_bytes(H, S), dtype=torch.uint8, device=device)
                mc = C.c_int(0)
                with torch.cuda.device(device):
                    _lib.check(L.hqmq_encode_lut_build(t["joint"].data_ptr(), H, S, lut.data_ptr(), lut.numel(),
                                                       ws.data_ptr(), ws.numel(), _lib.stream_ptr()), "hqmq_encode_lut_build")
                    _lib.check(L.hqmq_encode_lut_footprint(lut.data_ptr(), H, C.byref(mc), _lib.stream_ptr()),
                               "hqmq_encode_lut_footprint")
                t["lut"], t["lut_footprint"] = lut, mc.value
            self._tables[key] = t
        return t

    # ---- compressed representation ---------------------------------------------------------------
    def new_cache(self, B: int, T_cap: int, d_head: int, device, scale_dtype=torch.bfloat16,
                  with_outliers: bool = False, out_dtype=torch.bfloat16, out_cap: Optional[int] = None,
                  ofrag: bool = False, ofrag_cap: Optional[int] = None) -> PackedKV:
        if d_head % 4 != 0:
            raise ValueError(f"d_head={d_head} not divisible by 4")
        return PackedKV(B, self.n_heads, T_cap, d_head // 4, self.secondary_size, self.radius_bits, device,
                        scale_dtype=scale_dtype, with_outliers=with_outliers, out_dtype=out_dtype, out_cap=out_cap,
                        ofrag=ofrag, ofrag_cap=ofrag_cap)

    def _check_dst(self, x: torch.Tensor, out: PackedKV):
        """The library takes batch, heads and chunks per token from the destination planes: x must have that geometry."""
        B, H, _, d = x.shape
        if (B, H, d // 4) != (out.B, out.H, out.n_chunks) or d % 4:
            raise ValueError(f"x of shape {tuple(x.shape)} does not match the destination cache "
                             f"(B={out.B}, H={out.H}, d_head={out.n_chunks * 4})")
        if out.S != self.secondary_size or out.radius_bits != self.radius_bits:
            raise ValueError(f"destination cache is s{out.S}_r{out.radius_bits}, quantizer is "
                             f"s{self.secondary_size}_r{self.radius_bits}")
        if out.device != x.device:
            raise ValueError(f"x is on {x.device}, the destination cache on {out.device}")

    def _enc_args(self, x, layer_idx, kv, out, median_mult=None, search=0, med_out=None, med_in=None, quantile=None):
        """The hqmq_encode_args of one call (x already validated and laid out, ``out`` the destination cache)."""
        tb = self.tables(layer_idx, kv, x.device)
        B, H, T, d = x.shape
        a = _lib.EncodeArgs()
        a.struct_size = C.sizeof(_lib.EncodeArgs)
        a.x_dtype, a.x = _lib.dtype_enum(x.dtype), x.data_ptr()
        a.x_stride = (C.c_int64 * 3)(*x.stride()[:3])
        a.T_new, a.t_start = T, out.T
        a.qs, a.joint = tb["qs"].data_ptr(), tb["joint"].data_ptr()
        a.median_mult = float(median_mult) if median_mult is not None else 0.0
        a.quantile = float(quantile) if quantile is not None else 0.0      # 0: the median
        a.search = search
        a.dst = out.c_struct()
        a.med_out = med_out.data_ptr() if med_out is not None else None
        if med_in is not None:
            if median_mult is None:
                raise ValueError("med_in needs a median multiplier (Med3x encode)")
            if med_in.dtype != torch.float32 or med_in.numel() != H or med_in.device != x.device or not med_in.is_contiguous():
                raise ValueError("med_in must be a contiguous (H,) fp32 tensor on the device of x")
            a.med_in = med_in.data_ptr()
        a.lut, a.lut_footprint = tb["lut"].data_ptr(), tb["lut_footprint"]
        a._keep = (x, tb, out, med_out, med_in)     # the struct holds raw addresses: keep their owners alive with it
        return a

    def encode(self, x: torch.Tensor, layer_idx: int, kv: int, out: Optional[PackedKV] = None,
               median_mult: Optional[float] = None, scale_dtype: Optional[torch.dtype] = None,
               search: int = 0, med_out: Optional[torch.Tensor] = None, ofrag: Optional[bool] = None,
               check_status: bool = False, med_in: Optional[torch.Tensor] = None,
               quantile: Optional[float] = None) -> PackedKV:
        """Encode x (B, H, T_new, d) and append it to ``out`` (a fresh cache when None).

        ``ofrag``: also keep the flagged chunks of every complete 16-token block as tensor-core operand
        records for the decode-attention kernel (K tensors only use them).  Default: on for a fresh K
        cache with Med3x, off otherwise.  ``check_status``: synchronise and raise if the outlier side buffer
        overflowed (otherwise the caller may compare ``out_count`` with ``out_cap`` itself).  ``quantile``: flag
        against ``median_mult`` times ``torch.quantile(norms, quantile)`` per head instead of the median (the
        reference wrapper's "fraction" mode: quantile = 1 - fraction, median_mult = 1).  ``med_in``: (H,) fp32
        medians to flag against instead of this call's own (``hqmq_b200.dist.split_batch_median`` computes them
        when the batch entries of a head are spread over several GPUs)."""
        # Decode-time appends repeat one small call shape on one cache: the argument struct and the workspace of
        # such a call are kept with the cache, and a repeat only patches the input address and the write position
        # (calls on one cache are ordered on a stream anyway, since they append to the same planes).
        fast_key = None
        if out is not None and med_out is None and med_in is None and not check_status and x.dim() == 4 and x.shape[2] <= 64:
            fast_key = (id(self), layer_idx, kv, tuple(x.shape), x.dtype, x.stride(), median_mult, search, quantile)
            hit = out._enc_cache.get(fast_key)
            if hit is not None:
                a, ws, nbytes = hit
                T = x.shape[2]
                if out.T + T > out.T_cap:
                    raise _lib.HqmqError(f"hqmq_b200: cache capacity {out.T_cap} exceeded ({out.T} + {T})")
                a.x, a.t_start = x.data_ptr(), out.T
                with _lib.device_guard(x.device):
                    _lib.check(_lib.lib().hqmq_encode(C.byref(a), ws.data_ptr(), nbytes, _lib.stream_ptr()), "hqmq_encode")
                out.T += T
                return out
        why = self._unsupported()
        if why:
            raise NotImplementedError(f"hqmq_b200 accelerates the unit-magnitude linear-radius path only ({why})")
        _lib.require_cuda(x, "HQMQQuantizer.encode")
        _lib.check_device(x.device)
        B, H, T, d = x.shape
        if d % 4 != 0:
            raise ValueError(f"d_head={d} not divisible by 4")
        if H != self.n_heads:
            raise ValueError(f"x has {H} heads, quantizer has {self.n_heads}")
        x_given = x
        if x.stride(-1) != 1 or any(s % 4 for s in x.stride()[:3]):
            x = x.contiguous()
        if out is None:
            sd = scale_dtype or (x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.float32)
            od = x.dtype
            if ofrag is None:
                ofrag = kv == 0 and median_mult is not None
            out = self.new_cache(B, T, d, x.device, scale_dtype=sd, with_outliers=median_mult is not None,
                                 out_dtype=od, ofrag=bool(ofrag) and median_mult is not None)
        self._check_dst(x, out)
        if median_mult is not None and not out.with_outliers:
            raise ValueError("destination cache was created without outlier planes")
        if out.T + T > out.T_cap:
            raise _lib.HqmqError(f"hqmq_b200: cache capacity {out.T_cap} exceeded ({out.T} + {T})")
        if T == 0:              # appending nothing leaves the cache as it is (an empty tensor has no address to pass)
            return out
        a = self._enc_args(x, layer_idx, kv, out, median_mult, search, med_out, med_in, quantile)
        L = _lib.lib()
        with _lib.device_guard(x.device):
            nbytes = L.hqmq_encode_workspace_bytes(C.byref(a))
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
            _lib.check(L.hqmq_encode(C.byref(a), ws.data_ptr(), nbytes, _lib.stream_ptr()), "hqmq_encode")
            if check_status and nbytes and (_lib.read_status(ws) & 1):
                raise _lib.HqmqError(f"hqmq_b200: outlier side buffer too small (out_cap={out.out_cap} chunks per (b, h))")
        if fast_key is not None and x is x_given:
            a._keep = (a._keep[1], out)          # the tables and the planes, not the input tensor of this call
            out._enc_cache[fast_key] = (a, ws, nbytes)
        out.T += T
        return out

    def encode_pair(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int, out_k: PackedKV, out_v: PackedKV,
                    median_mult: Optional[float] = None, quantile: Optional[float] = None) -> Tuple[PackedKV, PackedKV]:
        """Append the keys and the values of one layer (the reference cache quantises both on every update,
        src/model_utils.py:29-32).  Same result as ``encode(k, layer_idx, 0, out=out_k)`` followed by
        ``encode(v, layer_idx, 1, out=out_v)``; a decode-time append (a few tokens per sequence) runs both tensors
        in one kernel launch (hqmq_encode_pair) instead of three per tensor."""
        small = (k.dim() == 4 and k.shape == v.shape and k.dtype == v.dtype and k.shape[2] <= 64 and k.is_cuda and v.is_cuda
                 and k.stride(-1) == 1 and v.stride(-1) == 1 and not any(s % 4 for s in k.stride()[:3] + v.stride()[:3]))
        if not small or k.shape[2] == 0:
            return (self.encode(k, layer_idx, 0, out=out_k, median_mult=median_mult, quantile=quantile),
                    self.encode(v, layer_idx, 1, out=out_v, median_mult=median_mult, quantile=quantile))
        T = k.shape[2]
        key = ("pair", id(self), id(out_v), layer_idx, tuple(k.shape), k.dtype, k.stride(), v.stride(), median_mult, quantile)
        hit = out_k._enc_cache.get(key)
        if hit is None:
            why = self._unsupported()
            if why:
                raise NotImplementedError(f"hqmq_b200 accelerates the unit-magnitude linear-radius path only ({why})")
            _lib.check_device(k.device)
            if k.shape[1] != self.n_heads:
                raise ValueError(f"x has {k.shape[1]} heads, quantizer has {self.n_heads}")
            for x, out in ((k, out_k), (v, out_v)):
                self._check_dst(x, out)
                if median_mult is not None and not out.with_outliers:
                    raise ValueError("destination cache was created without outlier planes")
            ak = self._enc_args(k, layer_idx, 0, out_k, median_mult, quantile=quantile)
            av = self._enc_args(v, layer_idx, 1, out_v, median_mult, quantile=quantile)
            with _lib.device_guard(k.device):
                nbytes = _lib.lib().hqmq_encode_pair_workspace_bytes(C.byref(ak), C.byref(av))
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=k.device)
            ak._keep, av._keep = (ak._keep[1], out_k), (av._keep[1], out_v)     # tables and planes, not this call's inputs
            hit = out_k._enc_cache[key] = (ak, av, ws, nbytes)
        ak, av, ws, nbytes = hit
        if out_k.T + T > out_k.T_cap or out_v.T + T > out_v.T_cap:
            raise _lib.HqmqError(f"hqmq_b200: cache capacity {out_k.T_cap} exceeded ({out_k.T} + {T})")
        ak.x, ak.t_start, av.x, av.t_start = k.data_ptr(), out_k.T, v.data_ptr(), out_v.T
        with _lib.device_guard(k.device):
            _lib.check(_lib.lib().hqmq_encode_pair(C.byref(ak), C.byref(av), ws.data_ptr(), nbytes, _lib.stream_ptr()),
                       "hqmq_encode_pair")
        out_k.T += T
        out_v.T += T
        return out_k, out_v

    def decode(self, packed: PackedKV, layer_idx: int, kv: int, dtype: torch.dtype = torch.float32,
               t0: int = 0, T: Optional[int] = None, scale_first: bool = False,
               merge_outliers: bool = True) -> torch.Tensor:
        """Dense (B, H, T, d) reconstruction of tokens [t0, t0+T) of a native cache."""
        T = packed.T - t0 if T is None else T
        dev = packed.device
        tb = self.tables(layer_idx, kv, dev)
        out = torch.empty(packed.B, packed.H, T, packed.n_chunks * 4, dtype=dtype, device=dev)
        a = _lib.DequantArgs()
        a.struct_size = C.sizeof(_lib.DequantArgs)
        a.layout = 0
        a.src_native = packed.c_struct()
        a.t0, a.T = t0, T
        a.r_qmax = packed.qmax
        a.scale_first = int(scale_first)
        a.joint_f32 = tb["joint"].data_ptr()
        a.out_dtype, a.out = _lib.dtype_enum(dtype), out.data_ptr()
        a.merge_outliers = int(merge_outliers and packed.with_outliers)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().hqmq_dequant(C.byref(a), _lib.stream_ptr()), "hqmq_dequant")
        return out

    def _qdq(self, x: torch.Tensor, layer_idx: int, kv: int, median_mult: Optional[float] = None,
             quantile: Optional[float] = None) -> torch.Tensor:
        """Fake-quantise: decode(encode(x)).  The scale plane is kept in fp32 and the radius is
        rebuilt as rq * (r_max / qmax), the reference's own order (src/quantizers/hqmq.py:210-216)."""
        B, H, T, d = x.shape
        if d % 4 != 0:
            raise ValueError(f"d_head={d} not divisible by 4")
        if T == 0 or B == 0:
            return x.clone()
        pk = self.new_cache(B, T, d, x.device, scale_dtype=torch.float32, with_outliers=median_mult is not None,
                            out_dtype=x.dtype if x.dtype != torch.float64 else torch.float32)
        self.encode(x, layer_idx, kv, out=pk, median_mult=median_mult, quantile=quantile)
        self._last_packed = pk
        return self.decode(pk, layer_idx, kv, dtype=x.dtype, scale_first=True)

    def quantize_K(self, k, layer_idx):
        return self._qdq(k, layer_idx, kv=0)

    def quantize_V(self, v, layer_idx):
        return self._qdq(v, layer_idx, kv=1)

    def bits_per_value(self):
        bits_dir = math.log2(24 * self.secondary_size)
        radius = 0 if self.magnitude_mode == "free" else self.radius_bits
        return (bits_dir + radius + self.jl_dim) / 4.0

    @property
    def name(self) -> str:
        parts = [f"HQMQ_s{self.secondary_size}_r{self.radius_bits}"]
        if self.jl_dim > 0:
            parts.append(f"jl{self.jl_dim}")
        if self.magnitude_mode != "unit":
            parts.append(self.magnitude_mode)
        if self.log_radius:
            parts.append("logr")
        if self.robust_radius_scale:
            parts.append("robust")
        return "_".join(parts)


class _OutlierStats:
    """Running mean of the per-call outlier rates (what the reference's wrapper keeps in ``_observed_outlier_rate``),
    from the caches' device counters, read (and synchronised) only on demand.  A call costs no device work: every
    cache remembers how many calls of which size it took since its counters were last read, and the flagged chunks
    of those calls are the growth of its counters.  Calls of one size on one cache share their growth evenly (exact
    for the sum of their rates, which is all a mean needs)."""

    def __init__(self):
        self._caches = []           # caches with calls that were not accounted yet
        self._counts = []           # (0-d device tensor: flagged chunks of one finished call, chunks of that call)
        self._sum_rates, self._n = 0.0, 0   # sum of the per-call rates, number of calls

    def begin(self, pk, total_chunks: int):
        """Before a call appends to ``pk`` (None: a fresh cache).  Calls of another size are accounted first."""
        if pk is None:
            return
        st = getattr(pk, "_stat_pending", None)
        if st is not None and st[1] != total_chunks:
            self._account(pk)
        elif st is None and pk.T > 0 and not hasattr(pk, "_stat_base"):
            pk._stat_base = float(pk.out_count.sum().item())      # a cache filled elsewhere: count from what it holds

    def end(self, pk, total_chunks: int):
        st = getattr(pk, "_stat_pending", None)
        if st is None:
            st = pk._stat_pending = [0, total_chunks]
            self._caches.append(pk)
        st[0] += 1

    def _account(self, pk):
        n_calls, total = pk._stat_pending
        pk._stat_pending = None
        now = float(pk.out_count.sum().item())
        self._sum_rates += (now - getattr(pk, "_stat_base", 0.0)) / max(1, total)
        self._n += n_calls
        pk._stat_base = now

    def push_count(self, count: torch.Tensor, total_chunks: int):
        """A finished one-shot call (fake-quant): only its count is kept, not its cache."""
        self._counts.append((count, total_chunks))
        if len(self._counts) >= 1024:
            self._sync()

    def _sync(self):
        for pk in self._caches:
            if getattr(pk, "_stat_pending", None) is not None:
                self._account(pk)
        self._caches = []
        for count, total in self._counts:
            self._sum_rates += float(count.item()) / max(1, total)
            self._n += 1
        self._counts = []

    @property
    def rate(self):
        self._sync()
        return self._sum_rates / self._n if self._n else 0.0

    @property
    def n(self):
        self._sync()
        return self._n


class OutlierAwareHQMQQuantizer(KVQuantizer):
    """Outlier extraction around HQMQQuantizer: chunks whose norm exceeds the per-call, per-head
    threshold keep their original values (src/quantizers/outlier_aware.py:28-114)."""

    def __init__(self, inner: HQMQQuantizer, outlier_fraction: float = 0.01, threshold_mode: str = "fraction",
                 median_mult: float = 20.0):
        assert isinstance(inner, HQMQQuantizer), "wrapper expects HQMQQuantizer"
        self.inner = inner
        self.outlier_fraction, self.threshold_mode, self.median_mult = outlier_fraction, threshold_mode, median_mult
        self.chunk_dim = inner.chunk_dim
        self._stats = _OutlierStats()

    @property
    def _observed_outlier_rate(self):
        return self._stats.rate

    @property
    def _n_observations(self):
        return self._stats.n

    def trainable_parameters(self):
        return self.inner.trainable_parameters()

    def set_training(self, training, tau=None):
        self.inner.set_training(training, tau=tau)

    def _refresh_rotations(self):
        self.inner._refresh_rotations()

    def _check_mode(self):
        if self.threshold_mode not in ("median_mult", "fraction"):
            raise ValueError(self.threshold_mode)

    def _thr(self) -> dict:
        """The threshold of a call as the encoder takes it (src/quantizers/outlier_aware.py:63-72): ``median_mult``
        times the per-head median, or ("fraction") the per-head quantile 1 - outlier_fraction itself."""
        if self.threshold_mode == "fraction":
            return dict(median_mult=1.0, quantile=1.0 - self.outlier_fraction)
        return dict(median_mult=self.median_mult)

    def encode(self, x, layer_idx, kv, out: Optional[PackedKV] = None, **kw) -> PackedKV:
        self._check_mode()
        total = x.shape[0] * x.shape[1] * x.shape[2] * (x.shape[3] // 4)
        if total:
            self._stats.begin(out, total)
        pk = self.inner.encode(x, layer_idx, kv, out=out, **self._thr(), **kw)
        if total:
            self._stats.end(pk, total)
        return pk

    def encode_pair(self, k, v, layer_idx, out_k: PackedKV, out_v: PackedKV):
        """Keys and values of one layer in one call (see ``HQMQQuantizer.encode_pair``), each with its own median."""
        self._check_mode()
        total = k.shape[0] * k.shape[1] * k.shape[2] * (k.shape[3] // 4)
        if total:
            self._stats.begin(out_k, total)
            self._stats.begin(out_v, total)
        pair = self.inner.encode_pair(k, v, layer_idx, out_k, out_v, **self._thr())
        if total:
            self._stats.end(out_k, total)
            self._stats.end(out_v, total)
        return pair

    def decode(self, packed, layer_idx, kv, **kw):
        return self.inner.decode(packed, layer_idx, kv, **kw)

    def _qdq(self, x, layer_idx, kv):
        self._check_mode()
        out = self.inner._qdq(x, layer_idx, kv, **self._thr())
        if x.shape[0] and x.shape[2]:
            self._stats.push_count(self.inner._last_packed.out_count.sum(), x.shape[0] * x.shape[1] * x.shape[2] * (x.shape[3] // 4))
        return out

    def quantize_K(self, k, layer_idx):
        return self._qdq(k, layer_idx, kv=0)

    def quantize_V(self, v, layer_idx):
        return self._qdq(v, layer_idx, kv=1)

    def bits_per_value(self):
        if self._n_observations > 0:
            p = self._observed_outlier_rate
        else:
            p = self.outlier_fraction if self.threshold_mode == "fraction" else 0.03
        return (1 - p) * self.inner.bits_per_value() + p * 16 + 1 / self.chunk_dim

    @property
    def name(self):
        if self.threshold_mode == "fraction":
            return f"Outlier{int(self.outlier_fraction * 100)}p_{self.inner.name}"
        return f"OutlierMed{self.median_mult:.0f}_{self.inner.name}"


class OutlierAwareGenericQuantizer(OutlierAwareHQMQQuantizer):
    """Type-agnostic outlier wrapper of the reference (src/quantizers/outlier_generic.py).  Only an
    HQMQQuantizer inner (optionally padded) is accelerated here; other inner quantizers belong to
    the reference's ablation baselines and are rejected."""

    def __init__(self, inner: KVQuantizer, chunk_dim: int = 4, outlier_fraction: float = 0.01,
                 threshold_mode: str = "median_mult", median_mult: float = 3.0):
        if not isinstance(inner, HQMQQuantizer):
            raise NotImplementedError("hqmq_b200: OutlierAwareGenericQuantizer supports an HQMQQuantizer inner only")
        if chunk_dim != 4:
            raise NotImplementedError("hqmq_b200: chunk_dim must be 4")
        super().__init__(inner, outlier_fraction=outlier_fraction, threshold_mode=threshold_mode,
                         median_mult=median_mult)

    @property
    def name(self):
        if self.threshold_mode == "fraction":
            return f"Outlier{int(self.outlier_fraction * 100)}p_{self.inner.__class__.__name__}"
        return f"OutlierMed{self.median_mult:.0f}_{self.inner.__class__.__name__}"


class PaddedHQMQQuantizer(KVQuantizer):
    """HQMQ for head dims not divisible by 4: zero-pad to the next multiple of 4, quantize,
    truncate (src/quantizers/hqmq_padded.py:19-86)."""

    def __init__(self, n_layers: int, n_heads: int, d_head: int, secondary_size: int = 24, radius_bits: int = 4,
                 device: str = "cuda", init: str = "random", seed: int = 42):
        self.d_head_orig = d_head
        self.d_head_padded = ((d_head + 3) // 4) * 4
        self.pad_count = self.d_head_padded - d_head
        self.chunk_dim = 4
        self.radius_bits, self.secondary_size = radius_bits, secondary_size
        self.inner = HQMQQuantizer(n_layers=n_layers, n_heads=n_heads, secondary_size=secondary_size,
                                   radius_bits=radius_bits, device=device, init=init, seed=seed)

    def trainable_parameters(self):
        return self.inner.trainable_parameters()

    def set_training(self, training, tau=None):
        self.inner.set_training(training, tau=tau)

    def _qdq(self, x, layer_idx, kv):
        B, H, T, d_h = x.shape
        if d_h != self.d_head_padded:
            assert d_h == self.d_head_orig, f"Expected d_head={self.d_head_orig}, got {d_h}"
            x = torch.nn.functional.pad(x, (0, self.pad_count))
        xq = self.inner._qdq(x, layer_idx, kv)
        return xq[..., :self.d_head_orig]

    def quantize_K(self, k, layer_idx):
        return self._qdq(k, layer_idx, kv=0)

    def quantize_V(self, v, layer_idx):
        return self._qdq(v, layer_idx, kv=1)

    def bits_per_value(self):
        return self.inner.bits_per_value() * self.d_head_padded / self.d_head_orig

    @property
    def name(self):
        return f"PaddedHQMQ_d{self.d_head_orig}to{self.d_head_padded}_{self.inner.name}"
