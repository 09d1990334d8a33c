"""Multi-GPU partitioning of the hot path (one process per GPU, torch.distributed).

The reference is single-GPU.  Both halves shard without any data-path collective over the units
(batch, KV head): the encoder's Med3x median couples only the batch entries of one head, and decode
attention is independent per (batch, KV head).  Three exchanges exist:
  * gathering the attention outputs of KV-head shards (an all_gather of (B, H_q/N, 1, d) tensors), and
  * for a cache split by SEQUENCE across GPUs (one very long context), merging the per-GPU partial
    results (o[d], m, l) of each query head: one all_gather of (B, H_q, 1, d+2) fp32 followed by the
    library's merge kernel, and
  * for a head whose BATCH entries are spread over several GPUs (more GPUs than KV heads): the encoder's
    Med3x median must still be the one over every batch entry of the head, so the three histogram levels
    of its radix select are summed over those GPUs (three all_reduce of 16 KB per head; integer sums, so
    every GPU derives identical bits).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def split_range(n: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous piece [lo, hi) of range(n) for `rank`; pieces differ by at most `align` items and
    every boundary except the last is a multiple of `align`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} / world {world}")
    blocks = (n + align - 1) // align
    base, rem = divmod(blocks, world)
    lo_b = rank * base + min(rank, rem)
    hi_b = lo_b + base + (1 if rank < rem else 0)
    return min(n, lo_b * align), min(n, hi_b * align)


def kv_head_shard(B: int, H_kv: int, world: int, rank: int):
    """(batch slice, head slice) of this rank: KV heads are split first (the Med3x median stays local
    to a GPU); when there are more GPUs than KV heads, each head's batch is split further."""
    if world <= H_kv:
        h0, h1 = split_range(H_kv, world, rank)
        return slice(0, B), slice(h0, h1)
    if world % H_kv:
        raise ValueError(f"world={world} must be a multiple of H_kv={H_kv} when it exceeds it")
    per_head = world // H_kv
    h = rank // per_head
    b0, b1 = split_range(B, per_head, rank % per_head)
    return slice(b0, b1), slice(h, h + 1)


def seq_shard(T: int, world: int, rank: int) -> Tuple[int, int]:
    """Token range of this rank for a sequence-split cache; boundaries fall on 16-token tiles."""
    return split_range(T, world, rank, align=16)


def gather_partials(partials: torch.Tensor, group=None) -> torch.Tensor:
    """all_gather of per-rank partial results (..., d+2) -> (world, ..., d+2)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(partials.shape), dtype=partials.dtype, device=partials.device)
    dist.all_gather_into_tensor(out.view(world * partials.shape[0], *partials.shape[1:]), partials.contiguous(),
                                group=group)
    return out


def gather_head_outputs(O_local: torch.Tensor, group=None) -> torch.Tensor:
    """Outputs of KV-head shards (B, H_q/N, T_q, d) -> (B, H_q, T_q, d) on every rank."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(O_local) for _ in range(world)]
    dist.all_gather(parts, O_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def seq_parallel_attention(Q: torch.Tensor, K_local, V_local, table_K, table_V, group=None,
                           softmax_scale: Optional[float] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Decode attention over a cache whose tokens are split across the ranks of `group` (flash-decoding
    across GPUs): local partials, one all_gather over NVLink, merge on every rank."""
    from .attention import combine_partials, fused_attention_packed
    B, Hq, Tq, d = Q.shape
    part = torch.empty(B, Hq, Tq, d + 2, dtype=torch.float32, device=Q.device)
    fused_attention_packed(Q, K_local, V_local, table_K, table_V, causal=False, softmax_scale=softmax_scale,
                           partials=part)
    allp = gather_partials(part, group)
    return combine_partials(allp, out_dtype or Q.dtype)


HIST_BINS = 2048      # bins per radix-select histogram of the library (two histograms per level and head)


def summed_radix_select(hist_level, level_view, select_level, group=None) -> None:
    """The exchange pattern of a median over values that live on several ranks: for each of the three digit
    levels, ``hist_level(level)`` histograms this rank's values into its own state, the level's counters
    (``level_view(level)``, an integer tensor view of that state) are summed over the ranks of ``group``, and
    ``select_level(level)`` narrows the search on the summed counters -- identically on every rank."""
    for level in range(3):
        hist_level(level)
        view = level_view(level)
        tmp = view.contiguous()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        if tmp.data_ptr() != view.data_ptr():
            view.copy_(tmp)
        select_level(level)


def split_batch_median(quant, x: torch.Tensor, layer_idx: int, kv: int, out, group=None,
                       n_total: Optional[int] = None) -> torch.Tensor:
    """Med3x medians (H,) fp32 of the chunk norms of x over ALL ranks of ``group``: every rank passes its own
    batch entries of the same H heads (same T_new not required; a rank may hold none).  ``quant`` is the
    outlier-aware wrapper, ``out`` the cache the following ``encode(..., med_in=...)`` call will append to.
    ``n_total`` = chunk norms per head over all ranks (computed with one more all_reduce when not given)."""
    import ctypes as C
    from . import _lib
    if getattr(quant, "threshold_mode", "median_mult") != "median_mult":
        raise NotImplementedError("split_batch_median: the batch of a head can be split over GPUs for threshold_mode='median_mult' only")
    inner, mult = quant.inner, float(quant.median_mult)
    B, H, T, d = x.shape
    inner._check_dst(x, out)
    if x.stride(-1) != 1 or any(s % 4 for s in x.stride()[:3]):
        x = x.contiguous()
    L = _lib.lib()
    dev = x.device
    a = inner._enc_args(x, layer_idx, kv, out, mult)
    nbytes = L.hqmq_med3x_state_bytes(H)
    state = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    hist = state[: H * 3 * 2 * HIST_BINS * 4].view(torch.int32).view(H, 3, 2, HIST_BINS)
    med = torch.empty(H, dtype=torch.float32, device=dev)
    if n_total is None:
        n = torch.tensor([B * T * (d // 4)], dtype=torch.int64, device=dev)
        dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
        n_total = int(n.item())

    def hist_level(level):
        with _lib.device_guard(dev):
            _lib.check(L.hqmq_med3x_hist(C.byref(a), level, state.data_ptr(), nbytes, _lib.stream_ptr()), "hqmq_med3x_hist")

    def select_level(level):
        with _lib.device_guard(dev):
            _lib.check(L.hqmq_med3x_select(H, level, n_total, mult, state.data_ptr(), nbytes, med.data_ptr(),
                                           _lib.stream_ptr()), "hqmq_med3x_select")

    summed_radix_select(hist_level, lambda level: hist[:, level], select_level, group)
    return med


def encode_split_batch(quant, x: torch.Tensor, layer_idx: int, kv: int, out=None, group=None, **kw):
    """``quant.encode`` for a rank that holds only some batch entries of its heads: the Med3x threshold is the
    one the reference would take over the whole batch (src/quantizers/outlier_aware.py:63-72).  Every rank of
    ``group`` must make the call."""
    inner = quant.inner
    B, H, T, d = x.shape
    if out is None:
        sd = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.float32
        out = inner.new_cache(B, max(T, 1), d, x.device, scale_dtype=sd, with_outliers=True, out_dtype=x.dtype,
                              ofrag=kv == 0)
    med = split_batch_median(quant, x, layer_idx, kv, out, group)
    return quant.encode(x, layer_idx, kv, out=out, med_in=med, **kw)


class PushExchange:
    """Sequence-split partials exchanged by direct stores into the peers' memory (see hqmq_exchange in
    include/hqmq_b200.h) instead of an all_gather: one small kernel per step stores this rank's block into
    every peer, one polls this GPU's own flag words, then the usual merge runs on the local receive buffer.

    Set-up (collective over ``group``, once): every rank allocates one buffer (receive slots + flag words),
    exports its CUDA IPC handle, and maps every peer's buffer with ITS OWN device current, so that its kernels
    can store into them.  ``rows`` = B * H_q * T_q rows of d + 2 floats per rank.  All ranks must call
    ``step`` the same number of times; ``close`` is collective too."""

    def __init__(self, rows: int, d: int, device, group=None, max_polls: int = 0):
        import ctypes as C
        from . import _lib
        self.group, self.rows, self.d = group, rows, d
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.block = rows * (d + 2)
        if self.block % 4:
            raise ValueError(f"rows * (d + 2) = {self.block} must be a multiple of 4 (16-byte slots)")
        if self.world > _lib.EXCHANGE_MAX_RANKS:
            raise ValueError(f"at most {_lib.EXCHANGE_MAX_RANKS} ranks")
        L = _lib.lib()
        dev = self.device = torch.device(device)
        recv_bytes, flag_bytes = L.hqmq_exchange_recv_bytes(self.world, self.block), L.hqmq_exchange_flag_bytes(self.world)
        self.buf = torch.zeros(recv_bytes + flag_bytes, dtype=torch.uint8, device=dev)     # one allocation, one handle
        self.recv = self.buf[:recv_bytes].view(torch.float32)
        self.flags = self.buf[recv_bytes:].view(torch.int32)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        handle, off = (C.c_ubyte * 64)(), C.c_int64(0)
        with _lib.device_guard(dev):
            _lib.check(L.hqmq_exchange_ipc_export(self.buf.data_ptr(), handle, C.byref(off)), "hqmq_exchange_ipc_export")
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (bytes(handle), int(off.value)), group=group)
        self._opened = []                      # peers' mapped allocations, closed in close()
        x = _lib.Exchange()
        x.struct_size = C.sizeof(_lib.Exchange)
        x.world, x.rank, x.block_floats = self.world, self.rank, self.block
        for p, (h, o) in enumerate(everyone):
            if p == self.rank:
                base = self.buf.data_ptr()
            else:
                mapped = C.c_void_p()
                with _lib.device_guard(dev):
                    _lib.check(L.hqmq_exchange_ipc_open((C.c_ubyte * 64).from_buffer_copy(h), C.byref(mapped)),
                               "hqmq_exchange_ipc_open")
                self._opened.append(mapped.value)
                base = mapped.value + o
            x.recv[p], x.flags[p] = base, base + recv_bytes
        with _lib.device_guard(dev):
            _lib.check(L.hqmq_exchange_verify(C.byref(x)), "hqmq_exchange_verify")
        self.x, self.max_polls, self.epoch = x, max_polls, 0
        dist.barrier(group=group)              # every rank has mapped every buffer before anyone stores into one

    def step(self, part: torch.Tensor, out: torch.Tensor, fused: bool = True) -> None:
        """Enqueue on the current stream: push ``part`` (rows, d + 2 fp32, contiguous) to all ranks, wait for all
        ranks' blocks of this step, merge them into ``out`` (rows, d) -- in one launch (``fused``) or as three."""
        import ctypes as C
        from . import _lib
        L = _lib.lib()
        if part.dtype != torch.float32 or part.numel() != self.block or not part.is_contiguous():
            raise ValueError("part must be contiguous fp32 with rows * (d + 2) elements")
        self.epoch += 1
        st = _lib.stream_ptr()
        if fused and self.rows + self.world <= 148 * 8:
            # one launch: the block goes out, the ranks' blocks are awaited (bounded) and merged
            _lib.check(L.hqmq_exchange_step(C.byref(self.x), part.data_ptr(), self.epoch, self.max_polls, self.status.data_ptr(),
                                            self.rows, self.d, _lib.dtype_enum(out.dtype), out.data_ptr(), st),
                       "hqmq_exchange_step")
            return
        _lib.check(L.hqmq_exchange_push(C.byref(self.x), part.data_ptr(), self.epoch, st), "hqmq_exchange_push")
        _lib.check(L.hqmq_exchange_wait(C.byref(self.x), self.epoch, self.max_polls, self.status.data_ptr(), st),
                   "hqmq_exchange_wait")
        src = self.recv.data_ptr() + (self.epoch & 1) * self.world * self.block * 4
        _lib.check(L.hqmq_combine_partials(src, self.world, self.rows, self.d, 1, _lib.dtype_enum(out.dtype),
                                           out.data_ptr(), st), "hqmq_combine_partials")

    def check(self) -> None:
        """Synchronise and raise if a wait ran out since the last check (bit r of the status = rank r missing)."""
        from . import _lib
        s = int(self.status.item()) & 0xffffffff
        if s:
            self.status.zero_()
            missing = [r for r in range(self.world) if s >> r & 1]
            raise _lib.HqmqError(f"hqmq_b200: exchange timed out waiting for the partials of ranks {missing} (-11)")

    def close(self) -> None:
        """Collective: nobody unmaps a buffer that a peer may still store into."""
        from . import _lib
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with _lib.device_guard(self.device):
            for base in self._opened:
                _lib.check(_lib.lib().hqmq_exchange_ipc_close(base), "hqmq_exchange_ipc_close")
        self._opened = []
        dist.barrier(group=self.group)
