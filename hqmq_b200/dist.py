"""Multi-GPU partitioning of the hot path (one process per GPU, torch.distributed).

The reference is single-GPU.  Both halves shard without any data-path collective over the units
(batch, KV head): the encoder's Med3x median couples only the batch entries of one head, and decode
attention is independent per (batch, KV head).  Only two exchanges exist:
  * gathering the attention outputs of KV-head shards (an all_gather of (B, H_q/N, 1, d) tensors), and
  * for a cache split by SEQUENCE across GPUs (one very long context), merging the per-GPU partial
    results (o[d], m, l) of each query head: one all_gather of (B, H_q, 1, d+2) fp32 followed by the
    library's merge kernel.
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
