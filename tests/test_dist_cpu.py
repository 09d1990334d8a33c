"""Host logic of the multi-GPU paths on CPU: partitioning, and the gather + merge of sequence-split
partial results exercised with two gloo ranks (the merge itself is checked with the oracle)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hqmq_b200 import dist as hd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_range_covers_everything():
    for n, world, align in [(10, 3, 1), (131072, 8, 16), (100, 8, 16), (5, 8, 1), (0, 2, 1), (33, 2, 16)]:
        pieces = [hd.split_range(n, world, r, align) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == n
        for (a, b), (c, d) in zip(pieces[:-1], pieces[1:]):
            assert b == c and a <= b and b % align == 0 or b == n
        blocks = [(b - a + align - 1) // align for a, b in pieces]
        assert max(blocks) - min(blocks) <= 1


def test_kv_head_shard():
    # 8 KV heads over 1/2/4/8 GPUs: heads only
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            bs, hs = hd.kv_head_shard(16, 8, world, r)
            assert bs == slice(0, 16)
            seen += list(range(hs.start, hs.stop))
        assert seen == list(range(8))
    # 4 KV heads over 8 GPUs: each head's batch is halved
    units = set()
    for r in range(8):
        bs, hs = hd.kv_head_shard(32, 4, 8, r)
        assert hs.stop - hs.start == 1 and bs.stop - bs.start == 16
        units |= {(b, hs.start) for b in range(bs.start, bs.stop)}
    assert len(units) == 32 * 4
    with pytest.raises(ValueError):
        hd.kv_head_shard(4, 3, 8, 0)


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    from oracle import hqmq_oracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        B, H, T, d = 2, 3, 64, 8
        s = torch.randn(B, H, T, generator=g) * 2          # scores in the exp2 domain
        v = torch.randn(B, H, T, d, generator=g)
        lo, hi = hd.seq_shard(T, world, rank)
        m = s[..., lo:hi].amax(-1)
        p = torch.exp2(s[..., lo:hi] - m[..., None])
        part = torch.cat([torch.einsum("bht,bhtd->bhd", p, v[:, :, lo:hi]), m[..., None], p.sum(-1, keepdim=True)], -1)
        allp = hd.gather_partials(part.unsqueeze(2))         # (world, B, H, 1, d+2)
        assert allp.shape == (world, B, H, 1, d + 2)
        # the gathered partials of every rank merge to the unsplit softmax (natural-log oracle: rescale m)
        ln2 = 0.6931471805599453
        merged = orc.combine_partials(allp[..., d] * ln2, allp[..., d + 1], allp[..., :d])
        full = torch.einsum("bht,bhtd->bhd", torch.softmax(s * ln2, -1), v).unsqueeze(2)
        ok = torch.allclose(merged, full, atol=1e-5)
        outs = hd.gather_head_outputs(torch.full((1, 2, 1, 4), float(rank)))
        ok = ok and outs.shape == (1, 2 * world, 1, 4) and float(outs[0, 2 * rank, 0, 0]) == rank
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sequence_split_gather_and_merge_two_ranks():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _radix_worker(rank, world, port, ret):
    """Two ranks hold different values of the same three 'heads'; a numpy stand-in of the library's histogram
    and select steps drives hd.summed_radix_select, whose result must be torch.quantile of the union."""
    sys.path.insert(0, ROOT)
    import numpy as np
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, counts = 3, (700, 1301)                       # uneven shares, odd total
        g = torch.Generator().manual_seed(5)
        allv = [torch.randn(H, c, generator=g).abs() * (1 + 10 * (torch.rand(H, c, generator=g) < 0.05)) for c in counts]
        mine = allv[rank].numpy().view(np.uint32)        # non-negative floats order like their bit patterns
        n_total = sum(counts)
        hist = torch.zeros(H, 3, 2, hd.HIST_BINS, dtype=torch.int32)
        prefix = np.zeros((H, 2), dtype=np.uint32)
        rank_in = np.array([[(n_total - 1) // 2, n_total // 2]] * H, dtype=np.int64)
        shifts, masks, fixed = (21, 10, 0), (0x7ff, 0x7ff, 0x3ff), (32, 21, 10)

        def hist_level(level):
            for h in range(H):
                for q in range(2):
                    keys = mine[h].astype(np.uint64)
                    sel = keys >> fixed[level] == np.uint64(prefix[h, q]) >> np.uint64(fixed[level]) if level else np.ones(keys.shape, bool)
                    dig = ((keys[sel] >> np.uint64(shifts[level])) & np.uint64(masks[level])).astype(np.int64)
                    hist[h, level, q] = torch.from_numpy(np.bincount(dig, minlength=hd.HIST_BINS).astype(np.int32))

        def select_level(level):
            for h in range(H):
                for q in range(2):
                    cum = np.cumsum(hist[h, level, q].numpy().astype(np.int64))
                    b = int(np.searchsorted(cum, rank_in[h, q], side="right"))
                    rank_in[h, q] -= cum[b - 1] if b else 0
                    prefix[h, q] |= np.uint32(b << shifts[level])

        hd.summed_radix_select(hist_level, lambda level: hist[:, level], select_level)
        a, b = torch.from_numpy(prefix.view(np.float32).copy()).unbind(1)
        med = a if n_total % 2 else b - (b - a) * 0.5
        want = torch.quantile(torch.cat(allv, 1), 0.5, dim=1)
        ret[rank] = bool(torch.equal(med, want))
    finally:
        dist.destroy_process_group()


def test_median_over_values_spread_across_two_ranks():
    world = 2
    port = 31500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_radix_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
