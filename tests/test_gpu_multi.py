"""The two multi-GPU exchanges over real GPUs (NCCL, one process per GPU): needs at least two GPUs, skipped
otherwise.  (a) A head's batch split over two GPUs: `encode_split_batch` must give each rank exactly its slice of
the single-GPU encode of the whole batch.  (b) Sequence-split partials pushed into the peer's memory must merge
to exactly what merging the gathered blocks gives, over several steps (both receive halves)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import hqmq_b200 as hqmq
    from hqmq_b200 import dist as hd
    from tests.util import make_kv
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # (a) split-batch Med3x
        B, H, T, d, S, br, Cm = 4, 2, 160, 128, 96, 4, 3.0
        x = make_kv("spiky", (B, H, T, d), seed=311, dtype=torch.bfloat16).to(dev)
        quant = hqmq.with_outlier_extraction(hqmq.HQMQ(1, H, S, br, device=dev), Cm)
        whole = quant.encode(x, 0, 0)
        b0, b1 = (0, 1) if rank == 0 else (1, B)                     # uneven shares
        mine = hd.encode_split_batch(quant, x[b0:b1], 0, 0)
        ok = all(torch.equal(g, w[b0:b1]) for g, w in zip(mine.to_reference(), whole.to_reference()))
        ok = ok and torch.equal(mine.out_count.view(b1 - b0, H), whole.out_count.view(B, H)[b0:b1])
        # (b) pushed exchange against the gathered merge
        rows, dd = 32, 128
        px = hd.PushExchange(rows, dd, dev)
        for step in range(3):
            g = torch.Generator().manual_seed(40 + step)
            parts = torch.cat([torch.randn(world, rows, dd, generator=g), torch.randn(world, rows, 1, generator=g) * 3,
                               torch.rand(world, rows, 1, generator=g) + 0.5], -1).to(dev)
            out = torch.empty(rows, dd, device=dev)
            px.step(parts[rank].contiguous(), out)
            want = hqmq.combine_partials(parts.view(world, 1, rows, 1, dd + 2), torch.float32).view(rows, dd)
            torch.cuda.synchronize()
            px.check()
            ok = ok and torch.equal(out, want)
        px.close()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_split_batch_encode_and_pushed_exchange_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = 33500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
