"""The NVLink push exchange of sequence-split partials, through the C ABI, with both ranks' buffers on ONE
device: the stores, epoch words, parity halves and the bounded wait are the same code that runs across GPUs
(there the peers' addresses are CUDA-IPC mappings).  The launches are issued in stream order -- pushes before
waits -- so no kernel ever waits for a later one."""
import ctypes as C

import pytest
import torch

from hqmq_b200 import _lib
from hqmq_b200.attention import combine_partials

pytestmark = pytest.mark.gpu


def _pair(world, block):
    L = _lib.lib()
    recv = [torch.zeros(L.hqmq_exchange_recv_bytes(world, block) // 4, device="cuda") for _ in range(world)]
    flags = [torch.zeros(L.hqmq_exchange_flag_bytes(world) // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    xs = []
    for r in range(world):
        x = _lib.Exchange()
        x.struct_size, x.world, x.rank, x.block_floats = C.sizeof(_lib.Exchange), world, r, block
        for p in range(world):
            x.recv[p], x.flags[p] = recv[p].data_ptr(), flags[p].data_ptr()
        xs.append(x)
    return xs, recv, flags


def _parts(world, rows, d, seed):
    g = torch.Generator().manual_seed(seed)
    o = torch.randn(world, rows, d, generator=g)
    m = torch.randn(world, rows, 1, generator=g) * 3
    l = torch.rand(world, rows, 1, generator=g) + 0.5
    return torch.cat([o, m, l], -1).cuda().contiguous()


def test_push_wait_merge_equals_gathered_merge():
    world, rows, d = 3, 32, 128
    block = rows * (d + 2)
    L = _lib.lib()
    xs, recv, flags = _pair(world, block)
    status = torch.zeros(world, dtype=torch.int32, device="cuda")
    st = _lib.stream_ptr()
    for epoch in (1, 2, 3):
        parts = _parts(world, rows, d, seed=epoch)
        want = combine_partials(parts.view(world, 1, rows, 1, d + 2), torch.float32).view(rows, d)
        for r in range(world):
            _lib.check(L.hqmq_exchange_push(C.byref(xs[r]), parts[r].data_ptr(), epoch, st), "push")
        for r in range(world):
            out = torch.empty(rows, d, device="cuda")
            _lib.check(L.hqmq_exchange_wait(C.byref(xs[r]), epoch, 0, status[r:].data_ptr(), st), "wait")
            src = recv[r].data_ptr() + (epoch & 1) * world * block * 4
            _lib.check(L.hqmq_combine_partials(src, world, rows, d, 1, _lib.dtype_enum(torch.float32), out.data_ptr(), st), "merge")
            assert torch.equal(out, want), (epoch, r)
    assert int(status.abs().sum()) == 0


def test_wait_gives_up_and_names_the_missing_rank():
    """Rank 1 never pushes: rank 0's wait runs out after a few polls, records bit 1 and returns; the device
    keeps working and a later complete step succeeds."""
    world, rows, d = 2, 4, 62
    block = rows * (d + 2)
    L = _lib.lib()
    xs, recv, flags = _pair(world, block)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = _lib.stream_ptr()
    parts = _parts(world, rows, d, seed=9)
    _lib.check(L.hqmq_exchange_push(C.byref(xs[0]), parts[0].data_ptr(), 1, st), "push")
    _lib.check(L.hqmq_exchange_wait(C.byref(xs[0]), 1, 64, status.data_ptr(), st), "wait")
    assert int(status.item()) == 0b10
    status.zero_()
    for r in range(world):
        _lib.check(L.hqmq_exchange_push(C.byref(xs[r]), parts[r].data_ptr(), 2, st), "push")
    _lib.check(L.hqmq_exchange_wait(C.byref(xs[0]), 2, 64, status.data_ptr(), st), "wait")
    assert int(status.item()) == 0


def test_exchange_arguments_are_validated():
    L = _lib.lib()
    xs, recv, flags = _pair(2, 8)
    assert L.hqmq_exchange_push(None, None, 1, None) == -1
    assert L.hqmq_exchange_push(C.byref(xs[0]), recv[0].data_ptr(), 0, None) == -1      # epoch 0 is the cleared state
    xs[0].block_floats = 6
    assert L.hqmq_exchange_push(C.byref(xs[0]), recv[0].data_ptr(), 1, None) == -4      # slots off 16-byte boundaries
    assert L.hqmq_exchange_recv_bytes(17, 8) == 0 and L.hqmq_exchange_flag_bytes(2) == 16
    xs[0].block_floats = 8
    assert L.hqmq_exchange_verify(C.byref(xs[0])) == 0 and L.hqmq_exchange_enable_peer(torch.cuda.current_device()) == 0
    handle, off = (C.c_ubyte * 64)(), C.c_int64(-1)
    assert L.hqmq_exchange_ipc_export(recv[0].data_ptr() + 16, handle, C.byref(off)) == 0      # an interior address
    assert off.value >= 16 and off.value % 16 == 0 and any(handle)
    assert L.hqmq_exchange_ipc_export(None, handle, C.byref(off)) == -1
    host = (C.c_float * 64)()
    xs[0].recv[1] = C.addressof(host)                                                    # not device memory
    assert L.hqmq_exchange_verify(C.byref(xs[0])) in (-1, -4)


def test_fused_step_equals_gathered_merge():
    """Push, wait and merge in one launch (hqmq_exchange_step).  On one device the launches that stand for the
    other ranks must not be waited for by an earlier launch, so the other ranks' blocks are pushed first (plain
    push), and a rank's fused step then finds their epoch words set and waits only for its own pushing CTAs,
    which never wait themselves."""
    world, rows, d = 3, 32, 128
    block = rows * (d + 2)
    L = _lib.lib()
    xs, recv, flags = _pair(world, block)
    status = torch.zeros(world, dtype=torch.int32, device="cuda")
    st = _lib.stream_ptr()
    for epoch in (1, 2, 3, 4):
        parts = _parts(world, rows, d, seed=20 + epoch)
        want = combine_partials(parts.view(world, 1, rows, 1, d + 2), torch.float32).view(rows, d)
        for r in range(1, world):
            _lib.check(L.hqmq_exchange_push(C.byref(xs[r]), parts[r].data_ptr(), epoch, st), "push")
        for r in range(world):          # rank 0 pushes inside its step; the later ranks push once more (same bytes)
            out = torch.empty(rows, d, device="cuda")
            _lib.check(L.hqmq_exchange_step(C.byref(xs[r]), parts[r].data_ptr(), epoch, 0, status[r:].data_ptr(), rows, d,
                                            _lib.dtype_enum(torch.float32), out.data_ptr(), st), "step")
            assert torch.equal(out, want), (epoch, r)
    assert int(status.abs().sum()) == 0
    # a 16-bit output rounds the same merge once
    out16 = torch.empty(rows, d, dtype=torch.bfloat16, device="cuda")
    for r in range(1, world):
        _lib.check(L.hqmq_exchange_push(C.byref(xs[r]), parts[r].data_ptr(), 5, st), "push")
    _lib.check(L.hqmq_exchange_step(C.byref(xs[0]), parts[0].data_ptr(), 5, 0, status.data_ptr(), rows, d,
                                    _lib.dtype_enum(torch.bfloat16), out16.data_ptr(), st), "step")
    assert torch.allclose(out16.float(), want.bfloat16().float(), rtol=1e-2, atol=1e-2)


def test_fused_step_gives_up_and_names_the_missing_rank():
    """Rank 1 never delivers: the waiting CTAs of rank 0's step run out of polls (a few milliseconds), set bit 1 of the
    status word and write NaN rows; the device keeps working and a complete step afterwards succeeds."""
    world, rows, d = 2, 4, 62
    block = rows * (d + 2)
    L = _lib.lib()
    xs, recv, flags = _pair(world, block)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = _lib.stream_ptr()
    parts = _parts(world, rows, d, seed=10)
    out = torch.zeros(rows, d, device="cuda")
    _lib.check(L.hqmq_exchange_step(C.byref(xs[0]), parts[0].data_ptr(), 1, 64, status.data_ptr(), rows, d,
                                    _lib.dtype_enum(torch.float32), out.data_ptr(), st), "step")
    assert int(status.item()) == 0b10 and torch.isnan(out).all()
    status.zero_()
    _lib.check(L.hqmq_exchange_push(C.byref(xs[1]), parts[1].data_ptr(), 2, st), "push")
    _lib.check(L.hqmq_exchange_step(C.byref(xs[0]), parts[0].data_ptr(), 2, 64, status.data_ptr(), rows, d,
                                    _lib.dtype_enum(torch.float32), out.data_ptr(), st), "step")
    want = combine_partials(parts.view(world, 1, rows, 1, d + 2), torch.float32).view(rows, d)
    assert int(status.item()) == 0 and torch.allclose(out, want, rtol=1e-6, atol=1e-6)
    assert L.hqmq_exchange_step(C.byref(xs[0]), parts[0].data_ptr(), 3, 0, status.data_ptr(), rows + 1, d, 0, out.data_ptr(), st) == -2
