"""Bounded barrier of the one-sided exchange, on ONE GPU: the "peer" flag arrays are local buffers, so no second
kernel is ever waited for.  A signal that is already there lets the barrier pass; a signal that nothing sets makes
the wait run out after a short limit, which must end in a status word — not in a trap — and leave the context
usable."""
import time

import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def setup(world, rank):
    flags = torch.zeros(world, world, dtype=torch.int32, device=DEV)  # row p = the flag array of rank p
    ptrs = torch.tensor([flags[p].data_ptr() for p in range(world)], dtype=torch.int64, device=DEV)
    status = torch.zeros(world, dtype=torch.int32).pin_memory()
    return flags, ptrs, status


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (8, 3)])
def test_barrier_passes_when_every_peer_has_signalled(world, rank):
    flags, ptrs, status = setup(world, rank)
    flags[rank, :] = 5  # every peer announced barrier 5 in my array
    flags[rank, rank] = 0
    ops.peer_barrier(ptrs, rank, world, 5, 200_000, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0] * world
    # my own announcement landed in flag `rank` of every peer's array, and nowhere else
    expect = torch.zeros(world, world, dtype=torch.int32)
    expect[:, rank] = 5
    expect[rank, :] = 5
    expect[rank, rank] = 0
    assert torch.equal(flags.cpu(), expect)
    # a peer that already ran ahead to a later barrier counts as arrived
    flags[rank, :] = 9
    ops.peer_barrier(ptrs, rank, world, 6, 200_000, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0] * world


def test_wait_that_runs_out_ends_in_a_status_word():
    world, rank = 4, 1
    flags, ptrs, status = setup(world, rank)
    flags[rank, 0] = 3
    flags[rank, 3] = 3  # peer 2 never signals
    t0 = time.perf_counter()
    ops.peer_barrier(ptrs, rank, world, 3, 50_000, status)  # 50 ms limit
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert status.tolist() == [0, 0, 3, 0]
    assert 0.04 < elapsed < 5.0
    # the context is still usable, and a later barrier whose signals are all there passes
    x = torch.arange(10, device=DEV).sum().item()
    assert x == 45
    status.zero_()
    flags[rank, :] = 4
    ops.peer_barrier(ptrs, rank, world, 4, 50_000, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0] * world


def test_status_on_the_device_and_argument_checks():
    world, rank = 2, 0
    flags, ptrs, _ = setup(world, rank)
    status = torch.zeros(world, dtype=torch.int32, device=DEV)
    ops.peer_barrier(ptrs, rank, world, 1, 20_000, status)  # nothing signals: 20 ms
    torch.cuda.synchronize()
    assert status.tolist() == [0, 1]
    with pytest.raises(RuntimeError):
        ops.peer_barrier(ptrs, 2, world, 1, 20_000, status)       # rank outside the world
    with pytest.raises(RuntimeError):
        ops.peer_barrier(ptrs, 0, world, 0, 20_000, status)       # epoch 0 is the flags' initial value
    with pytest.raises(RuntimeError):
        ops.peer_barrier(ptrs, 0, world, 1, 0, status)            # no limit
    with pytest.raises(RuntimeError):
        ops.peer_barrier(ptrs, 0, world, 1, 20_000, torch.zeros(world, dtype=torch.int32))  # pageable host memory
    # a world of one launches nothing
    one = torch.zeros(1, dtype=torch.int64, device=DEV)
    ops.peer_barrier(one, 0, 1, 1, 20_000, status[:1].contiguous())
