"""The flag barrier of the fused multi-GPU modes on ONE GPU: the peers' arrivals are written by the host, so the kernel's
epoch bookkeeping, its flag stores and its bounded wait are checked without a second rank.  (A missing peer is a flag
that nothing sets: the wait runs out, the status says so, and the context stays usable.)"""
import ctypes as C

import pytest
import torch

import baracuda_b200 as bq
from baracuda_b200 import _lib

pytestmark = pytest.mark.gpu


def _flags(world):
    words = _lib.load().baracuda_q_peer_barrier_flag_bytes() // 4
    bufs = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
    return bufs, (C.c_void_p * world)(*[b.data_ptr() for b in bufs])


def test_barrier_passes_when_every_peer_has_arrived_and_keeps_its_epoch():
    lib = _lib.load()
    world, rank = 4, 1
    bufs, ptrs = _flags(world)
    for epoch in (1, 2, 3):
        for peer in range(world):
            if peer != rank:
                bufs[rank][peer] = epoch  # the peers' stores into this rank's buffer
        assert lib.baracuda_q_peer_barrier_run(ptrs, rank, world, 0, None) == 0
        torch.cuda.synchronize()
        assert bq.device_status() == 0
        assert int(bufs[rank][16].item()) == epoch
        for peer in range(world):
            assert int(bufs[peer][rank].item()) == epoch  # this rank's arrival reached every buffer, its own included


def test_a_peer_one_barrier_ahead_does_not_block():
    lib = _lib.load()
    world, rank = 2, 0
    bufs, ptrs = _flags(world)
    bufs[rank][1] = 2  # the peer already stands at the next barrier
    assert lib.baracuda_q_peer_barrier_run(ptrs, rank, world, 0, None) == 0
    torch.cuda.synchronize()
    assert bq.device_status() == 0 and int(bufs[rank][16].item()) == 1


def test_missing_peer_times_out_with_a_status_and_the_context_survives(oracle):
    lib = _lib.load()
    world, rank = 2, 0
    bufs, ptrs = _flags(world)
    assert lib.baracuda_q_peer_barrier_run(ptrs, rank, world, 1 << 21, None) == 0  # about a millisecond
    torch.cuda.synchronize()
    assert bq.device_status() == 301
    assert bq.device_status() == 0  # read and clear
    # the context is as usable as before
    x = torch.arange(1024, device="cuda", dtype=torch.float32)
    assert float(x.sum().item()) == 1023 * 1024 / 2


def test_barrier_argument_rules():
    lib = _lib.load()
    bufs, ptrs = _flags(2)
    assert lib.baracuda_q_peer_barrier_run(None, 0, 2, 0, None) == 2
    assert lib.baracuda_q_peer_barrier_run(ptrs, 2, 2, 0, None) == 2
    assert lib.baracuda_q_peer_barrier_run(ptrs, 0, 9, 0, None) == 2
    bad = (C.c_void_p * 2)(bufs[0].data_ptr(), None)
    assert lib.baracuda_q_peer_barrier_run(bad, 0, 2, 0, None) == 2
