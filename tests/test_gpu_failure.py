"""Failure detection on the GPU without a fault: a bounded wait that runs out.

The rank barrier waits (at most two seconds of the device's global timer) for a flag that
nothing sets; the kernel must return normally, record where it gave up in the status record
and leave the context usable for the next launch.  No trap, no bad address, no endless loop.
"""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

WAIT_TIMEOUT, SITE_RANK_BARRIER = 1, 5


def _barrier(flag_table, rank, world, epoch, phase, status):
    from mega_moe import _native as N
    N.check(N.lib().mm_rank_barrier(flag_table.data_ptr(), rank, world, epoch, phase,
                                    status.data_ptr(), N.stream_ptr()), "mm_rank_barrier")


def _read(status):
    from mega_moe import _native as N
    rec = N.StatusRecord()
    N.check(N.lib().mm_status_read(status.data_ptr(), C.byref(rec), N.stream_ptr()),
            "mm_status_read")
    return rec


def test_rank_barrier_wait_runs_out_and_reports():
    from mega_moe import _native as N
    world, rank, epoch = 2, 0, 7
    # this "rank"'s flag words: the own slot is already at the epoch, the peer's never arrives
    flags = torch.tensor([epoch, 0], dtype=torch.int32, device=DEV)
    # every entry of the peer table points at the local words: no second GPU is involved
    table = torch.tensor([flags.data_ptr()] * world, dtype=torch.int64, device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)

    t0 = time.time()
    _barrier(table, rank, world, epoch, 2, status)      # phase 2: wait only
    torch.cuda.synchronize()                             # the kernel returns by itself
    waited = time.time() - t0
    assert 1.0 < waited < 20.0, waited

    rec = _read(status)
    assert rec.code == WAIT_TIMEOUT and rec.site == SITE_RANK_BARRIER
    assert rec.slot == 1 and rec.want == epoch and rec.seen == 0

    # the context is still usable: reset the record, let the "peer" arrive, wait again
    N.check(N.lib().mm_status_reset(status.data_ptr(), N.stream_ptr()), "mm_status_reset")
    flags[1] = epoch
    t0 = time.time()
    _barrier(table, rank, world, epoch, 2, status)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert _read(status).code == 0


def test_rank_barrier_signal_then_wait_completes():
    """Phases 1 (signal) and 2 (wait) of the split barrier on one rank's own words."""
    world, rank, epoch = 1, 0, 3
    flags = torch.zeros(1, dtype=torch.int32, device=DEV)
    table = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    _barrier(table, rank, world, epoch, 1, status)
    _barrier(table, rank, world, epoch, 2, status)
    torch.cuda.synchronize()
    assert int(flags[0]) == epoch and _read(status).code == 0
