"""Failure detection without touching a GPU: the signalling protocol model
with withheld and corrupted signals, heartbeats with a rank that goes quiet,
and a collective that one rank never joins."""
import time

import pytest
import torch
import torch.distributed as dist

from jaxdecomp_b200.parallel.protocol import (
    OK,
    STALE_EPOCH,
    TIMEOUT_PEER_SIGNAL,
    FlagBoard,
    HealthMonitor,
    PeerDeadError,
)
from jaxdecomp_b200.utils.testing import run_ranks


def test_protocol_model_normal_rounds_and_wraparound():
    fb = FlagBoard(4)
    for _ in range(5):
        assert all(r.code == OK for r in fb.barrier_all())
    fb.counter = [0xFFFFFFFE] * 4
    for r in range(4):
        fb.slots[r] = [0xFFFFFFFE] * 4
    for _ in range(4):  # crosses 2^32
        assert all(r.code == OK for r in fb.barrier_all())
    assert fb.counter[0] == 2


def test_protocol_model_withheld_signal_times_out_with_peer_and_epochs():
    fb = FlagBoard(4, drop=lambda src, dst, epoch: src == 2 and dst == 0 and epoch == 3)
    assert all(r.code == OK for r in fb.barrier_all())
    assert all(r.code == OK for r in fb.barrier_all())
    res = fb.barrier_all()
    assert res[0].code == TIMEOUT_PEER_SIGNAL and res[0].peer == 2 and res[0].expected == 3 and res[0].seen == 2
    assert all(r.code == OK for r in res[1:])


def test_protocol_model_corrupted_epoch_is_reported_as_stale():
    fb = FlagBoard(3)
    fb.barrier_all()
    for r in range(3):
        fb.signal(r, 2)
    fb.slots[1][0] = 40  # rank 0's slot on rank 1 jumps far ahead of the epoch in progress
    res = [fb.wait(r, 2) for r in range(3)]
    assert res[1].code == STALE_EPOCH and res[1].peer == 0 and res[1].seen == 40
    assert res[0].code == OK and res[2].code == OK


def _heartbeat_worker(rank, world):
    mon = HealthMonitor(period=0.05, max_age=0.6)
    dist.barrier()
    time.sleep(0.3)
    mon.check()  # everyone alive
    dist.barrier()
    if rank == 3:
        mon.stop()  # this rank goes quiet between steps (no collective in flight)
        time.sleep(2.0)
        return
    time.sleep(1.2)
    with pytest.raises(PeerDeadError) as ei:
        mon.check()
    assert ei.value.ranks == [3]
    mon.stop()


def test_heartbeat_detects_quiet_rank():
    run_ranks(_heartbeat_worker, 4)


def _public_heartbeat_worker(rank, world):
    import jaxdecomp_b200 as jd

    jd.check_peers()  # no monitor yet: nothing to check
    jd.init(heartbeat=0.05, heartbeat_max_age=0.6)
    dist.barrier()
    time.sleep(0.3)
    jd.check_peers()
    dist.barrier()
    if rank == 1:
        jd.finalize()  # stops publishing; the rank leaves between steps
        time.sleep(2.0)
        return
    time.sleep(1.2)
    with pytest.raises(PeerDeadError) as ei:
        jd.check_peers()
    assert ei.value.ranks == [1]
    jd.finalize()
    jd.check_peers()  # the monitor is gone again


def test_heartbeat_through_init_and_check_peers():
    run_ranks(_public_heartbeat_worker, 3)


def _missing_rank_worker(rank, world):
    t = torch.ones(4)
    dist.all_reduce(t)
    if rank == 1:
        return  # never joins the next collective
    t0 = time.time()
    try:
        dist.all_reduce(t)
    except Exception:  # noqa: BLE001
        assert time.time() - t0 < 30
        raise
    raise AssertionError("collective completed although a rank never joined")


def test_collective_with_missing_rank_raises_within_timeout():
    t0 = time.time()
    with pytest.raises(Exception):
        run_ranks(_missing_rank_worker, 3, env={"JD_TEST_PG_TIMEOUT": "5"}, timeout=60)
    assert time.time() - t0 < 60
