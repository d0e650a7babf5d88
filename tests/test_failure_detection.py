"""Failure detection without any GPU fault: stalled peers are simulated on the host (a rank that stops
beating, a rank that exits, a fake clock) and collectives fail through short process-group timeouts."""
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist

from gradient_compression_b200.parallel.watchdog import DictStore, PeerStalled, StepWatchdog


def test_watchdog_detects_a_peer_that_stops_beating_fake_clock():
    now = [0.0]
    store = DictStore()
    a = StepWatchdog(store, 0, 2, timeout_s=10, clock=lambda: now[0])
    b = StepWatchdog(store, 1, 2, timeout_s=10, clock=lambda: now[0])
    for step in range(1, 4):
        now[0] += 1
        a.beat(step), b.beat(step)
        a.poll_once(), b.poll_once()
    now[0] += 5
    a.beat(4)             # rank 1 falls silent from here on
    a.poll_once()
    a.check()
    now[0] += 20
    a.poll_once()
    with pytest.raises(PeerStalled) as e:
        a.beat(5)
    assert e.value.rank == 1 and e.value.last_step == 3


def test_watchdog_thread_and_peer_that_never_joins():
    store = DictStore()
    wd = StepWatchdog(store, 0, 2, timeout_s=0.2, poll_s=0.02).start()
    try:
        deadline = time.time() + 5
        while wd.error is None and time.time() < deadline:
            time.sleep(0.02)
        with pytest.raises(PeerStalled):
            wd.check()
    finally:
        wd.stop()


def _exiting_rank_body(rank, world):
    x = torch.ones(4)
    dist.all_reduce(x)
    assert float(x[0]) == world
    if rank == 1:
        return                      # leaves between steps, nothing in flight
    from gradient_compression_b200.reducers import NoneAllReducer

    red = NoneAllReducer("cpu")
    t0 = time.time()
    with pytest.raises(Exception):  # the short group timeout ends the collective with an error
        red.reduce([torch.ones(4)], [torch.empty(4)])
        dist.barrier()
    assert time.time() - t0 < 60


def _short_timeout_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        _exiting_rank_body(rank, world)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_collective_with_a_departed_rank_errors_instead_of_hanging():
    import torch.multiprocessing as mp

    from tests.conftest import free_port

    mp.spawn(_short_timeout_worker, args=(2, free_port()), nprocs=2, join=True)


def test_collective_timeout_exception_fields():
    from gradient_compression_b200.parallel.comm import CollectiveTimeout

    e = CollectiveTimeout(0, 0x21, 3)
    assert e.peer == 3 and "rank 3" in str(e) and "0x21" in str(e)
