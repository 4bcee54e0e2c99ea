"""Failure detection of the expert-parallel path, on the host only (no GPU is faulted or hung).

* the polling wait behind moe_ep_set_deadline_ms, driven by a clock through a debug hook;
* join_ranks: a rank that never arrives is reported to the others within the deadline, before any
  collective is started (gloo ranks on CPU; the missing rank simply never checks in).
"""
import ctypes as C
import os
import sys
import time

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

from rustingbrain_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_the_polling_wait_returns_ok_before_the_deadline_and_timeout_after_it():
    L = _lib.lib()
    gave_up = C.c_int32(-1)
    t0 = time.monotonic()
    assert L.moe_debug_deadline_wait(20, 2000, C.byref(gave_up)) == _lib.OK and gave_up.value == 0
    assert 0.015 <= time.monotonic() - t0 < 1.0            # it returned when the condition came true, not at the deadline
    t0 = time.monotonic()
    assert L.moe_debug_deadline_wait(5000, 60, C.byref(gave_up)) == _lib.TIMEOUT and gave_up.value == 1
    assert 0.05 <= time.monotonic() - t0 < 1.0             # ... and gave up at the deadline, not when it would have come true
    assert L.moe_debug_deadline_wait(30, 0, C.byref(gave_up)) == _lib.OK   # 0 = no deadline


def _join_worker(rank, world, port, absent, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from rustingbrain_b200.ep import join_ranks, RankMissing
        join_ranks(10.0)                                   # everybody is here: returns at once
        t0 = time.monotonic()
        if rank in absent:
            time.sleep(1.5)                                # never checks in for the second round
            ret[rank] = "absent"
        else:
            try:
                join_ranks(0.4)
                ret[rank] = "joined"
            except RankMissing as e:
                ret[rank] = "missing after %.1f s: %s" % (time.monotonic() - t0, e)
    finally:
        # no collective here: the store-based check-in is the only traffic, so an absent rank hangs nobody
        time.sleep(0.2)
        dist.destroy_process_group()


@pytest.mark.parametrize("world,absent", [(2, (1,)), (3, (2,)), (2, ())])
def test_a_rank_that_never_arrives_is_noticed_on_the_host_within_the_deadline(world, absent):
    port = 29400 + (os.getpid() % 500) + 7 * world + len(absent)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_join_worker, args=(world, port, absent, ret), nprocs=world, join=True)
        ret = dict(ret)
    for r in range(world):
        if r in absent:
            assert ret[r] == "absent"
        elif absent:
            assert ret[r].startswith("missing after 0.") and "Timeout" in ret[r], ret[r]
            assert "%d of %d ranks" % (world - len(absent), world) in ret[r]
        else:
            assert ret[r] == "joined"
