"""Expert-parallel host logic on CPU: two gloo ranks exchange rows according to the library's plan.

Each rank routes its own tokens with the CPU checker, the count matrix is all-gathered,
`moe_ep_plan` gives every rank its send offsets and receive rows, and the rows are moved
with gloo send/recv exactly as the library moves them with NCCL.  The rows that arrive for
each local expert must be the rows a single rank would have dispatched to that expert from
the concatenated batch (stable order: source rank, then slot).
"""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import OracleMoe
        from helpers import seeded_weights
        from rustingbrain_b200.ep import exchange_plan
        d, E, k, F, T = 16, 8, 3, 8, 37 + 5 * rank
        w = seeded_weights(d, E, F, False, 4, std=0.5, router_std=0.7)
        ora = OracleMoe(d, E, k, F)
        ora.set_weights(w["router"], w["gate"], w["up"], w["down"])
        x = np.random.Generator(np.random.Philox(100 + rank)).standard_normal((T, d)).astype(np.float32)
        ora.forward(x)
        _, _, counts, token_of, _ = ora.routing()
        gathered = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts.astype(np.int32)))
        counts_all = torch.stack(gathered).numpy()
        plan = exchange_plan(counts_all, rank)
        El = E // world
        send = x[token_of]                        # compact expert-major send buffer
        recv = np.full((plan["rows"], d), np.nan, np.float32)
        ops = []
        keep = []
        for p in range(world):
            for l in range(El):
                e = p * El + l
                n_out = int(counts_all[rank, e])
                n_in = int(counts_all[p, rank * El + l])
                lo = int(plan["send_off"][e])
                ro = int(plan["recv_row"][p, l])
                if p == rank:
                    recv[ro:ro + n_out] = send[lo:lo + n_out]
                    continue
                if n_out:
                    t = torch.from_numpy(np.ascontiguousarray(send[lo:lo + n_out]))
                    keep.append(t)
                    ops.append(dist.P2POp(dist.isend, t, p))
                if n_in:
                    t = torch.empty(n_in, d)
                    keep.append((t, ro, n_in))
                    ops.append(dist.P2POp(dist.irecv, t, p))
        for r in (dist.batch_isend_irecv(ops) if ops else []):
            r.wait()
        for item in keep:
            if isinstance(item, tuple):
                t, ro, n = item
                recv[ro:ro + n] = t.numpy()
        # what one device would do with every rank's tokens
        xs = [torch.zeros(37 + 5 * r, d) for r in range(world)]
        dist.all_gather_object(obj := [None] * world, x)
        whole = np.concatenate(obj)
        ref = OracleMoe(d, E, k, F)
        ref.set_weights(w["router"], w["gate"], w["up"], w["down"])
        ref.forward(whole)
        _, _, c_ref, tok_ref, _ = ref.routing()
        off = np.concatenate([[0], np.cumsum(c_ref)])
        ok = True
        for l in range(El):
            e = rank * El + l
            want = whole[tok_ref[off[e]:off[e + 1]]]
            got = recv[plan["local_row0"][l]:plan["local_row0"][l] + plan["local_counts"][l]]
            ok &= plan["local_counts"][l] == c_ref[e] and np.array_equal(got, want)
            ok &= plan["local_row0"][l] % 128 == 0
        ok &= plan["send_off"][-1] == T * k
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_matches_single_rank_dispatch():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_plan_shapes_and_offsets():
    sys.path.insert(0, ROOT)
    from rustingbrain_b200.ep import exchange_plan
    counts = np.array([[3, 0, 200, 1], [5, 129, 0, 0]], np.int32)
    p0, p1 = exchange_plan(counts, 0), exchange_plan(counts, 1)
    assert p0["send_off"].tolist() == [0, 3, 3, 203, 204] and p1["send_off"].tolist() == [0, 5, 134, 134, 134]
    assert p0["local_counts"].tolist() == [8, 129] and p0["local_row0"].tolist() == [0, 128, 384]
    assert p0["recv_row"].tolist() == [[0, 128], [3, 128]] and p0["local_tiles"].tolist() == [0, 1, 3]
    assert p1["local_counts"].tolist() == [200, 1] and p1["rows"] == 256 + 128
    assert p1["recv_row"].tolist() == [[0, 256], [200, 257]]


def test_wrapper_needs_a_process_group():
    """The expert-parallel wrapper refuses to build before torch.distributed is initialised
    (a rank that never joined must not get as far as creating a communicator)."""
    import torch.distributed as dist
    from rustingbrain_b200 import MoeConfig
    from rustingbrain_b200.ep import ExpertParallelMoe
    assert not dist.is_initialized()
    with pytest.raises(RuntimeError, match="torch.distributed"):
        ExpertParallelMoe(64, MoeConfig(4, 2, 32))


def test_plan_rejects_inconsistent_arguments():
    from rustingbrain_b200.ep import exchange_plan
    counts = np.zeros((2, 6), np.int32)
    with pytest.raises(ValueError):
        exchange_plan(counts, rank=2)            # no such rank
    with pytest.raises(ValueError):
        exchange_plan(np.zeros((4, 6), np.int32), rank=0)   # 6 experts do not split over 4 ranks
