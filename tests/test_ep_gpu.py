"""Expert parallelism on real GPUs: N ranks against one CPU checker over the concatenated batch."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _world():
    """Every visible GPU takes part, as 2, 4 or 8 ranks (8 experts: at 8 ranks each rank owns one)."""
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 1


def _worker(rank, world, port, precision, transport, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import OracleMoe, ROUTER, GATE, UP, DOWN, SHARED_GATE
        from helpers import seeded_weights, rel_l2
        from rustingbrain_b200 import MoeConfig
        from rustingbrain_b200.ep import ExpertParallelMoe
        d, E, k, F = 256, 8, 2, 96
        Ts = [200 + 56 * r for r in range(world)]
        tol = 1e-5 if precision == "f32" else 2e-2
        w = seeded_weights(d, E, F, True, 21, std=0.05, router_std=0.05)
        if precision != "f32":
            rb = lambda a: torch.from_numpy(a).bfloat16().float().numpy()
            w = dict(w, gate=rb(w["gate"]), up=rb(w["up"]), down=rb(w["down"]), shared=tuple(rb(s) for s in w["shared"]))
        layer = ExpertParallelMoe(d, MoeConfig(E, k, F, True), precision=precision, max_tokens=max(Ts), device=rank,
                                  capacity_factor=2.0, transport=transport)
        layer.set_weight(ROUTER, 0, w["router"])
        for e in layer.owned_experts():
            layer.set_weight(GATE, e, w["gate"][e]); layer.set_weight(UP, e, w["up"][e]); layer.set_weight(DOWN, e, w["down"][e])
        for i, s in enumerate(w["shared"]):
            layer.set_weight(SHARED_GATE + i, 0, s)
        gens = [np.random.Generator(np.random.Philox(50 + r)) for r in range(world)]
        xs = [g.standard_normal((T, d)).astype(np.float32) for g, T in zip(gens, Ts)]
        gys = [g.standard_normal((T, d)).astype(np.float32) for g, T in zip(gens, Ts)]
        dt = torch.float32 if precision == "f32" else torch.bfloat16
        x = torch.from_numpy(xs[rank]).cuda().to(dt)
        gy = torch.from_numpy(gys[rank]).cuda().to(dt)
        if os.environ.get("MOE_B200_OVERLAP", "0") != "0":
            # passes on other data first: with overlap their weight gradients may still run while the
            # checked pass dispatches, and the double-buffered halves alternate
            for scale in (0.5, -1.5):
                _, c0 = layer.forward_train(x * scale)
                layer.zero_grad()
                layer.backward(c0, gy * scale)
        y, cache = layer.forward_train(x)
        layer.zero_grad()
        gx = layer.backward(cache, gy)
        logits = layer.router_cache(Ts[rank])[0]
        all_logits = [None] * world
        dist.all_gather_object(all_logits, logits)
        # single-device checker over the concatenated batch, fed the devices' own logits
        rnd = (lambda a: torch.from_numpy(a).to(dt).float().numpy())
        ora = OracleMoe(d, E, k, F, True)
        ora.set_weights(w["router"], w["gate"], w["up"], w["down"], w["shared"])
        yo = ora.forward(rnd(np.concatenate(xs)), logits=np.concatenate(all_logits))
        gxo = ora.backward(rnd(np.concatenate(gys)))
        lo, hi = sum(Ts[:rank]), sum(Ts[:rank + 1])
        ok = True
        e_dev = cache.routing()[0]
        ok &= np.array_equal(e_dev, ora.routing()[0][lo:hi])
        ok &= rel_l2(y.float().cpu().numpy(), yo[lo:hi]) <= tol
        ok &= rel_l2(gx.float().cpu().numpy(), gxo[lo:hi]) <= tol
        a, z = ora.losses()
        ok &= abs(cache.aux_loss() - a) <= 1e-4 * abs(a) and abs(cache.z_loss() - z) <= 1e-4 * abs(z)
        for e in layer.owned_experts():
            for which in (GATE, UP, DOWN):
                ok &= rel_l2(layer.get_grad(which, e), ora.get_grad(which, e)) <= tol
        ok &= rel_l2(layer.get_grad(ROUTER), ora.get_grad(ROUTER)) <= max(tol, 1e-4)
        ok &= rel_l2(layer.get_grad(SHARED_GATE), ora.get_grad(SHARED_GATE)) <= tol
        # a second backward without zero_grad accumulates (Param.grad semantics, accumulate_step
        # transformer.rs:1519): every gradient doubles, the replicated ones included
        if os.environ.get("MOE_B200_OVERLAP", "0") == "0":
            first = {(which, e): layer.get_grad(which, e).copy() for e in layer.owned_experts() for which in (GATE, UP, DOWN)}
            first[(ROUTER, 0)] = layer.get_grad(ROUTER).copy()
            first[(SHARED_GATE, 0)] = layer.get_grad(SHARED_GATE).copy()
            layer.backward(cache, gy)
            for (which, e), g1 in first.items():
                ok &= rel_l2(layer.get_grad(which, e), 2 * g1) <= 1e-5
        ret[rank] = bool(ok)
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("precision,transport,overlap", [
    ("f32", "nccl", "0"), ("bf16", "nccl", "0"), ("f32", "peer", "0"), ("bf16", "peer", "0"),
    ("bf16", "peer", "1"), ("bf16", "peer", "2"), ("bf16", "nccl", "2"),
    ("bf16", "peer", "0-rowperslot")])   # the gradient push with one row per slot instead of one per destination rank
def test_expert_parallel_matches_single_device(precision, transport, overlap, monkeypatch):
    if overlap.endswith("-rowperslot"):
        overlap = overlap.split("-")[0]
        monkeypatch.setenv("MOE_B200_EP_DEDUP", "0")
    monkeypatch.setenv("MOE_B200_OVERLAP", overlap)   # read by the spawned ranks' copy of the library
    world = _world()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = 29700 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, precision, transport, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def _overflow_worker(rank, world, port, transport, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from helpers import seeded_weights
        from oracle import ROUTER, GATE, UP, DOWN
        from rustingbrain_b200 import MoeConfig, InvalidInput
        from rustingbrain_b200.ep import ExpertParallelMoe
        d, E, k, F, T = 128, 8, 2, 64, 1024
        w = seeded_weights(d, E, F, False, 3, std=0.05, router_std=0.05)
        # room for 1.1 x the balanced share (plus group padding): enough for a balanced batch, not for
        # one whose every token goes to the same rank
        layer = ExpertParallelMoe(d, MoeConfig(E, k, F, False), precision="bf16", max_tokens=T, device=rank,
                                  capacity_factor=1.1, transport=transport)
        router = w["router"].copy()
        router[:, d - 1] = 0.0
        router[:E // world, d - 1] = 8.0          # a constant input column sends every token to rank 0's experts
        layer.set_weight(ROUTER, 0, router)
        for e in layer.owned_experts():
            layer.set_weight(GATE, e, w["gate"][e]); layer.set_weight(UP, e, w["up"][e]); layer.set_weight(DOWN, e, w["down"][e])
        g = np.random.Generator(np.random.Philox(70 + rank))
        x = g.standard_normal((T, d)).astype(np.float32)
        x[:, d - 1] = 1.0
        refused = False
        try:
            layer.forward_train(torch.from_numpy(x).cuda().bfloat16())
            layer.synchronize()                    # the peer transport reports through a device flag
        except InvalidInput as e:
            refused = "ep_capacity_factor" in str(e)
        # nothing was written past a buffer and the handle is not poisoned: a balanced batch still runs
        x[:, d - 1] = 0.0
        y, cache = layer.forward_train(torch.from_numpy(x).cuda().bfloat16())
        layer.synchronize()
        counts = cache.routing()[2]
        ok = refused and bool(torch.isfinite(y.float()).all()) and int(counts.sum()) == T * k
        if not ok:
            print("rank", rank, "refused", refused, "counts", counts.tolist(), flush=True)
        ret[rank] = bool(ok)
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_rows_beyond_a_ranks_capacity_are_refused_on_every_rank(transport):
    """Dropless routing: when one rank's experts receive more rows than its buffers hold, every rank
    gets InvalidInput (nobody sends), no memory is touched out of bounds and the handles stay usable."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    port = 29900 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_overflow_worker, args=(2, port, transport, ret), nprocs=2, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_one_process_can_hold_layers_on_two_devices():
    """The opt-in to large dynamic shared memory is a per-device attribute of the tensor-core kernels: a second
    device used from the same process must get it too (bf16 layer -> grouped GEMM; head_dim 128 cache -> the
    decode-attention kernel with 96 KB of shared memory)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import seeded_weights
    from rustingbrain_b200 import MoeConfig, MoeLayer
    from rustingbrain_b200.kv_attention import KvCache
    d, E, k, F, T = 128, 4, 2, 64, 96
    w = seeded_weights(d, E, F, False, 5, std=0.05, router_std=0.05)
    x = np.random.Generator(np.random.Philox(9)).standard_normal((T, d)).astype(np.float32)
    outs = []
    for dev in (0, 1):
        torch.cuda.set_device(dev)
        layer = MoeLayer(d, MoeConfig(E, k, F), precision="bf16", max_tokens=T, device=dev, training=False)
        layer.set_weights(w["router"], w["gate"], w["up"], w["down"], None)
        y = layer.forward(torch.from_numpy(x).to("cuda:%d" % dev).bfloat16())
        layer.synchronize()
        outs.append(y.float().cpu().numpy())
        cache = KvCache(2, 4, 2, 128, capacity=64, precision="bf16", device=dev)
        q = torch.randn(2, 4 * 128, device="cuda:%d" % dev).bfloat16()
        kv = torch.randn(2, 2 * 128, device="cuda:%d" % dev).bfloat16()
        out = cache.forward_cached(q, kv, kv.clone())
        torch.cuda.synchronize(dev)
        assert bool(torch.isfinite(out.float()).all())
        layer.close()
    torch.cuda.set_device(0)
    assert np.array_equal(outs[0], outs[1])
