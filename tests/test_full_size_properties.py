"""Benchmark configurations 3 (16384 tokens, d_model 2048, 64 experts top-8 + shared, d_ff 1408,
Zipf-like router bias) and 4 (one rank's 32768 tokens, d_model 4096, 64 experts top-8, d_ff 1536,
uniform expected load) at their full sizes in bf16, checked through properties that do not need the
CPU checker to run the whole batch:

* routing of the whole batch equals the checker's routing of the device's own logits;
* the forward and the input gradient of a token depend on that token alone (load-balancing and
  z-loss weights are 0 here), so a subset of tokens run through the checker must reproduce the
  device's rows for those tokens;
* weight gradients are sums over tokens: the gradient of the whole batch equals the sum of the
  gradients of its two halves;
* two runs are bitwise equal (no float atomics anywhere).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from helpers import rel_l2
import oracle
from oracle import OracleMoe, ROUTER, GATE, UP, DOWN, SHARED_GATE, SHARED_DOWN
from rustingbrain_b200 import MoeConfig, MoeLayer

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


def _round_bf16(a):
    return torch.from_numpy(a).bfloat16().float().numpy()


@pytest.mark.parametrize("T,d,E,k,F,shared,zipf,seed", [(16384, 2048, 64, 8, 1408, True, True, 123),
                                                        (32768, 4096, 64, 8, 1536, False, False, 2024)])
def test_full_size_properties(T, d, E, k, F, shared, zipf, seed):
    g = np.random.Generator(np.random.Philox(seed))
    cfg = MoeConfig(E, k, F, shared, 0.0, 0.0)
    dev = MoeLayer(d, cfg, precision="bf16", max_tokens=T)
    ora = OracleMoe(d, E, k, F, shared, 0.0, 0.0)

    def put(which, e, rows, cols, std=0.02):
        w = _round_bf16((g.standard_normal((rows, cols)) * std).astype(np.float32))
        dev.set_weight(which, e, w)
        ora.set_weight(which, e, w)

    # router: N(0, 1/sqrt(d)) columns plus a bias column realising 1.5 * log(1 / rank)
    r = (g.standard_normal((E, d)) / np.sqrt(d)).astype(np.float32)
    r[:, d - 1] = 1.5 * np.log(1.0 / np.arange(1, E + 1)) if zipf else 0.0
    dev.set_weight(ROUTER, 0, r)
    ora.set_weight(ROUTER, 0, r)
    for e in range(E):
        put(GATE, e, F, d); put(UP, e, F, d); put(DOWN, e, d, F)
    if shared:
        for i, (rows, cols) in enumerate(((F, d), (F, d), (d, F))):
            put(SHARED_GATE + i, 0, rows, cols)

    x = _round_bf16(g.standard_normal((T, d)).astype(np.float32))
    x[:, d - 1] = 1.0
    gy = _round_bf16(g.standard_normal((T, d)).astype(np.float32))
    xd, gyd = torch.from_numpy(x).cuda().bfloat16(), torch.from_numpy(gy).cuda().bfloat16()

    y, cache = dev.forward_train(xd)
    dev.zero_grad()
    gx = dev.backward(cache, gyd)
    y, gx = y.float().cpu().numpy(), gx.float().cpu().numpy()
    logits = dev.router_cache(T)[0]
    e_dev, g_dev, counts, token_of, slot_of = cache.routing()

    # 1. routing of the whole batch (the checker's route() is cheap: T x E)
    e_ref, g_ref = oracle.route(oracle.softmax_rows(logits)[0], k)
    assert np.array_equal(e_dev, e_ref)
    assert np.max(np.abs(g_dev - g_ref)) <= 1e-6
    assert counts.sum() == T * k
    if zipf:
        assert counts[0] > 4 * counts[-1]                                  # the skew is there
    order = np.lexsort((np.arange(T * k), e_dev.ravel()))                  # stable sort of the slots by expert
    assert np.array_equal(slot_of, order.astype(np.int32)) and np.array_equal(token_of, (order // k).astype(np.int32))

    # 2. a subset of tokens through the checker reproduces the device's rows
    sub = np.arange(7, T, T // 192)
    yo = ora.forward(x[sub], logits=logits[sub])
    ora.zero_grad()
    gxo = ora.backward(gy[sub])
    assert rel_l2(y[sub], yo) <= BF16_TOL
    assert rel_l2(gx[sub], gxo) <= BF16_TOL

    # 3. weight gradients add up over a split of the batch
    picks = [(GATE, 0), (UP, 1), (DOWN, 2), (GATE, 40), (DOWN, 63), (ROUTER, 0)]
    if shared:
        picks += [(SHARED_GATE, 0), (SHARED_DOWN, 0)]
    whole = {p: dev.get_grad(*p) for p in picks}
    halves = {p: 0.0 for p in picks}
    for lo, hi in ((0, T // 2), (T // 2, T)):
        _, c = dev.forward_train(xd[lo:hi])
        dev.zero_grad()
        dev.backward(c, gyd[lo:hi])
        for p in picks:
            halves[p] = halves[p] + dev.get_grad(*p)
    for p in picks:
        assert rel_l2(halves[p], whole[p]) <= 2e-3, p

    # 4. determinism
    y2, c2 = dev.forward_train(xd)
    dev.zero_grad()
    gx2 = dev.backward(c2, gyd)
    assert np.array_equal(y2.float().cpu().numpy(), y) and np.array_equal(gx2.float().cpu().numpy(), gx)
    for p in picks[:3]:
        assert np.array_equal(dev.get_grad(*p), whole[p])
