"""Layer forward / backward against the CPU checker, through the C ABI.

Tolerances are the ones the task states: relative L2 <= 1e-5 for the f32 layer,
<= 2e-2 for the bf16 layer (checker evaluated in f32 on the same bf16-rounded
inputs and weights).  Routing is compared bit for bit on the device's own logits.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from gpu_common import make_pair, to_dev, to_np, assert_routing_equal
from helpers import ramp, rel_l2
from oracle import ROUTER, GATE, UP, DOWN, SHARED_GATE, SHARED_UP, SHARED_DOWN
from rustingbrain_b200 import InvalidInput, InvalidConfig, MoeConfig, MoeLayer

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 2e-2


def _fwd_bwd(dev, ora, x, gy, precision, valid=None):
    xd = to_dev(x, precision)
    y, cache = dev.forward_train(xd, valid=valid)
    logits = dev.router_cache(x.shape[0])[0]
    xo = to_np(xd)
    yo = ora.forward(xo, valid=valid, logits=logits)   # same logits -> same routing decisions
    assert_routing_equal(cache, ora)
    dev.zero_grad()
    ora.zero_grad()
    gyd = to_dev(gy, precision)
    gx = dev.backward(cache, gyd)
    gxo = ora.backward(to_np(gyd))
    return to_np(y), yo, to_np(gx), gxo, cache


def _check_grads(dev, ora, E, shared, tol):
    for e in range(E):
        for which in (GATE, UP, DOWN):
            assert rel_l2(dev.get_grad(which, e), ora.get_grad(which, e)) <= tol, (which, e)
    if shared:
        for which in (SHARED_GATE, SHARED_UP, SHARED_DOWN):
            assert rel_l2(dev.get_grad(which), ora.get_grad(which)) <= tol, which


@pytest.mark.parametrize("T,d,E,k,F,shared", [(3, 6, 4, 2, 5, True), (3, 4, 3, 2, 4, False), (9, 8, 6, 3, 4, False),
                                              (7, 8, 4, 1, 6, True), (70, 16, 5, 2, 12, True)])
def test_f32_tiny_forward_backward(T, d, E, k, F, shared):
    dev, ora, _ = make_pair(d, E, k, F, shared, seed=T, precision="f32", max_tokens=T, std=0.5, router_std=0.5)
    x = ramp(T * d, 29, 17, 8, (T, d))
    gy = ramp(T * d, 13, 11, 5, (T, d))
    y, yo, gx, gxo, cache = _fwd_bwd(dev, ora, x, gy, "f32")
    assert rel_l2(y, yo) <= F32_TOL
    assert rel_l2(gx, gxo) <= F32_TOL
    _check_grads(dev, ora, E, shared, F32_TOL)
    # the router gradient depends on logits computed in a different summation order
    assert rel_l2(dev.get_grad(ROUTER), ora.get_grad(ROUTER)) <= 1e-4
    a, z = ora.losses()
    assert abs(cache.aux_loss() - a) <= 1e-5 * abs(a) and abs(cache.z_loss() - z) <= 1e-5 * abs(z) + 1e-9


def test_f32_padding_rows_and_gradient_accumulation():
    T, d, E, k, F = 10, 8, 4, 2, 6
    dev, ora, _ = make_pair(d, E, k, F, True, seed=3, precision="f32", max_tokens=T, std=0.5, router_std=0.5)
    x = ramp(T * d, 29, 17, 8, (T, d))
    gy = ramp(T * d, 19, 13, 6, (T, d))
    valid = np.array([1, 1, 0, 1, 0, 1, 1, 1, 0, 1], np.uint8)
    y, yo, gx, gxo, cache = _fwd_bwd(dev, ora, x, gy, "f32", valid=valid)
    assert rel_l2(y, yo) <= F32_TOL and rel_l2(gx, gxo) <= F32_TOL
    e = cache.routing()[0]
    assert np.all(e[valid == 0] == -1)
    # a second backward accumulates (Param.grad semantics): gradients double
    g1 = dev.get_grad(GATE, 0).copy()
    dev.backward(cache, to_dev(gy, "f32"))
    assert rel_l2(dev.get_grad(GATE, 0), 2 * g1) <= 1e-6
    dev.zero_grad()
    assert np.all(dev.get_grad(GATE, 0) == 0)


def test_unrouted_experts_get_exactly_zero_gradient():  # moe.rs:861-893
    from helpers import one_hot_router, one_hot_rows
    dev, ora, w = make_pair(4, 4, 1, 4, aux_w=0.0, z_w=0.0, seed=10, precision="f32", max_tokens=3, std=0.5)
    r = one_hot_router(4, 4, 30.0)
    dev.set_weight(ROUTER, 0, r)
    x = one_hot_rows([0, 0, 0], 4)
    y, cache = dev.forward_train(to_dev(x, "f32"))
    dev.zero_grad()
    dev.backward(cache, to_dev(np.ones((3, 4), np.float32), "f32"))
    assert np.any(dev.get_grad(GATE, 0) != 0)
    for e in (1, 2, 3):
        assert np.all(dev.get_grad(GATE, e) == 0)
    assert cache.load_fractions().tolist() == [1.0, 0.0, 0.0, 0.0]  # moe.rs:801


def test_f32_config1_forward():
    """Benchmark configuration 1: 2048 tokens, d 512, 8 experts top-2, F 1408, no shared expert, N(0,0.02) seed 42 / N(0,1) seed 7."""
    T, d, E, k, F = 2048, 512, 8, 2, 1408
    dev, ora, _ = make_pair(d, E, k, F, False, seed=42, precision="f32", max_tokens=T, training=False)
    x = np.random.Generator(np.random.Philox(7)).standard_normal((T, d)).astype(np.float32)
    y, cache = dev.forward_train(to_dev(x, "f32"))
    logits = dev.router_cache(T)[0]
    yo = ora.forward(x, logits=logits)
    assert_routing_equal(cache, ora)
    assert rel_l2(to_np(y), yo) <= F32_TOL
    a, z = ora.losses()
    assert abs(cache.aux_loss() - a) <= 1e-5 * abs(a) and abs(cache.z_loss() - z) <= 1e-5 * abs(z)
    aux_dev, z_dev = cache.aux_loss(), cache.z_loss()
    ora.forward(x)   # the checker's own router product: logits agree to f32 rounding
    assert rel_l2(logits, ora.router_cache()[0]) <= 1e-5
    # the host-buffer entry point gives the same answer and is deterministic
    y2, _ = dev.forward_train(x)
    y3, _ = dev.forward_train(x)
    assert np.array_equal(y2, y3) and np.array_equal(y2, to_np(y))


@pytest.mark.parametrize("T,d,E,k,F,shared", [(300, 256, 8, 2, 160, True), (1000, 512, 16, 4, 352, False)])
def test_bf16_forward_backward(T, d, E, k, F, shared):
    dev, ora, _ = make_pair(d, E, k, F, shared, seed=5, precision="bf16", max_tokens=T, std=0.05, router_std=0.05)
    g = np.random.Generator(np.random.Philox(T))
    x = g.standard_normal((T, d)).astype(np.float32)
    gy = g.standard_normal((T, d)).astype(np.float32)
    y, yo, gx, gxo, cache = _fwd_bwd(dev, ora, x, gy, "bf16")
    assert rel_l2(y, yo) <= BF16_TOL
    assert rel_l2(gx, gxo) <= BF16_TOL
    _check_grads(dev, ora, E, shared, BF16_TOL)
    assert rel_l2(dev.get_grad(ROUTER), ora.get_grad(ROUTER)) <= BF16_TOL
    # determinism: no float atomics anywhere, two runs are bitwise equal
    y2, cache2 = dev.forward_train(to_dev(x, "bf16"))
    assert np.array_equal(to_np(y2), y)


def test_bf16_zipf_skew_with_empty_experts():
    """Config-3-like skew at reduced size: some experts get no rows at all, some get most."""
    T, d, E, k, F = 512, 256, 64, 8, 64
    dev, ora, w = make_pair(d, E, k, F, True, seed=123, precision="bf16", max_tokens=T, std=0.05)
    g = np.random.Generator(np.random.Philox(123))
    x = g.standard_normal((T, d)).astype(np.float32)
    x[:, d - 1] = 1.0
    r = (g.standard_normal((E, d)) / np.sqrt(d)).astype(np.float32)
    r[:, d - 1] = 4.0 * np.log(1.0 / np.arange(1, E + 1))
    dev.set_weight(ROUTER, 0, r)
    ora.set_weight(ROUTER, 0, r)
    gy = g.standard_normal((T, d)).astype(np.float32)
    y, yo, gx, gxo, cache = _fwd_bwd(dev, ora, x, gy, "bf16")
    counts = cache.routing()[2]
    assert (counts == 0).any() and counts.max() > 3 * np.median(counts[counts > 0])
    assert rel_l2(y, yo) <= BF16_TOL and rel_l2(gx, gxo) <= BF16_TOL
    _check_grads(dev, ora, E, True, BF16_TOL)


def test_adam_step_matches_the_checker():  # gpu_transformer.rs:1652 accepts 1e-3 after one step
    T, d, E, k, F = 12, 8, 4, 2, 6
    dev, ora, _ = make_pair(d, E, k, F, True, seed=9, precision="f32", max_tokens=T, std=0.5, router_std=0.5)
    x = ramp(T * d, 29, 17, 8, (T, d))
    gy = ramp(T * d, 13, 11, 5, (T, d))
    _fwd_bwd(dev, ora, x, gy, "f32")
    dev.step_adam(lr=1e-2, step=1)
    ora.adam_step(lr=1e-2, step=1)
    dev.synchronize()
    for e in range(E):
        for which in (GATE, UP, DOWN):
            np.testing.assert_allclose(dev.get_weight(which, e), ora.get_weight(which, e), atol=1e-3)
    m_d, v_d = dev.get_moments(DOWN, 1)
    m_o, v_o = ora.get_moments(DOWN, 1)
    assert rel_l2(m_d, m_o) <= 1e-5 and rel_l2(v_d, v_o) <= 1e-5
    assert np.all(dev.get_grad(DOWN, 1) == 0)


@pytest.mark.parametrize("kind", ["sgd", "lion"])
def test_sgd_and_lion_steps_match_the_checker(kind):  # param.rs:557-561, 590-613; gpu_transformer.rs:1855-1884 accepts 1e-3
    T, d, E, k, F = 12, 8, 4, 2, 6
    dev, ora, _ = make_pair(d, E, k, F, True, seed=10, precision="f32", max_tokens=T, std=0.5, router_std=0.5)
    x = ramp(T * d, 29, 17, 8, (T, d))
    gy = ramp(T * d, 13, 11, 5, (T, d))
    for _ in range(2):                       # the second Lion step reads the moment the first one left
        _fwd_bwd(dev, ora, x, gy, "f32")
        if kind == "sgd":
            dev.step_sgd(lr=0.05, scale=0.5)
            ora.sgd_step(lr=0.05, scale=0.5)
        else:
            dev.step_lion(lr=1e-2, weight_decay=0.1)
            ora.lion_step(lr=1e-2, wd=0.1)
    dev.synchronize()
    # a sign taken the wrong way round is off by twice the learning rate; entries whose smoothed gradient is
    # within rounding of zero may differ by one learning rate, so the band is checked on the rest
    for e in range(E):
        for which in (GATE, UP, DOWN):
            a, b = dev.get_weight(which, e), ora.get_weight(which, e)
            if kind == "sgd":
                np.testing.assert_allclose(a, b, atol=1e-5)
            else:
                assert np.mean(np.abs(a - b) > 1e-4) <= 0.02
    if kind == "lion":
        m_d, v_d = dev.get_moments(DOWN, 1)
        m_o, v_o = ora.get_moments(DOWN, 1)
        assert rel_l2(m_d, m_o) <= 1e-4 and np.all(v_d == 0)
    assert np.all(dev.get_grad(DOWN, 1) == 0)


def test_errors_follow_the_reference():
    cfg = MoeConfig(4, 2, 6)
    layer = MoeLayer(8, cfg, precision="f32", max_tokens=4)
    with pytest.raises(InvalidInput):      # moe.rs:248-253
        layer.forward(torch.zeros(3, 7, device="cuda"))
    with pytest.raises(InvalidInput):
        layer.forward(torch.zeros(5, 8, device="cuda"))   # more rows than max_tokens
    with pytest.raises(InvalidConfig):     # batch.rs:262-266
        layer.forward(torch.zeros(3, 8, device="cuda"), valid=np.ones(2, np.uint8))
    with pytest.raises(InvalidConfig):
        MoeLayer(40, cfg, precision="bf16", max_tokens=4)  # shape rule of the tensor-core path
    y = layer.forward(torch.zeros(0, 8, device="cuda"))    # empty batch is fine
    assert tuple(y.shape) == (0, 8)
    inf = MoeLayer(8, cfg, precision="f32", max_tokens=4, training=False)
    with pytest.raises(InvalidConfig):
        inf.backward(inf.forward_train(torch.zeros(2, 8, device="cuda"))[1], torch.zeros(2, 8, device="cuda"))
