"""Pins the CPU checker against the reference's own closed-form tests.

Each case restates a `#[test]` of the reference crate (cited by file:line) on
fixtures that need no RNG, so the checker is anchored to the reference's
behaviour and not only to itself.
"""
import numpy as np
import pytest

import oracle
from oracle import OracleMoe, ROUTER, GATE
from helpers import ramp, he_uniform_weights, one_hot_router, one_hot_rows


def make(d, E, k, F, shared=False, aux_w=0.01, z_w=1e-3, seed=1):
    m = OracleMoe(d, E, k, F, shared, aux_w, z_w)
    w = he_uniform_weights(d, E, F, shared, seed)
    m.set_weights(w["router"], w["gate"], w["up"], w["down"], w["shared"])
    return m, w


def test_invalid_top_k_is_rejected():  # moe.rs:705-710
    for E, k in ((4, 0), (4, 5), (0, 1)):
        with pytest.raises(ValueError):
            OracleMoe(8, E, k, 6)


def test_wrong_width_is_invalid_input():  # moe.rs:248-253
    m, _ = make(8, 4, 2, 6)
    with pytest.raises(ValueError):
        m.forward(np.zeros((3, 7), np.float32))


def test_routing_picks_the_highest_probability_experts():  # moe.rs:712-723
    e, g = oracle.route(np.array([[0.1, 0.3, 0.05, 0.5, 0.05]], np.float32), 2)
    assert e.tolist() == [[3, 1]]
    np.testing.assert_allclose(g[0], [0.5 / 0.8, 0.3 / 0.8], rtol=1e-6)


def test_ties_resolve_to_the_lowest_index():  # moe.rs:575-579
    e, g = oracle.route(np.full((1, 6), 1 / 6, np.float32), 3)
    assert e.tolist() == [[0, 1, 2]]


def test_gate_weights_sum_to_one_per_token():  # moe.rs:725-741
    x = np.random.Generator(np.random.Philox(3)).standard_normal((7, 8)).astype(np.float32)
    for k in range(1, 5):
        m, _ = make(8, 4, k, 6, seed=3)
        m.forward(x)
        _, gates, _, _, _ = m.routing()
        assert np.all(np.abs(gates.sum(1) - 1.0) < 1e-5)


def test_top_one_gates_are_exactly_one():  # moe.rs:743-754
    m, _ = make(8, 4, 1, 6, seed=4)
    m.forward(np.random.Generator(np.random.Philox(4)).standard_normal((6, 8)).astype(np.float32))
    _, gates, _, _, _ = m.routing()
    assert np.all(np.abs(gates - 1.0) < 1e-6)


def test_every_token_reaches_exactly_top_k_experts():  # moe.rs:756-765
    m, _ = make(8, 6, 3, 4, seed=5)
    m.forward(np.random.Generator(np.random.Philox(5)).standard_normal((9, 8)).astype(np.float32))
    expert_of, _, counts, token_of, slot_of = m.routing()
    assert counts.sum() == 27 and len(token_of) == 27
    for t in range(9):
        assert len(set(expert_of[t])) == 3
    # stable bucketing (moe.rs:266-274): slots ascend inside each expert
    start = 0
    for e in range(6):
        s = slot_of[start:start + counts[e]]
        assert np.all(np.diff(s) > 0) and np.all(expert_of.ravel()[s] == e)
        assert np.all(token_of[start:start + counts[e]] == s // 3)
        start += counts[e]


def test_balanced_routing_reaches_the_minimum_of_the_load_balancing_loss():  # moe.rs:767-787
    m, _ = make(4, 4, 1, 4, z_w=0.0, seed=6)
    m.set_weight(ROUTER, 0, one_hot_router(4, 4, 30.0))
    m.forward(one_hot_rows([0, 1, 2, 3], 4))
    aux, z = m.losses()
    assert abs(aux - 0.01) < 1e-3 and z == 0.0
    counts = m.routing()[2]
    assert np.all(np.abs(counts / counts.sum() - 0.25) < 1e-6)


def test_imbalanced_routing_costs_more_than_balanced_routing():  # moe.rs:789-802
    m, _ = make(4, 4, 1, 4, z_w=0.0, seed=6)
    m.set_weight(ROUTER, 0, one_hot_router(4, 4, 30.0))
    m.forward(one_hot_rows([0, 0, 0, 0], 4))
    aux, _ = m.losses()
    assert abs(aux - 0.04) < 1e-3 and aux > 0.01
    assert m.routing()[2].tolist() == [4, 0, 0, 0]


def test_the_z_loss_grows_with_the_router_logits():  # moe.rs:804-825
    x = one_hot_rows([0, 1, 2, 3], 4)
    zs = []
    for strength in (1.0, 20.0):
        m, _ = make(4, 4, 1, 4, seed=7)
        m.set_weight(ROUTER, 0, one_hot_router(4, 4, strength))
        m.forward(x)
        zs.append(m.losses()[1])
    assert zs[1] > zs[0] > 0.0


def test_a_disabled_z_loss_is_zero():  # moe.rs:827-836
    m, _ = make(8, 4, 2, 6, z_w=0.0, seed=8)
    m.forward(np.random.Generator(np.random.Philox(8)).standard_normal((4, 8)).astype(np.float32))
    assert m.losses()[1] == 0.0


def test_the_shared_expert_contributes_to_every_token():  # moe.rs:838-859
    x = np.random.Generator(np.random.Philox(9)).standard_normal((4, 8)).astype(np.float32)
    plain, w = make(8, 4, 1, 6, seed=9)
    with_shared = OracleMoe(8, 4, 1, 6, True)
    ws = he_uniform_weights(8, 1, 6, True, 99)["shared"]
    with_shared.set_weights(w["router"], w["gate"], w["up"], w["down"], ws)
    a, b = plain.forward(x), with_shared.forward(x)
    assert np.all(np.any(np.abs(a - b) > 1e-6, axis=1))


def test_padding_rows_are_routed_nowhere():  # batch.rs:247-249, moe.rs:559-562, gpu_model.rs:4078-4118
    logits = ramp(20, 37, 23, 11, (4, 5))
    probs, lse = oracle.softmax_rows(logits)
    assert np.all(np.abs(probs.sum(1) - 1) < 1e-5)
    mx = logits.max(1)
    np.testing.assert_allclose(lse, mx + np.log(np.exp(logits - mx[:, None]).sum(1)), atol=1e-5)
    valid = np.array([1, 1, 1, 0], np.uint8)
    e, g = oracle.route(probs, 2, valid)
    assert e[3].tolist() == [-1, -1] and g[3].tolist() == [0.0, 0.0]
    for r in range(3):
        order = sorted(range(5), key=lambda i: (-probs[r, i], i))[:2]
        assert e[r].tolist() == order
        np.testing.assert_allclose(g[r], probs[r, order] / probs[r, order].sum(), atol=1e-6)


def test_padding_is_excluded_from_the_losses_and_router_gradient():
    m, _ = make(6, 4, 2, 5, seed=21)
    x = ramp(30, 29, 17, 8, (5, 6))
    valid = np.array([1, 0, 1, 1, 0], np.uint8)
    m.forward(x, valid)
    aux_p, z_p = m.losses()
    m2, _ = make(6, 4, 2, 5, seed=21)
    m2.forward(x[valid.astype(bool)])
    aux, z = m2.losses()
    assert abs(aux - aux_p) < 1e-7 and abs(z - z_p) < 1e-7
    gi = m.backward(np.zeros((5, 6), np.float32))
    assert np.all(gi[1] == 0) and np.all(gi[4] == 0)


def test_gradients_reach_only_the_experts_a_token_was_routed_to():  # moe.rs:861-893
    m, _ = make(4, 4, 1, 4, aux_w=0.0, z_w=0.0, seed=10)
    m.set_weight(ROUTER, 0, one_hot_router(4, 4, 30.0))
    m.forward(one_hot_rows([0, 0, 0], 4))
    m.backward(np.ones((3, 4), np.float32))
    assert np.any(m.get_grad(GATE, 0) != 0)
    for e in (1, 2, 3):
        assert np.all(m.get_grad(GATE, e) == 0)


def test_backward_matches_finite_differences():  # moe.rs:895-931
    m, _ = make(6, 4, 2, 5, shared=True, aux_w=0.0, z_w=0.0, seed=11)
    x = ramp(18, 29, 17, 8, (3, 6))
    m.forward(x)
    gi = m.backward(np.ones((3, 6), np.float32))
    eps = np.float32(1e-3)
    for idx in range(18):
        b = x.copy().ravel()
        b[idx] += eps
        hi = m.forward(b.reshape(3, 6)).sum(dtype=np.float32)
        b[idx] -= 2 * eps
        lo = m.forward(b.reshape(3, 6)).sum(dtype=np.float32)
        assert abs(gi.ravel()[idx] - (hi - lo) / (2 * eps)) < 2e-2


def test_router_weight_gradient_matches_finite_differences():  # moe.rs:933-971
    m, w = make(4, 3, 2, 4, aux_w=0.0, z_w=0.0, seed=12)
    x = ramp(12, 13, 11, 5, (3, 4))
    m.forward(x)
    m.backward(np.ones((3, 4), np.float32))
    analytic = m.get_grad(ROUTER).ravel()
    eps = np.float32(1e-3)
    for idx in range(analytic.size):
        r = w["router"].copy().ravel()
        r[idx] += eps
        m.set_weight(ROUTER, 0, r.reshape(3, 4))
        hi = m.forward(x).sum(dtype=np.float32)
        r[idx] -= 2 * eps
        m.set_weight(ROUTER, 0, r.reshape(3, 4))
        lo = m.forward(x).sum(dtype=np.float32)
        assert abs(analytic[idx] - (hi - lo) / (2 * eps)) < 2e-2


def test_auxiliary_loss_gradient_matches_finite_differences():  # moe.rs:973-1013
    m, w = make(4, 3, 2, 4, seed=13)
    x = ramp(16, 19, 13, 6, (4, 4))
    m.forward(x)
    m.backward(np.zeros((4, 4), np.float32))
    analytic = m.get_grad(ROUTER).ravel()
    eps = np.float32(1e-3)
    for idx in range(analytic.size):
        r = w["router"].copy().ravel()
        r[idx] += eps
        m.set_weight(ROUTER, 0, r.reshape(3, 4))
        m.forward(x)
        hi = np.float32(sum(m.losses()))
        r[idx] -= 2 * eps
        m.set_weight(ROUTER, 0, r.reshape(3, 4))
        m.forward(x)
        lo = np.float32(sum(m.losses()))
        assert abs(analytic[idx] - (hi - lo) / (2 * eps)) < 1e-3


def test_swiglu_matches_its_definition_and_finite_differences():  # ffn.rs:274-321,345-352
    assert abs(oracle.silu(0.0)) < 1e-6 and abs(oracle.silu(10.0) - 10.0) < 1e-3
    for g in (-2.0, -0.3, 0.0, 0.7, 3.0):
        num = (oracle.silu(g + 1e-3) - oracle.silu(g - 1e-3)) / 2e-3
        assert abs(oracle.silu_derivative(g) - num) < 2e-3  # gpu_model.rs:4040-4043
    # one expert, top-1, no aux terms: the layer is a SwiGLU with gate 1
    m, w = make(4, 1, 1, 6, aux_w=0.0, z_w=0.0, seed=2)
    x = np.array([[0.5, -1.0, 2.0, 0.25], [-0.75, 1.5, 0.1, -0.3]], np.float32)
    y = m.forward(x)
    g = x @ w["gate"][0].T
    u = x @ w["up"][0].T
    ref = (g / (1 + np.exp(-g)) * u) @ w["down"][0].T
    np.testing.assert_allclose(y, ref, rtol=1e-5, atol=1e-6)
    gi = m.backward(np.ones_like(y))
    for idx in range(x.size):
        b = x.copy().ravel()
        b[idx] += 1e-3
        hi = m.forward(b.reshape(2, 4)).sum(dtype=np.float32)
        b[idx] -= 2e-3
        lo = m.forward(b.reshape(2, 4)).sum(dtype=np.float32)
        assert abs(gi.ravel()[idx] - (hi - lo) / 2e-3) < 1e-2


def test_int8_rows_follow_the_reference_scheme():  # quantized.rs:201-237
    w = (np.arange(12, dtype=np.float32) * np.float32(0.37) - 2.0).reshape(3, 4)
    x = np.array([[0.5, -1.5, 2.0, 0.25], [1.0, 1.0, -1.0, 0.0]], np.float32)
    q, s = oracle.quantize_rows(w)
    assert np.all(np.abs(oracle.q8_matmul(x, q, s) - x @ w.T) < 0.05)
    np.testing.assert_allclose(s, np.abs(w).max(1) / 127.0, rtol=1e-7)
    assert np.all(np.abs(q) <= 127) and np.all(np.abs(q).max(1) == 127)
    qz, sz = oracle.quantize_rows(np.zeros((2, 3), np.float32))
    assert np.all(qz == 0) and np.all(sz == 0)
    w2 = np.array([[0.5, -1.0, 0.25], [4.0, -2.0, 0.0]], np.float32)
    q2, s2 = oracle.quantize_rows(w2)
    assert np.all(np.abs(q2[1] * s2[1] - w2[1]) < 4.0 / 127.0)


def test_quantized_layer_tracks_the_float_layer():  # transformer.rs:2202-2280 (fake-quant == quantized)
    m, w = make(16, 4, 2, 12, shared=True, seed=31)
    x = np.random.Generator(np.random.Philox(31)).standard_normal((8, 16)).astype(np.float32)
    y = m.forward(x)
    m.quantize(include_router=False)
    yq = m.forward(x)
    assert np.linalg.norm(yq - y) / np.linalg.norm(y) < 0.03


def test_adam_step_follows_the_reference_rule():  # param.rs:562-589
    m, w = make(4, 2, 1, 3, seed=41)
    x = ramp(12, 13, 11, 5, (3, 4))
    m.forward(x)
    m.backward(np.ones((3, 4), np.float32))
    g = m.get_grad(ROUTER).astype(np.float64)
    m.adam_step(lr=1e-2, step=1)
    mm, vv = m.get_moments(ROUTER)
    np.testing.assert_allclose(mm, 0.1 * g, rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(vv, 0.001 * g * g, rtol=1e-4, atol=1e-12)
    upd = w["router"] - 1e-2 * (0.1 * g / 0.1) / (np.sqrt(0.001 * g * g / 0.001) + 1e-8)
    np.testing.assert_allclose(m.get_weight(ROUTER), upd, rtol=1e-4, atol=1e-6)
    assert np.all(m.get_grad(ROUTER) == 0)  # step clears the gradient


def test_lion_step_follows_the_reference_known_answers():  # param.rs:996-1018
    import oracle
    value, grad, m = (np.array([v], np.float32) for v in (1.0, 0.5, 0.0))
    oracle.lion_apply(value, grad, m, lr=0.1)               # Optimizer::lion(0.1): betas 0.9 / 0.99, no decay
    assert abs(value[0] - 0.9) < 1e-6 and abs(m[0] - 0.005) < 1e-7 and grad[0] == 0
    grad[0] = -0.5
    oracle.lion_apply(value, grad, m, lr=0.1)
    assert abs(value[0] - 1.0) < 1e-6 and abs(m[0] - -0.00005) < 1e-7
    # a vanished smoothed gradient moves nothing (optimizers.rs:45-58) and decay is decoupled
    value, grad, m = (np.array([v], np.float32) for v in (2.0, 0.0, 0.0))
    oracle.lion_apply(value, grad, m, lr=0.1)
    assert value[0] == 2.0
    oracle.lion_apply(value, grad, m, lr=0.1, wd=0.5)
    assert abs(value[0] - 1.9) < 1e-6


def test_sgd_and_lion_layer_steps_follow_the_rule():  # param.rs:557-561, 590-613
    for kind in ("sgd", "lion"):
        m, w = make(4, 2, 1, 3, seed=43)
        x = ramp(12, 13, 11, 5, (3, 4))
        m.forward(x)
        m.backward(np.ones((3, 4), np.float32))
        g = m.get_grad(ROUTER).astype(np.float32)
        if kind == "sgd":
            m.sgd_step(lr=0.25, scale=0.5)
            want = w["router"] - np.float32(0.25) * g * np.float32(0.5)
        else:
            m.lion_step(lr=1e-2, wd=0.1)
            want = w["router"] - np.float32(1e-2) * (np.sign(g) + np.float32(0.1) * w["router"])
            mm, vv = m.get_moments(ROUTER)
            np.testing.assert_allclose(mm, 0.01 * g, rtol=1e-5, atol=1e-9)
            assert np.all(vv == 0)                          # Lion keeps one moment
        np.testing.assert_allclose(m.get_weight(ROUTER), want, rtol=1e-6, atol=1e-7)
        assert np.all(m.get_grad(ROUTER) == 0)
