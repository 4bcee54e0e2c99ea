"""Low-rank adapters on the expert projections (the reference's add_lora / merge_lora over a MoE layer).

The checker has no adapter code of its own: it is given the folded weights W + scale * up * down, which
is the form the reference's device path computes with (gpu_model.rs:1390-1428), and the adapter
gradients are derived from its weight gradient with the identities of Lora::backward
(param.rs:690-709): d up = scale * dW * down^T, d down = scale * up^T * dW.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from gpu_common import make_pair, to_dev, to_np
from helpers import rel_l2
from oracle import GATE, UP, DOWN, SHARED_GATE, SHARED_UP, SHARED_DOWN, ROUTER
from rustingbrain_b200 import InvalidConfig, InvalidInput, MoeConfig, MoeLayer

pytestmark = pytest.mark.gpu


def _adapters(g, shapes, rank):
    out = {}
    for key, (rows, cols) in shapes.items():
        out[key] = ((g.standard_normal((rank, cols)) * 0.2).astype(np.float32),
                    (g.standard_normal((rows, rank)) * 0.2).astype(np.float32))
    return out


@pytest.mark.parametrize("precision,tol", [("f32", 1e-5), ("bf16", 2e-2)])
def test_adapters_match_the_folded_checker(precision, tol):
    T, d, E, k, F, rank, alpha = 96, 64, 4, 2, 48, 4, 8.0
    dev, ora, w = make_pair(d, E, k, F, shared=True, precision=precision, max_tokens=T, seed=17, std=0.1, router_std=0.1)
    dev.lora_attach(rank, alpha)
    scale = alpha / rank
    g = np.random.Generator(np.random.Philox(31))
    shapes = {}
    for e in range(E):
        shapes[(GATE, e)] = (F, d); shapes[(UP, e)] = (F, d); shapes[(DOWN, e)] = (d, F)
    shapes[(SHARED_GATE, 0)] = (F, d); shapes[(SHARED_UP, 0)] = (F, d); shapes[(SHARED_DOWN, 0)] = (d, F)
    ad = _adapters(g, shapes, rank)
    base = {}
    for (which, e), (down, up) in ad.items():
        dev.lora_set(which, e, down, up)
        base[(which, e)] = ora.get_weight(which, e).copy()
        ora.set_weight(which, e, base[(which, e)] + np.float32(scale) * (up @ down))
        d2, u2 = dev.lora_get(which, e)
        assert np.array_equal(d2, down) and np.array_equal(u2, up)
    x = g.standard_normal((T, d)).astype(np.float32)
    gy = g.standard_normal((T, d)).astype(np.float32)
    xd = to_dev(x, precision)
    y, cache = dev.forward_train(xd)
    yo = ora.forward(to_np(xd), logits=dev.router_cache(T)[0])
    dev.zero_grad(); ora.zero_grad()
    gyd = to_dev(gy, precision)
    gx = dev.backward(cache, gyd)
    gxo = ora.backward(to_np(gyd))
    assert rel_l2(to_np(y), yo) <= tol and rel_l2(to_np(gx), gxo) <= tol
    for (which, e), (down, up) in ad.items():
        dW = ora.get_grad(which, e)
        gd, gu = dev.lora_get_grad(which, e)
        assert rel_l2(gu, scale * dW @ down.T) <= max(tol, 2e-5), (which, e)
        assert rel_l2(gd, scale * up.T @ dW) <= max(tol, 2e-5), (which, e)
        # the base weight the caller reads back is still the frozen one
        assert np.array_equal(dev.get_weight(which, e), base[(which, e)]) or precision != "f32"

    # one Adam step moves the adapters only
    before = dev.get_weight(GATE, 1).copy()
    gd, gu = dev.lora_get_grad(DOWN, 2)
    down0, up0 = dev.lora_get(DOWN, 2)
    lr, b1, b2, eps = 1e-2, 0.9, 0.999, 1e-8
    dev.step_adam(lr=lr, beta1=b1, beta2=b2, eps=eps, step=1)

    def adam(wv, gv):
        m = (1 - b1) * gv
        v = (1 - b2) * gv * gv
        return wv - lr * (m / (1 - b1)) / (np.sqrt(v / (1 - b2)) + eps)

    down1, up1 = dev.lora_get(DOWN, 2)
    assert np.allclose(down1, adam(down0, gd), rtol=1e-4, atol=1e-6)
    assert np.allclose(up1, adam(up0, gu), rtol=1e-4, atol=1e-6)
    assert np.array_equal(dev.get_weight(GATE, 1), before)           # frozen
    assert np.array_equal(dev.get_weight(ROUTER, 0), w["router"])     # frozen, never adapted

    # merging keeps the function and removes the adapters
    y1, _ = dev.forward_train(xd)
    dev.lora_merge()
    y2, _ = dev.forward_train(xd)
    assert rel_l2(to_np(y2), to_np(y1)) <= (1e-6 if precision == "f32" else 1e-2)
    with pytest.raises(InvalidConfig):
        dev.lora_get(GATE, 0)


def test_adapter_errors():
    dev = MoeLayer(64, MoeConfig(4, 2, 32), precision="f32", max_tokens=8)
    with pytest.raises(InvalidConfig):
        dev.lora_get_grad(GATE, 0)                 # nothing attached
    with pytest.raises(InvalidConfig):
        dev.lora_attach(0)
    with pytest.raises(InvalidConfig):
        dev.lora_attach(65)
    dev.lora_attach(2)
    with pytest.raises(InvalidConfig):
        dev.lora_attach(2)                         # already attached
    with pytest.raises(InvalidInput):
        dev.lora_get(ROUTER, 0)                    # the router takes no adapter (moe.rs:502-504)
    with pytest.raises(InvalidInput):
        dev.lora_get(SHARED_GATE, 0)               # no shared expert in this layer
    q = MoeLayer(64, MoeConfig(4, 2, 64), precision="q8", max_tokens=8, training=False)
    with pytest.raises(InvalidConfig):
        q.lora_attach(2)
