"""The RMSNorm checker against the reference's own tests (norm.rs:138-216).  No GPU."""
import numpy as np

from oracle import norm as ora


def test_forward_normalizes_to_unit_rms():  # norm.rs:138-147
    y = ora.forward(np.array([[1.0, 2.0, 3.0, 4.0]], np.float32), np.ones(4, np.float32), 1e-6)
    assert abs((y * y).sum() / 4.0 - 1.0) < 1e-4


def test_forward_does_not_subtract_the_mean():  # norm.rs:149-159
    y = ora.forward(np.full((1, 3), 5.0, np.float32), np.ones(3, np.float32), 1e-6)
    assert np.abs(y - 1.0).max() < 1e-4


def test_weight_scales_each_channel():  # norm.rs:161-170
    y = ora.forward(np.ones((1, 2), np.float32), np.array([2.0, 0.5], np.float32), 1e-6)
    assert abs(y[0, 0] - 2.0) < 1e-4 and abs(y[0, 1] - 0.5) < 1e-4


def _fd(fn, base, eps=1e-3):
    out = np.zeros(base.size)
    flat = base.reshape(-1)
    for i in range(base.size):
        hi, lo = flat.copy(), flat.copy()
        hi[i] += eps; lo[i] -= eps
        out[i] = (fn(hi.reshape(base.shape)) - fn(lo.reshape(base.shape))) / (2 * eps)
    return out.reshape(base.shape)


def test_backward_matches_finite_differences():  # norm.rs:172-196, same inputs and tolerance
    w = np.array([1.5, 0.5, -2.0, 1.0], np.float32)
    x = np.array([[0.3, -1.2, 2.5, 0.1], [-0.7, 0.4, 1.1, -1.9]], np.float32)
    gx, _ = ora.backward(x, w, np.ones_like(x), 1e-6)
    numeric = _fd(lambda v: float(ora.forward(v.astype(np.float32), w, 1e-6).sum(dtype=np.float32)), x)
    assert np.abs(gx - numeric).max() < 1e-2


def test_weight_gradient_matches_finite_differences():  # norm.rs:198-216
    x = np.array([[0.5, -1.0, 2.0], [1.5, 0.25, -0.5]], np.float32)
    w = np.ones(3, np.float32)
    _, gw = ora.backward(x, w, np.ones_like(x), 1e-6)
    numeric = _fd(lambda v: float(ora.forward(x, v.astype(np.float32), 1e-6).sum(dtype=np.float32)), w)
    assert np.abs(gw - numeric).max() < 1e-2


def test_the_weight_gradient_accumulates_and_tiles_add_in_order():  # norm.rs:8-14, 112-117
    g = np.random.Generator(np.random.Philox(3))
    x = g.standard_normal((70, 16)).astype(np.float32)
    gy = g.standard_normal((70, 16)).astype(np.float32)
    w = g.standard_normal(16).astype(np.float32)
    _, once = ora.backward(x, w, gy, 1e-6)
    _, twice = ora.backward(x, w, gy, 1e-6, grad_weight=once)
    assert np.allclose(twice, 2 * once, rtol=1e-6)
    inv = ora.inverse_rms(x, 1e-6)
    assert np.allclose(once, (gy * x * inv[:, None]).sum(axis=0), rtol=1e-5, atol=1e-6)
