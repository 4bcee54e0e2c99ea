"""Router from given logits: top-k indices, counts and the permutation are bit-exact against the checker."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from gpu_common import make_pair, to_dev, assert_routing_equal
from helpers import ramp

pytestmark = pytest.mark.gpu


def _run(T, E, k, logits, valid=None, d=16, F=8):
    dev, ora, _ = make_pair(d, E, k, F, max_tokens=max(T, 1), training=False)
    x = np.random.Generator(np.random.Philox(5)).standard_normal((T, d)).astype(np.float32)
    lg = torch.from_numpy(logits).cuda()
    _, cache = dev.forward_train(to_dev(x, "f32"), valid=valid, logits=lg)
    ora.forward(x, valid=valid, logits=logits)
    assert_routing_equal(cache, ora)
    _, probs, lse = dev.router_cache(T)
    _, p_o, l_o = ora.router_cache()
    assert np.array_equal(probs, p_o), "probabilities differ in %d places" % int((probs != p_o).sum())
    np.testing.assert_allclose(lse, l_o, rtol=0, atol=2e-6)
    a_d, z_d = cache.aux_loss(), cache.z_loss()
    a_o, z_o = ora.losses()
    assert abs(a_d - a_o) <= 1e-5 * abs(a_o) + 1e-9 and abs(z_d - z_o) <= 1e-5 * abs(z_o) + 1e-9
    return cache


def test_reference_ramp_with_a_padding_row():  # gpu_model.rs:4052-4137
    logits = ramp(20, 37, 23, 11, (4, 5))
    cache = _run(4, 5, 2, logits, valid=np.array([1, 1, 1, 0], np.uint8))
    e, g = cache.routing()[:2]
    assert e[3].tolist() == [-1, -1] and g[3].tolist() == [0.0, 0.0]


@pytest.mark.parametrize("k", [1, 2, 3, 4])
def test_small_layers(k):  # moe.rs:725-765
    logits = np.random.Generator(np.random.Philox(k)).standard_normal((7, 4)).astype(np.float32)
    cache = _run(7, 4, k, logits)
    e, g, c = cache.routing()[:3]
    assert c.sum() == 7 * k and np.all(np.abs(g.sum(1) - 1) < 1e-5)
    if k == 1:
        assert np.all(g == 1.0)


def test_ties_and_near_ties():
    T, E, k = 96, 16, 4
    g = np.random.Generator(np.random.Philox(11))
    logits = g.standard_normal((T, E)).astype(np.float32)
    logits[0] = 0.25                      # all equal: experts 0..k-1
    logits[1, :] = logits[1, 0]           # all equal again
    logits[2, 5] = logits[2, 9]           # exact pair
    for t in range(3, 40):                # pairs one ulp apart
        a, b = g.integers(0, E, 2)
        logits[t, b] = np.nextafter(logits[t, a], np.float32(np.inf))
    logits[40:48] = np.round(logits[40:48] * 2) / 2   # many exact ties on a coarse grid
    cache = _run(T, E, k, logits)
    assert cache.routing()[0][0].tolist() == [0, 1, 2, 3]


def test_config1_shape_routing():
    T, E, k = 2048, 8, 2
    logits = np.random.Generator(np.random.Philox(7)).standard_normal((T, E)).astype(np.float32)
    _run(T, E, k, logits)


def test_config3_shape_routing_with_zipf_bias():
    T, E, k = 16384, 64, 8
    g = np.random.Generator(np.random.Philox(123))
    logits = (g.standard_normal((T, E)) + 1.5 * np.log(1.0 / np.arange(1, E + 1))).astype(np.float32)
    cache = _run(T, E, k, logits)
    counts = cache.routing()[2]
    assert counts.sum() == T * k and counts[0] > 4 * counts[-1]


def test_ragged_token_counts_and_all_padding():
    for T in (1, 63, 64, 65, 130):
        logits = np.random.Generator(np.random.Philox(T)).standard_normal((T, 6)).astype(np.float32)
        valid = (np.arange(T) % 3 != 1).astype(np.uint8)
        _run(T, 6, 3, logits, valid=valid)
    logits = np.random.Generator(np.random.Philox(3)).standard_normal((5, 6)).astype(np.float32)
    cache = _run(5, 6, 2, logits, valid=np.zeros(5, np.uint8))
    assert cache.routing()[2].sum() == 0 and cache.auxiliary_loss() == 0.0


def test_the_largest_expert_count():
    """256 experts (the library's limit): 64 per lane in the four-lane top-k scan, more statistics
    columns than threads in the small-batch finalize."""
    for T, k in ((300, 4), (5000, 16)):
        logits = np.random.Generator(np.random.Philox(256 + T)).standard_normal((T, 256)).astype(np.float32)
        logits[::7] = np.round(logits[::7] * 4) / 4       # ties across lane ranges
        _run(T, 256, k, logits)
