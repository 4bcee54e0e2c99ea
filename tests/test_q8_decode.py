"""int8 expert weights on the decode path against the checker's Quantized restatement."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from helpers import rel_l2
from gpu_common import assert_routing_equal
from oracle import OracleMoe, ROUTER, GATE, UP, DOWN, SHARED_GATE, SHARED_UP, SHARED_DOWN
from rustingbrain_b200 import MoeConfig, MoeLayer, InvalidConfig

pytestmark = pytest.mark.gpu


def _pair(T, d, E, k, F, shared, seed):
    g = np.random.Generator(np.random.Philox(seed))
    dev = MoeLayer(d, MoeConfig(E, k, F, shared), precision="q8", max_tokens=T, training=False)
    ora = OracleMoe(d, E, k, F, shared)
    router = (g.standard_normal((E, d)) * 0.05).astype(np.float32)
    dev.set_weight(ROUTER, 0, router)
    ora.set_weight(ROUTER, 0, router)

    def put(which, expert, rows, cols):
        q = g.integers(-127, 128, (rows, cols)).astype(np.int8)      # benchmark configuration 5: uniform in [-127, 127]
        s = g.uniform(1e-3, 4e-3, rows).astype(np.float32)           # scales uniform in [1e-3, 4e-3]
        dev.set_weight_q8(which, expert, q, s)
        ora.set_weight_q8(which, expert, q, s)

    for e in range(E):
        put(GATE, e, F, d); put(UP, e, F, d); put(DOWN, e, d, F)
    if shared:
        put(SHARED_GATE, 0, F, d); put(SHARED_UP, 0, F, d); put(SHARED_DOWN, 0, d, F)
    x = g.standard_normal((T, d)).astype(np.float32)
    return dev, ora, x


@pytest.mark.parametrize("T,d,E,k,F,shared", [(64, 1024, 16, 2, 2816, True),   # benchmark configuration 5
                                              (200, 128, 4, 2, 96, True),      # many rows per expert, padded d_ff
                                              (5, 64, 8, 1, 64, False),        # most experts empty
                                              (33, 256, 64, 8, 64, True)])     # the widest shape of the one-launch routing
def test_q8_forward_matches_the_quantized_checker(T, d, E, k, F, shared):
    dev, ora, x = _pair(T, d, E, k, F, shared, seed=9)
    xd = torch.from_numpy(x).cuda().bfloat16()
    y, cache = dev.forward_train(xd)
    logits = dev.router_cache(T)[0]
    yo = ora.forward(xd.float().cpu().numpy(), logits=logits)
    assert np.array_equal(cache.routing()[0], ora.routing()[0])
    assert np.array_equal(cache.routing()[2], ora.routing()[2])
    assert rel_l2(y.float().cpu().numpy(), yo) <= 2e-2
    y2 = dev.forward(xd)
    assert torch.equal(y, y2)


def test_padding_rows_of_a_decode_batch_are_routed_nowhere():  # batch.rs:225-269 through the one-launch routing
    T, d, E, k, F = 40, 128, 16, 2, 96
    dev, ora, x = _pair(T, d, E, k, F, True, seed=13)
    valid = np.ones(T, np.uint8)
    valid[[0, 7, 8, 31, 39]] = 0
    xd = torch.from_numpy(x).cuda().bfloat16()
    y, cache = dev.forward_train(xd, valid=valid)
    logits = dev.router_cache(T)[0]
    yo = ora.forward(xd.float().cpu().numpy(), valid=valid, logits=logits)
    assert_routing_equal(cache, ora)             # expert_of, counts and the permutation bit-equal, gates to 1e-6
    assert np.all(cache.routing()[0][valid == 0] == -1)
    a_o, z_o = ora.losses()
    assert abs(cache.auxiliary_loss() - (a_o + z_o)) <= 1e-6 * max(1.0, abs(a_o + z_o))
    keep = valid != 0
    assert rel_l2(y.float().cpu().numpy()[keep], yo[keep]) <= 2e-2


def test_a_quantized_router_routes_like_the_checkers():  # transformer.rs:899-910: quantize() includes the router
    T, d, E, k, F = 48, 128, 8, 2, 64
    dev, ora, x = _pair(T, d, E, k, F, True, seed=12)
    g = np.random.Generator(np.random.Philox(13))
    q = g.integers(-127, 128, (E, d)).astype(np.int8)
    s = g.uniform(1e-3, 4e-3, E).astype(np.float32)
    dev.set_weight_q8(ROUTER, 0, q, s)
    ora.set_weight_q8(ROUTER, 0, q, s)
    np.testing.assert_allclose(dev.get_weight(ROUTER), q.astype(np.float32) * s[:, None], rtol=0, atol=0)
    xd = torch.from_numpy(x).cuda().bfloat16()
    y, cache = dev.forward_train(xd)
    logits = dev.router_cache(T)[0]
    yo = ora.forward(xd.float().cpu().numpy(), logits=logits)
    assert np.array_equal(cache.routing()[0], ora.routing()[0])
    assert rel_l2(y.float().cpu().numpy(), yo) <= 2e-2
    # the devices' own logits are those of the quantized router to bf16 rounding of its weights
    want = xd.float().cpu().numpy() @ (q.astype(np.float32) * s[:, None]).T
    assert rel_l2(logits, want) <= 1e-2


def test_activations_beyond_the_f16_range_saturate_instead_of_becoming_infinite():
    """The int8 kernels multiply in f16: a bf16 activation (or hidden value) beyond 65504 is clamped to +-65504 when
    the token tile is staged, so an outlier gives a finite row and leaves the other rows of the batch alone."""
    T, d, E, k, F = 8, 64, 4, 2, 64
    dev, ora, x = _pair(T, d, E, k, F, False, seed=4)
    x[3, 7] = 3.0e6
    x[5, 9] = -1.0e30
    xd = torch.from_numpy(x).cuda().bfloat16()
    y, cache = dev.forward_train(xd)
    assert bool(torch.isfinite(y.float()).all())
    logits = dev.router_cache(T)[0]
    yo = ora.forward(xd.float().cpu().numpy(), logits=logits)
    others = [t for t in range(T) if t not in (3, 5)]
    assert rel_l2(y.float().cpu().numpy()[others], yo[others]) <= 2e-2


def test_a_quantized_layer_refuses_to_train():  # transformer.rs:2202-2280: quantizing is one-way
    with pytest.raises(InvalidConfig):
        MoeLayer(64, MoeConfig(4, 2, 64), precision="q8", max_tokens=8, training=True)


def test_the_tensor_core_variant_passes_the_same_parity_cases():
    """MOE_B200_Q8_TC=1 routes both projections through the tcgen05 kernel (decode_q8_tc.cu); the switch is read
    once per process, so the parity cases above run again in a child process with it set."""
    import os, subprocess, sys
    env = dict(os.environ, MOE_B200_Q8_TC="1")
    here = os.path.dirname(os.path.abspath(__file__))
    out = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_q8_decode.py"), "-q", "-x",
                          "-k", "matches_the_quantized_checker", "-p", "no:cacheprovider"],
                         env=env, cwd=os.path.dirname(here), capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "4 passed" in out.stdout
