"""moe_route_noalloc: the routing step for callers that must not let the library allocate.

Such a caller (a runtime that owns the whole device through its own arena, or a serving loop
that cannot take the device-wide stall of a cudaMalloc) passes every buffer itself; the scratch
the step needs sits in a static array inside the library.  The results must equal what the
ordinary handle-based entry points give for the same logits, on two calls in a row (the second
call reuses the scratch the first one left behind).
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from rustingbrain_b200 import MoeConfig, MoeLayer, _lib

pytestmark = pytest.mark.gpu


def _by_handle(T, E, k, logits, valid):
    layer = MoeLayer(32, MoeConfig(E, k, 32), precision="f32", max_tokens=T, training=False)
    x = torch.zeros(T, 32, device="cuda")
    _, cache = layer.forward_train(x, valid=valid, logits=torch.from_numpy(logits).cuda())
    e, g, c, _, _ = cache.routing()
    _, p, l = layer.router_cache(T)
    out = (e, g, c, p, l, np.array([cache.aux_loss(), cache.z_loss()], np.float32))
    layer.close()
    return out


def _no_alloc(T, E, k, logits, valid):
    lg = torch.from_numpy(logits).cuda()
    v = torch.from_numpy(valid).cuda() if valid is not None else None
    probs = torch.empty(T, E, device="cuda")
    lse = torch.empty(T, device="cuda")
    e = torch.empty(T * k, dtype=torch.int32, device="cuda")
    g = torch.empty(T * k, device="cuda")
    c = torch.empty(E, dtype=torch.int32, device="cuda")
    losses = torch.empty(2, device="cuda")
    msg = C.create_string_buffer(256)
    rc = _lib.lib().moe_route_noalloc(lg.data_ptr(), v.data_ptr() if v is not None else None, T, E, k, 0.01, 1e-3,
                                      probs.data_ptr(), lse.data_ptr(), e.data_ptr(), g.data_ptr(), c.data_ptr(),
                                      losses.data_ptr(), C.c_void_p(torch.cuda.current_stream().cuda_stream), msg, 256)
    assert rc == 0, msg.value
    torch.cuda.synchronize()
    return (e.cpu().numpy().reshape(T, k), g.cpu().numpy().reshape(T, k), c.cpu().numpy(), probs.cpu().numpy(),
            lse.cpu().numpy(), losses.cpu().numpy())


def test_two_calls_in_a_row_match_the_handle_based_routing():
    cases = [(3000, 64, 8, 123, True), (517, 16, 2, 7, False)]   # the second call is smaller: stale scratch must not leak
    for T, E, k, seed, masked in cases:
        g = np.random.Generator(np.random.Philox(seed))
        logits = (g.standard_normal((T, E)) + 1.5 * np.log(1.0 / np.arange(1, E + 1))).astype(np.float32)
        valid = (np.arange(T) % 5 != 2).astype(np.uint8) if masked else None
        want = _by_handle(T, E, k, logits, valid)
        got = _no_alloc(T, E, k, logits, valid)
        for a, b in zip(got[:5], want[:5]):
            assert np.array_equal(a, b)                       # integers, gates, probabilities: bit for bit
        np.testing.assert_allclose(got[5], want[5], rtol=1e-6)


def test_it_matches_the_cpu_checker_directly():
    """The same step against the CPU restatement of the reference's route / softmax_rows / auxiliary_losses
    (moe.rs:553-656), not only against the library's other entry point."""
    from oracle import OracleMoe
    T, E, k, d = 1500, 32, 4, 8
    g = np.random.Generator(np.random.Philox(11))
    logits = (g.standard_normal((T, E)) * 2.0).astype(np.float32)
    logits[5] = logits[5, 0]                                   # an all-equal row: ties go to the lowest index
    valid = (np.arange(T) % 7 != 3).astype(np.uint8)
    ora = OracleMoe(d, E, k, 8, False)
    ora.forward(np.zeros((T, d), np.float32), valid=valid, logits=logits)
    e_o, g_o, c_o, _, _ = ora.routing()
    got = _no_alloc(T, E, k, logits, valid)
    assert np.array_equal(got[0], np.asarray(e_o).reshape(T, k)) and np.array_equal(got[2], c_o)
    assert np.max(np.abs(got[1] - np.asarray(g_o).reshape(T, k))) <= 1e-6
    a, z = ora.losses()
    np.testing.assert_allclose(got[5], [a, z], rtol=1e-5)


def test_sizes_beyond_the_static_scratch_are_rejected():
    msg = C.create_string_buffer(256)
    one = torch.zeros(1, device="cuda")
    rc = _lib.lib().moe_route_noalloc(one.data_ptr(), None, 16385, 8, 2, 0.01, 1e-3, one.data_ptr(), one.data_ptr(),
                                      one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(), None, msg, 256)
    assert rc == _lib.INVALID_INPUT and b"16384" in msg.value
    rc = _lib.lib().moe_route_noalloc(one.data_ptr(), None, 64, 65, 2, 0.01, 1e-3, one.data_ptr(), one.data_ptr(),
                                      one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(), None, msg, 256)
    assert rc == _lib.INVALID_INPUT
