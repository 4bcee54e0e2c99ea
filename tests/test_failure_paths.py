"""The bounded waits of the grouped tensor-core GEMM, made to run out without faulting or hanging anything.

A debug hook starves ONE launch: its producer issues no load and every barrier wait gets a limit of about a
millisecond.  The waits give up, the kernel records a code, frees its tensor memory and returns; the handle
reports Timeout (the reference's fail-closed model: the failing call poisons the context,
gpu_transformer.rs:160-195) and, once the error is cleared, computes the same result as before.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from gpu_common import make_pair, to_dev
from rustingbrain_b200 import NetworkError, Timeout, _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pair", [0, 1, 2], ids=["one_sm", "two_sm", "wide"])
def test_a_starved_gemm_reports_timeout_and_the_handle_recovers(pair):
    T, d, E, k, F = 256, 256, 8, 2, 128
    dev, ora, _ = make_pair(d, E, k, F, False, seed=6, precision="bf16", max_tokens=T, std=0.05, router_std=0.05)
    x = to_dev(np.random.Generator(np.random.Philox(8)).standard_normal((T, d)).astype(np.float32), "bf16")
    _lib.lib().moe_debug_set_tc_pair(pair)
    try:
        y0, _ = dev.forward_train(x)
        dev.synchronize()
        _lib.lib().moe_debug_starve_next_gemm(2_000_000)      # about 1 ms of clock cycles
        dev.forward_train(x)                                   # asynchronous: the launch itself succeeds
        with pytest.raises(Timeout, match="bounded device-side wait"):
            dev.synchronize()
        with pytest.raises(NetworkError):                      # sticky until cleared
            dev.forward_train(x)
        dev.clear_error()
        y1, _ = dev.forward_train(x)
        dev.synchronize()
        assert torch.equal(y0, y1)                             # tensor memory was released: the next launch got all of it
    finally:
        _lib.lib().moe_debug_set_tc_pair(3)   # back to the per-launch choice
        dev.close()
