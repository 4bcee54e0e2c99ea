"""Committed golden vectors of the attention and RMSNorm checkers (tests/golden/make_golden_blocks.py)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden_blocks as mg  # noqa: E402
from helpers import rel_l2  # noqa: E402


def _load(name):
    return np.load(os.path.join(HERE, "golden", name + ".npz"))


@pytest.mark.parametrize("name", sorted(mg.ATTENTION))
def test_attention_checker_reproduces_its_golden_vectors(name):
    want, got = _load(name), mg.run_attention(name)
    for key in ("merged", "keys", "values"):
        assert rel_l2(got[key], want[key]) <= 1e-6, key


@pytest.mark.parametrize("name", sorted(mg.RMSNORM))
def test_rmsnorm_checker_reproduces_its_golden_vectors(name):
    want, got = _load(name), mg.run_rmsnorm(name)
    for key in ("y", "gx", "gw"):
        assert rel_l2(got[key], want[key]) <= 1e-6, key


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(mg.ATTENTION))
def test_device_attention_matches_the_golden_vectors(name):
    import torch
    from rustingbrain_b200.kv_attention import KvCache
    H, Hkv, hd, prompt, steps = mg.ATTENTION[name]
    want = _load(name)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    cache = KvCache(1, H, Hkv, hd, capacity=64, precision="f32")
    out = [cache.forward_cached(dev(want["q"][:prompt]), dev(want["k"][:prompt]), dev(want["v"][:prompt]),
                                rows_per_sequence=prompt).cpu().numpy()]
    for t in range(prompt, prompt + steps):
        out.append(cache.forward_cached(dev(want["q"][t:t + 1]), dev(want["k"][t:t + 1]), dev(want["v"][t:t + 1])).cpu().numpy())
    assert np.abs(np.concatenate(out) - want["merged"]).max() <= 1e-5
    keys, values = cache.keys_values(0)
    assert rel_l2(keys, want["keys"]) <= 1e-5 and np.array_equal(values, want["values"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(mg.RMSNORM))
def test_device_rmsnorm_matches_the_golden_vectors(name):
    import torch
    from rustingbrain_b200.norm import RmsNorm
    rows, d, eps = mg.RMSNORM[name]
    want = _load(name)
    norm = RmsNorm(d, eps)
    norm.weight.copy_(torch.from_numpy(want["w"]))
    x, gy = torch.from_numpy(want["x"]).cuda(), torch.from_numpy(want["gy"]).cuda()
    assert rel_l2(norm.forward(x).cpu().numpy(), want["y"]) <= 1e-5
    assert rel_l2(norm.backward(x, gy).cpu().numpy(), want["gx"]) <= 1e-5
    assert rel_l2(norm.grad.cpu().numpy(), want["gw"]) <= 1e-5
