"""Writes tests/golden/attention_*.npz and rmsnorm_*.npz from the numpy checkers (oracle/attention.py,
oracle/norm.py), after they have been pinned by the reference's own tests
(tests/test_kv_attention_oracle.py, tests/test_rmsnorm_oracle.py).

The reference crate cannot be executed in the build image (no Rust toolchain), so these vectors freeze
the pinned checkers: they catch regressions of the checkers and give the device paths fixed targets.
Inputs are closed-form ramps in the style of the reference's fixtures (moe.rs:905-911), no RNG.

    python tests/golden/make_golden_blocks.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from helpers import ramp  # noqa: E402
from oracle import attention as att  # noqa: E402
from oracle import norm as nrm  # noqa: E402

ATTENTION = {
    # name: (num_heads, kv_heads, head_dim, prompt rows, decode steps)
    "attention_gqa": (4, 2, 8, 3, 4),
    "attention_mha64": (2, 2, 64, 5, 2),
}
RMSNORM = {
    # name: (rows, d_model, eps)
    "rmsnorm_small": (5, 16, 1e-6),
    "rmsnorm_tiles": (70, 64, 1e-5),       # three tiles of 32 rows, the last one ragged
}


def attention_inputs(name):
    H, Hkv, hd, prompt, steps = ATTENTION[name]
    rows = prompt + steps
    return (ramp(rows * H * hd, 29, 17, 8, (rows, H * hd)), ramp(rows * Hkv * hd, 31, 19, 9, (rows, Hkv * hd)),
            ramp(rows * Hkv * hd, 23, 13, 6, (rows, Hkv * hd)))


def run_attention(name):
    """Prefill of `prompt` rows, then `steps` single-row decode steps; merged heads of every row."""
    H, Hkv, hd, prompt, steps = ATTENTION[name]
    q, k, v = attention_inputs(name)
    cache = att.KvCacheOracle(H, Hkv, hd, 64)
    out = [cache.forward_cached(q[:prompt], k[:prompt], v[:prompt])]
    for t in range(prompt, prompt + steps):
        out.append(cache.forward_cached(q[t:t + 1], k[t:t + 1], v[t:t + 1]))
    return {"q": q, "k": k, "v": v, "merged": np.concatenate(out), "keys": cache.keys, "values": cache.values}


def rmsnorm_inputs(name):
    rows, d, _ = RMSNORM[name]
    return (ramp(rows * d, 29, 17, 8, (rows, d)) * np.float32(1.5), ramp(rows * d, 7, 23, 11, (rows, d)),
            ramp(d, 5, 11, 4) * np.float32(0.5) + np.float32(1.0))


def run_rmsnorm(name):
    x, gy, w = rmsnorm_inputs(name)
    eps = RMSNORM[name][2]
    gx, gw = nrm.backward(x, w, gy, eps)
    return {"x": x, "gy": gy, "w": w, "y": nrm.forward(x, w, eps), "gx": gx, "gw": gw}


if __name__ == "__main__":
    for name in ATTENTION:
        np.savez(os.path.join(HERE, name + ".npz"), **run_attention(name))
    for name in RMSNORM:
        np.savez(os.path.join(HERE, name + ".npz"), **run_rmsnorm(name))
    print("wrote", ", ".join(sorted(list(ATTENTION) + list(RMSNORM))))
