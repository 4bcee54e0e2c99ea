"""Writes tests/golden/*.npz from the CPU checker (oracle/), after the checker has been
pinned by the reference's own known-answer tests (tests/test_oracle_known_answers.py).

The reference crate cannot be executed in the build image (no Rust toolchain), so these
vectors freeze the pinned checker rather than a run of the crate: they catch regressions of
the checker and give the device path fixed targets.  Inputs are the reference's closed-form
ramps (moe.rs:905-911, 942-948, 976-982), so every value is reproducible without an RNG.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from helpers import ramp  # noqa: E402
from oracle import OracleMoe, ROUTER, GATE, UP, DOWN  # noqa: E402

CASES = {
    # name: (T, d, E, k, F, shared, aux_w, z_w, valid)
    "fd_shared": (3, 6, 4, 2, 5, True, 0.0, 0.0, None),        # moe.rs:895-931
    "router_fd": (3, 4, 3, 2, 4, False, 0.0, 0.0, None),       # moe.rs:933-971
    "aux_fd": (4, 4, 3, 2, 4, False, 0.01, 1e-3, None),        # moe.rs:973-1013
    "padded": (10, 8, 4, 2, 6, True, 0.01, 1e-3, [1, 1, 0, 1, 0, 1, 1, 1, 0, 1]),
    "wide": (48, 32, 8, 3, 40, True, 0.01, 1e-3, None),
}


def weights(d, E, F, shared):
    """Closed-form weights: scaled ramps with different strides per matrix."""
    w = {"router": ramp(E * d, 31, 19, 9, (E, d)) * np.float32(0.7),
         "gate": np.stack([ramp(F * d, 7 + 2 * e, 23, 11, (F, d)) for e in range(E)]) * np.float32(0.6),
         "up": np.stack([ramp(F * d, 5 + 2 * e, 29, 14, (F, d)) for e in range(E)]) * np.float32(0.6),
         "down": np.stack([ramp(d * F, 3 + 2 * e, 31, 15, (d, F)) for e in range(E)]) * np.float32(0.6),
         "shared": None}
    if shared:
        w["shared"] = (ramp(F * d, 37, 41, 20, (F, d)) * np.float32(0.5), ramp(F * d, 43, 47, 23, (F, d)) * np.float32(0.5),
                       ramp(d * F, 53, 59, 29, (d, F)) * np.float32(0.5))
    return w


def run_case(name):
    T, d, E, k, F, shared, aux_w, z_w, valid = CASES[name]
    w = weights(d, E, F, shared)
    m = OracleMoe(d, E, k, F, shared, aux_w, z_w)
    m.set_weights(w["router"], w["gate"], w["up"], w["down"], w["shared"])
    x = ramp(T * d, 29, 17, 8, (T, d))
    gy = ramp(T * d, 13, 11, 5, (T, d))
    v = None if valid is None else np.array(valid, np.uint8)
    y = m.forward(x, valid=v)
    gx = m.backward(gy)
    expert_of, gates, counts, token_of, slot_of = m.routing()
    logits, probs, lse = m.router_cache()
    aux, z = m.losses()
    out = dict(x=x, gy=gy, y=y, gx=gx, expert_of=expert_of, gates=gates, counts=counts, token_of=token_of,
               slot_of=slot_of, logits=logits, probs=probs, lse=lse, losses=np.array([aux, z], np.float32),
               g_router=m.get_grad(ROUTER), g_gate0=m.get_grad(GATE, 0), g_up1=m.get_grad(UP, 1),
               g_down2=m.get_grad(DOWN, 2), valid=np.zeros(0, np.uint8) if v is None else v)
    return out


if __name__ == "__main__":
    for name in CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **run_case(name))
        print("wrote", name)
