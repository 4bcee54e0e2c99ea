"""Helpers shared by the GPU parity tests: paired checker / device layers on the same weights."""
import numpy as np
import torch

from oracle import OracleMoe
from rustingbrain_b200 import MoeConfig, MoeLayer
from rustingbrain_b200 import _lib
from helpers import seeded_weights


def make_pair(d, E, k, F, shared=False, aux_w=0.01, z_w=1e-3, seed=1, precision="f32", max_tokens=64, std=0.02,
              router_std=None, weights=None, training=True):
    w = weights or seeded_weights(d, E, F, shared, seed, std=std, router_std=router_std)
    if precision != "f32":
        # both sides see the same bf16-representable expert weights
        rb = lambda a: torch.from_numpy(a).bfloat16().float().numpy()
        w = dict(w, gate=rb(w["gate"]), up=rb(w["up"]), down=rb(w["down"]),
                 shared=tuple(rb(s) for s in w["shared"]) if w["shared"] is not None else None)
    cfg = MoeConfig(E, k, F, shared, aux_w, z_w)
    dev = MoeLayer(d, cfg, precision=precision, max_tokens=max_tokens, training=training)
    dev.set_weights(w["router"], w["gate"], w["up"], w["down"], w["shared"])
    ora = OracleMoe(d, E, k, F, shared, aux_w, z_w)
    ora.set_weights(w["router"], w["gate"], w["up"], w["down"], w["shared"])
    return dev, ora, w


def to_dev(a, precision):
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    return t if precision == "f32" else t.bfloat16()


def to_np(t):
    return t.float().cpu().numpy()


def assert_routing_equal(cache, ora):
    """Integers bit-exact; gates to 1e-6 (they are quotients of identical f32 values)."""
    e_d, g_d, c_d, t_d, s_d = cache.routing()
    e_o, g_o, c_o, t_o, s_o = ora.routing()
    assert np.array_equal(e_d, e_o), "top-k indices differ on %d slots" % int((e_d != e_o).sum())
    assert np.array_equal(c_d, c_o), "per-expert counts differ"
    assert np.array_equal(t_d, t_o) and np.array_equal(s_d, s_o), "permutation differs"
    assert np.max(np.abs(g_d - g_o), initial=0.0) <= 1e-6
