"""Shared fixtures: seeded weights, closed-form ramps and the error measure."""
import numpy as np


def rel_l2(a, b):
    """||a-b||_2 / ||b||_2 with b the checker's answer (0 when both vanish)."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    den = np.linalg.norm(b)
    num = np.linalg.norm(a - b)
    return 0.0 if num == 0 else num / max(den, 1e-30)


def ramp(n, mul, mod, div, shape=None):
    """The reference's RNG-free fixtures, e.g. ((i*29)%17)/8-1 (moe.rs:905-911)."""
    i = np.arange(n, dtype=np.int64)
    v = ((i * mul) % mod).astype(np.float32) / np.float32(div) - np.float32(1.0)
    return v.reshape(shape) if shape else v


def seeded_weights(d, E, F, shared, seed, std=0.02, router_std=None):
    """router [E,d], gate/up [E,F,d], down [E,d,F], shared triple or None; N(0,std)."""
    g = np.random.Generator(np.random.Philox(seed))
    rs = std if router_std is None else router_std
    w = {
        "router": (g.standard_normal((E, d)) * rs).astype(np.float32),
        "gate": (g.standard_normal((E, F, d)) * std).astype(np.float32),
        "up": (g.standard_normal((E, F, d)) * std).astype(np.float32),
        "down": (g.standard_normal((E, d, F)) * std).astype(np.float32),
        "shared": None,
    }
    if shared:
        w["shared"] = ((g.standard_normal((F, d)) * std).astype(np.float32),
                       (g.standard_normal((F, d)) * std).astype(np.float32),
                       (g.standard_normal((d, F)) * std).astype(np.float32))
    return w


def he_uniform_weights(d, E, F, shared, seed):
    """U(+-sqrt(2/fan_in)) like the reference's Linear::new (param.rs:240-246), own RNG stream."""
    g = np.random.Generator(np.random.Philox(seed))

    def u(rows, cols):
        b = np.sqrt(2.0 / cols)
        return g.uniform(-b, b, (rows, cols)).astype(np.float32)

    w = {
        "gate": np.stack([u(F, d) for _ in range(E)]),
        "up": np.stack([u(F, d) for _ in range(E)]),
        "down": np.stack([u(d, F) for _ in range(E)]),
        "shared": (u(F, d), u(F, d), u(d, F)) if shared else None,
    }
    w["router"] = u(E, d)
    return w


def one_hot_router(E, d, strength):
    """moe.rs:678-686: a scaled identity, so a one-hot row t goes to expert t % E."""
    w = np.zeros((E, d), np.float32)
    for e in range(E):
        w[e, e % d] = strength
    return w


def one_hot_rows(rows, width):
    x = np.zeros((len(rows), width), np.float32)
    for r, c in enumerate(rows):
        x[r, c] = 1.0
    return x
