"""The attention checker against the known answers and properties of the reference's own tests
(rope.rs:232-298, attention.rs:1276-1362).  No GPU."""
import math

import numpy as np
import pytest

from oracle import attention as ora


def test_position_zero_is_the_identity():  # rope.rs:232-240
    cos, sin = ora.rope_tables(4, 8, 10000.0)
    x = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    assert np.array_equal(ora.rope_apply(x, 1, 0, cos, sin), x)


def test_rotation_matches_the_hand_computed_example():  # rope.rs:242-254: head_dim 2, base 1 -> angle = position
    cos, sin = ora.rope_tables(2, 4, 1.0)
    out = ora.rope_apply(np.array([[1.0, 0.0]], np.float32), 1, 1, cos, sin)
    assert abs(out[0, 0] - math.cos(1.0)) < 1e-6 and abs(out[0, 1] - math.sin(1.0)) < 1e-6


def test_inverse_norm_and_relative_distance():  # rope.rs:256-298
    cos, sin = ora.rope_tables(8, 16, 10000.0)
    x = (np.arange(48, dtype=np.float32) * np.float32(0.1)).reshape(3, 16)
    back = ora.rope_apply(ora.rope_apply(x, 2, 5, cos, sin), 2, 5, cos, sin, direction=-1.0)
    assert np.abs(back - x).max() < 1e-5
    cos, sin = ora.rope_tables(6, 32, 10000.0)
    v = np.array([[0.5, -1.0, 2.0, 0.25, -0.75, 1.5]], np.float32)
    assert abs((ora.rope_apply(v, 1, 17, cos, sin) ** 2).sum() - (v ** 2).sum()) < 1e-4
    cos, sin = ora.rope_tables(4, 64, 10000.0)
    q = np.array([[0.3, -1.1, 0.7, 2.0]], np.float32)
    k = np.array([[1.3, 0.2, -0.9, 0.4]], np.float32)
    score = lambda a, b: float((ora.rope_apply(q, 1, a, cos, sin) * ora.rope_apply(k, 1, b, cos, sin)).sum())
    assert abs(score(3, 1) - score(20, 18)) < 1e-4


def test_applying_past_the_table_is_an_error():  # rope.rs:300-309, 311-314
    cos, sin = ora.rope_tables(2, 4, 10000.0)
    with pytest.raises(ValueError, match="SequenceTooLong: length 5"):
        ora.rope_apply(np.zeros((3, 2), np.float32), 1, 2, cos, sin)
    with pytest.raises(ValueError):
        ora.rope_tables(3, 8, 10000.0)


def _qkv(rows, H, Hkv, hd, seed):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.standard_normal((rows, H * hd)).astype(np.float32), g.standard_normal((rows, Hkv * hd)).astype(np.float32),
            g.standard_normal((rows, Hkv * hd)).astype(np.float32))


@pytest.mark.parametrize("H,Hkv", [(4, 2), (2, 2), (2, 1)])
def test_a_cached_decode_reproduces_the_full_sequence_forward(H, Hkv):  # attention.rs:1318-1340
    q, k, v = _qkv(6, H, Hkv, 4, seed=11)
    want = ora.full_sequence(q, k, v, H, Hkv, 4, 32)
    cache = ora.KvCacheOracle(H, Hkv, 4, 32)
    for t in range(6):
        got = cache.forward_cached(q[t:t + 1], k[t:t + 1], v[t:t + 1])
        assert len(cache) == t + 1
        assert np.abs(got[0] - want[t]).max() < 1e-5


def test_a_prefill_then_decode_reproduces_the_full_sequence_forward():  # attention.rs:1342-1362
    q, k, v = _qkv(5, 2, 2, 4, seed=12)
    want = ora.full_sequence(q, k, v, 2, 2, 4, 32)
    cache = ora.KvCacheOracle(2, 2, 4, 32)
    got = cache.forward_cached(q[:3], k[:3], v[:3])
    assert np.abs(got - want[:3]).max() < 1e-5
    for t in range(3, 5):
        assert np.abs(cache.forward_cached(q[t:t + 1], k[t:t + 1], v[t:t + 1])[0] - want[t]).max() < 1e-5


def test_grouped_heads_read_their_own_kv_head():  # attention.rs:1108, 1143: kv head = head / group_size
    q, k, v = _qkv(3, 4, 2, 4, seed=13)
    base = ora.full_sequence(q, k, v, 4, 2, 4, 16)
    v2 = v.copy()
    v2[:, 4:] += 1.0                     # only kv head 1 changes -> only query heads 2 and 3 move
    moved = ora.full_sequence(q, k, v2, 4, 2, 4, 16)
    assert np.array_equal(base[:, :8], moved[:, :8]) and not np.allclose(base[:, 8:], moved[:, 8:])
