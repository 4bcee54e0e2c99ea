"""Batched KV-cache decode attention on the device against the checker (oracle/attention.py)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from helpers import rel_l2
from oracle import attention as ora
from rustingbrain_b200 import InvalidConfig, InvalidInput
from rustingbrain_b200.kv_attention import KvCache

pytestmark = pytest.mark.gpu


def _qkv(rows, H, Hkv, hd, seed):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.standard_normal((rows, H * hd)).astype(np.float32), g.standard_normal((rows, Hkv * hd)).astype(np.float32),
            g.standard_normal((rows, Hkv * hd)).astype(np.float32))


def _dev(a, precision):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.bfloat16() if precision == "bf16" else t


@pytest.mark.parametrize("H,Hkv,hd", [(4, 2, 8), (2, 2, 8), (2, 1, 16), (8, 2, 64), (4, 4, 128), (2, 1, 256), (3, 1, 32)])
def test_a_cached_decode_reproduces_the_full_sequence_forward(H, Hkv, hd):  # attention.rs:1318-1340
    T = 6
    q, k, v = _qkv(T, H, Hkv, hd, seed=11)
    want = ora.full_sequence(q, k, v, H, Hkv, hd, 32)
    cache = KvCache(1, H, Hkv, hd, capacity=32, precision="f32")
    for t in range(T):
        got = cache.forward_cached(_dev(q[t:t + 1], "f32"), _dev(k[t:t + 1], "f32"), _dev(v[t:t + 1], "f32"))
        assert cache.lengths() == [t + 1]
        assert np.abs(got.cpu().numpy()[0] - want[t]).max() < 1e-5      # the reference's own tolerance


def test_a_prefill_then_decode_reproduces_the_full_sequence_forward():  # attention.rs:1342-1362
    q, k, v = _qkv(5, 2, 2, 8, seed=12)
    want = ora.full_sequence(q, k, v, 2, 2, 8, 32)
    cache = KvCache(1, 2, 2, 8, capacity=32, precision="f32")
    got = cache.forward_cached(_dev(q[:3], "f32"), _dev(k[:3], "f32"), _dev(v[:3], "f32"), rows_per_sequence=3)
    assert np.abs(got.cpu().numpy() - want[:3]).max() < 1e-5
    for t in range(3, 5):
        got = cache.forward_cached(_dev(q[t:t + 1], "f32"), _dev(k[t:t + 1], "f32"), _dev(v[t:t + 1], "f32"))
        assert np.abs(got.cpu().numpy()[0] - want[t]).max() < 1e-5


@pytest.mark.parametrize("precision,tol", [("f32", 1e-5), ("bf16", 2e-2)])
def test_sequences_of_different_lengths_advance_together(precision, tol):
    """Every sequence against its own single-sequence checker: prefill of different lengths (one sequence
    per call), then decode steps for all of them at once; long enough for several slices per sequence."""
    S, H, Hkv, hd = 5, 8, 2, 64
    prompt = [700, 1, 333, 1024, 64]
    steps = 3
    cache = KvCache(S, H, Hkv, hd, capacity=1100, precision=precision)
    oracles = [ora.KvCacheOracle(H, Hkv, hd, 1100) for _ in range(S)]
    rnd = lambda a: _dev(a, precision).float().cpu().numpy()        # the checker sees the values the device sees
    for s in range(S):
        q, k, v = _qkv(prompt[s], H, Hkv, hd, seed=100 + s)
        got = cache.forward_cached(_dev(q, precision), _dev(k, precision), _dev(v, precision),
                                   rows_per_sequence=prompt[s], first_sequence=s, n_sequences=1)
        want = oracles[s].forward_cached(rnd(q), rnd(k), rnd(v))
        assert rel_l2(got.float().cpu().numpy(), want) <= tol
    assert cache.lengths() == prompt
    for step in range(steps):
        q, k, v = _qkv(S, H, Hkv, hd, seed=200 + step)
        got = cache.forward_cached(_dev(q, precision), _dev(k, precision), _dev(v, precision)).float().cpu().numpy()
        for s in range(S):
            want = oracles[s].forward_cached(rnd(q[s:s + 1]), rnd(k[s:s + 1]), rnd(v[s:s + 1]))
            assert rel_l2(got[s:s + 1], want) <= tol, (step, s)
    assert cache.lengths() == [p + steps for p in prompt]
    # the cache holds the rotated keys and the values as appended (attention.rs:15-17)
    keys, values = cache.keys_values(2)
    assert rel_l2(keys, oracles[2].keys) <= (1e-5 if precision == "f32" else 1e-2)
    assert rel_l2(values, oracles[2].values) <= (1e-6 if precision == "f32" else 1e-2)


@pytest.mark.parametrize("H,Hkv,hd,rows", [(8, 1, 128, 1), (16, 2, 128, 3), (4, 4, 64, 5), (32, 2, 64, 1)])
def test_bf16_cache_on_the_tensor_core_kernel(H, Hkv, hd, rows):
    """bf16 caches with head_dim 64 / 128 take the mma.sync kernel: groups of 1 to 16 query heads, several new
    rows per step (more than 16 queries per kv head means more than one pass), histories that end inside a block."""
    S = 3
    cache = KvCache(S, H, Hkv, hd, capacity=600, precision="bf16")
    oracles = [ora.KvCacheOracle(H, Hkv, hd, 600) for _ in range(S)]
    rnd = lambda a: _dev(a, "bf16").float().cpu().numpy()
    for s, n in enumerate((1, 77, 530)):
        q, k, v = _qkv(n, H, Hkv, hd, seed=300 + s)
        cache.forward_cached(_dev(q, "bf16"), _dev(k, "bf16"), _dev(v, "bf16"), rows_per_sequence=n, first_sequence=s, n_sequences=1)
        oracles[s].forward_cached(rnd(q), rnd(k), rnd(v))
    for step in range(2):
        q, k, v = _qkv(S * rows, H, Hkv, hd, seed=400 + step)
        got = cache.forward_cached(_dev(q, "bf16"), _dev(k, "bf16"), _dev(v, "bf16"), rows_per_sequence=rows).float().cpu().numpy()
        for s in range(S):
            sl = slice(s * rows, (s + 1) * rows)
            want = oracles[s].forward_cached(rnd(q[sl]), rnd(k[sl]), rnd(v[sl]))
            assert rel_l2(got[sl], want) <= 2e-2, (step, s)


def test_clear_and_truncate_and_a_restarted_sequence():
    S, H, Hkv, hd = 3, 4, 2, 32
    cache = KvCache(S, H, Hkv, hd, capacity=64, precision="f32")
    q, k, v = _qkv(S * 4, H, Hkv, hd, seed=5)
    cache.forward_cached(_dev(q, "f32"), _dev(k, "f32"), _dev(v, "f32"), rows_per_sequence=4)
    assert cache.lengths() == [4, 4, 4]
    cache.clear(1)
    assert cache.lengths() == [4, 0, 4]
    cache.truncate(2, sequence=2)
    assert cache.lengths() == [4, 0, 2]
    with pytest.raises(InvalidInput):
        cache.truncate(3, sequence=2)
    # the restarted sequence decodes from position 0 again
    o = ora.KvCacheOracle(H, Hkv, hd, 64)
    q1, k1, v1 = _qkv(2, H, Hkv, hd, seed=6)
    got = cache.forward_cached(_dev(q1, "f32"), _dev(k1, "f32"), _dev(v1, "f32"), rows_per_sequence=2,
                               first_sequence=1, n_sequences=1)
    assert np.abs(got.cpu().numpy() - o.forward_cached(q1, k1, v1)).max() < 1e-5


def test_without_rotation_and_errors():
    H, Hkv, hd = 2, 1, 8
    cache = KvCache(1, H, Hkv, hd, capacity=4, rope=False, precision="f32")
    o = ora.KvCacheOracle(H, Hkv, hd, 4, rope=False)
    q, k, v = _qkv(3, H, Hkv, hd, seed=8)
    got = cache.forward_cached(_dev(q, "f32"), _dev(k, "f32"), _dev(v, "f32"), rows_per_sequence=3)
    assert np.abs(got.cpu().numpy() - o.forward_cached(q, k, v)).max() < 1e-5
    with pytest.raises(InvalidInput, match="SequenceTooLong"):          # rope.rs:194-200
        cache.forward_cached(_dev(q[:2], "f32"), _dev(k[:2], "f32"), _dev(v[:2], "f32"), rows_per_sequence=2)
    assert cache.lengths() == [3]                                        # nothing was appended
    for bad in (dict(num_heads=3, kv_heads=2), dict(num_heads=2, kv_heads=4), dict(head_dim=7), dict(num_heads=0)):
        kw = dict(sequences=1, num_heads=4, kv_heads=2, head_dim=8, capacity=8)
        kw.update(bad)
        with pytest.raises(InvalidConfig):                               # attention.rs:173-186, rope.rs:72-76
            KvCache(**kw)


@pytest.mark.parametrize("precision,hd", [("bf16", 64), ("f32", 32)])
def test_a_replayed_step_that_runs_into_the_end_of_a_cache_is_skipped_not_written(precision, hd):
    """A step replayed from a CUDA graph advances the device lengths only, so only the device can see
    a replay that no longer fits.  The kernels then store nothing, leave the length alone, return zeros
    for that sequence and mark it; kv_cache_lengths reports the mark as SequenceTooLong and clears it.
    The other sequence of the cache keeps stepping and its rows are untouched by the skipped one."""
    from rustingbrain_b200 import InvalidInput
    S, H, Hkv, cap = 2, 4, 2, 8
    dt = torch.bfloat16 if precision == "bf16" else torch.float32
    cache = KvCache(S, H, Hkv, hd, capacity=cap, precision=precision)
    gen = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=gen).to(dt)
    # sequence 0 starts with 5 positions, sequence 1 with 2
    cache.forward_cached(rnd(5, H * hd), rnd(5, Hkv * hd), rnd(5, Hkv * hd), rows_per_sequence=5, first_sequence=0, n_sequences=1)
    cache.forward_cached(rnd(2, H * hd), rnd(2, Hkv * hd), rnd(2, Hkv * hd), rows_per_sequence=2, first_sequence=1, n_sequences=1)
    q, k, v = rnd(S, H * hd), rnd(S, Hkv * hd), rnd(S, Hkv * hd)
    q0, out = q.clone(), torch.empty_like(q)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        cache.forward_cached(q, k, v, out=out)             # lengths 6 and 3 (warm-up before the capture)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        cache.forward_cached(q, k, v, out=out)             # captured, not run
    for _ in range(2):                                     # 7 / 4, then 8 / 5: sequence 0 is now full
        q.copy_(q0); graph.replay()
    torch.cuda.synchronize()
    before = cache.keys_values(0)
    assert cache.lengths() == [cap, 5]
    q.copy_(q0); graph.replay()                            # sequence 0 has no room; sequence 1 goes to 6
    torch.cuda.synchronize()
    assert float(out[0].float().abs().max()) == 0.0 and float(out[1].float().abs().max()) > 0.0
    with pytest.raises(InvalidInput, match="SequenceTooLong"):
        cache.lengths()
    assert cache.lengths() == [cap, 6]                     # reported once; the length never passed capacity
    after = cache.keys_values(0)
    assert np.array_equal(before[0], after[0]) and np.array_equal(before[1], after[1])
    k1, _ = cache.keys_values(1)
    assert k1.shape[0] == 6
    cache.truncate(4, sequence=0)                          # room again: the same graph steps it normally
    q.copy_(q0); graph.replay()
    torch.cuda.synchronize()
    assert cache.lengths() == [5, 7] and float(out[0].float().abs().max()) > 0.0
