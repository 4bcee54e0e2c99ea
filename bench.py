"""Benchmark of the MoE layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg4|cfg3|cfg1] [--impl reference]

One "step" is one forward + backward pass of the layer over one batch of synthetic
tokens.  Prints ONE JSON line (rank 0).  The default workload is the expert-parallel
configuration the metric is quoted on (32768 tokens per GPU, d_model 4096, 64 experts
top-8, SwiGLU d_ff 1536, bf16); `--workload cfg3` is the 1-GPU fine-grained layer
(16384 tokens, d 2048, 64 experts top-8 + shared expert, d_ff 1408, Zipf-skewed router).

`--impl reference` times the CPU restatement of the reference's own (rayon) MoE path
on the host cores instead; it is the one place this file executes code under oracle/
besides the `cpu_baseline` leg.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "cfg4": dict(T=32768, d=4096, E=64, k=8, F=1536, shared=False, seed=2024, precision="bf16", zipf=False,
                 name="expert-parallel MoE layer fwd+bwd bf16: 32768 tokens/GPU, d_model 4096, 64 experts top-8, d_ff 1536"),
    "cfg3": dict(T=16384, d=2048, E=64, k=8, F=1408, shared=True, seed=123, precision="bf16", zipf=True,
                 name="fine-grained MoE layer fwd+bwd bf16: 16384 tokens, d_model 2048, 64 experts top-8 + shared, d_ff 1408, Zipf router"),
    # reduced copy of cfg3's shapes (same tile shapes, a quarter of the rows and experts) for ncu captures
    "prof": dict(T=8192, d=2048, E=16, k=4, F=1408, shared=True, seed=123, precision="bf16", zipf=False,
                 name="profiling case: 8192 tokens, d_model 2048, 16 experts top-4 + shared, d_ff 1408"),
    # cfg3's token rows (16384 x top-8, d 2048) with few narrow experts: same dispatch/combine traffic, ~3 GB on the device
    "hbm": dict(T=16384, d=2048, E=8, k=8, F=256, shared=False, seed=123, precision="bf16", zipf=False,
                name="HBM-kernel profiling case: 16384 tokens, d_model 2048, 8 experts top-8, d_ff 256"),
    "cfg5": dict(T=64, d=1024, E=16, k=2, F=2816, shared=True, seed=9, precision="q8", zipf=False,
                 name="KV-cached decode step through a quantized MoE layer: 64 sequences x 1 token, d_model 1024, 16 experts top-2 + shared, d_ff 2816, int8 weights"),
    # the attention half of the same decode step: 64 caches of 4096 positions, d_model 1024 = 16 query heads x 64,
    # 4 key/value heads (the head split of the reference's README model scaled to d_model 1024), bf16 cache
    "cfg5_attn": dict(S=64, H=16, Hkv=4, hd=64, history=4096, precision="attn", seed=9,
                      name="KV-cached decode attention: 64 sequences x 1 token over 4096 cached positions, 16 query heads, 4 kv heads, head_dim 64, bf16 cache"),
    # the normalisation in front of the layer, on cfg 4's activations (268 MB per tensor in bf16: larger than L2)
    "rmsnorm": dict(T=32768, d=4096, precision="rmsnorm", seed=2024,
                    name="RMSNorm forward + backward bf16: 32768 tokens, d_model 4096"),
    # The 55M language model workload is a whole-model train_step; only its MoE layers are on this path.  One of its
    # six MoE blocks (layers 2..7: 8 experts top-2, expert d_ff 352 + shared, 8 x 1024 tokens), forward +
    # backward + Adam, bf16 GEMMs over f32 master weights.
    "cfg2": dict(T=8192, d=512, E=8, k=2, F=352, shared=True, seed=42, precision="bf16", zipf=False, adam=True,
                 name="one MoE block of the 55M language model, fwd+bwd+Adam bf16: 8192 tokens, d_model 512, 8 experts top-2 + shared, d_ff 352"),
    # the whole 55M-parameter language model of the reference's README: train_step (forward + backward + Adam) over
    # 8 sequences of 1024 tokens, bf16 products over f32 master weights; 6 of its 8 blocks are MoE blocks
    "cfg2_model": dict(precision="model", batch=8, seq=1024, seed=42,
                       name="55.2M-parameter MoE language model, full train_step bf16/f32-master: vocab 32000, d_model 512, 8 layers, GQA 8/2 x 64, dense d_ff 1408, 8 experts top-2 (d_ff 352) + shared on layers 2..7, batch 8 x seq 1024"),
    "cfg1": dict(T=2048, d=512, E=8, k=2, F=1408, shared=False, seed=42, precision="f32", zipf=False,
                 name="MoE layer fwd+bwd f32: 2048 tokens, d_model 512, 8 experts top-2, d_ff 1408"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sustained=p["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, src="fallback")


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        rows = [l.split(",") for l in open(self.file.name).read().strip().splitlines() if l.count(",") >= 8]
        os.unlink(self.file.name)
        if not rows:
            return out
        sm = [float(r[1]) for r in rows if r[1].strip().replace(".", "").isdigit()]
        out["sm_mhz"] = float(np.median(sm)) if sm else None
        out["sm_max_mhz"] = float(rows[0][2]) if rows[0][2].strip().replace(".", "").isdigit() else None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for i, nm in enumerate(names):
            if any(r[5 + i].strip().lower().startswith("active") for r in rows):
                out["reasons"].append(nm)
        out["samples"] = len(rows)
        return out


def make_inputs(torch, w, rank, device):
    g = torch.Generator(device=device)
    g.manual_seed(w["seed"] + rank)
    dt = torch.float32 if w["precision"] == "f32" else torch.bfloat16
    x = torch.randn(w["T"], w["d"], generator=g, device=device, dtype=torch.float32)
    if w["zipf"]:
        x[:, -1] = 1.0
    gy = torch.randn(w["T"], w["d"], generator=g, device=device, dtype=torch.float32)
    return x.to(dt), gy.to(dt)


def load_weights(torch, layer, w, device, experts=None):
    """N(0, 0.02) weights from the workload's seed, generated on the device, expert by expert."""
    from rustingbrain_b200 import _lib
    g = torch.Generator(device=device)
    d, E, F = w["d"], w["E"], w["F"]
    g.manual_seed(w["seed"])
    router = torch.randn(E, d, generator=g, device=device) * (1.0 / np.sqrt(d) if w["zipf"] else 0.02)
    if w["zipf"]:   # per-expert bias 1.5*log(1/rank) through a constant-one input column
        router[:, -1] = 1.5 * torch.log(1.0 / torch.arange(1, E + 1, device=device, dtype=torch.float32))
    layer.set_weight(_lib.W_ROUTER, 0, router)
    for e in range(E):
        g.manual_seed(w["seed"] * 1000 + e)
        wg = torch.randn(F, d, generator=g, device=device) * 0.02
        wu = torch.randn(F, d, generator=g, device=device) * 0.02
        wd = torch.randn(d, F, generator=g, device=device) * 0.02
        if experts is None or e in experts:
            layer.set_weight(_lib.W_GATE, e, wg)
            layer.set_weight(_lib.W_UP, e, wu)
            layer.set_weight(_lib.W_DOWN, e, wd)
    if w["shared"]:
        g.manual_seed(w["seed"] * 1000 + E)
        layer.set_weight(_lib.W_SHARED_GATE, 0, torch.randn(F, d, generator=g, device=device) * 0.02)
        layer.set_weight(_lib.W_SHARED_UP, 0, torch.randn(F, d, generator=g, device=device) * 0.02)
        layer.set_weight(_lib.W_SHARED_DOWN, 0, torch.randn(d, F, generator=g, device=device) * 0.02)


def oracle_layer(w, sample_tokens, threads=None):
    """CPU restatement with the workload's shapes; weights N(0,0.02) from numpy (same distribution)."""
    import oracle
    from oracle import OracleMoe
    if threads:
        oracle.lib().orc_set_threads(threads)
    d, E, k, F = w["d"], w["E"], w["k"], w["F"]
    m = OracleMoe(d, E, k, F, w["shared"])
    g = np.random.Generator(np.random.Philox(w["seed"]))
    router = (g.standard_normal((E, d)) * (1.0 / np.sqrt(d) if w["zipf"] else 0.02)).astype(np.float32)
    if w["zipf"]:
        router[:, -1] = 1.5 * np.log(1.0 / np.arange(1, E + 1))
    m.set_weight(oracle.ROUTER, 0, router)
    base = (g.standard_normal((3, max(F, d), max(F, d))) * 0.02).astype(np.float32)
    for e in range(E):   # one draw, rolled per expert: distribution, not values, is what the timing needs
        r = np.roll(base, e * 7, axis=2)
        m.set_weight(oracle.GATE, e, np.ascontiguousarray(r[0, :F, :d]))
        m.set_weight(oracle.UP, e, np.ascontiguousarray(r[1, :F, :d]))
        m.set_weight(oracle.DOWN, e, np.ascontiguousarray(r[2, :d, :F]))
    if w["shared"]:
        m.set_weight(oracle.SHARED_GATE, 0, np.ascontiguousarray(base[0, :F, :d]))
        m.set_weight(oracle.SHARED_UP, 0, np.ascontiguousarray(base[1, :F, :d]))
        m.set_weight(oracle.SHARED_DOWN, 0, np.ascontiguousarray(base[2, :d, :F]))
    x = g.standard_normal((sample_tokens, d)).astype(np.float32)
    if w["zipf"]:
        x[:, -1] = 1.0
    gy = g.standard_normal((sample_tokens, d)).astype(np.float32)
    return m, x, gy


def host_threads():
    """Every core this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def time_oracle(w, sample_tokens, steps, warmup, budget_s=150.0):
    """Times forward + backward of the CPU restatement on `sample_tokens` tokens of the workload's shape, on all
    host threads.  The sample is the same at every GPU count (the large workloads use 2048 tokens per pass, so
    that the experts' weights are not re-streamed from memory for a few rows each); when `steps` passes of it
    would not fit in `budget_s`, fewer are timed and that number is returned.
    """
    import oracle
    threads = host_threads()
    m, x, gy = oracle_layer(w, sample_tokens, threads=threads)
    t0 = time.perf_counter()
    m.forward(x); m.backward(gy)                             # first touch: pages in weights, allocates gradients
    first = time.perf_counter() - t0
    warm = warmup if first * (warmup + 1) < 0.3 * budget_s else 0
    for _ in range(warm):
        m.forward(x); m.backward(gy)
    t0 = time.perf_counter()
    m.forward(x); m.backward(gy)
    one = time.perf_counter() - t0
    timed = int(max(1, min(steps, (budget_s - first * (1 + warm)) // max(one, 1e-9))))
    total = one
    for _ in range(timed - 1):
        t0 = time.perf_counter()
        m.forward(x); m.backward(gy)
        total += time.perf_counter() - t0
    dt = total / timed
    return sample_tokens / dt, dt, oracle.lib().orc_max_threads(), sample_tokens, timed


def reference_sample(w):
    """Tokens per pass of the CPU arm: the whole batch for the small workloads, 2048 tokens for the large ones."""
    return min(w["T"], 2048)


def run_reference(args, w):
    """The reference's CPU path (restated in oracle/) on the host cores, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if w["precision"] == "model":
        # the checker's train_step (numpy + the C++ MoE restatement) on a bounded sample: 2 sequences of 128 tokens
        import oracle
        from oracle import transformer as T
        oracle.lib().orc_set_threads(host_threads())
        c = T.default_config()
        m = T.OracleLm(c, T.seeded_model_weights(c, w["seed"]))
        g = np.random.Generator(np.random.Philox(w["seed"]))
        batch = T.TokenBatch([list(g.integers(0, 32000, 128)) for _ in range(2)])
        m.train_step(batch)
        steps = max(1, min(args.steps, 3))
        t0 = time.perf_counter()
        for _ in range(steps):
            m.train_step(batch)
        dt = (time.perf_counter() - t0) / steps
        v = batch.rows / dt
        print(json.dumps({"impl": "reference", "metric": "language-model tokens/s (train_step: forward + backward + Adam)", "value": v,
                          "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": w["name"], "sample": "2 sequences of 128 tokens per step", "steps_timed": steps},
                          "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": host_threads(), "kind": "port",
                                           "sample": "train_step on 2 x 128 tokens: numpy (BLAS threads) + the C++ MoE restatement"},
                          "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return
    if w["precision"] == "attn":
        # the checker's single-sequence decode step (numpy, one thread), scaled to the workload's sequences
        from oracle import attention as ora
        H, Hkv, hd, L, S = w["H"], w["Hkv"], w["hd"], w["history"], w["S"]
        g = np.random.Generator(np.random.Philox(w["seed"]))
        o = ora.KvCacheOracle(H, Hkv, hd, L + 8)
        o.keys = g.standard_normal((L - 1, Hkv * hd)).astype(np.float32)
        o.values = g.standard_normal((L - 1, Hkv * hd)).astype(np.float32)
        q, k, v = (g.standard_normal((1, n * hd)).astype(np.float32) for n in (H, Hkv, Hkv))
        ts = []
        for it in range(min(args.warmup, 1) + max(args.steps, 1)):
            o.keys, o.values = o.keys[:L - 1], o.values[:L - 1]
            t0 = time.perf_counter(); o.forward_cached(q, k, v); ts.append(time.perf_counter() - t0)
        us = float(np.median(ts[min(args.warmup, 1):])) * 1e6 * S
        print(json.dumps({"impl": "reference", "metric": "p50 microseconds per KV-cached attention decode step (64 sequences)",
                          "value": us, "unit": "us", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic", "config": {"workload": w["name"]},
                          "cpu_baseline": {"value": us, "unit": "us", "cores": 1, "kind": "port",
                                           "sample": "one sequence's decode step at the workload's history, times %d sequences" % S},
                          "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return
    value, dt, cores, sample, timed = time_oracle(w, reference_sample(w), max(args.steps, 1), min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "MoE-layer tokens/s (forward + backward)", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "sample": "%d tokens per step" % sample, "steps_timed": timed},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": "%d tokens of the workload's shape per step, forward + backward, %d host threads, %d steps timed"
                                   % (sample, cores, timed)},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_decode(args, w):
    """Latency of one quantized MoE layer on a decode-sized batch (p50 over graph replays)."""
    import torch
    from rustingbrain_b200 import MoeConfig, MoeLayer, _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    T, d, E, F = w["T"], w["d"], w["E"], w["F"]
    g = np.random.Generator(np.random.Philox(w["seed"]))

    def build_layer():
        layer = MoeLayer(d, MoeConfig(E, w["k"], F, w["shared"]), precision="q8", max_tokens=T, training=False)
        layer.set_weight(_lib.W_ROUTER, 0, (g.standard_normal((E, d)) * 0.02).astype(np.float32))

        def put(which, e, rows, cols):
            layer.set_weight_q8(which, e, g.integers(-127, 128, (rows, cols)).astype(np.int8),
                                g.uniform(1e-3, 4e-3, rows).astype(np.float32))
        for e in range(E):
            put(_lib.W_GATE, e, F, d); put(_lib.W_UP, e, F, d); put(_lib.W_DOWN, e, d, F)
        put(_lib.W_SHARED_GATE, 0, F, d); put(_lib.W_SHARED_UP, 0, F, d); put(_lib.W_SHARED_DOWN, 0, d, F)
        return layer

    layer = build_layer()
    x = torch.from_numpy(g.standard_normal((T, d)).astype(np.float32)).to(dev).bfloat16()
    y = torch.empty_like(x)
    side = torch.cuda.Stream()

    def capture(lay):
        with torch.cuda.stream(side):
            for _ in range(5):
                lay.forward(x, out=y)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            lay.forward(x, out=y)
        return gr

    with torch.cuda.stream(side):
        for _ in range(5):
            layer.forward(x, out=y)
    torch.cuda.synchronize()
    counts = layer._routing(T)[2]
    l0 = _lib.lib().moe_debug_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        layer.forward(x, out=y)
    per_layer = _lib.lib().moe_debug_launch_count() - l0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # larger than L2: weights come from HBM each time
    reps = max(args.steps, 1) * 50
    times = []
    for _ in range(max(args.warmup, 3) * 10):
        graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); graph.replay(); e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    clocks = sampler.stop()
    times = np.array(times)
    p50 = float(np.percentile(times, 50))
    # A decoder walks through its layers: the kernels' code and the small buffers stay in L2 from layer to layer,
    # only the weights are new.  Second protocol: two layers with weights of their own (2 x 152 MB > L2) take
    # turns, no flush.
    layer2 = build_layer()
    pair = [graph, capture(layer2)]
    for i in range(40):
        pair[i % 2].replay()
    torch.cuda.synchronize()
    turns = []
    for i in range(min(reps, 400)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); pair[i % 2].replay(); e1.record()
        e1.synchronize()
        turns.append(e0.elapsed_time(e1) * 1e3)
    layer2.close()
    active = int((counts > 0).sum()) + 1
    wbytes = active * 3 * d * F                  # int8 weights of the active experts + shared
    pk = peaks()
    line = {"metric": "p50 microseconds per quantized MoE layer (decode, 64 rows)", "value": p50, "unit": "us",
            "n_gpus": 1, "steps": reps, "warmup": max(args.warmup, 3) * 10, "ms_per_step": p50 / 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "int8 weights, bf16 activations",
            "data": "synthetic", "config": {"workload": w["name"], "l2": "256 MB buffer written between replays",
                                            "graph": "one CUDA graph per layer, %d kernels" % per_layer},
            "clocks": clocks, "gpu_launches": int(per_layer * reps), "p90_us": float(np.percentile(times, 90)),
            "p50_us_two_layers_taking_turns_no_flush": float(np.percentile(np.array(turns), 50)),
            "roofline": {"bound": "hbm", "achieved": wbytes / (p50 * 1e-6) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                         "frac": wbytes / (p50 * 1e-6) / 1e9 / pk["hbm"], "traffic": None,
                         "note": "int8 weight bytes of the %d active experts + shared (%.0f MB) / whole-layer p50" % (active - 1, wbytes / 1e6)}}
    layer.close()
    return line


def run_decode_attention(args, w):
    """One decode step of the batched KV-cache attention at a fixed history (p50 over replays).  Every step
    rotates and appends one row per sequence and streams every cached key and value once."""
    import torch
    from rustingbrain_b200 import _lib
    from rustingbrain_b200.kv_attention import KvCache
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    S, H, Hkv, hd, L = w["S"], w["H"], w["Hkv"], w["hd"], w["history"]
    # Two caches take turns: between two steps on the same cache the other one's 268 MB of keys and values pass
    # through the 126 MB L2, so every step reads from HBM without a flush whose dirty lines would have to be
    # written back under the step (the flushed variant is measured too and reported beside it).
    caches = [KvCache(S, H, Hkv, hd, capacity=L + 8, precision="bf16") for _ in range(2)]
    gen = torch.Generator(device=dev).manual_seed(w["seed"])
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=gen).bfloat16()
    chunk = 512                                  # prefill in pieces: the history only has to be there
    for cache in caches:
        for p0 in range(0, L - 1, chunk):
            n = min(chunk, L - 1 - p0)
            cache.forward_cached(rnd(S * n, H * hd), rnd(S * n, Hkv * hd), rnd(S * n, Hkv * hd), rows_per_sequence=n)
    q, k, v = rnd(S, H * hd), rnd(S, Hkv * hd), rnd(S, Hkv * hd)
    out = torch.empty_like(q)
    q0 = q.clone()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    reps = max(args.steps, 1) * 50
    side = torch.cuda.Stream()
    graphs = []
    per_step = 0
    for cache in caches:
        with torch.cuda.stream(side):
            for _ in range(3):
                cache.truncate(L - 1); q.copy_(q0); cache.forward_cached(q, k, v, out=out)
        torch.cuda.synchronize()
        cache.truncate(L - 1)
        l0 = _lib.lib().moe_debug_launch_count()
        graph = torch.cuda.CUDAGraph()           # the decode step as a serving loop would replay it
        with torch.cuda.graph(graph, stream=side):
            cache.forward_cached(q, k, v, out=out)
        per_step = _lib.lib().moe_debug_launch_count() - l0
        graphs.append(graph)

    def measure(n_warm, n_timed, flushed):
        ts, smp = [], None
        for it in range(n_warm + n_timed):
            if it == n_warm:
                torch.cuda.synchronize()
                smp = ClockSampler(0)
            cache, graph = caches[it % 2], graphs[it % 2]
            cache.truncate(L - 1)                # the same step every time: history L - 1, one new row
            q.copy_(q0)
            if flushed:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); graph.replay(); e1.record()
            e1.synchronize()
            if smp is not None:
                ts.append(e0.elapsed_time(e1) * 1e3)
        return np.array(ts), smp.stop()

    times, clocks = measure(max(args.warmup, 3) * 10, reps, False)
    flushed_times, _ = measure(10, min(reps, 200), True)
    for cache in caches:
        assert cache.lengths() == [L] * S        # also brings the host copy of the lengths back in line
    launches = per_step * reps
    times = np.array(times)
    p50 = float(np.percentile(times, 50))
    kv_bytes = 2 * S * L * Hkv * hd * 2          # every cached key and value once, bf16
    pk = peaks()
    line = {"metric": "p50 microseconds per KV-cached attention decode step (64 sequences)", "value": p50, "unit": "us",
            "n_gpus": 1, "steps": reps, "warmup": max(args.warmup, 3) * 10, "ms_per_step": p50 / 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 cache, f32 softmax",
            "data": "synthetic", "config": {"workload": w["name"],
                                            "l2": "inputs larger than L2: two caches of %.0f MB take turns, no flush" % (kv_bytes / 1e6),
                                            "graph": "one CUDA graph per step, %d kernels (attention incl. rotate + append, merge)" % per_step},
            "clocks": clocks, "gpu_launches": int(launches), "p90_us": float(np.percentile(times, 90)),
            "p50_us_with_256MB_flush_before_each_step": float(np.percentile(flushed_times, 50)),
            "roofline": {"bound": "hbm", "achieved": kv_bytes / (p50 * 1e-6) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                         "frac": kv_bytes / (p50 * 1e-6) / 1e9 / pk["hbm"], "traffic": None,
                         "note": "cached keys + values (%.0f MB) / whole-step p50" % (kv_bytes / 1e6)}}
    print(json.dumps(line))


def run_rmsnorm(args, w):
    """RMSNorm forward + backward over activations larger than L2; each direction timed with CUDA events."""
    import torch
    from rustingbrain_b200 import _lib
    from rustingbrain_b200.norm import RmsNorm
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    T, d = w["T"], w["d"]
    gen = torch.Generator(device=dev).manual_seed(w["seed"])
    x = torch.randn(T, d, device=dev, generator=gen).bfloat16()
    gy = torch.randn(T, d, device=dev, generator=gen).bfloat16()
    norm = RmsNorm(d, 1e-6)
    y = torch.empty_like(x)
    steps, warm = max(args.steps, 1), max(args.warmup, 3)
    for _ in range(warm):
        norm.forward(x, out=y); norm.backward(x, gy)
    torch.cuda.synchronize()
    l0 = _lib.lib().moe_debug_launch_count()
    sampler = ClockSampler(0)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * steps)]
    for i in range(steps):
        ev[3 * i].record(); norm.forward(x, out=y); ev[3 * i + 1].record(); norm.backward(x, gy); ev[3 * i + 2].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    launches = _lib.lib().moe_debug_launch_count() - l0
    fwd = float(np.mean([ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(steps)]))
    bwd = float(np.mean([ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(steps)]))
    tensor = T * d * 2
    pk = peaks()
    fb, bb = 2 * tensor / (fwd * 1e-3) / 1e9, 3 * tensor / (bwd * 1e-3) / 1e9
    line = {"metric": "RMSNorm tokens/s (forward + backward)", "value": T / ((fwd + bwd) * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": warm, "ms_per_step": fwd + bwd, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations, f32 arithmetic", "data": "synthetic",
            "config": {"workload": w["name"], "l2": "inputs larger than L2 (%.0f MB per tensor)" % (tensor / 1e6)},
            "clocks": clocks, "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": bb, "peak": pk["hbm"], "unit": "GB/s", "frac": bb / pk["hbm"], "traffic": None,
                         "note": "backward: x and grad_y read, grad_x written (%.0f MB) / %.3f ms; forward: %.0f MB / %.3f ms = %.0f GB/s = %.2f"
                                 % (3 * tensor / 1e6, bwd, 2 * tensor / 1e6, fwd, fb, fb / pk["hbm"])}}
    print(json.dumps(line))


def ep_parity_check(torch, dist, w, rank, world, local):
    """N ranks against ONE CPU checker over the concatenated batch, before anything is timed: 256 tokens per
    rank of the workload's d_model / experts / top-k with a small d_ff, forward + backward.  The checker is fed
    the devices' own router logits, so routing must be equal bit for bit; outputs, input gradients and weight
    gradients must agree within the bf16 tolerance.  Returns the dict that goes into the JSON line."""
    import oracle
    from oracle import OracleMoe
    from rustingbrain_b200 import MoeConfig, _lib
    from rustingbrain_b200.ep import ExpertParallelMoe
    d, E, k, shared, F, T = w["d"], w["E"], w["k"], w["shared"], 64, 256
    f32 = w["precision"] == "f32"
    tol = 1e-5 if f32 else 2e-2
    dt = torch.float32 if f32 else torch.bfloat16
    rnd = (lambda a: a) if f32 else (lambda a: torch.from_numpy(a).bfloat16().float().numpy())
    g = np.random.Generator(np.random.Philox(w["seed"] + 77))
    router = (g.standard_normal((E, d)) * 0.02).astype(np.float32)
    gate = rnd((g.standard_normal((E, F, d)) * 0.02).astype(np.float32))
    up = rnd((g.standard_normal((E, F, d)) * 0.02).astype(np.float32))
    down = rnd((g.standard_normal((E, d, F)) * 0.02).astype(np.float32))
    sh = tuple(rnd((g.standard_normal(sz) * 0.02).astype(np.float32)) for sz in ((F, d), (F, d), (d, F))) if shared else None
    layer = ExpertParallelMoe(d, MoeConfig(E, k, F, shared), precision=w["precision"], max_tokens=T, device=local,
                              capacity_factor=2.0)
    layer.set_weight(_lib.W_ROUTER, 0, router)
    for e in layer.owned_experts():
        layer.set_weight(_lib.W_GATE, e, gate[e]); layer.set_weight(_lib.W_UP, e, up[e]); layer.set_weight(_lib.W_DOWN, e, down[e])
    if shared:
        for i, m in enumerate(sh):
            layer.set_weight(_lib.W_SHARED_GATE + i, 0, m)
    gens = [np.random.Generator(np.random.Philox(w["seed"] + 1000 + r)) for r in range(world)]
    xs = [rnd(gen.standard_normal((T, d)).astype(np.float32)) for gen in gens]
    gys = [rnd(gen.standard_normal((T, d)).astype(np.float32)) for gen in gens]
    dev = torch.device("cuda", local)
    x = torch.from_numpy(xs[rank]).to(dev).to(dt)
    gy = torch.from_numpy(gys[rank]).to(dev).to(dt)
    y, cache = layer.forward_train(x)
    layer.zero_grad()
    gx = layer.backward(cache, gy)
    logits = layer.router_cache(T)[0]
    all_logits = [None] * world
    dist.all_gather_object(all_logits, logits)
    oracle.lib().orc_set_threads(max(1, host_threads() // world))
    ora = OracleMoe(d, E, k, F, shared)
    ora.set_weights(router, gate, up, down, sh)
    yo = ora.forward(np.concatenate(xs), logits=np.concatenate(all_logits))
    gxo = ora.backward(np.concatenate(gys))
    lo, hi = rank * T, (rank + 1) * T

    def rel(a, b):
        a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
        return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))

    e_dev, _, c_dev, _, _ = cache.routing()
    mine = {"routing_equal": bool(np.array_equal(e_dev, ora.routing()[0][lo:hi])),
            "rel_l2_y": rel(y.float().cpu().numpy(), yo[lo:hi]), "rel_l2_grad_x": rel(gx.float().cpu().numpy(), gxo[lo:hi])}
    gw = 0.0
    for e in layer.owned_experts():
        for which in (_lib.W_GATE, _lib.W_UP, _lib.W_DOWN):
            gw = max(gw, rel(layer.get_grad(which, e), ora.get_grad(which, e)))
    gw = max(gw, rel(layer.get_grad(_lib.W_ROUTER), ora.get_grad(_lib.W_ROUTER)))
    if shared:
        gw = max(gw, rel(layer.get_grad(_lib.W_SHARED_GATE), ora.get_grad(_lib.W_SHARED_GATE)))
    mine["rel_l2_grad_w"] = gw
    a, z = ora.losses()
    mine["loss_err"] = max(abs(cache.aux_loss() - a) / max(abs(a), 1e-30), abs(cache.z_loss() - z) / max(abs(z), 1e-30))
    layer.close()
    every = [None] * world
    dist.all_gather_object(every, mine)
    out = {"ranks": world, "tokens_per_rank": T, "d_model": d, "experts": E, "top_k": k, "d_ff": F, "tol": tol,
           "routing_equal": all(m["routing_equal"] for m in every)}
    for key in ("rel_l2_y", "rel_l2_grad_x", "rel_l2_grad_w", "loss_err"):
        out[key] = max(m[key] for m in every)
    out["ok"] = bool(out["routing_equal"] and out["rel_l2_y"] <= tol and out["rel_l2_grad_x"] <= tol
                     and out["rel_l2_grad_w"] <= tol and out["loss_err"] <= 1e-3)
    return out


def run_layer(args, w, torch, dist, world, rank, local, device, with_e2e, with_cpu):
    """One workload of the layer: timed steps with resident inputs, the host-buffer leg, rooflines."""
    from rustingbrain_b200 import MoeConfig, MoeLayer, _lib
    cfg = MoeConfig(w["E"], w["k"], w["F"], w["shared"])
    if world > 1:
        from rustingbrain_b200.ep import ExpertParallelMoe
        layer = ExpertParallelMoe(w["d"], cfg, precision=w["precision"], max_tokens=w["T"], device=local)
        load_weights(torch, layer, w, device, experts=set(layer.owned_experts()))
    else:
        layer = MoeLayer(w["d"], cfg, precision=w["precision"], max_tokens=w["T"], device=local, training=True)
        load_weights(torch, layer, w, device)
    x, gy = make_inputs(torch, w, rank, device)
    y = torch.empty_like(x)
    gx = torch.empty_like(x)

    def step():
        _, cache = layer.forward_train(x, out=y)
        layer.zero_grad()
        layer.backward(cache, gy, out=gx)
        if w.get("adam"):
            step.n += 1
            layer.step_adam(lr=3e-4, step=step.n)

    step.n = 0

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = _lib.lib().moe_debug_launch_count()
    layer.profile(True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = _lib.lib().moe_debug_launch_count() - launches0
    prof = layer.profile_read()
    layer.profile(False)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * w["T"] / (ms * 1e-3)

    # ---- end to end through the host-buffer entry points (copies inside the timed region) ----
    e2e = None
    if with_e2e:
        xh = torch.empty(w["T"], w["d"], dtype=torch.float32).pin_memory()
        gh = torch.empty(w["T"], w["d"], dtype=torch.float32).pin_memory()
        xh.copy_(x.float().cpu()); gh.copy_(gy.float().cpu())
        host = layer
        xn, gn = xh.numpy(), gh.numpy()
        yn = torch.empty(w["T"], w["d"], dtype=torch.float32).pin_memory().numpy()
        gxn = torch.empty(w["T"], w["d"], dtype=torch.float32).pin_memory().numpy()
        e2e_steps = max(1, min(args.steps, 10))
        for _ in range(2):
            _, c = host.forward_train(xn, out=yn); host.zero_grad(); host.backward(c, gn, out=gxn)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            yh, c = host.forward_train(xn, out=yn)
            host.zero_grad()
            gxh = host.backward(c, gn, out=gxn)
            aux = c.auxiliary_loss()
        barrier()
        dt = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([dt], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        nbytes = w["T"] * w["d"] * 4
        e2e = {"value": world * w["T"] / dt, "unit": "tokens/s", "h2d_bytes_per_step": 2 * nbytes,
               "d2h_bytes_per_step": 2 * nbytes + 8, "ms_per_step": dt * 1e3, "steps": e2e_steps}
    layer.close()
    del layer, x, gy, y, gx
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    pk = peaks()
    R = w["T"] * w["k"]
    gemm_stages = ("gemm_gate_up", "gemm_down", "dgrad_down", "wgrad_down", "dgrad_gate_up", "wgrad_gate_up")
    gemm_ms = sum(prof[s][0] for s in gemm_stages)
    gemm_launches = sum(prof[s][1] for s in gemm_stages)
    gemm_flops = 18.0 * R * w["d"] * w["F"] * args.steps      # 6RdF forward, twice that backward
    es = 4 if w["precision"] == "f32" else 2
    if w["precision"] == "f32":
        roof = {"bound": "hbm", "achieved": None, "peak": pk["hbm"], "unit": "GB/s", "frac": None, "traffic": None,
                "note": "f32 configuration (1e-5 parity bar): forward expert products on tcgen05 with three bf16 pieces per operand "
                        "(6 x the bf16 FLOPs), backward as f32 FMA on the CUDA cores; no single roofline applies to the step"}
    else:
        ach = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        # Operand and result bytes of the six launches (every matrix once): activations R x {d, F, 2F} in
        # bf16, weights in bf16, weight gradients in f32.  The ncu capture of the reduced case measured
        # DRAM read+write at 0.95 of these bytes (profiles/grouped_gemm_prof_case.md); traffic scales with
        # rows and experts, so the full-size figure is that ratio times the bytes below.
        d_, F_, E_ = w["d"], w["F"], w["E"] // world
        Rl = R   # rows per rank (balanced routing: every rank serves as many rows as it sends)
        gemm_bytes = (2 * (Rl * d_ + E_ * 2 * F_ * d_ + Rl * 3 * F_) + 2 * (Rl * F_ + E_ * d_ * F_ + Rl * d_)
                      + 2 * (Rl * d_ + E_ * d_ * F_ + Rl * 4 * F_) + 2 * (Rl * d_ + Rl * F_) + 4 * E_ * d_ * F_
                      + 2 * (Rl * 2 * F_ + E_ * 2 * F_ * d_ + Rl * d_) + 2 * (Rl * 2 * F_ + Rl * d_) + 4 * E_ * 2 * F_ * d_)
        roof = {"bound": "tensor", "achieved": ach, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                "frac": ach / pk["tf_sustained"] if ach else None, "traffic": 0.95 * gemm_bytes / 6.0,
                "traffic_unit": "bytes per launch (mean of the 6), ncu DRAM bytes of the reduced case scaled by rows",
                "algorithmic_bytes_per_launch": gemm_bytes / 6.0,
                "kernel": "grouped_gemm_wide_kernel (256x256 tiles; 5 of the 6 launches per step: gate|up, down, gate|up dgrad, "
                          "2 wgrad) and grouped_gemm_kernel (128x256 tiles; the down dgrad with the SwiGLU-backward epilogue)",
                "launches": gemm_launches, "ms_per_launch": gemm_ms / max(gemm_launches, 1),
                "flops_per_step": gemm_flops / args.steps, "peak_source": pk["src"] + " sustained bf16",
                "frac_of_measured_burst": ach / pk["tf_burst"] if ach else None,
                "frac_of_nominal_2250": ach / 2250.0 if ach else None}
    hbm = {}
    alg_bytes = {"permute": (w["T"] + 1.0 * R) * w["d"] * es, "combine": (R + w["T"] * (2 if w["shared"] else 1)) * w["d"] * es,
                 "grad_gather": (w["T"] + 2.0 * R) * w["d"] * es, "unpermute": (R + w["T"] * (3 if w["shared"] else 2)) * w["d"] * es,
                 "router": w["T"] * w["d"] * es + w["T"] * w["k"] * 8}
    for name, b in alg_bytes.items():
        t, n = prof[name]
        if t > 0:
            gbs = b * n / (t * 1e-3) / 1e9
            hbm[name] = {"ms": t / n, "GB/s": gbs, "frac": gbs / pk["hbm"]}
    line = {
        "metric": "MoE-layer tokens/s (forward + backward)", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w["precision"], "data": "synthetic",
        "config": {"workload": w["name"], "tokens_per_gpu": w["T"], "l2": "inputs larger than L2 (%.0f MB activations per pass)" % (w["T"] * w["d"] * es / 1e6),
                   "parallelism": "ep%d" % world if world > 1 else "single"},
        "clocks": clocks, "gpu_launches": int(launches), "roofline": roof, "hbm_kernels": hbm,
        "stage_ms_per_step": {k: v[0] / args.steps for k, v in prof.items() if v[1]},
    }
    if e2e:
        line["e2e"] = e2e
    if with_cpu:
        v, dt, cores, sample, timed = time_oracle(w, reference_sample(w), 2, 0, budget_s=30.0)
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": "%d tokens of the workload's shape, forward + backward, %.1f s per pass, %d passes timed"
                                          % (sample, dt, timed)}
    return line


def run_model(args, w):
    """train_step of the 55M model through the model-level C ABI: ids go up from the host and the loss comes back
    every step, so this number is end to end by construction."""
    import torch
    from rustingbrain_b200 import _lib
    from rustingbrain_b200.transformer import TransformerLm, TokenBatch
    torch.cuda.set_device(0)
    B, S = w["batch"], w["seq"]
    model = TransformerLm.builder().max_batch_rows(B * S).seed(w["seed"]).build()
    total, active = model.parameter_counts()
    g = np.random.Generator(np.random.Philox(w["seed"]))
    batch = TokenBatch([list(g.integers(0, 32000, S)) for _ in range(B)])
    steps, warm = max(args.steps, 1), max(args.warmup, 3)
    for _ in range(warm):
        loss = model.train_step_batch(batch)
    model.synchronize()
    l0 = _lib.lib().moe_debug_launch_count()
    sampler = ClockSampler(0)
    phases = np.zeros(4)
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = model.train_step_batch(batch)
        phases += np.array(model.last_step_ms())
    model.synchronize()
    wall = (time.perf_counter() - t0) / steps * 1e3
    clocks = sampler.stop()
    launches = _lib.lib().moe_debug_launch_count() - l0
    phases /= steps
    dev_ms = float(phases.sum())
    tokens = B * S
    flops = (6.0 * active + 12.0 * 8 * S * 512) * tokens      # the reference's own formula (docs/baseline.md:15)
    pk = peaks()
    ach = flops / (dev_ms * 1e-3) / 1e12
    line = {"metric": "language-model tokens/s (train_step: forward + backward + Adam)", "value": tokens / (wall * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warm, "ms_per_step": wall, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 products, f32 master weights", "data": "synthetic",
            "config": {"workload": w["name"], "parameters_total": total, "parameters_active": active,
                       "l2": "activations of a step (about 2 GB) are larger than L2"},
            "clocks": clocks, "gpu_launches": int(launches), "device_ms_per_step": dev_ms,
            "phase_ms": {"forward": float(phases[0]), "head_and_loss": float(phases[1]), "backward": float(phases[2]), "adam": float(phases[3])},
            "loss": {"lm_loss": loss.lm_loss, "auxiliary_loss": loss.auxiliary_loss},
            "reference_published": {"value": 36302, "unit": "tokens/s", "hardware": "RTX 3060 12 GB", "batch": "16 x 512 tokens",
                                    "note": "the reference's own figure for this model on other hardware and another batch shape "
                                            "(docs/baseline.md:21); context only, vs_baseline stays null"},
            "roofline": {"bound": "tensor", "achieved": ach, "peak": pk["tf_sustained"], "unit": "TFLOP/s", "frac": ach / pk["tf_sustained"],
                         "traffic": None, "flops_per_step": flops,
                         "note": "whole step: 6 x active parameters + attention, per token; device time of the four phases"},
            "e2e": {"value": tokens / (wall * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": tokens * 9, "d2h_bytes_per_step": 4,
                    "ms_per_step": wall, "note": "the step takes host token ids and returns the host loss: the same number as value"}}
    model.close()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="cfg4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the cfg3 / cfg5 legs the default 1-GPU run appends")
    ap.add_argument("--no-parity", action="store_true", help="skip the N-rank parity leg of a multi-GPU run")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
        return
    if w["precision"] == "q8":
        print(json.dumps(run_decode(args, w)))
        return
    if w["precision"] == "model":
        print(json.dumps(run_model(args, w)))
        return
    if w["precision"] == "attn":
        run_decode_attention(args, w)
        return
    if w["precision"] == "rmsnorm":
        run_rmsnorm(args, w)
        return

    import torch
    import torch.distributed as dist

    # libraries (NCCL) may print banners on stdout; keep it clean for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    args.warmup = max(args.warmup, 3)

    # ---- correctness of the N-rank path, before anything is timed ----
    parity = None
    if world > 1 and not args.no_parity:
        parity = ep_parity_check(torch, dist, w, rank, world, local)
        if not parity["ok"]:
            if rank == 0:
                os.dup2(real_stdout, 1)
                print(json.dumps({"error": "expert-parallel parity check failed", "ep_parity": parity}), flush=True)
            dist.destroy_process_group()
            sys.exit(3)

    line = run_layer(args, w, torch, dist, world, rank, local, device, not args.no_e2e, world == 1 and not args.no_cpu_baseline)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    if parity is not None:
        line["ep_parity"] = parity

    # ---- the two other single-GPU configurations the targets are written for, a few steps each ----
    if world == 1 and args.workload == "cfg4" and not args.no_extra:
        extra = {}
        short = argparse.Namespace(**vars(args))
        short.steps, short.warmup = min(args.steps, 10), 3
        c3 = run_layer(short, WORKLOADS["cfg3"], torch, dist, 1, 0, local, device, False, False)
        extra["cfg3"] = {k: c3[k] for k in ("value", "unit", "ms_per_step", "steps", "roofline", "hbm_kernels", "clocks", "config")}
        short.steps = 4
        c5 = run_decode(short, WORKLOADS["cfg5"])
        extra["cfg5"] = {k: c5[k] for k in ("value", "unit", "steps", "roofline", "clocks", "config", "p90_us",
                                               "p50_us_two_layers_taking_turns_no_flush")}
        line["extra"] = extra
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    print(json.dumps(line), flush=True)
    if world > 1:
        os.dup2(2, 1)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
