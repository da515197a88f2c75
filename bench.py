#!/usr/bin/env python3
"""Decode and prefill throughput of llaisys_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The model has the layer sizes of the Qwen2-1.5B shape (DeepSeek-R1-Distill-Qwen-1.5B's
config) with seeded random bfloat16 weights; requests are seeded uniform-random token ids.
A "step" is one decode step.  The run times K decode steps of a batch of 8 sequences that hold
2,048 tokens each (context 4,096), and reports on one JSON line:

  value      decoded tokens a second at batch 8, timed on the device with CUDA events
  e2e        the same through the Python entry point (generate_batch: host token ids in,
             host token ids out, every step a pinned host-to-device copy of the step's
             description and a device-to-host read of the chosen tokens)
  prefill    one step over 2,048 prompt tokens: tokens a second, and its flops over the time
             over the peak of its dtype
  roofline   the decode step's bytes (every weight it uses once, and the cache of the live
             requests) over its time, against the measured copy bandwidth
  points     decode tokens a second at batch 1 and batch 64

`--shape 7b|32b` runs the same measurement at the two larger shapes, and `--workload own` runs
such a shape's own workload (16 prompts of 256..4096 tokens and 256 decode steps; 64 prompts of
512..2048 tokens and 128 steps) end to end through the generation loop; the reported metric of
the default run does not change.

Between timed steps nothing flushes L2: each decode step streams the 3.1 GB of weights, which
is larger than L2 (126 MB), so no step finds its inputs cached.  Peaks come from
MEASURED_PEAKS.json beside this file when it exists, else from the fallback figures below.
"""
from __future__ import annotations

import argparse
import contextlib
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN2_1_5B = {
    "architectures": ["Qwen2ForCausalLM"],
    "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "intermediate_size": 8960, "vocab_size": 151936, "max_position_embeddings": 131072,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False,
    "use_sliding_window": False, "sliding_window": 4096, "max_window_layers": 21,
    "eos_token_id": 151643,
}
# The other two large shapes that xsmccc/llaisys' Qwen2 code path serves; `--shape` selects them for
# measurements beside the default one (the reported metric stays that of the default shape).
SHAPES = {
    "1.5b": ("Qwen2-1.5B shape (DeepSeek-R1-Distill-Qwen-1.5B config)", QWEN2_1_5B),
    "7b": ("Qwen2.5-7B shape", dict(QWEN2_1_5B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
                                    num_key_value_heads=4, intermediate_size=18944, vocab_size=152064,
                                    max_position_embeddings=32768, rope_theta=1e6, max_window_layers=28)),
    "32b": ("Qwen2.5-32B shape", dict(QWEN2_1_5B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=40,
                                      num_key_value_heads=8, intermediate_size=27648, vocab_size=152064,
                                      max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-5,
                                      max_window_layers=64)),
}
PROMPT_LEN, CONTEXT, PREFILL_TOKENS = 2048, 4096, 2048
# Untimed decode steps between the prefill that fills the cache and the warm-up.  After a prefill burst at the power
# limit the device runs its next 40 to 70 ms at reduced clocks (measured: steps of 1.35, then 1.20, then 1.12 ms at
# batch 8); the decode measurements are of the steady state behind that.
SETTLE_STEPS = 64
# The two larger shapes' own workloads: (requests, shortest prompt, longest prompt, decode steps).  The prompts
# of unequal lengths go through one prefill step together, then every request decodes that many tokens.
OWN_WORKLOADS = {"7b": (16, 256, 4096, 256), "32b": (64, 512, 2048, 128)}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in d.items() if k in out and isinstance(v, (int, float))})
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs.

    The program is started before the warm-up steps and waited for until its first line has come, so that its
    start-up (a process to create, the management library to load) does not run beside the timed steps, where it
    was measured to take tenths of a millisecond per step from a host that enqueues 64-sequence steps.  region()
    marks the timed steps; the summary is over the samples that arrived between its start and shortly after its
    end (all samples since the start of the program if the region was shorter than a sampling period)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    PERIOD_MS = 50

    def __init__(self):
        self.rows, self.proc, self.t0, self.t1 = [], None, None, None
        self.first = threading.Event()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", str(self.PERIOD_MS)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            self.first.wait(timeout=5.0)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))
            self.first.set()

    def region_start(self):
        self.t0 = time.perf_counter()

    def region_end(self):
        self.t1 = time.perf_counter()

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.12)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        rows = [r for t, r in self.rows if self.t0 is not None and self.t0 <= t <= (self.t1 or t) + 1.5 * self.PERIOD_MS / 1e3]
        if not rows:
            rows = [r for _, r in self.rows]
        sm = [int(r[0]) for r in rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def linear_params(cfg, layers):
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    dh = H // cfg["num_attention_heads"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * dh
    per_layer = qkv * H + cfg["num_attention_heads"] * dh * H + 3 * I * H
    return per_layer * layers, cfg["vocab_size"] * H


def filled_slots(engine, batch, rng, vocab):
    """`batch` slots that hold PROMPT_LEN cached tokens each, put there by real prefill steps of up to
    eight sequences (the cache is filled the way serving fills it, through the step function)."""
    from llaisys_b200.engine import StepEntry
    slots = [engine.acquire() for _ in range(batch)]
    for i in range(0, batch, 8):
        engine.step([StepEntry(s, rng.integers(0, vocab, size=PROMPT_LEN).tolist(), []) for s in slots[i:i + 8]])
    return slots


def profile_run(args, model, cfg, rng) -> int:
    """Two uncaptured steps inside a cudaProfilerStart/Stop range, after a warm-up outside it."""
    import torch

    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.engine import Engine, StepEntry
    V = cfg.vocab_size
    engine = Engine(model, CacheConfig(max_tokens=max(args.batch, 1) * CONTEXT, max_seqs=max(args.batch, 1)), use_graphs=False)
    if args.profile == "prefill":
        def once():
            s = engine.acquire()
            engine.step([StepEntry(s, rng.integers(0, V, size=PREFILL_TOKENS).tolist(), [PREFILL_TOKENS - 1])])
            engine.release(s)
    else:
        slots = filled_slots(engine, args.batch, rng, V)

        def once():
            engine.step([StepEntry(s, [int(rng.integers(0, V))], [0]) for s in slots])
    for _ in range(2):
        once()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(2):
        once()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    engine.check()
    return 0


def timeline_run(args, model, cfg, rng) -> int:
    """Per-kernel timeline of whole steps as the device ran them (torch.profiler / CUPTI, no ncu): decode steps
    are replayed from their CUDA graph with programmatic dependent launch, as in serving.  Prints each kernel's
    total, and one layer's launches with their start offsets and durations; a kernel's own share of the layer
    is its end minus its predecessor's end (kernels start early and wait)."""
    import collections
    import tempfile

    import torch
    from torch.profiler import ProfilerActivity, profile

    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.engine import Engine, StepEntry
    V, B = cfg.vocab_size, max(args.batch, 1)
    engine = Engine(model, CacheConfig(max_tokens=B * CONTEXT, max_seqs=B))
    if args.timeline == "prefill":
        prompt = rng.integers(0, V, size=PREFILL_TOKENS).tolist()

        def once():
            s = engine.acquire()
            engine.step([StepEntry(s, prompt, [PREFILL_TOKENS - 1])])
            engine.release(s)
    else:
        slots = filled_slots(engine, B, rng, V)

        def once():
            engine.step([StepEntry(s, [int(rng.integers(0, V))], [0]) for s in slots])
    for _ in range(4):
        once()
    torch.cuda.synchronize()
    steps = 3
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            once()
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "trace.json")
        prof.export_chrome_trace(path)
        with open(path) as f:
            events = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    engine.check()
    events.sort(key=lambda e: e["ts"])
    last = events[-(len(events) // steps):]                  # the last step's kernels
    totals = collections.defaultdict(lambda: [0, 0.0])
    busy_end, gaps = last[0]["ts"], 0.0
    for e in last:
        name = e["name"].replace("(anonymous namespace)::", "").replace("void ", "")[:64]
        totals[name][0] += 1
        totals[name][1] += e["dur"]
        gaps += max(0.0, e["ts"] - busy_end)
        busy_end = max(busy_end, e["ts"] + e["dur"])
    print(f"{args.timeline} step: {len(last)} kernels, span {busy_end - last[0]['ts']:.1f} us, idle gaps {gaps:.1f} us")
    for name, (n, t) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
        print(f"{t:9.1f} us  n={n:4d}  avg {t / n:7.2f}  {name}")
    per_layer = max(1, (len(last) - 3) // max(1, cfg.num_hidden_layers))
    start = min(len(last) - 1, 1 + per_layer * (cfg.num_hidden_layers // 2))
    print("one layer from the middle of the step: start offset, duration, end, own share (end - previous end), kernel")
    t0, prev_end = last[start]["ts"], None
    for e in last[start:start + per_layer + 1]:
        end = e["ts"] + e["dur"] - t0
        own = "" if prev_end is None else f"{end - prev_end:7.2f}"
        print(f"  +{e['ts'] - t0:7.2f} {e['dur']:7.2f} {end:8.2f} {own:>7}  {e['name'].replace('(anonymous namespace)::', '')[:60]}  grid={e['args'].get('grid')}")
        prev_end = end
    return 0


STAMP_NAMES = {
    "gemm": ("gemm_tc.cu", ["set up", "input ready (grid dependency)", "first stage full", "all products issued", "accumulator ready",
                            "own partial rows pushed", "peers' partial rows received", "end"]),
    "attention": ("attention_mma.cu", ["set up", "projections ready (grid dependency)", "queries staged", "tiles walked",
                                       "warps' sums in shared memory", "merged pieces pushed", "peers' pieces received", "stored"]),
    "mlp": ("mlp_tc.cu", ["-", "activations ready (grid dependency)", "first tile of Wd issued", "last tile of Wd issued",
                          "last reduction issued", "reductions complete"]),
    "gate_up": ("gemm_tc2.cu", ["start", "first tile: accumulators ready", "first 32 tokens computed", "(warp joined)", "first 32 tokens stored",
                                "all tokens stored", "accumulators handed back", "second tile: accumulators ready",
                                "second tile: accumulators handed back"]),
    "qkv": ("gemm_tc2.cu", ["start", "first tile: accumulator ready", "first 32 tokens computed", "(warp joined)", "first 32 tokens stored",
                            "all tokens stored", "accumulator handed back", "second tile: accumulator ready",
                            "second tile: accumulator handed back"]),
    "down": ("gemm_tc2.cu", ["start", "first unit: accumulator ready", "second 32 tokens staged", "the reduction before has read its buffer",
                             "reduction issued", "all reductions issued", "accumulator handed back", "second unit: accumulator ready",
                             "second unit: accumulator handed back"]),
}


def stamps_run(args, model, cfg, rng) -> int:
    """Cycle stamps from inside one kernel of the decode step, in its place in the step (replayed from its CUDA graph):
    per stamp the minimum, median and maximum over the kernel's blocks, in SM cycles after the block saw its grid
    dependency resolve.  All stamps of a block read one SM's cycle counter.  Stamps that one thread takes are in
    program order; a stamp is not ordered with another thread's unless data flows between them (the clock read is
    no memory operation, so a barrier alone does not hold it in place).  A stamp costs a clock read and a store."""
    import numpy as np
    import torch

    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.engine import Engine, StepEntry
    from llaisys_b200.kernels import ops

    if args.stamps in ("gate_up", "down", "qkv"):
        # one of the prefill's two largest products alone (--tokens tokens on pairs of SMs): how long a tile's epilogue
        # takes (and, for gate/up, keeps the tensor cores waiting), in SM cycles after the block started
        from llaisys_b200 import kernels
        source, names = STAMP_NAMES[args.stamps]
        if args.stamps == "gate_up":
            x = torch.randn(args.tokens, cfg.hidden_size, device="cuda:0", dtype=torch.bfloat16)
            w = torch.randn(2 * cfg.intermediate_size, cfg.hidden_size, device="cuda:0", dtype=torch.bfloat16) * 0.02

            def product():
                kernels.linear_swiglu(x, w)
        elif args.stamps == "qkv":
            n_qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
            x = torch.randn(args.tokens, cfg.hidden_size, device="cuda:0", dtype=torch.bfloat16)
            w = torch.randn(n_qkv, cfg.hidden_size, device="cuda:0", dtype=torch.bfloat16) * 0.02
            bias = torch.randn(n_qkv, device="cuda:0", dtype=torch.bfloat16)

            def product():
                kernels.linear(x, w, bias)
        else:
            x = torch.randn(args.tokens, cfg.intermediate_size, device="cuda:0", dtype=torch.bfloat16)
            w = torch.randn(cfg.hidden_size, cfg.intermediate_size, device="cuda:0", dtype=torch.bfloat16) * 0.02
            stream = torch.zeros(args.tokens, cfg.hidden_size, device="cuda:0", dtype=torch.float32)

            def product():
                kernels.linear_into(x, w, None, stream)
        for _ in range(3):
            product()
        buf = torch.zeros((1 << 12, 16), dtype=torch.int64, device="cuda:0")
        ops.set_stamps(source, buf, 0)
        product()
        torch.cuda.synchronize()
        ops.set_stamps(source, None)
        st = buf.cpu().numpy().astype(np.float64)
        st = st[st[:, 1] != 0]
        print(f"{args.stamps}: {len(st)} blocks; SM cycles after the block's start ({args.tokens} tokens)")
        for i, name in enumerate(names):
            col = (st[:, i] - st[:, 0])[st[:, i] != 0]
            if i and len(col):
                print(f"  {name:40s} min {col.min():8.0f}   median {np.median(col):8.0f}   max {col.max():8.0f}")
        return 0

    B = args.batch
    engine = Engine(model, CacheConfig(max_tokens=B * CONTEXT, max_seqs=B))
    slots = filled_slots(engine, B, rng, cfg.vocab_size)

    def steps(n):
        for _ in range(n):
            engine.step([StepEntry(s, [int(rng.integers(0, cfg.vocab_size))], [0]) for s in slots])

    steps(SETTLE_STEPS)
    source, names = STAMP_NAMES[args.stamps]
    blocks = 0
    if args.stamps == "gemm":                      # the q/k/v product's grid, of all the launches of that module in a step
        n_qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
        bn, splits = ops.tc_plan(B, n_qkv, cfg.hidden_size, engine.sm_count)
        blocks = -(-n_qkv // 128) * -(-B // bn) * splits
    buf = torch.zeros((1 << 16, 16), dtype=torch.int64, device="cuda:0")
    ops.set_stamps(source, buf, blocks)
    steps(8)
    torch.cuda.synchronize()
    ops.set_stamps(source, None)
    engine.check()
    st = buf.cpu().numpy().astype(np.float64)
    st = st[st[:, 1] != 0]
    print(f"{args.stamps}: {len(st)} blocks of the last launch that stamped; SM cycles after the grid dependency resolved (batch {B})")
    for i, name in enumerate(names):
        if name == "-" or not (st[:, i] != 0).any():
            continue
        col = (st[:, i] - st[:, 1])[st[:, i] != 0]
        print(f"  {name:36s} min {col.min():8.0f}   median {np.median(col):8.0f}   max {col.max():8.0f}")
    return 0


def products_run(args, cfg) -> int:
    """The four matrix products of a layer timed alone at --tokens tokens, with every kernel that takes them:
    the one-CTA tcgen05 kernel and, for more than 256 tokens, the paired-SM kernel (which the library chooses)."""
    import torch

    from llaisys_b200.kernels import ops
    dev = torch.device("cuda:0")
    T, H, I = args.tokens, cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim

    reps = 20

    def graph_of(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        return g

    def replay_us(g):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps * 1e3

    print(f"{SHAPES[args.shape][0]}, {T} tokens: microseconds per launch (TFLOP/s); {reps} launches in a CUDA graph, "
          "the kernels taking turns five times, median")
    for name, N, K, dual in (("q/k/v", qkv, H, False), ("output", H, cfg.num_attention_heads * cfg.head_dim, False),
                             ("gate/up + SwiGLU", 2 * I, H, True), ("down", H, I, False)):
        x = (torch.randn(T, K, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        run = (lambda plan: ops.linear_swiglu(x, w, plan=plan)) if dual else (lambda plan: ops.linear(x, w, None, plan=plan))
        plans = [("one CTA per tile", ops.tc_plan(T, N // 2 if dual else N, K, ops._sm_count(dev), dual))]
        if T > 256:
            plans.append(("paired SMs", ("pair",)))
        graphs = [(label, graph_of(lambda plan=plan: run(plan))) for label, plan in plans]
        # for scale only: the library's product of the same operands (cuBLAS through torch.matmul; for gate/up
        # without the SwiGLU, writing [T, 2I])
        wt = w.t()
        graphs.append(("cuBLAS, for scale", graph_of(lambda: torch.matmul(x, wt))))
        times = {label: [] for label, _ in graphs}
        for _ in range(5):
            for label, g in graphs:
                times[label].append(replay_us(g))
        cells = []
        for label, _ in graphs:
            us = statistics.median(times[label])
            cells.append(f"{label} {us:.1f} ({2 * T * N * K / us / 1e6:.0f})")
        print(f"  {name:18s} " + "   ".join(cells))
    print("error word", ops.tc_error(dev))
    return 0


def own_workload(args, model, cfg, cfg_dict, layers, full_layers, shape_name, pk, pk_src, rng) -> int:
    """A shape's own workload through the generation loop (host token ids in and out): prompts of unequal
    lengths in one prefill step, then the stated number of decode steps.  Run twice; the second run is timed."""
    import torch

    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.engine import Engine
    from llaisys_b200.engine.generate import GenerationLoop
    from llaisys_b200.sampling import Sampler, SamplingParams

    n_req, lo, hi, steps = OWN_WORKLOADS[args.shape]
    lengths = rng.integers(lo, hi + 1, size=n_req).tolist()
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in lengths]
    room = sum(-(-(n + steps + 1) // 64) * 64 for n in lengths)
    engine = Engine(model, CacheConfig(max_tokens=room, max_seqs=n_req))
    for timed in (False, True):
        loop = GenerationLoop(engine, Sampler(SamplingParams(top_k=1)), stop_ids=[])
        torch.cuda.synchronize()
        with ClockSampler() as clk:
            clk.region_start()
            t0 = time.perf_counter()
            out = loop.run(prompts, max_new_tokens=steps + 1)
            marks = loop.step_marks
            clk.region_end()
        engine.check()
    assert all(len(g.tokens) == steps + 1 for g in out) and loop.batches_run == 1
    T = sum(lengths)
    prefill_s, decode_s = marks[0] - t0, marks[-1] - marks[0]
    lin, head = linear_params(cfg_dict, layers)
    attn_flops = layers * 4 * cfg.num_attention_heads * cfg.head_dim * sum(n * (n + 1) // 2 for n in lengths)
    prefill_flops = 2 * T * lin + 2 * n_req * head + attn_flops
    weight_bytes = model.weight_bytes() - model.embedding.weight.numel() * 2 + n_req * cfg.hidden_size * 2
    kv_bytes = (T + n_req * steps // 2) * engine.cache.bytes_per_token()
    ms = decode_s * 1e3 / steps
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    print(json.dumps({
        "metric": f"decode tok/s of the {shape_name}'s own workload, end to end through the generation loop",
        "value": round(n_req * steps / decode_s, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": steps,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), seeded uniform-random token ids",
        "config": {"model": shape_name, "layers": layers, "layers_of_config": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": n_req,
                   "prompt_len_min": min(lengths), "prompt_len_max": max(lengths), "prompt_tokens": T,
                   "decode_steps": steps, "cache_tokens": room, "parallelism": "single GPU", "peaks": pk_src},
        "clocks": clk.summary(),
        "prefill": {"value": round(T / prefill_s, 1), "tokens": T, "ms": round(prefill_s * 1e3, 2),
                    "frac": round(prefill_flops / prefill_s / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }))
    return 0


REF_DIR = os.environ.get("LLAISYS_REF_DIR") or os.path.join(ROOT, "baseline", "_ref")
REF_SOURCES = ["src/utils/*.cpp", "src/device/*.cpp", "src/device/cpu/*.cpp", "src/core/*/*.cpp", "src/tensor/*.cpp",
               "src/ops/*/*.cpp", "src/ops/*/cpu/*.cpp", "src/llaisys/*.cc", "src/models/qwen2/*.cpp"]


def build_reference(src: str) -> str:
    """Copies an unmodified checkout of xsmccc/llaisys to baseline/_ref and compiles its C++ sources with g++ into
    the shared library that its Python package loads (the project builds with xmake, which is not installed; the
    compiler, the optimisation level and the source list are those of tests/golden/make_golden.py).  Returns the
    folder to put on sys.path."""
    import glob
    import shutil
    if os.path.exists(REF_DIR):
        shutil.rmtree(REF_DIR)
    shutil.copytree(src, REF_DIR, ignore=shutil.ignore_patterns(".git"))
    srcs = []
    for pat in REF_SOURCES:
        srcs += sorted(glob.glob(os.path.join(REF_DIR, pat)))
    lib = os.path.join(REF_DIR, "python", "llaisys", "libllaisys", "libllaisys.so")
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", f"-I{os.path.join(REF_DIR, 'include')}", *srcs, "-o", lib])
    return os.path.join(REF_DIR, "python")


def reference_arm(args) -> int:
    """xsmccc/llaisys itself, unmodified, through its own public API (`llaisys.models.Qwen2(folder).generate`,
    python/llaisys/models/qwen2.py:212-283) on the one device it implements, the CPU.

    What can and cannot be the same as our arm: the layer sizes and the layer count are the benchmark's
    (Qwen2-1.5B shape, random weights), but that project serves ONE sequence, feeds it ONE token per call of its
    C function (prompt included, src/models/qwen2/qwen2.cpp:53-87) in float32 through scalar loops on one core, and
    has no CUDA path (every NVIDIA entry point is TO_BE_IMPLEMENTED).  A 2,048-token prompt would take hours, a
    batch does not exist.  So this arm measures decode tokens a second at batch 1, float32, after a prompt of
    `warmup` tokens, and says so in `config` (same_config: false); the ratio of the two arms is not a speed-up at
    equal work."""
    import glob
    import tempfile
    lib = os.path.join(REF_DIR, "python", "llaisys", "libllaisys", "libllaisys.so")
    why = None
    try:
        if args.reference_src:
            build_reference(args.reference_src)
        if not os.path.exists(lib):
            why = ("baseline/_ref holds no built copy of xsmccc/llaisys (pip cannot install it: no setup.py or pyproject.toml; "
                   "build it with: python bench.py --impl reference --reference-src <checkout>)")
    except (OSError, subprocess.CalledProcessError) as e:
        why = f"building xsmccc/llaisys with g++ failed: {type(e).__name__}: {e}"
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    import numpy as np
    steps, prompt_len = min(args.steps, 32), max(args.warmup, 3)
    cfg = dict(QWEN2_1_5B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    L, H, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkvh = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    dh = H // nh
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,), "lm_head.weight": (V, H)}
    for l in range(L):
        q = f"model.layers.{l}."
        shapes.update({q + "input_layernorm.weight": (H,), q + "post_attention_layernorm.weight": (H,),
                       q + "self_attn.q_proj.weight": (nh * dh, H), q + "self_attn.q_proj.bias": (nh * dh,),
                       q + "self_attn.k_proj.weight": (nkvh * dh, H), q + "self_attn.k_proj.bias": (nkvh * dh,),
                       q + "self_attn.v_proj.weight": (nkvh * dh, H), q + "self_attn.v_proj.bias": (nkvh * dh,),
                       q + "self_attn.o_proj.weight": (H, nh * dh), q + "mlp.gate_proj.weight": (I, H),
                       q + "mlp.up_proj.weight": (I, H), q + "mlp.down_proj.weight": (H, I)})
    # that project prints its progress on standard output: send it to standard error, so that this arm prints one line
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        with tempfile.TemporaryDirectory() as tmp:
            # float32 N(0, 0.02) weights (norm weights 1 + N), written tensor by tensor
            import struct
            header, off = {}, 0
            for name, shape in shapes.items():
                n = int(np.prod(shape)) * 4
                header[name] = {"dtype": "F32", "shape": list(shape), "data_offsets": [off, off + n]}
                off += n
            raw = json.dumps(header).encode()
            raw += b" " * (-len(raw) % 8)
            rng = np.random.default_rng(0)
            with open(os.path.join(tmp, "model.safetensors"), "wb") as f:
                f.write(struct.pack("<Q", len(raw)) + raw)
                for name, shape in shapes.items():
                    x = rng.standard_normal(size=shape, dtype=np.float32) * np.float32(0.02)
                    if name.endswith("norm.weight"):
                        x += np.float32(1.0)
                    f.write(x.tobytes())
            cfg_out = dict(cfg, torch_dtype="float32")
            cfg_out["max_position_embeddings"] = 4096           # its cache has this many rows per layer
            with open(os.path.join(tmp, "config.json"), "w") as f:
                json.dump(cfg_out, f)
            sys.path.insert(0, os.path.join(REF_DIR, "python"))
            import llaisys
            model = llaisys.models.Qwen2(tmp, llaisys.DeviceType.CPU)
            prompt = rng.integers(0, V, size=prompt_len).tolist()
            out = model.generate(prompt, max_new_tokens=1)       # the prompt, one token per call, and the first new token
            t0 = time.perf_counter()
            more = model.generate([out[-1]], max_new_tokens=steps)      # goes on in the same cache: `steps` calls of one token
            dt = time.perf_counter() - t0
            done = len(more) - 1
    except Exception as e:              # no room for the 7 GB folder, a missing package: say which
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps({"impl": "reference", "unavailable": f"running xsmccc/llaisys on the CPU failed: {type(e).__name__}: {e}"}))
        return 0
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    print(json.dumps({
        "impl": "reference",
        "metric": "decode tok/s @ batch 1 (Qwen2-1.5B shape, float32, CPU: the only device and batch xsmccc/llaisys serves)",
        "value": round(done / dt, 4), "unit": "tokens/s", "n_gpus": 0, "steps": done, "warmup": prompt_len,
        "ms_per_step": round(dt / done * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic: seeded random weights N(0,0.02), seeded uniform-random token ids",
        "config": {"model": SHAPES["1.5b"][0], "layers": L, "layers_of_config": QWEN2_1_5B["num_hidden_layers"], "hidden": H,
                   "heads": nh, "kv_heads": nkvh, "head_dim": dh, "intermediate": I, "vocab": V, "global_batch": 1,
                   "prompt_len": prompt_len, "device": "cpu", "same_config": False,
                   "why_not_same": "no batching, one token per call, no CUDA path: batch 8 and 2,048-token prompts do not exist there",
                   "build": "g++ -std=c++17 -O2 of the unmodified sources under baseline/_ref"},
    }))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--reference-src", default=os.environ.get("LLAISYS_REFERENCE_SRC"),
                    help="with --impl reference: a checkout of xsmccc/llaisys to copy to baseline/_ref and build there first")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="1.5b", help="layer sizes (default: the benchmark's)")
    ap.add_argument("--workload", choices=["uniform", "own"], default="uniform",
                    help="own: the 7b / 32b shape's own workload (unequal prompts in one prefill step, then decoding) "
                         "through the generation loop, instead of the benchmark's equal 2,048-token prompts")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / batch 64 points and the end-to-end run")
    ap.add_argument("--profile", choices=["decode", "prefill"], default=None,
                    help="for a profiler: warm up, then run two uncaptured steps of this kind between "
                         "cudaProfilerStart and cudaProfilerStop, print nothing else")
    ap.add_argument("--products", action="store_true",
                    help="time a layer's four matrix products alone at --tokens tokens, with each kernel that takes them")
    ap.add_argument("--tokens", type=int, default=PREFILL_TOKENS, help="tokens for --products")
    ap.add_argument("--prompt-len", type=int, default=None,
                    help="for measurements beside the reported one: tokens every sequence holds before decoding, and tokens of "
                         "the timed prefill step (default 2,048; the cache is sized for twice as many per sequence)")
    ap.add_argument("--stamps", choices=["gemm", "attention", "mlp", "gate_up", "down", "qkv"], default=None,
                    help="cycle stamps from inside one kernel of the decode step (the q/k/v product, decode attention or the "
                         "one-launch feed-forward), in its place in the step replayed from its CUDA graph, or (gate_up, down, qkv) from one "
                         "of the prefill's products alone at --tokens tokens; builds that kernel with -DLLB_STAMPS=1")
    ap.add_argument("--timeline", choices=["decode", "prefill"], default=None,
                    help="print the per-kernel timeline of a step (torch.profiler, no ncu) instead of measuring")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.stamps:
        os.environ["LLAISYS_STAMPS"] = "1"           # read when the package is imported, below
    if args.gpus != 1:
        print(f"bench.py: llaisys_b200 is a single-GPU library; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.workload == "own" and args.shape not in OWN_WORKLOADS:
        print(f"bench.py: --workload own needs --shape {' or '.join(sorted(OWN_WORKLOADS))}")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.prompt_len:
        g = globals()
        g["PROMPT_LEN"], g["CONTEXT"], g["PREFILL_TOKENS"] = args.prompt_len, 2 * args.prompt_len, args.prompt_len

    import numpy as np
    import torch

    from llaisys_b200 import kernels
    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.config import config_from_dict
    from llaisys_b200.engine import DecoderModel, Engine, StepEntry
    from llaisys_b200.engine.generate import GenerationLoop
    from llaisys_b200.parts import BuildEnv
    from llaisys_b200.sampling import Sampler, SamplingParams
    from llaisys_b200.weights import RandomSource, load_weights

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    shape_name, shape = SHAPES[args.shape]
    cfg_dict = dict(shape)
    full_layers = cfg_dict["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg_dict["num_hidden_layers"] = layers
    cfg = config_from_dict(cfg_dict)
    if args.products:
        return products_run(args, cfg)
    model = DecoderModel(cfg.to_spec(), BuildEnv(torch.bfloat16, dev))
    load_weights(model, RandomSource(model.expected_tensors(), seed=0, dtype=torch.bfloat16, device=dev))
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)
    V = cfg.vocab_size

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    if args.profile:
        return profile_run(args, model, cfg, rng)
    if args.timeline:
        return timeline_run(args, model, cfg, rng)
    if args.stamps:
        return stamps_run(args, model, cfg, rng)
    if args.workload == "own":
        return own_workload(args, model, cfg, cfg_dict, layers, full_layers, shape_name, pk, pk_src, rng)

    # ---- prefill: one step over 2,048 tokens
    engine = Engine(model, CacheConfig(max_tokens=max(64, args.batch) * CONTEXT, max_seqs=max(64, args.batch)))
    prompt = rng.integers(0, V, size=PREFILL_TOKENS).tolist()

    def prefill_once():
        s = engine.acquire()
        engine.step([StepEntry(s, prompt, [PREFILL_TOKENS - 1])])
        engine.release(s)

    for _ in range(3):
        prefill_once()
    torch.cuda.synchronize()
    reps = 8                       # back to back: the host enqueues a step while the device still runs the one before
    a, b = events()
    a.record()
    for _ in range(reps):
        prefill_once()
    b.record()
    torch.cuda.synchronize()
    prefill_ms = a.elapsed_time(b) / reps
    lin, head = linear_params(cfg_dict, layers)
    dh, nh = cfg.head_dim, cfg.num_attention_heads
    attn_flops = layers * 4 * nh * dh * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)
    prefill_flops = 2 * PREFILL_TOKENS * lin + 2 * head + attn_flops
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode at a given batch: sequences that already hold PROMPT_LEN tokens each
    def decode(batch, steps, warmup, clocks=True):
        slots = filled_slots(engine, batch, rng, V)
        warmup += SETTLE_STEPS
        toks = rng.integers(0, V, size=(warmup + steps, batch)).tolist()
        sampler = Sampler(SamplingParams(top_k=1))
        with (ClockSampler() if clocks else contextlib.nullcontext()) as clk:      # up and sampling before the warm-up
            for i in range(warmup):
                sampler.on_device(engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, toks[i])]), slots, [i] * batch)
            torch.cuda.synchronize()
            n0 = kernels.launch_count()
            a, b = events()
            # a collection of the host's garbage (the prompts of the fill are a few hundred thousand objects) inside a
            # region of some tens of milliseconds shows as milliseconds of idle device: collect before, not during
            gc.collect()
            gc.disable()
            if clk:
                clk.region_start()
            a.record()
            for i in range(warmup, warmup + steps):
                sampler.on_device(engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, toks[i])]), slots, [i] * batch)
            b.record()
            torch.cuda.synchronize()
            gc.enable()
            if clk:
                clk.region_end()
        ms = a.elapsed_time(b) / steps
        launches = kernels.launch_count() - n0
        ctx = PROMPT_LEN + warmup + steps // 2            # mean cached length over the timed steps
        for s in slots:
            engine.release(s)
        engine.check()
        return ms, launches, clk.summary() if clk else None, ctx

    ms, launches, clocks, ctx_len = decode(args.batch, args.steps, args.warmup)
    value = args.batch * 1e3 / ms
    weight_bytes = model.weight_bytes() - model.embedding.weight.numel() * 2 + args.batch * cfg.hidden_size * 2
    kv_bytes = args.batch * ctx_len * engine.cache.bytes_per_token()
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4)}

    points, e2e = {}, None
    if not args.no_points:
        for b in (1, 64):
            m, _, _, _ = decode(b, max(8, args.steps), 3, clocks=False)
            points[f"decode_b{b}"] = round(b * 1e3 / m, 1)
        # ---- end to end through the generation loop: host ids in, host ids out
        prompts = [rng.integers(0, V, size=PROMPT_LEN).tolist() for _ in range(args.batch)]
        loop = GenerationLoop(engine, Sampler(SamplingParams(top_k=1)), stop_ids=[])
        n = SETTLE_STEPS + args.warmup + args.steps
        loop.run(prompts, max_new_tokens=n + 1)
        marks = loop.step_marks
        dt = marks[-1] - marks[-1 - args.steps]
        meta_ints = 3 * args.batch + (args.batch + 1) + 3 * args.batch + 1 + args.batch * (CONTEXT // 64)
        e2e = {"value": round(args.batch * args.steps / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": 4 * meta_ints, "d2h_bytes_per_step": 4 * args.batch}

    out = {
        "metric": f"decode tok/s @ batch {args.batch} ({shape_name.split(' shape')[0]} shape, bf16, {PROMPT_LEN}-token prompts, context {CONTEXT})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), seeded uniform-random token ids",
        "config": {"model": shape_name, "layers": layers,
                   "layers_of_config": full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "settle_steps": SETTLE_STEPS,
                   "parallelism": "single GPU", "l2": f"no flush: each step streams {weight_bytes / 1e9:.1f} GB of weights, larger than L2",
                   "peaks": pk_src},
        "clocks": clocks, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
    }
    if e2e:
        out["e2e"] = e2e
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
