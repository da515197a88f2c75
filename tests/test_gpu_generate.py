"""Generation through the Python entry point and the command line, and replay through bin/trace_run."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import CONFIGS, Oracle, compare, make_folder, random_requests, tolerance

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


class Folders:
    """Model folders per configuration; the bfloat16 runs get a milder attention gain (see
    test_gpu_engine.GAIN for why)."""

    def __init__(self, tmp):
        self._tmp, self._made = tmp, {}

    def get(self, name, dtype="float32"):
        gain = 5.0 if dtype == "bfloat16" else 8.0
        if (name, gain) not in self._made:
            self._made[(name, gain)] = make_folder(self._tmp / f"{name}{int(gain)}", CONFIGS[name],
                                                   seed=7 + ord(name), attn_gain=gain)
        return self._made[(name, gain)]

    def __getitem__(self, name):
        return self.get(name)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return Folders(tmp_path_factory.mktemp("gen"))


def _greedy_is_consistent(oracle, prompt, new, dtype, config):
    """Every generated token must be the plain arg-max at its place, or, where the two best plain
    logits are closer than the precision's tolerance, one of the tokens within that tolerance."""
    seq = list(prompt) + list(new)
    ref = oracle.logits(seq[:-1])
    tol = tolerance(dtype, config, ref)
    for i, tok in enumerate(new):
        row = ref[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - 2 * tol, f"token {i} ({tok}) is not a maximum of the plain logits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from llaisys_b200.models import DeviceType, Qwen2
    cfg = CONFIGS[name]
    folder = folders.get(name, dtype)
    oracle = Oracle(folder)
    model = Qwen2(folder, DeviceType.NVIDIA, dtype=dtype, max_tokens=64 * 4)
    prompts = random_requests(cfg, [5, 9, 2, 30, 1, 17], seed=3)
    # the cache holds four rooms of 64: the six requests take two batches, slots are used again
    outs = model.generate_batch(prompts, max_new_tokens=8, top_k=1, stop_ids=[])
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    for p, new in zip(prompts, outs):
        assert len(new) == 8
        _greedy_is_consistent(oracle, p, new, td, cfg)
    if dtype == "float32":
        for p, new in zip(prompts[:3], outs):
            assert new == plain.generate_greedy(p, oracle.config, oracle.weights, 8)
    # the single-request signature of the reference: prompt + new tokens
    assert model.generate(prompts[0], max_new_tokens=8) == prompts[0] + outs[0]
    # a stop token ends a request early and is kept
    stop = outs[1][2]
    cut = model.generate_batch(prompts[:3], max_new_tokens=8, stop_ids=[stop])
    first = outs[1].index(stop)
    assert cut[1] == outs[1][:first + 1]
    assert not model.engine.cache.live_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_loop_one_step_ahead_of_the_host_decides_like_the_plain_loop(folders, dtype):
    """With the chosen tokens kept on the device the loop launches a step before it has seen the last tokens;
    tokens, reasons, steps per request and the slots given back must be those of the loop that waits."""
    from llaisys_b200.engine.generate import GenerationLoop
    from llaisys_b200.models import Qwen2
    from llaisys_b200.sampling import Sampler, SamplingParams
    cfg = CONFIGS["B"]
    model = Qwen2(folders.get("B", dtype), dtype=dtype, max_tokens=64 * 3)
    prompts = random_requests(cfg, [3, 11, 1, 25, 6, 2, 40], seed=9)
    for params, seed in ((SamplingParams(top_k=1), 0), (SamplingParams(temperature=0.9, top_k=0, top_p=0.95), 5)):
        free = GenerationLoop(model.engine, Sampler(params, seed), stop_ids=[])
        free.pipelined = False
        base = free.run(prompts, 10)
        # stop tokens that some requests meet early, some late, some never; a limit of one token; a long limit
        stops = sorted({base[0].tokens[0], base[1].tokens[4], base[3].tokens[9]})
        for max_new in (1, 2, 10):
            waiting = GenerationLoop(model.engine, Sampler(params, seed), stop_ids=stops)
            waiting.pipelined = False
            want = waiting.run(prompts, max_new)
            ahead = GenerationLoop(model.engine, Sampler(params, seed), stop_ids=stops)
            assert ahead.pipelined
            got = ahead.run(prompts, max_new)
            assert [(g.tokens, g.reason) for g in got] == [(g.tokens, g.reason) for g in want]
            assert ahead.batches_run == waiting.batches_run
            assert not model.engine.cache.live_slots
    model.engine.check()


def test_sampling_generation_is_reproducible_and_batch_independent(folders):
    from llaisys_b200.models import Qwen2
    model = Qwen2(folders["B"], dtype="float32", max_tokens=64 * 8)
    prompts = random_requests(CONFIGS["B"], [1, 7, 13, 20], seed=4)
    a = model.generate_batch(prompts, max_new_tokens=12, top_k=0, top_p=1.0, temperature=0.7, seed=11, stop_ids=[])
    b = model.generate_batch(prompts, max_new_tokens=12, top_k=0, top_p=1.0, temperature=0.7, seed=11, stop_ids=[])
    c = model.generate_batch(prompts, max_new_tokens=12, top_k=0, top_p=1.0, temperature=0.7, seed=12, stop_ids=[])
    assert a == b and a != c
    one_by_one = model.generate_batch(prompts, max_new_tokens=12, top_k=0, top_p=1.0, temperature=0.7, seed=11,
                                      stop_ids=[], max_batch=1)
    assert one_by_one == a                      # a request's draws do not depend on its company
    # every sampled token follows the rule given the plain logits and the documented uniform
    from llaisys_b200 import kernels
    oracle = Oracle(folders["B"])
    r = 2
    seq = prompts[r] + a[r]
    ref = oracle.logits(seq[:-1])
    agree = sum(plain.sample(ref[len(prompts[r]) - 1 + i], 0.7, 0, 1.0, kernels.uniform(11, r, i)) == tok
                for i, tok in enumerate(a[r]))
    assert agree >= 11


def test_command_line(folders, tmp_path):
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    # --test: the engine's tokens against the CPU model's, in both precisions
    for dtype in ("float32", "bfloat16"):
        out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folders.get("A", dtype)), "--tokens", "5,17,3,200",
                              "--max_steps", "6", "--test", "--dtype", dtype], env=env, capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        assert "Test passed" in out.stdout and "Tokens:" in out.stdout
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["B"]))
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--random-weights", str(cfg), "--seed", "3", "--tokens", "1,2,3",
                          "--max_steps", "4", "--temperature", "0.9", "--top_k", "20", "--top_p", "0.9"],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    # a file of requests of unequal lengths, generated as a batch and checked against the CPU model
    (tmp_path / "batch.txt").write_text("5,17,3,200,7,7,7,7,7\n[9, 8]\n1\n")
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folders["B"]), "--batch-file", str(tmp_path / "batch.txt"),
                          "--max_steps", "5", "--test", "--dtype", "float32"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("Tokens:") == 3 and "Test passed" in out.stdout
    # the same request on the CPU device gives the same tokens
    gpu = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folders["A"]), "--tokens", "5,17,3", "--max_steps", "4",
                          "--top_k", "1", "--dtype", "float32"], env=env, capture_output=True, text=True, timeout=600)
    cpu = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--device", "cpu", "--model", str(folders["A"]), "--tokens", "5,17,3",
                          "--max_steps", "4", "--top_k", "1"], env=env, capture_output=True, text=True, timeout=600)
    assert gpu.returncode == 0 and cpu.returncode == 0, gpu.stderr[-1000:] + cpu.stderr[-1000:]
    line = lambda o: o.stdout.split("Tokens:")[1].splitlines()[1]
    assert line(gpu) == line(cpu)


# ----------------------------------------------------------------------------- bin/trace_run
def _trace_lines(requests, batches, prompt_lens):
    """Steps of a trace: batches one after another; per batch the prompts in one step, then one
    token each; a request is ended in the step that feeds its last token."""
    lines, step, order = [], 0, []
    for batch in batches:
        fed = {r: prompt_lens[r] for r in batch}
        live = list(batch)
        entries = [{"id": f"r{r}", "tokens": requests[r][:fed[r]], "want": list(range(fed[r]))} for r in live]
        rows = [(r, p) for r in live for p in range(fed[r])]
        while live:
            done = [r for r in live if fed[r] >= len(requests[r])]
            lines.append(json.dumps({"step": step, "entries": entries, "end": [f"r{r}" for r in done]}))
            order.append((step, rows))
            step += 1
            live = [r for r in live if r not in done]
            entries = [{"id": f"r{r}", "tokens": [requests[r][fed[r]]], "want": [0]} for r in live]
            rows = [(r, fed[r]) for r in live]
            for r in live:
                fed[r] += 1
    return lines, order


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(folders, tmp_path, dtype):
    name = "B"
    cfg = CONFIGS[name]
    requests = random_requests(cfg, [1, 7, 70, 20, 40], seed=8)
    batches = [[0, 2, 4], [1, 3]]
    prompt_lens = [1, 3, 38, 20, 8]            # request 2: its last 32 tokens one by one; request 3: whole
    lines, order = _trace_lines(requests, batches, prompt_lens)
    lines.insert(3, json.dumps({"step": 1000, "entries": [], "end": []}))        # a step with nothing in it
    out_dir = tmp_path / "out"
    room = max(sum(-(-len(requests[r]) // 64) * 64 for r in b) for b in batches)
    folder = folders.get(name, dtype)
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(room)], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [json.loads(l)["step"] for l in lines]
    got = {}
    for step, rows in order:
        data = np.frombuffer((out_dir / f"{step}.f32").read_bytes(), dtype="<f4").reshape(len(rows), cfg["vocab_size"])
        for i, key in enumerate(rows):
            got[key] = data[i]
    assert not (out_dir / "1000.f32").exists()
    compare(got, Oracle(folder), requests, torch.float32 if dtype == "float32" else torch.bfloat16, cfg, "trace_run")
