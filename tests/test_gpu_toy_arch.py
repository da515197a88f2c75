"""Another architecture, registered from here, goes through everything a user touches (model
folder, engine, entry point, command line, trace replay) without an edit inside the package,
and agrees with its own plain implementation.  The architecture and its parts are in toy_arch.py."""
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import toy_arch
from helpers import run_batches, run_chunked, run_whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
ENV = dict(os.environ, PYTHONPATH=os.pathsep.join([str(ROOT), str(ROOT / "tests")]), LLAISYS_PLUGINS="toy_arch")


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from llaisys_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    path = write_random_model(tmp_path_factory.mktemp("toy"), toy_arch.TOY, seed=4, dtype="float32")
    f = SafetensorsFile(path / "model.safetensors")
    # N(0, 0.02) weights leave every softmax flat: scale the matrices so that keys, routing and state matter
    is_norm = re.compile(r"(\.n\d|^fn)\.weight$")
    write_safetensors(path / "model.safetensors", {n: f.get(n) * (1.0 if is_norm.search(n) else 8.0) for n in f.entries})
    return path


def _check(got, requests, cfg, w, what):
    for r, toks in enumerate(requests):
        ref = toy_arch.plain_logits(toks, cfg, w)
        for p in range(len(toks)):
            err = float(np.abs(got[(r, p)] - ref[p]).max())
            assert err < 1e-4, f"{what}: request {r} position {p}: max |diff| {err:.3e}"
    assert float(np.std(ref)) > 1e-2


def test_the_architecture_builds_from_its_folder(folder):
    from llaisys_b200.config import known_architectures, load_config
    from llaisys_b200.engine import DecoderModel
    from llaisys_b200.parts import BuildEnv
    assert "ToyForCausalLM" in known_architectures()
    cfg = load_config(folder)
    assert type(cfg).__name__ == "ToyConfig"
    model = DecoderModel(cfg.to_spec(), BuildEnv(torch.float32, torch.device("cuda:0")))
    assert [len(b.sublayers) for b in model.blocks] == [3, 2, 2]
    # users of the cache: the mixers of the five entries of the run order
    assert model.call_users == [(0,), (1,), (2,), (3,), (4,)]
    assert model.state_sizes() == [0, 40, 0, 40, 0] and model.cache_of() == [None, None, None, None, 2]
    needs = model.kv_needs()
    assert (needs[0].key_dim, needs[0].value_dim, needs[0].window) == (12, 6, 70) and needs[1] is None
    assert {"l0.wide.v.weight", "l0.routed.experts.1.weight", "l1.mean.mix.weight", "l2.attn.k_proj.weight"} <= set(model.expected_tensors())


def test_engine_against_the_toys_plain_implementation(folder):
    from helpers import build_engine
    cfg, w = plain.load_model_folder(folder)
    rng = np.random.default_rng(0)
    requests = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in (150, 9, 70)]
    engine = build_engine(folder, torch.float32, max_tokens=64 * 6, max_seqs=3)
    assert not engine.use_graphs                                   # the toy parts read back from the device
    assert len(engine.cache.k_pools) == 2 and engine.cache.v_pools[0].shape[-1] == 6 and set(engine.cache.state) == {1, 3}
    assert engine.cache.k_pools[1].shape[0] == 1                   # one cache for both runs of layer 2
    _check(run_whole(engine, requests), requests, cfg, w, "whole")
    _check(run_chunked(engine, requests, [40, 30, 1, 65]), requests, cfg, w, "chunked")
    # together, the shorter ones ending earlier, in slots whose pages and state the runs above used
    _check(run_batches(engine, requests, [[0, 1, 2]], [100, 3, 50]), requests, cfg, w, "batch")
    assert not engine.cache.live_slots


def test_generation_command_line_and_replay(folder, tmp_path):
    from llaisys_b200.models import CausalLM
    cfg, w = plain.load_model_folder(folder)
    prompt = [3, 14, 15, 9, 26, 5]
    model = CausalLM(folder, dtype="float32", max_tokens=256)
    out = model.generate(prompt, max_new_tokens=6, top_k=1)
    assert out[:len(prompt)] == prompt and len(out) == len(prompt) + 6
    ref = toy_arch.plain_logits(out[:-1], cfg, w)
    for i, tok in enumerate(out[len(prompt):]):
        row = ref[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - 2e-4, f"generated token {i} is not the plain arg-max"
    del model

    # the command line, as a process of its own that learns of the architecture through LLAISYS_PLUGINS
    run = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folder), "--tokens", ",".join(map(str, prompt)),
                          "--max_steps", "6", "--dtype", "float32", "--top_k", "1"], env=ENV, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert str(out) in run.stdout
    no_plugin = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--model", str(folder), "--tokens", "1", "--max_steps", "1"],
                               env=dict(ENV, LLAISYS_PLUGINS=""), capture_output=True, text=True, timeout=600)
    assert no_plugin.returncode != 0 and "unknown architecture" in no_plugin.stderr

    # replay: two requests start together, the shorter one ends first
    reqs = [out, [7, 7, 2, 40, 11]]
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": reqs[0][:4], "want": [0, 1, 2, 3]},
                                                 {"id": "b", "tokens": reqs[1][:2], "want": [0, 1]}], "end": []})]
    rows = [[(0, p) for p in range(4)] + [(1, p) for p in range(2)]]
    for s in range(1, len(reqs[0]) - 3):
        entries, keys, end = [{"id": "a", "tokens": [reqs[0][3 + s]], "want": [0]}], [(0, 3 + s)], []
        if 1 + s < len(reqs[1]):
            entries.append({"id": "b", "tokens": [reqs[1][1 + s]], "want": [0]})
            keys.append((1, 1 + s))
            if 2 + s == len(reqs[1]):
                end.append("b")
        lines.append(json.dumps({"step": s, "entries": entries, "end": end}))
        rows.append(keys)
    out_dir = tmp_path / "out"
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out_dir),
                           "--max-tokens", "128"], input="\n".join(lines) + "\n", env=ENV, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = {}
    for s, keys in enumerate(rows):
        data = np.frombuffer((out_dir / f"{s}.f32").read_bytes(), dtype="<f4").reshape(len(keys), cfg["vocab_size"])
        for i, key in enumerate(keys):
            got[key] = data[i]
    _check(got, reqs, cfg, w, "trace_run")
