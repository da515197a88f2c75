"""The package's CPU operators put together as a model (models/cpu_model.py) against the plain
implementation: whole prompts, prompt then single tokens, greedy generation, and the command
line on --device cpu.  No GPU is needed."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_qwen2 as plain
from helpers import CONFIGS, make_folder, random_requests
from llaisys_b200.models.cpu_model import CpuModel

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_logits_whole_and_token_by_token(tmp_path, name):
    cfg = CONFIGS[name]
    folder = make_folder(tmp_path, cfg, seed=11, store="float32", attn_gain=8.0)
    config, weights = plain.load_model_folder(folder)
    model = CpuModel.from_folder(folder)
    toks = random_requests(cfg, [150], seed=1)[0]
    ref = plain.forward_logits(toks, config, weights)
    whole = model.step(toks)
    assert whole.dtype == np.float32 and np.abs(whole - ref).max() < 1e-4
    model.reset()
    cut = np.concatenate([model.step(toks[:100])] + [model.step([t]) for t in toks[100:]])
    assert np.abs(cut - ref).max() < 1e-4
    prompt = toks[:7]
    stop = config.get("eos_token_id", [])
    stop = stop if isinstance(stop, list) else [stop]
    assert model.generate(prompt, 6, stop) == plain.generate_greedy(prompt, config, weights, 6, stop)


def test_parts_it_does_not_know_are_refused():
    from llaisys_b200.config import config_from_dict
    import dataclasses
    spec = config_from_dict(CONFIGS["A"]).to_spec()
    odd = dataclasses.replace(spec, final_norm=dataclasses.replace(spec.final_norm, kind="layer_norm"))
    with pytest.raises(NotImplementedError, match="layer_norm"):
        CpuModel(odd, {})


def test_command_line_on_the_cpu(tmp_path):
    folder = make_folder(tmp_path / "m", CONFIGS["A"], seed=5, store="float32", attn_gain=8.0)
    config, weights = plain.load_model_folder(folder)
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    (tmp_path / "batch.txt").write_text("5,17,3,200\n[9, 8, 7]\n")
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--device", "cpu", "--model", str(folder), "--batch-file",
                          str(tmp_path / "batch.txt"), "--max_steps", "5", "--top_k", "1"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    for prompt in ([5, 17, 3, 200], [9, 8, 7]):
        assert str(prompt + plain.generate_greedy(prompt, config, weights, 5, [255])) in out.stdout
    out = subprocess.run([sys.executable, "-m", "llaisys_b200.cli", "--device", "cpu", "--model", str(folder), "--tokens", "1"],
                         env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode != 0 and "greedily" in out.stderr
