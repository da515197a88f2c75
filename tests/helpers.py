"""Shared by the tests: the two tiny configurations, model folders, the plain oracle's logits,
and the three ways of cutting requests into steps."""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

import plain_qwen2 as plain

# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 160, "vocab_size": 256, "max_position_embeddings": 512,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": True,
    "use_sliding_window": False, "eos_token_id": 255,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 144, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 24, "intermediate_size": 232, "vocab_size": 384, "max_position_embeddings": 640,
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1, "eos_token_id": [383, 382],
}
# A third one for the window's edge across pages: head size 48, one kv head, window of 70 keys.
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 136, "vocab_size": 200, "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-6, "rope_theta": 50000.0, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 0,
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def make_folder(tmp, config: dict, seed: int, store="bfloat16", attn_gain: float = 1.0) -> Path:
    """A model folder with seeded random weights.  attn_gain > 1 scales the query and key
    projections so that attention scores spread out and single keys matter: with plain
    N(0, 0.02) weights every softmax is nearly flat and a lost key would hardly show."""
    from llaisys_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    folder = write_random_model(Path(tmp), config, seed, store)
    if attn_gain != 1.0:
        f = SafetensorsFile(folder / "model.safetensors")
        out = {}
        for name in f.entries:
            t = f.get(name).clone()
            if ".q_proj." in name or ".k_proj." in name:
                t = (t.float() * attn_gain).to(t.dtype)
            out[name] = t
        write_safetensors(folder / "model.safetensors", out)
    return folder


def random_requests(config: dict, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, config["vocab_size"], size=n).tolist() for n in lengths]


class Oracle:
    """Plain logits of whole requests, computed once per request."""

    def __init__(self, folder):
        self.config, self.weights = plain.load_model_folder(folder)
        self._memo = {}

    def logits(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward_logits(list(tokens), self.config, self.weights)
        return self._memo[key]


def tolerance(dtype: torch.dtype, config: dict, ref: np.ndarray) -> float:
    """Largest allowed |engine - plain| over a logits array.

    float32: 1e-4 absolute.  bfloat16: activations are rounded to 8 significant bits
    (unit round-off u = 2^-9) about six times per layer and twice outside; the errors add up
    like a random walk, so a logit carries about u * sqrt(6 L + 2) of the logits' typical size.
    The bound is eight times that, times the root mean square of the reference logits."""
    if dtype == torch.float32:
        return 1e-4
    u = 2.0 ** -9
    L = config["num_hidden_layers"]
    return 8 * u * math.sqrt(6 * L + 2) * float(np.sqrt(np.mean(ref ** 2)))


def build_engine(folder, dtype: torch.dtype, max_tokens: int, max_seqs=None, use_graphs=True):
    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.config import load_config
    from llaisys_b200.engine import build_engine as be
    from llaisys_b200.weights import FolderSource
    cfg = load_config(folder)
    return be(cfg.to_spec(), dtype, "cuda:0", CacheConfig(max_tokens=max_tokens, max_seqs=max_seqs), FolderSource(folder),
              use_graphs=use_graphs)


# ----------------------------------------------------------------------------- schedules
# Each returns {(request index, position): logits row (numpy float32)} for every position.

def run_whole(engine, requests):
    from llaisys_b200.engine import StepEntry
    got = {}
    for r, toks in enumerate(requests):
        slot = engine.acquire()
        out = engine.step([StepEntry(slot, toks, list(range(len(toks))))]).cpu().numpy()
        engine.check()
        engine.release(slot)
        for p in range(len(toks)):
            got[(r, p)] = out[p]
    return got


def run_tail_by_one(engine, requests, tail=32):
    from llaisys_b200.engine import StepEntry
    got = {}
    for r, toks in enumerate(requests):
        slot = engine.acquire()
        head = max(0, len(toks) - tail)
        if head:
            out = engine.step([StepEntry(slot, toks[:head], list(range(head)))]).cpu().numpy()
            for p in range(head):
                got[(r, p)] = out[p]
        for p in range(head, len(toks)):
            got[(r, p)] = engine.step([StepEntry(slot, [toks[p]], [0])]).cpu().numpy()[0]
        engine.check()
        engine.release(slot)
    return got


def run_batches(engine, requests, batches, prompt_lens):
    """batches: lists of request indices that start together.  A request's first
    prompt_lens[r] tokens go in the first step, the rest one per step; shorter requests end
    earlier and give their slot back while the others go on."""
    from llaisys_b200.engine import StepEntry
    got = {}
    for batch in batches:
        slot = {r: engine.acquire() for r in batch}
        fed = {r: prompt_lens[r] for r in batch}
        entries = [StepEntry(slot[r], requests[r][:fed[r]], list(range(fed[r]))) for r in batch]
        out = engine.step(entries).cpu().numpy()
        row = 0
        for r in batch:
            for p in range(fed[r]):
                got[(r, p)] = out[row]
                row += 1
        live = list(batch)
        while True:
            for r in [r for r in live if fed[r] >= len(requests[r])]:
                engine.release(slot.pop(r))
                live.remove(r)
            if not live:
                break
            out = engine.step([StepEntry(slot[r], [requests[r][fed[r]]], [0]) for r in live]).cpu().numpy()
            for i, r in enumerate(live):
                got[(r, fed[r])] = out[i]
                fed[r] += 1
        engine.check()
    return got


def run_chunked(engine, requests, cuts):
    """Each request alone, its tokens fed in several multi-token steps: `cuts` lists the portion
    lengths tried in turn (the last one is repeated until the request is used up), so a portion
    meets history in the slot and, on a window layer, a ring that has already wrapped."""
    from llaisys_b200.engine import StepEntry
    got = {}
    for r, toks in enumerate(requests):
        slot = engine.acquire()
        at, i = 0, 0
        while at < len(toks):
            n = min(cuts[min(i, len(cuts) - 1)], len(toks) - at)
            out = engine.step([StepEntry(slot, toks[at:at + n], list(range(n)))]).cpu().numpy()
            for p in range(n):
                got[(r, at + p)] = out[p]
            at, i = at + n, i + 1
        engine.check()
        engine.release(slot)
    return got


def run_mixed(engine, requests, plans):
    """All requests live together; plans[r] lists the portion lengths request r brings step by
    step (0: it sits this step out).  In one step some requests bring a single token onto
    history, others a fresh prompt, others a further portion.  A request whose plan is used up
    ends and frees its slot while the others go on."""
    from llaisys_b200.engine import StepEntry
    got = {}
    slot = {r: engine.acquire() for r in range(len(requests))}
    fed = {r: 0 for r in slot}
    step = 0
    while slot:
        entries, who = [], []
        for r in sorted(slot):
            plan = plans[r]
            n = plan[step] if step < len(plan) else 1
            n = min(n, len(requests[r]) - fed[r])
            if n > 0:
                entries.append(StepEntry(slot[r], requests[r][fed[r]:fed[r] + n], list(range(n))))
                who.append((r, n))
        if entries:
            out = engine.step(entries).cpu().numpy()
            row = 0
            for r, n in who:
                for p in range(n):
                    got[(r, fed[r] + p)] = out[row]
                    row += 1
                fed[r] += n
        for r in [r for r in slot if fed[r] >= len(requests[r])]:
            engine.release(slot.pop(r))
        step += 1
    engine.check()
    return got


def compare(got, oracle: Oracle, requests, dtype, config, what=""):
    """Asserts every logits row against the plain implementation; reports the first wrong place."""
    worst, worst_at = 0.0, None
    for r, toks in enumerate(requests):
        ref = oracle.logits(toks)
        tol = tolerance(dtype, config, ref)
        for p in range(len(toks)):
            assert (r, p) in got, f"{what}: no logits for request {r} position {p}"
            err = float(np.abs(got[(r, p)].astype(np.float64) - ref[p]).max())
            assert np.isfinite(err), f"{what}: non-finite logits at request {r} position {p}"
            assert err <= tol, (f"{what}: first wrong place is request {r} (length {len(toks)}) position {p}: "
                                f"max |diff| {err:.3e} > {tol:.3e}")
            if err / tol > worst:
                worst, worst_at = err / tol, (r, p, err)
    return worst, worst_at
