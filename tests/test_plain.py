"""The plain implementation against xsmccc/llaisys' own CPU code (recorded under tests/golden/)
and against its own invariants."""
import importlib.util
import json
from pathlib import Path

import numpy as np

import plain_qwen2 as plain

GOLDEN = Path(__file__).with_name("golden")


def _golden(name="tiny_a"):
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rec = json.loads((GOLDEN / f"{name}_reference.json").read_text())
    weights = {k: v.astype(np.float64) for k, v in mod.tiny_weights(rec["config"], rec["seed"], rec.get("gain", 1.0)).items()}
    return rec, weights


def test_logits_match_reference_operators():
    rec, w = _golden()
    want = np.array(rec["logits"]).reshape(rec["logits_shape"])
    got = plain.forward_logits(rec["prompt"], rec["config"], w)
    assert np.abs(got - want).max() < 2e-6


def test_greedy_tokens_match_reference_model():
    rec, w = _golden()
    n = len(rec["prompt"])
    assert rec["generated"][:n] == rec["prompt"]
    got = plain.generate_greedy(rec["prompt"], rec["config"], w, max_new_tokens=8)
    assert got == rec["generated"][n:]


def test_window_layers_match_the_reference_operator_on_sliced_keys():
    """Case B: theta 1e6, eps 1e-5, head size 24, 6 heads on 2, an untied head, and a window of 8 keys
    from layer 1 on, where the recorded logits come from that project's own self_attention called per
    query row on keys and values sliced to the window.  21 tokens: most rows have lost keys to the window."""
    rec, w = _golden("tiny_b")
    cfg = rec["config"]
    assert cfg["sliding_window"] == 8 and cfg["max_window_layers"] == 1 and len(rec["prompt"]) > 2 * cfg["sliding_window"]
    want = np.array(rec["logits"]).reshape(rec["logits_shape"])
    got = plain.forward_logits(rec["prompt"], cfg, w)
    # that project computes in float32: with scores spread over +-10 (the gain) its own rounding is a few 1e-6 of
    # logits near 1; a window that is off by one key moves the logits by 0.5
    assert np.abs(got - want).max() < 1e-5
    # the window matters in this case: without it, or one key longer or shorter, the logits are other logits
    for other in (dict(cfg, use_sliding_window=False), dict(cfg, sliding_window=9), dict(cfg, sliding_window=7),
                  dict(cfg, max_window_layers=2)):
        assert np.abs(plain.forward_logits(rec["prompt"], other, w) - want).max() > 1e-3
    # that project's model applies no window: its greedy tokens are those of the plain model without one
    n = len(rec["prompt"])
    got = plain.generate_greedy(rec["prompt"], dict(cfg, use_sliding_window=False), w, max_new_tokens=8)
    assert got == rec["generated"][n:]


def test_attention_decode_equals_last_row_of_whole():
    rng = np.random.default_rng(3)
    q, k, v = rng.normal(size=(7, 6, 8)), rng.normal(size=(7, 2, 8)), rng.normal(size=(7, 2, 8))
    whole = plain.self_attention(q, k, v, 0.3, window=3)
    last = plain.self_attention(q[-1:], k, v, 0.3, window=3)
    assert np.allclose(whole[-1:], last)
    # a window as long as the sequence is no window
    assert np.allclose(plain.self_attention(q, k, v, 0.3, window=7), plain.self_attention(q, k, v, 0.3))


def test_window_sees_exactly_w_keys():
    # one key dominates: once it leaves the window the output must stop following its value
    T, d, W = 12, 4, 5
    q = np.ones((T, 1, d))
    k = np.zeros((T, 1, d))
    k[2] = 50.0
    v = np.zeros((T, 1, d))
    v[2] = 1.0
    out = plain.self_attention(q, k, v, 1.0, window=W)[:, 0, 0]
    assert out[2] > 0.99 and out[2 + W - 1] > 0.99 and abs(out[2 + W]) < 1e-12


def test_rope_is_a_rotation_and_relative():
    rng = np.random.default_rng(0)
    x, y = rng.normal(size=(1, 1, 16)), rng.normal(size=(1, 1, 16))
    for theta in (1e4, 1e6):
        a = plain.rope(x, [5], theta)
        assert np.allclose(np.linalg.norm(a), np.linalg.norm(x))
        d1 = (plain.rope(x, [9], theta) * plain.rope(y, [4], theta)).sum()
        d2 = (plain.rope(x, [105], theta) * plain.rope(y, [100], theta)).sum()
        assert np.allclose(d1, d2)
    assert np.allclose(plain.rope(x, [0], 1e4), x)


def test_sampling_rules():
    logits = np.log(np.array([0.1, 0.4, 0.2, 0.3]))
    assert plain.sample(logits, temperature=0.0) == 1
    assert plain.sample(logits, top_k=1, u=0.99) == 1
    # inverse CDF in index order: cdf = .1 .5 .7 1
    assert [plain.sample(logits, u=u) for u in (0.0, 0.09, 0.11, 0.49, 0.51, 0.71, 0.999)] == [0, 0, 1, 1, 2, 3, 3]
    # top_k=2 keeps {1, 3}: cdf over kept = .4/.7, 1
    assert [plain.sample(logits, top_k=2, u=u) for u in (0.0, 0.5, 0.6, 0.99)] == [1, 1, 3, 3]
    # top_p=0.5: sorted .4 .3 .2 .1; prefix mass before each: 0 .4 .7 -> keep {1, 3}
    assert [plain.sample(logits, top_p=0.5, u=u) for u in (0.0, 0.5, 0.6, 0.99)] == [1, 1, 3, 3]
    # a low temperature sharpens
    assert plain.sample(logits, temperature=0.01, u=0.9) == 1


def test_safetensors_reader_roundtrip(tmp_path):
    import struct
    a = np.arange(6, dtype="<f4").reshape(2, 3)
    bf = (np.array([1.0, -2.5, 3.0], dtype="<f4").view("<u4") >> 16).astype("<u2")
    blobs = a.tobytes() + bf.tobytes()
    header = {"a": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]},
              "b": {"dtype": "BF16", "shape": [3], "data_offsets": [24, 30]},
              "__metadata__": {"format": "pt"}}
    h = json.dumps(header).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + blobs)
    got = plain.read_safetensors(tmp_path / "m.safetensors")
    assert np.array_equal(got["a"], a) and np.array_equal(got["b"], [1.0, -2.5, 3.0])
