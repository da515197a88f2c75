"""The engine at the layer sizes that the benchmark runs (the 1.5B, 7B and 32B shapes of the
architecture), against the plain implementation: the kernels' plans for these widths, head
counts and groups are the ones that serving uses, which the tiny configurations never reach.

One or two layers and a small vocabulary keep the plain float64
model within seconds; every size of a layer is the shape's own."""
import pytest
import torch

from helpers import (Oracle, build_engine, compare, make_folder, random_requests, run_batches, run_chunked, run_mixed,
                     run_tail_by_one)

pytestmark = pytest.mark.gpu

SHAPES = {
    "1.5b": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 1536,
             "num_attention_heads": 12, "num_key_value_heads": 2, "intermediate_size": 8960, "vocab_size": 20011,
             "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
             "tie_word_embeddings": False, "use_sliding_window": False, "sliding_window": 4096},
    "7b": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 3584,
           "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 5000,
           "max_position_embeddings": 32768, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
           "tie_word_embeddings": False, "use_sliding_window": False},
    "32b": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 5120,
            "num_attention_heads": 40, "num_key_value_heads": 8, "intermediate_size": 27648, "vocab_size": 3001,
            "max_position_embeddings": 32768, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
            "tie_word_embeddings": False, "use_sliding_window": False},
}
LENGTHS = {"1.5b": [130, 40, 67], "7b": [100, 35, 64], "32b": [70, 20, 33]}


@pytest.fixture(scope="module", params=sorted(SHAPES))
def shape(request, tmp_path_factory):
    name = request.param
    # Query and key projections are scaled so that a score's standard deviation (0.0004 gain^2
    # hidden_size with N(0, 0.02) weights) is 0.6 at every width, which is what the 1.5B shape has
    # unscaled.  The error that a score's own bfloat16 rounding sends through the softmax grows
    # with that spread, and the bound of helpers.tolerance counts roundings of activations only:
    # an emulation that rounds a plain float32 model at the engine's rounding points is as far from
    # the plain model as the engine is (both leave the bound together when the spread is tripled).
    gain = (1536.0 / SHAPES[name]["hidden_size"]) ** 0.5
    folder = make_folder(tmp_path_factory.mktemp(f"shape{name.replace('.', '_')}"), SHAPES[name], seed=7, attn_gain=gain)
    return name, folder, Oracle(folder), random_requests(SHAPES[name], LENGTHS[name], seed=11)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_then_decoding(shape, dtype):
    name, folder, oracle, requests = shape
    cfg = SHAPES[name]
    engine = build_engine(folder, dtype, max_tokens=sum(-(-len(r) // 64) * 64 for r in requests))
    prompt_lens = [len(r) - cut for r, cut in zip(requests, (12, 5, 9))]
    got = run_batches(engine, requests, [[0, 1, 2]], prompt_lens)
    worst = compare(got, oracle, requests, dtype, cfg, f"{name} batch")
    print(f"{name} {dtype} batch: worst error/tolerance {worst}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portions_and_mixed_steps(shape, dtype):
    """A prompt fed in portions across a page edge, and steps that mix single tokens, a fresh prompt
    and a further portion, at the benchmark's layer sizes."""
    name, folder, oracle, requests = shape
    cfg = SHAPES[name]
    engine = build_engine(folder, dtype, max_tokens=sum(-(-len(r) // 64) * 64 for r in requests), max_seqs=3)
    compare(run_chunked(engine, requests, [30, 35, 1, 64]), oracle, requests, dtype, cfg, f"{name} portions")
    plans = [[40, 1, 1, 30, 1], [0, 0, 20], [1, 1, 33, 0, 20]]
    compare(run_mixed(engine, requests, plans), oracle, requests, dtype, cfg, f"{name} mixed steps")
    assert not engine.cache.live_slots


def test_tail_by_one_in_bfloat16(shape):
    name, folder, oracle, requests = shape
    engine = build_engine(folder, torch.bfloat16, max_tokens=192)
    compare(run_tail_by_one(engine, requests[:1], tail=8), oracle, requests[:1], torch.bfloat16, SHAPES[name],
            f"{name} tail-by-one")


def test_a_prompt_of_some_hundred_tokens_in_bfloat16(shape):
    """More than 256 tokens in a step: the products run on pairs of SMs, attention over several row blocks."""
    name, folder, oracle, _ = shape
    requests = random_requests(SHAPES[name], [600 if name == "1.5b" else 300, 70], seed=31)
    engine = build_engine(folder, torch.bfloat16, max_tokens=sum(-(-len(r) // 64) * 64 for r in requests))
    got = run_batches(engine, requests, [[0, 1]], [len(r) - 2 for r in requests])
    compare(got, oracle, requests, torch.bfloat16, SHAPES[name], f"{name} long prompt")
