"""Sizes that take the less travelled paths of the kernels: head sizes that are no power of two
or above 128, as many key/value heads as query heads or a single one, a width and an
intermediate size that are no multiple of 8 (no tensor-core product, no 16-byte accesses), odd
vocabularies, a window that is no multiple of a page.  Each configuration goes through the
engine whole and with its last tokens one by one, in both dtypes, against the plain model."""
import pytest
import torch

from helpers import Oracle, build_engine, compare, make_folder, random_requests, run_batches, run_tail_by_one

pytestmark = pytest.mark.gpu

ODD = {
    # head size 80 (tensor-core decode and prefill kernels at a size that is no power of two), every query head its own keys
    "E": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 400, "num_attention_heads": 5,
          "num_key_value_heads": 5, "intermediate_size": 344, "vocab_size": 1001, "max_position_embeddings": 512,
          "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False,
          "use_sliding_window": True, "sliding_window": 33, "max_window_layers": 1},
    # head size 160 (above what the tensor-core attention takes), one key/value head, an intermediate size that is no multiple of 8
    "F": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 320, "num_attention_heads": 2,
          "num_key_value_heads": 1, "intermediate_size": 150, "vocab_size": 515, "max_position_embeddings": 300,
          "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": True, "use_sliding_window": False},
    # a width that is no multiple of 8, head size 20, a head size given apart from the width (5 * 20 = 100 != 108)
    "G": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 108, "num_attention_heads": 5,
          "num_key_value_heads": 1, "head_dim": 20, "intermediate_size": 72, "vocab_size": 203, "max_position_embeddings": 256,
          "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False, "use_sliding_window": False},
}
LENGTHS = {"E": [100, 7, 66], "F": [130, 3, 64], "G": [90, 65, 1]}


@pytest.fixture(scope="module", params=sorted(ODD))
def odd(request, tmp_path_factory):
    name = request.param
    folder = make_folder(tmp_path_factory.mktemp(f"odd{name}"), ODD[name], seed=ord(name), attn_gain=3.0)
    return name, folder, Oracle(folder), random_requests(ODD[name], LENGTHS[name], seed=23)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_odd_sizes_batch_and_tail(odd, dtype):
    name, folder, oracle, requests = odd
    cfg = ODD[name]
    engine = build_engine(folder, dtype, max_tokens=sum(-(-len(r) // 64) * 64 for r in requests))
    got = run_batches(engine, requests, [[0, 1, 2]], [max(1, len(r) - 10) for r in requests])
    compare(got, oracle, requests, dtype, cfg, f"{name} batch")
    compare(run_tail_by_one(engine, requests[:1], tail=12), oracle, requests[:1], dtype, cfg, f"{name} tail-by-one")
