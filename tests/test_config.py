import json

import pytest

from helpers import TINY_A, TINY_B
from llaisys_b200.config import (ConfigError, Qwen2Config, config_from_dict, known_architectures, load_config,
                                 register_architecture)


def test_reads_own_keys():
    c = config_from_dict(TINY_B)
    assert isinstance(c, Qwen2Config)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 144, 6, 2)
    assert (c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (24, 232, 384, 640)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.eos_token_id == (383, 382)
    a = config_from_dict(TINY_A)
    assert a.head_dim == 16 and a.tie_word_embeddings and a.eos_token_id == (255,)


def test_window_layers():
    c = config_from_dict(TINY_B)
    assert [c.layer_window(l) for l in range(3)] == [None, 8, 8]
    assert [config_from_dict(TINY_A).layer_window(l) for l in range(2)] == [None, None]
    d = dict(TINY_B, use_sliding_window=False)
    assert all(config_from_dict(d).layer_window(l) is None for l in range(3))
    d = dict(TINY_B)
    del d["max_window_layers"]          # absent: no layer is windowed
    assert all(config_from_dict(d).layer_window(l) is None for l in range(3))


def test_spec_chooses_parts_layer_by_layer():
    spec = config_from_dict(TINY_B).to_spec()
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2]
    assert [[sub.category for sub in l.sublayers] for l in spec.layers] == [["mixer", "ffn"]] * 3
    assert [l.mixers()[0].params["window"] for l in spec.layers] == [None, 8, 8]
    m = spec.layers[1].sublayers[0].part
    assert spec.layers[1].sublayers[0].norm.prefix == "model.layers.1.input_layernorm"
    assert m.kind == "gqa_attention" and m.prefix == "model.layers.1.self_attn"
    assert m.params["position"].kind == "rope_half_split" and m.params["position"].params["theta"] == 1e6
    assert abs(m.params["scale"] - 24 ** -0.5) < 1e-12
    ffn = spec.layers[0].sublayers[1].part
    assert ffn.kind == "swiglu_mlp" and ffn.params["intermediate_size"] == 232
    assert spec.final_norm.params["eps"] == 1e-5 and spec.head.params["tied_to"] is None
    assert config_from_dict(TINY_A).to_spec().head.params["tied_to"] == "model.embed_tokens.weight"
    assert spec.stop_token_ids == (383, 382)


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "max_position_embeddings", "vocab_size", "rms_norm_eps",
                                 "rope_theta"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch, word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"hidden_size": 66}, "head_dim"), ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"), ({"rope_theta": -1}, "rope_theta"), ({"vocab_size": 0}, "positive"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding_window"), ({"num_hidden_layers": 2.5}, "integer"),
])
def test_inconsistent_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY_A, **patch))


def test_unknown_architecture_lists_known():
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["NopeForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    assert "Qwen2ForCausalLM" in known_architectures()


def test_roundtrip_and_folder(tmp_path):
    c = config_from_dict(TINY_B)
    assert config_from_dict(c.to_dict()) == c
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert load_config(tmp_path) == config_from_dict(TINY_A)
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nowhere")


def test_another_architecture_registers():
    @register_architecture("ToyForCausalLM")
    class Toy:
        @classmethod
        def from_dict(cls, d):
            return cls()
    try:
        assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), Toy)
    finally:
        from llaisys_b200.config import registry
        del registry._ARCHITECTURES["ToyForCausalLM"]
