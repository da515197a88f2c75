import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TINY_A, TINY_B, make_folder
from llaisys_b200.config import load_config
from llaisys_b200.engine import DecoderModel
from llaisys_b200.parts import BuildEnv
from llaisys_b200.weights import (FolderSource, SafetensorsFile, WeightsError, check_tensors, kept_dtype,
                                  load_weights, write_random_model, write_safetensors)


def _model(folder, dtype=torch.bfloat16):
    return DecoderModel(load_config(folder).to_spec(), BuildEnv(dtype, torch.device("cpu")))


def _rewrite(folder, fn):
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.get(n).clone() for n in f.entries}
    fn(tensors)
    write_safetensors(folder / "model.safetensors", tensors)


def test_random_folder_is_complete_and_seeded(tmp_path):
    a = make_folder(tmp_path / "a", TINY_A, 0)
    b = make_folder(tmp_path / "b", TINY_A, 0)
    c = make_folder(tmp_path / "c", TINY_A, 1)
    assert (a / "config.json").exists() and (a / "model.safetensors").exists()
    fa, fb, fc = (SafetensorsFile(x / "model.safetensors") for x in (a, b, c))
    assert set(fa.entries) == set(_model(a).expected_tensors())
    assert "lm_head.weight" not in fa.entries                      # tied
    for n in fa.entries:
        assert torch.equal(fa.get(n), fb.get(n))
    assert not torch.equal(fa.get("model.norm.weight"), fc.get("model.norm.weight"))
    assert all(dt == "BF16" for dt, _ in fa.entries.values())
    w = fa.get("model.layers.0.mlp.up_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    assert abs(float(fa.get("model.norm.weight").float().mean()) - 1.0) < 0.02
    assert "lm_head.weight" in SafetensorsFile(make_folder(tmp_path / "d", TINY_B, 1) / "model.safetensors").entries


def test_plain_reader_agrees_with_ours(tmp_path):
    folder = make_folder(tmp_path, TINY_B, 1)
    _, w = plain.load_model_folder(folder)
    f = SafetensorsFile(folder / "model.safetensors")
    for n in f.entries:
        assert np.array_equal(w[n], f.get(n).double().numpy())


def test_one_error_lists_everything(tmp_path):
    folder = make_folder(tmp_path, TINY_B, 1)

    def damage(t):
        del t["model.layers.1.self_attn.k_proj.bias"]
        del t["model.norm.weight"]
        t["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
        t["rotary.inv_freq"] = torch.zeros(4)
        t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(232, 144, dtype=torch.bfloat16)
        t["model.embed_tokens.weight"] = torch.zeros(384, 144, dtype=torch.int32)
    _rewrite(folder, damage)
    with pytest.raises(WeightsError) as ei:
        check_tensors(_model(folder), FolderSource(folder))
    e = ei.value
    assert e.missing == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.mlp.up_proj.weight", "rotary.inv_freq"]
    assert e.wrong_shape == {"model.layers.0.mlp.down_proj.weight": ((232, 144), (144, 232))}
    assert list(e.wrong_kind) == ["model.embed_tokens.weight"]
    msg = str(e)
    for word in ("k_proj.bias", "model.norm.weight", "layers.7", "inv_freq", "[232, 144]", "[144, 232]", "stored as I32"):
        assert word in msg


def test_tied_head_may_be_present_untied_must(tmp_path):
    a = make_folder(tmp_path / "a", TINY_A, 0)
    _rewrite(a, lambda t: t.__setitem__("lm_head.weight", t["model.embed_tokens.weight"].clone()))
    check_tensors(_model(a), FolderSource(a))                     # a copy of the tied head is tolerated
    b = make_folder(tmp_path / "b", TINY_B, 1)
    _rewrite(b, lambda t: t.__delitem__("lm_head.weight"))
    with pytest.raises(WeightsError, match="lm_head.weight"):
        check_tensors(_model(b), FolderSource(b))


def test_kept_dtypes(tmp_path):
    assert kept_dtype("BF16", torch.bfloat16) == torch.bfloat16 and kept_dtype("F16", torch.bfloat16) == torch.bfloat16
    assert kept_dtype("F32", torch.bfloat16) == torch.float32 and kept_dtype("BF16", torch.float32) == torch.float32
    assert kept_dtype("I64", torch.bfloat16) == torch.int32
    folder = make_folder(tmp_path, TINY_A, 0)
    _rewrite(folder, lambda t: t.__setitem__("model.norm.weight", t["model.norm.weight"].float()))
    m = _model(folder, torch.bfloat16)
    load_weights(m, FolderSource(folder))
    assert m.final_norm.weight.dtype == torch.float32            # stored in 32-bit: stays so
    assert m.blocks[0].mixer.w_qkv.dtype == torch.bfloat16 and m.blocks[0].mixer.w_qkv.shape == (128, 64)
    assert m.blocks[0].ffn.gate_up.shape == (320, 64)
    assert m.head.weight is m.embedding.weight                   # tied: one tensor
    m32 = _model(folder, torch.float32)
    load_weights(m32, FolderSource(folder))
    assert m32.blocks[1].ffn.down.dtype == torch.float32


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        FolderSource(tmp_path)
    (tmp_path / "x.safetensors").write_bytes(b"\x05")
    with pytest.raises(ValueError):
        FolderSource(tmp_path)
