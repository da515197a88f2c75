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
    # operands of products follow the model; what enters 32-bit arithmetic only stays 32-bit if stored so
    assert kept_dtype("F32", torch.bfloat16) == torch.bfloat16 and kept_dtype("F32", torch.bfloat16, "vector") == torch.float32
    assert kept_dtype("BF16", torch.bfloat16, "vector") == torch.bfloat16 and kept_dtype("BF16", torch.float32) == torch.float32
    assert kept_dtype("I64", torch.bfloat16) == torch.int32
    folder = make_folder(tmp_path, TINY_A, 0)

    def to32(t):
        for n in ("model.norm.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.bias",
                  "model.layers.1.mlp.down_proj.weight"):
            t[n] = t[n].float()
    _rewrite(folder, to32)
    m = _model(folder, torch.bfloat16)
    load_weights(m, FolderSource(folder))
    mixer, ffn = m.blocks[0].sublayers[0].part, m.blocks[0].sublayers[1].part
    assert m.final_norm.weight.dtype == torch.float32            # a norm's weight stored in 32-bit: stays so
    assert mixer.b_qkv.dtype == torch.float32                    # one of the three biases is 32-bit: the fused bias is
    assert mixer.w_qkv.dtype == torch.bfloat16 and mixer.w_qkv.shape == (128, 64)      # matrices follow the model
    assert m.blocks[1].sublayers[1].part.down.dtype == torch.bfloat16
    assert ffn.gate_up.shape == (320, 64)
    assert m.head.weight is m.embedding.weight                   # tied: one tensor
    m32 = _model(folder, torch.float32)
    load_weights(m32, FolderSource(folder))
    assert m32.blocks[1].sublayers[1].part.down.dtype == torch.float32


def test_random_weights_are_a_function_of_seed_name_and_element():
    from llaisys_b200.parts import TensorDecl
    from llaisys_b200.weights import RandomSource
    from llaisys_b200.weights.rng import normal, tensor_key
    decls = {"a.weight": TensorDecl((40, 30)), "n.weight": TensorDecl((30,), init="one_plus_normal", use="vector")}
    src = RandomSource(decls, seed=5, dtype=torch.float32)
    a = src.get("a.weight")
    assert torch.equal(a, RandomSource({"a.weight": decls["a.weight"]}, 5, torch.float32).get("a.weight"))   # company does not matter
    assert not torch.equal(a, RandomSource(decls, 6, torch.float32).get("a.weight"))
    # any piece of a tensor can be made alone
    assert (normal(tensor_key(5, "a.weight"), 100, first=333, std=0.02) == a.reshape(-1)[333:433].numpy()).all()
    assert abs(float(a.std()) - 0.02) < 2e-3 and abs(float(src.get("n.weight").mean()) - 1.0) < 2e-2
    big = normal(tensor_key(1, "x"), 200000)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1) < 0.01 and abs((big ** 4).mean() - 3) < 0.1 and abs(big).max() > 3.5


def test_deferred_tensors_are_made_one_at_a_time(tmp_path):
    from llaisys_b200.weights import Deferred
    alive, peak = [0], [0]

    def make(i):
        alive[0] += 1
        peak[0] = max(peak[0], alive[0])
        t = torch.full((4, 3), float(i))
        import weakref
        weakref.finalize(t, lambda: alive.__setitem__(0, alive[0] - 1))
        return t
    write_safetensors(tmp_path / "d.safetensors", [(f"t{i}", Deferred(torch.float32, (4, 3), lambda i=i: make(i))) for i in range(5)])
    f = SafetensorsFile(tmp_path / "d.safetensors")
    assert [float(f.get(f"t{i}")[0, 0]) for i in range(5)] == [0.0, 1.0, 2.0, 3.0, 4.0] and peak[0] == 1
    with pytest.raises(ValueError, match="declared"):
        write_safetensors(tmp_path / "e.safetensors", [("t", Deferred(torch.float32, (2,), lambda: torch.zeros(3)))])


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        FolderSource(tmp_path)
    (tmp_path / "x.safetensors").write_bytes(b"\x05")
    with pytest.raises(ValueError):
        FolderSource(tmp_path)
