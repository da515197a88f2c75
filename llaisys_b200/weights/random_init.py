"""The random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.registry import config_from_dict
from ..engine.model import DecoderModel
from ..parts.base import BuildEnv
from .loader import RandomSource
from .safetensors_io import Deferred, write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "f32": torch.float32}


def write_random_model(folder, config: dict, seed: int, dtype="bfloat16") -> Path:
    """config: the architecture's config.json as a dict (with `architectures`).  Returns the folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    store = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    model = DecoderModel(cfg.to_spec(), BuildEnv(dtype=store, device=torch.device("cpu")))
    src = RandomSource(model.expected_tensors(), seed, store)
    out = dict(config)
    out["torch_dtype"] = "bfloat16" if store == torch.bfloat16 else "float32"
    (folder / "config.json").write_text(json.dumps(out, indent=1))
    kept = {n: (store if d.kind == "float" else torch.int32) for n, d in src.decls.items()}
    write_safetensors(folder / "model.safetensors",
                      [(n, Deferred(kept[n], src.decls[n].shape, lambda n=n: src.get(n))) for n in sorted(src.decls)],
                      metadata={"format": "pt", "seed": seed})
    return folder
