"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

xsmccc/llaisys reads num_hidden_layers, hidden_size, num_attention_heads, num_key_value_heads,
intermediate_size, max_position_embeddings, vocab_size, rms_norm_eps and rope_theta (all
required) and eos_token_id (python/llaisys/models/qwen2.py:50-64) into LlaisysQwen2Meta
(include/llaisys/models/qwen2.h:7-12) and from there into Qwen2Config
(src/models/qwen2/qwen2_impl.hpp:9-42); its head size is hidden_size // heads (:67).  Read here
in addition: head_dim, tie_word_embeddings, use_sliding_window / sliding_window /
max_window_layers, attention_bias, hidden_act, rope_scaling (only to refuse what is not built).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Optional, Tuple

from .registry import register_architecture
from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec

_REQUIRED = ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
             "intermediate_size", "max_position_embeddings", "vocab_size", "rms_norm_eps", "rope_theta")


@register_architecture("Qwen2ForCausalLM")
@dataclass(frozen=True)
class Qwen2Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    max_position_embeddings: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    head_dim: int
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    attention_bias: bool = True
    eos_token_id: Tuple[int, ...] = ()

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required keys {missing}")

        def as_int(key, v):
            if isinstance(v, bool) or not isinstance(v, int):
                raise ConfigError(f"config key {key!r} must be an integer, got {v!r}")
            return v

        ints = {k: as_int(k, d[k]) for k in _REQUIRED[:7]}
        for k, v in ints.items():
            if v <= 0:
                raise ConfigError(f"config key {k!r} must be positive, got {v}")
        nh, nkvh, H = ints["num_attention_heads"], ints["num_key_value_heads"], ints["hidden_size"]
        if nh % nkvh:
            raise ConfigError(f"num_attention_heads={nh} is not a multiple of num_key_value_heads={nkvh}")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if H % nh:
                raise ConfigError(f"hidden_size={H} is not a multiple of num_attention_heads={nh} and no head_dim is given")
            head_dim = H // nh
        head_dim = as_int("head_dim", head_dim)
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim={head_dim} must be positive and even (rotary pairs)")
        eps, theta = float(d["rms_norm_eps"]), float(d["rope_theta"])
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"rms_norm_eps={eps} must be positive")
        if not (theta > 0 and math.isfinite(theta)):
            raise ConfigError(f"rope_theta={theta} must be positive")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"rope_scaling={d['rope_scaling']!r} is not supported (plain rotary encoding only)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported (the feed-forward is SwiGLU with silu)")
        use_win = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window")
        mwl = d.get("max_window_layers")
        if use_win:
            if window is None or as_int("sliding_window", window) <= 0:
                raise ConfigError("use_sliding_window is set but sliding_window is not a positive integer")
            if mwl is not None and as_int("max_window_layers", mwl) < 0:
                raise ConfigError("max_window_layers must not be negative")
        eos = d.get("eos_token_id")
        if eos is None:
            eos = ()
        elif isinstance(eos, (list, tuple)):
            eos = tuple(as_int("eos_token_id", e) for e in eos)
        else:
            eos = (as_int("eos_token_id", eos),)
        return cls(**ints, rms_norm_eps=eps, rope_theta=theta, head_dim=head_dim,
                   tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                   use_sliding_window=use_win,
                   sliding_window=None if window is None else int(window),
                   max_window_layers=None if mwl is None else int(mwl),
                   attention_bias=bool(d.get("attention_bias", True)),
                   eos_token_id=eos)

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) != 1 else self.eos_token_id[0]
        if not self.eos_token_id:
            del d["eos_token_id"]
        d["hidden_act"] = "silu"
        return {k: v for k, v in d.items() if v is not None}

    # ------------------------------------------------------------------ derived
    def layer_window(self, layer: int) -> Optional[int]:
        """Layer l keeps a window iff use_sliding_window and l >= max_window_layers
        (max_window_layers absent: no layer is windowed)."""
        if not self.use_sliding_window:
            return None
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return self.sliding_window if layer >= first else None

    def to_spec(self) -> ModelSpec:
        H, dh = self.hidden_size, self.head_dim
        layers = []
        for l in range(self.num_hidden_layers):
            p = f"model.layers.{l}"
            position = PartSpec("rope_half_split", {"head_dim": dh, "theta": self.rope_theta})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": H, "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads, "head_dim": dh,
                "qkv_bias": self.attention_bias, "out_bias": False,
                "scale": 1.0 / math.sqrt(dh),              # src/models/qwen2/attention.hpp:67
                "window": self.layer_window(l), "position": position,
            }, prefix=f"{p}.self_attn")
            ffn = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": self.intermediate_size},
                           prefix=f"{p}.mlp")
            norm = {"size": H, "eps": self.rms_norm_eps}
            layers.append(LayerSpec.pair(
                "pre_norm_residual", mixer=mixer, ffn=ffn,
                mixer_norm=PartSpec("rms_norm", norm, prefix=f"{p}.input_layernorm"),
                ffn_norm=PartSpec("rms_norm", norm, prefix=f"{p}.post_attention_layernorm")))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=H,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H},
                               prefix="model.embed_tokens"),
            layers=tuple(layers),
            order=tuple(CallSpec(layer=l) for l in range(self.num_hidden_layers)),
            final_norm=PartSpec("rms_norm", {"size": H, "eps": self.rms_norm_eps}, prefix="model.norm"),
            head=PartSpec("lm_head", {
                "vocab_size": self.vocab_size, "hidden_size": H,
                "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None,
            }, prefix="lm_head"),
            stop_token_ids=self.eos_token_id)
