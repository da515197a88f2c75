"""A toy architecture that lives outside the package: its configuration class, its parts and a
plain whole-sequence implementation of it, all defined here, in torch and numpy.

It is not a model of anyone's.  It exists to show that the framework takes another
architecture without an edit to its files: importing this module registers
"ToyForCausalLM" and its parts (programs started as child processes import it through the
LLAISYS_PLUGINS environment variable).  Its layers differ from the built-in architecture in
every way the framework leaves open:

  layer 0  three sub-layers: an attention mixer whose keys and values have different widths
           (it reads and writes its cache pages itself), a feed-forward with routing, and the
           built-in SwiGLU feed-forward
  layer 1  a mixer with fixed-size state of its own (a running mean; no keys), then SwiGLU
  layer 2  the built-in attention with a position encoding that is not a rotation (an offset
           that grows with the position), then SwiGLU
  order    0, 1, 2, 1, 2: layer 1 runs twice (two states per sequence), and the second run of
           layer 2 reads the keys and values that its first run stored
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass

import numpy as np
import torch

import plain_qwen2 as plain
from llaisys_b200.config import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec, register_architecture
from llaisys_b200.parts import FeedForward, KVNeed, Mixer, PositionEncoding, TensorDecl, register_part

OFFSET = 0.01      # the toy position encoding adds OFFSET * position to every query and key element


@register_part("mixer", "toy_running_mean")
class RunningMean(Mixer):
    """out[t] = W mean(x[0..t]): the only memory is the running sum per sequence."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.h = spec.params["hidden_size"]

    def state_size(self):
        return self.h

    def tensors(self):
        return {"mix.weight": TensorDecl((self.h, self.h))}

    def load(self, tensors):
        self.w = tensors["mix.weight"]

    def forward(self, x, ctx, call):
        state = ctx.state(call)
        out = torch.empty_like(x)
        for b, (slot, n, start) in enumerate(zip(ctx.slots, ctx.n_new, ctx.seq_start.tolist())):
            run = state[slot] + torch.cumsum(x[start:start + n].float(), dim=0)
            state[slot] = run[-1]
            pos = torch.arange(ctx.lens_before[b] + 1, ctx.lens_before[b] + n + 1, device=x.device)[:, None]
            out[start:start + n] = ((run / pos) @ self.w.float().T).to(x.dtype)
        return out


@register_part("mixer", "toy_wide_attention")
class WideAttention(Mixer):
    """Causal attention whose keys are `key_dim` wide and whose values are `value_dim` wide, with an
    optional window.  It stores and reads its pages through ctx.kv(call) itself."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.h, self.nh, self.nkv, self.dk, self.dv, self.window = (p["hidden_size"], p["num_heads"], p["num_kv_heads"],
                                                                    p["key_dim"], p["value_dim"], p.get("window"))

    def kv_need(self):
        return KVNeed(self.nkv, self.dk, self.dv, self.window)

    def tensors(self):
        return {"q.weight": TensorDecl((self.nh * self.dk, self.h)), "k.weight": TensorDecl((self.nkv * self.dk, self.h)),
                "v.weight": TensorDecl((self.nkv * self.dv, self.h)), "o.weight": TensorDecl((self.h, self.nh * self.dv))}

    def load(self, tensors):
        self.t = {n: w.float() for n, w in tensors.items()}

    def forward(self, x, ctx, call):
        from llaisys_b200.cache import PAGE
        kv = ctx.kv(call)
        xf = x.float()
        q = (xf @ self.t["q.weight"].T).view(-1, self.nh, self.dk)
        k = (xf @ self.t["k.weight"].T).view(-1, self.nkv, self.dk)
        v = (xf @ self.t["v.weight"].T).view(-1, self.nkv, self.dv)
        out = torch.empty((x.shape[0], self.nh, self.dv), dtype=torch.float32, device=x.device)
        tables = kv.page_table.tolist()
        group = self.nh // self.nkv
        for b, (n, start, before) in enumerate(zip(ctx.n_new, ctx.seq_start.tolist(), ctx.lens_before)):
            for i in range(n):                       # one token at a time: store it, then attend over what is kept
                pos = before + i
                page = tables[b][(pos // PAGE) % kv.ring]
                kv.k[page, :, pos % PAGE] = k[start + i].to(kv.k.dtype)
                kv.v[page, :, pos % PAGE] = v[start + i].to(kv.v.dtype)
                lo = 0 if self.window is None else max(0, pos - self.window + 1)
                idx = torch.arange(lo, pos + 1, device=x.device)
                pages = torch.tensor([tables[b][(j // PAGE) % kv.ring] for j in range(lo, pos + 1)], device=x.device)
                ks = kv.k[pages, :, idx % PAGE].float()         # [keys, kv heads, dk]
                vs = kv.v[pages, :, idx % PAGE].float()
                for h in range(self.nh):
                    s = (ks[:, h // group] @ q[start + i, h]) / math.sqrt(self.dk)
                    out[start + i, h] = torch.softmax(s, 0) @ vs[:, h // group]
        return (out.view(x.shape[0], -1) @ self.t["o.weight"].T).to(x.dtype)


@register_part("ffn", "toy_routed")
class Routed(FeedForward):
    """y = sum_e softmax(R x)_e (E_e x): a router and two experts, tensors with indexed names."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.h = spec.params["hidden_size"]

    def tensors(self):
        return {"router.weight": TensorDecl((2, self.h)), "experts.0.weight": TensorDecl((self.h, self.h)),
                "experts.1.weight": TensorDecl((self.h, self.h))}

    def load(self, tensors):
        self.t = tensors

    def forward(self, x, ctx):
        xf = x.float()
        gate = torch.softmax(xf @ self.t["router.weight"].float().T, dim=-1)
        ys = torch.stack([xf @ self.t[f"experts.{i}.weight"].float().T for i in (0, 1)], dim=-1)
        return (ys * gate[:, None, :]).sum(-1).to(x.dtype)


@register_part("position", "toy_offset")
class Offset(PositionEncoding):
    """Adds OFFSET * position to every query and key element: not a rotation, so it hands out no
    tables and the attention part has to call apply() and store the keys in a pass of its own."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.dh = spec.params["head_dim"]

    def apply(self, qkv, num_heads, num_kv_heads, ctx):
        qk = qkv[:, :(num_heads + num_kv_heads) * self.dh]
        qk += (OFFSET * ctx.tok_pos.to(torch.float32))[:, None].to(qkv.dtype)


@register_architecture("ToyForCausalLM")
@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    ffn_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    head_dim: int
    eps: float
    max_positions: int
    window: int | None = None

    @classmethod
    def from_dict(cls, d):
        try:
            return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d or k != "window"})
        except KeyError as e:
            raise ConfigError(f"toy config lacks {e}") from None

    def to_dict(self):
        d = {k: v for k, v in asdict(self).items() if v is not None}
        d["architectures"] = [self.architecture]
        return d

    def to_spec(self) -> ModelSpec:
        H = self.hidden_size
        norm = lambda p: PartSpec("rms_norm", {"size": H, "eps": self.eps}, prefix=p)
        mlp = lambda p: PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": self.ffn_size}, prefix=p)
        wide = PartSpec("toy_wide_attention", {"hidden_size": H, "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads,
                                               "key_dim": self.key_dim, "value_dim": self.value_dim, "window": self.window},
                        prefix="l0.wide")
        l0 = LayerSpec("pre_norm_residual", (SubLayerSpec("mixer", wide, norm("l0.n0")),
                                             SubLayerSpec("ffn", PartSpec("toy_routed", {"hidden_size": H}, prefix="l0.routed"), norm("l0.n1")),
                                             SubLayerSpec("ffn", mlp("l0.mlp"), norm("l0.n2"))))
        l1 = LayerSpec.pair("pre_norm_residual", PartSpec("toy_running_mean", {"hidden_size": H}, prefix="l1.mean"), norm("l1.n0"),
                            mlp("l1.mlp"), norm("l1.n1"))
        att = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads,
                                         "head_dim": self.head_dim, "qkv_bias": False, "scale": 1 / math.sqrt(self.head_dim),
                                         "window": None, "position": PartSpec("toy_offset", {"head_dim": self.head_dim})},
                       prefix="l2.attn")
        l2 = LayerSpec.pair("pre_norm_residual", att, norm("l2.n0"), mlp("l2.mlp"), norm("l2.n1"))
        return ModelSpec(self.architecture, vocab_size=self.vocab_size, hidden_size=H, max_positions=self.max_positions,
                         embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H}, prefix="emb"),
                         layers=(l0, l1, l2),
                         order=(CallSpec(0), CallSpec(1), CallSpec(2), CallSpec(1), CallSpec(2, cache_of=2)),
                         final_norm=norm("fn"),
                         head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": H, "tied_to": "emb.weight"},
                                       prefix="head"))


TOY = {"architectures": ["ToyForCausalLM"], "vocab_size": 90, "hidden_size": 40, "ffn_size": 56, "num_heads": 4,
       "num_kv_heads": 2, "key_dim": 12, "value_dim": 6, "head_dim": 10, "eps": 1e-5, "max_positions": 512, "window": 70}


# ----------------------------------------------------------------------------- the toy, plain and whole
def plain_logits(tokens, cfg: dict, w: dict) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence in float64, no cache, one branch per part."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_heads"], cfg["num_kv_heads"]
    T = len(tokens)
    pos = np.arange(T)
    x = plain.embedding(tokens, w["emb.weight"])

    def mlp(h, p):
        return plain.mlp_block(h, w, p + ".")

    def layer0(x):
        h = plain.rms_norm(x, w["l0.n0.weight"], cfg["eps"])
        q = (h @ w["l0.wide.q.weight"].T).reshape(T, nh, cfg["key_dim"])
        k = (h @ w["l0.wide.k.weight"].T).reshape(T, nkv, cfg["key_dim"])
        v = (h @ w["l0.wide.v.weight"].T).reshape(T, nkv, cfg["value_dim"])
        o = plain.self_attention(q, k, v, 1 / math.sqrt(cfg["key_dim"]), cfg.get("window"))
        x = x + o.reshape(T, -1) @ w["l0.wide.o.weight"].T
        h = plain.rms_norm(x, w["l0.n1.weight"], cfg["eps"])
        logit = h @ w["l0.routed.router.weight"].T
        gate = np.exp(logit - logit.max(-1, keepdims=True))
        gate /= gate.sum(-1, keepdims=True)
        x = x + sum(gate[:, e:e + 1] * (h @ w[f"l0.routed.experts.{e}.weight"].T) for e in (0, 1))
        return x + mlp(plain.rms_norm(x, w["l0.n2.weight"], cfg["eps"]), "l0.mlp")

    def layer1(x):
        h = plain.rms_norm(x, w["l1.n0.weight"], cfg["eps"])
        x = x + (np.cumsum(h, axis=0) / (pos + 1)[:, None]) @ w["l1.mean.mix.weight"].T
        return x + mlp(plain.rms_norm(x, w["l1.n1.weight"], cfg["eps"]), "l1.mlp")

    def layer2(x):
        dh = cfg["head_dim"]
        h = plain.rms_norm(x, w["l2.n0.weight"], cfg["eps"])
        q = (h @ w["l2.attn.q_proj.weight"].T).reshape(T, nh, dh) + OFFSET * pos[:, None, None]
        k = (h @ w["l2.attn.k_proj.weight"].T).reshape(T, nkv, dh) + OFFSET * pos[:, None, None]
        v = (h @ w["l2.attn.v_proj.weight"].T).reshape(T, nkv, dh)
        keep = layer2.__dict__.setdefault("kv", (k, v))          # the second run reads the first run's keys and values
        o = plain.self_attention(q, keep[0], keep[1], 1 / math.sqrt(dh))
        x = x + o.reshape(T, -1) @ w["l2.attn.o_proj.weight"].T
        return x + mlp(plain.rms_norm(x, w["l2.n1.weight"], cfg["eps"]), "l2.mlp")

    for layer in (layer0, layer1, layer2, layer1, layer2):
        x = layer(x)
    return plain.rms_norm(x, w["fn.weight"], cfg["eps"]) @ w["emb.weight"].T
