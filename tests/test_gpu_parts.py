"""Each part alone, and parts that are not in the package: a mixer with state of its own, defined
here, is registered, built into a model next to attention layers, loaded and stepped."""
import math

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TINY_B

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _env(dtype):
    from llaisys_b200.parts import BuildEnv
    return BuildEnv(dtype, DEV)


def _ctx(cache, slots, n_new, tokens=None, want=()):
    from llaisys_b200.engine import StepContext
    for s, n in zip(slots, n_new):
        cache.book.reserve(s, n)
    tokens = tokens if tokens is not None else [0] * sum(n_new)
    shape = StepContext.shape_of(cache, slots, n_new, list(want), bucket=False)
    ctx = StepContext(cache, DEV, *shape, torch.zeros(1, dtype=torch.int32, device=DEV))
    ctx.load(slots, n_new, tokens, list(want))
    return ctx


def _commit(cache, slots, n_new):
    for s, n in zip(slots, n_new):
        cache.book.commit(s, n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    norm = build_part("norm", PartSpec("rms_norm", {"size": 50, "eps": 1e-3}, prefix="n"), _env(dtype))
    assert {k: v.shape for k, v in norm.tensors().items()} == {"weight": (50,)}
    rng = np.random.default_rng(0)
    w, x, d = 1 + rng.normal(size=50) * 0.1, rng.normal(size=(4, 50)), rng.normal(size=(4, 50))
    norm.load({"weight": torch.from_numpy(w).to(dtype).to(DEV)})
    res = torch.from_numpy(x).float().to(DEV)
    out = norm.forward(res, torch.from_numpy(d).to(dtype).to(DEV))
    wr, dr = (torch.from_numpy(a).to(dtype).double().numpy() for a in (w, d))
    want = plain.rms_norm(torch.from_numpy(x).float().double().numpy() + dr, wr, 1e-3)
    assert out.dtype == dtype and np.abs(out.double().cpu().numpy() - want).max() < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    ffn = build_part("ffn", PartSpec("swiglu_mlp", {"hidden_size": 40, "intermediate_size": 56}, prefix="f"), _env(dtype))
    rng = np.random.default_rng(1)
    ws = {n: rng.normal(size=d.shape) * 0.3 for n, d in ffn.tensors().items()}
    ffn.load({n: torch.from_numpy(w).to(dtype).to(DEV) for n, w in ws.items()})
    x = rng.normal(size=(9, 40))
    got = ffn.forward(torch.from_numpy(x).to(dtype).to(DEV), None)
    r = {n: torch.from_numpy(w).to(dtype).double().numpy() for n, w in ws.items()}
    xr = torch.from_numpy(x).to(dtype).double().numpy()
    want = plain.linear(plain.swiglu(plain.linear(xr, r["gate_proj.weight"]), plain.linear(xr, r["up_proj.weight"])),
                        r["down_proj.weight"])
    assert np.abs(got.double().cpu().numpy() - want).max() < (1e-4 if dtype == torch.float32 else 0.15)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 6])
def test_attention_part_prefill_then_decode(dtype, window):
    """The mixer alone over its own cache: 70 tokens at once, then 5 one by one, against the
    plain attention block over the whole 75."""
    from llaisys_b200.cache import CacheConfig, PagedCache
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    H, nh, nkvh, dh, theta = 48, 6, 3, 8, 3000.0
    spec = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkvh, "head_dim": dh,
                                      "qkv_bias": True, "scale": 1 / math.sqrt(dh), "window": window,
                                      "position": PartSpec("rope_half_split", {"head_dim": dh, "theta": theta})}, prefix="a")
    att = build_part("mixer", spec, _env(dtype))
    rng = np.random.default_rng(2)
    # sharp scores under float32; milder under bfloat16, where a score's rounding error grows with its size
    qk = 0.6 if dtype == torch.float32 else 0.15
    ws = {n: rng.normal(size=d.shape) * (qk if "q_proj" in n or "k_proj" in n else 0.2) for n, d in att.tensors().items()}
    att.load({n: torch.from_numpy(w).to(dtype).to(DEV) for n, w in ws.items()})
    cache = PagedCache([att.kv_need()], [None], [0], CacheConfig(max_tokens=128), dtype, DEV)
    x = rng.normal(size=(75, H))
    xt = torch.from_numpy(x).to(dtype).to(DEV)
    slot = cache.acquire()
    ctx = _ctx(cache, [slot], [70])
    outs = [att.forward(xt[:70], ctx, 0)]
    _commit(cache, [slot], [70])
    for t in range(70, 75):
        ctx = _ctx(cache, [slot], [1])
        outs.append(att.forward(xt[t:t + 1], ctx, 0))
        _commit(cache, [slot], [1])
    got = torch.cat(outs).double().cpu().numpy()
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkvh, "head_dim": dh, "hidden_size": H, "rope_theta": theta}
    r = {"a." + n: torch.from_numpy(w).to(dtype).double().numpy() for n, w in ws.items()}
    want = plain.attention_block(torch.from_numpy(x).to(dtype).double().numpy(), np.arange(75), cfg, r, "a.", window)
    # bfloat16: four roundings on the way (projections, rotation, attention output, output projection)
    bound = 2e-5 if dtype == torch.float32 else 8 * 2.0 ** -9 * 2 * float(np.sqrt(np.mean(want ** 2)))
    assert np.abs(got - want).max() < bound


def test_rope_part_table_grows():
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    rope = build_part("position", PartSpec("rope_half_split", {"head_dim": 16, "theta": 1e4}), _env(torch.float32))
    c1, _ = rope.table(10)
    c2, s2 = rope.table(500)
    assert c2.shape[0] >= 500 and torch.equal(c2[:10], c1[:10])
    j = np.arange(8)
    ang = 499 / np.power(1e4, 2 * j / 16)
    assert np.abs(c2[499].double().cpu().numpy() - np.cos(ang)).max() < 1e-7
    assert np.abs(s2[499].double().cpu().numpy() - np.sin(ang)).max() < 1e-7


# ----------------------------------------------------------------------------- a toy architecture
def _register_toys():
    """A mixer whose only memory is a running sum per sequence (fixed-size state, no keys), a
    feed-forward with a routed choice between two matrices, and a position encoding that adds a
    learned vector per position to the queries and keys.  All defined here, in torch."""
    from llaisys_b200.parts import FeedForward, Mixer, PositionEncoding, TensorDecl, register_part

    @register_part("mixer", "toy_running_sum")
    class RunningSum(Mixer):
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

    @register_part("ffn", "toy_routed")
    class Routed(FeedForward):
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.h = spec.params["hidden_size"]

        def tensors(self):
            return {"router.weight": TensorDecl((2, self.h)), "experts.0.weight": TensorDecl((self.h, self.h)),
                    "experts.1.weight": TensorDecl((self.h, self.h))}

        def load(self, tensors):
            self.t = tensors

        def forward(self, x, ctx):
            choice = (x.float() @ self.t["router.weight"].float().T).argmax(-1)
            y0, y1 = (x.float() @ self.t[f"experts.{i}.weight"].float().T for i in (0, 1))
            return torch.where(choice[:, None] == 0, y0, y1).to(x.dtype)

    @register_part("position", "toy_learned_offset")
    class LearnedOffset(PositionEncoding):
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.dh = spec.params["head_dim"]

        def apply(self, qkv, num_heads, num_kv_heads, ctx, append=None):
            from llaisys_b200 import kernels
            T = qkv.shape[0]
            qk = qkv[:, :(num_heads + num_kv_heads) * self.dh].view(T, -1, self.dh)
            qk += (0.01 * ctx.tok_pos.to(qkv.dtype))[:, None, None]
            if append is not None:
                kernels.rope_append(qkv, num_heads, num_kv_heads, self.dh, tok_pos=ctx.tok_pos, append=append, err=ctx.err)


def _toy_spec():
    """Layer 0: running-sum mixer + routed feed-forward.  Layer 1: attention with the toy position
    encoding.  Run order 0, 1, 0, 1: both layers run twice, and the second attention call reads
    the first one's cache."""
    from llaisys_b200.config import CallSpec, LayerSpec, ModelSpec, PartSpec
    H = 32
    norm = lambda p: PartSpec("rms_norm", {"size": H, "eps": 1e-5}, prefix=p)
    l0 = LayerSpec("pre_norm_residual", PartSpec("toy_running_sum", {"hidden_size": H}, prefix="l0.mixer"), norm("l0.n1"),
                   PartSpec("toy_routed", {"hidden_size": H}, prefix="l0.ffn"), norm("l0.n2"))
    l1 = LayerSpec("pre_norm_residual",
                   PartSpec("gqa_attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 1, "head_dim": 8,
                                              "qkv_bias": False, "scale": 0.3, "window": None,
                                              "position": PartSpec("toy_learned_offset", {"head_dim": 8})}, prefix="l1.attn"),
                   norm("l1.n1"), PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": 24}, prefix="l1.mlp"), norm("l1.n2"))
    return ModelSpec("ToyForCausalLM", vocab_size=50, hidden_size=H, max_positions=256,
                     embedding=PartSpec("token_embedding", {"vocab_size": 50, "hidden_size": H}, prefix="emb"),
                     layers=(l0, l1), order=(CallSpec(0), CallSpec(1), CallSpec(0), CallSpec(1, cache_of=1)),
                     final_norm=norm("fn"), head=PartSpec("lm_head", {"vocab_size": 50, "hidden_size": H, "tied_to": "emb.weight"}, prefix="head"))


def test_toy_parts_register_build_and_step():
    from llaisys_b200.cache import CacheConfig
    from llaisys_b200.engine import DecoderModel, Engine, StepEntry
    from llaisys_b200.parts import BuildEnv, known_parts
    from llaisys_b200.weights import RandomSource, load_weights
    _register_toys()
    assert "toy_running_sum" in known_parts("mixer") and "toy_routed" in known_parts("ffn")
    model = DecoderModel(_toy_spec(), BuildEnv(torch.float32, DEV))
    names = set(model.expected_tensors())
    assert {"l0.mixer.mix.weight", "l0.ffn.experts.1.weight", "l1.attn.q_proj.weight"} <= names and "head.weight" not in names
    assert model.state_sizes() == [32, 0, 32, 0] and [n is not None for n in model.kv_needs()] == [False, True, False, True]
    load_weights(model, RandomSource(model.expected_tensors(), seed=3, dtype=torch.float32, std=0.3))
    engine = Engine(model, CacheConfig(max_tokens=256, max_seqs=3))
    assert len(engine.cache.k_pools) == 1 and engine.cache.k_pools[0].shape[0] == 1        # one cache for both attention calls
    assert set(engine.cache.state) == {0, 2}
    assert not engine.use_graphs                     # the toy parts read back from the device: never captured
    toks = np.random.default_rng(0).integers(0, 50, size=90).tolist()
    a = engine.acquire()
    whole = engine.step([StepEntry(a, toks, list(range(90)))])
    engine.release(a)
    # the same tokens cut differently, next to another sequence, in a slot whose state was used before
    b, c = engine.acquire(), engine.acquire()
    assert b == a
    rows = [engine.step([StepEntry(b, toks[:70], list(range(70))), StepEntry(c, [1, 2, 3], [])])]
    for t in range(70, 90):
        entries = [StepEntry(b, [toks[t]], [0])] + ([StepEntry(c, [4], [])] if t < 75 else [])
        rows.append(engine.step(entries))
        if t == 74:
            engine.release(c)
    engine.check()
    cut = torch.cat(rows)
    assert torch.isfinite(whole).all() and float((whole - cut).abs().max()) < 1e-4
    assert float(whole.std()) > 1e-3
