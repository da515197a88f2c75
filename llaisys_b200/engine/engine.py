"""The step function: a batch of sequences, their next tokens, logits at the wanted places."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..cache.kv import CacheConfig, PagedCache
from ..cache.slots import CacheError
from ..config.spec import ModelSpec
from ..parts.base import BuildEnv
from .context import StepContext
from .model import DecoderModel


class StepError(RuntimeError):
    """A step that cannot run: a token id outside the vocabulary, a position beyond the model's
    limit, an unknown slot.  The cache is left as it was before the step."""


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the indices among these
    tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


def _require_cuda(device: torch.device):
    if device.type != "cuda":
        raise RuntimeError("llaisys_b200 runs on a CUDA device (B200, sm_100a) only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; llaisys_b200 has no CPU path")


class Engine:
    """A model, its cache and the step function over them.

    step() runs exactly the tokens it is given, as one packed batch, against what earlier
    steps left in the cache, and returns the logits at the wanted places.  Sequences are
    identified by slots from acquire(); release() gives a slot and its pages back.
    """

    def __init__(self, model: DecoderModel, cache_config: CacheConfig):
        self.model, self.spec, self.env = model, model.spec, model.env
        _require_cuda(self.env.device)
        self.cache = PagedCache(model.kv_needs(), model.cache_of(), model.state_sizes(), cache_config,
                                self.env.dtype, self.env.device)
        self.sm_count = torch.cuda.get_device_properties(self.env.device).multi_processor_count
        self.steps_run = 0

    # ---- limits the generation loop plans with
    @property
    def max_tokens(self) -> int:
        return self.cache.n_pages * self.page

    @property
    def max_seqs(self) -> int:
        return self.cache.n_slots

    @property
    def max_positions(self) -> int:
        return self.spec.max_positions

    @property
    def page(self) -> int:
        from ..cache.kv import PAGE
        return PAGE

    # ---- sequences
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step
    def step(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        """Returns float32 logits [sum(len(e.want)), vocab] in the order of the entries and of
        their `want` lists (None if nothing is wanted)."""
        if not entries:
            return None
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise StepError(f"a slot appears twice in one step: {slots}")
        n_new = [len(e.tokens) for e in entries]
        if min(n_new) < 1:
            raise StepError("every sequence of a step brings at least one token")
        tokens, out_rows, base = [], [], 0
        for e, n in zip(entries, n_new):
            for t in e.tokens:
                if not (0 <= int(t) < self.spec.vocab_size):
                    raise StepError(f"token id {t} is outside the vocabulary (0..{self.spec.vocab_size - 1})")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"wanted index {w} is outside the {n} tokens of slot {e.slot}")
            tokens += [int(t) for t in e.tokens]
            out_rows += [base + int(w) for w in e.want]
            base += n
        book = self.cache.book
        for s, n in zip(slots, n_new):
            if book.length(s) + n > self.spec.max_positions:
                raise StepError(f"slot {s} would reach {book.length(s) + n} positions; the model allows "
                                f"{self.spec.max_positions}")
        # reserve pages for all sequences or for none
        before = {s: [list(p) for p in book.seqs[s].pages] for s in slots}
        try:
            for s, n in zip(slots, n_new):
                book.reserve(s, n)
        except CacheError:
            for s in slots:
                for g, old in enumerate(before[s]):
                    for p in book.seqs[s].pages[g][len(old):]:
                        book.pools[g].give_back(p)
                    book.seqs[s].pages[g] = old
            raise
        with torch.cuda.device(self.env.device):
            ctx = StepContext(self.cache, slots, n_new, tokens, out_rows, self.env.device, self.sm_count)
            logits = self.model.forward(ctx)
            for s, n in zip(slots, n_new):
                book.commit(s, n)
            self.steps_run += 1
            self._last_ctx = ctx
        return logits

    def check(self) -> None:
        """Waits for the device and raises if a kernel of the last step flagged an error."""
        ctx = getattr(self, "_last_ctx", None)
        if ctx is None:
            return
        code = int(ctx.err.item())
        from ..kernels import tc_error
        tc = tc_error(self.env.device)
        if tc:
            raise StepError(f"a tensor-core kernel gave up a bounded wait (code {tc}); its output is not valid")
        if code:
            what = {1: "a token id outside the embedding table", 2: "a position outside the rotary table"}
            raise StepError(f"device-side check failed in the last step: {what.get(code, code)}")


def build_engine(spec: ModelSpec, dtype: torch.dtype, device, cache_config: CacheConfig, source) -> Engine:
    """Builds the model of `spec`, binds its weights from `source` (see weights.loader) and
    wraps it with a cache."""
    from ..weights.loader import load_weights
    device = torch.device(device)
    model = DecoderModel(spec, BuildEnv(dtype=dtype, device=device))
    load_weights(model, source)
    return Engine(model, cache_config)
