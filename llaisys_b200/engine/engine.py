"""The step function: a batch of sequences, their next tokens, logits at the wanted places."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import diagnostics
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

    A step in which every sequence brings one token (decode) has the same launches whenever its
    shape (sequences, wanted rows, page-table widths) is the same, so its launches are captured
    in a CUDA graph the first time the shape is met and replayed afterwards; the step's
    description is copied into the same device buffer each time.  This only removes launch
    overhead: the kernels, the cache and the results are those of the uncaptured step.
    Models with parts that are not `capturable` always run uncaptured.
    """

    MAX_GRAPHS = 64
    STAGES = 8

    def __init__(self, model: DecoderModel, cache_config: CacheConfig, use_graphs: bool = True):
        self.model, self.spec, self.env = model, model.spec, model.env
        _require_cuda(self.env.device)
        self.cache = PagedCache(model.kv_needs(), model.cache_of(), model.state_sizes(), cache_config,
                                self.env.dtype, self.env.device)
        self.sm_count = torch.cuda.get_device_properties(self.env.device).multi_processor_count
        self.err = torch.zeros(1, dtype=torch.int32, device=self.env.device)
        # with kernel timers on, steps run uncaptured: a replayed graph has no launches to put events around
        self.use_graphs = use_graphs and model.capturable() and not diagnostics.timers.enabled
        # The longest sequence a slot can reach: the model's limit, and the cache's room unless every
        # group keeps a window only (rings never run out of pages).  Parts size their tables for it once;
        # a captured step has their addresses, so they must not move afterwards.
        self.position_limit = self.spec.max_positions
        if any(r is None for r in self.cache.rings):
            self.position_limit = min(self.position_limit, self.cache.n_pages * self.page)
        model.prepare(self.position_limit)
        diagnostics.log.info("engine: %s, %s on %s, %d layers in the run order, positions up to %d, graphs %s",
                             self.spec.architecture, str(self.env.dtype).replace("torch.", ""), self.env.device,
                             len(self.spec.order),
                             self.position_limit, "on" if self.use_graphs else "off")
        # the last sampled token of every slot, for steps that take their tokens from the device (see feed())
        self.fed_tokens = torch.zeros(self.cache.n_slots, dtype=torch.int32, device=self.env.device)
        self._last_ctx = None
        self._graphs = {}                      # shape -> [context, graph or None, logits]
        self._stages = [[None, None] for _ in range(self.STAGES)]
        self._stage_i = 0
        self.steps_run = 0
        self.graph_replays = 0

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
    def _staging(self, n: int):
        """A pinned host buffer of the ring, free again (its last copy has run)."""
        i = self._stage_i % self.STAGES
        self._stage_i += 1
        buf, ev = self._stages[i]
        if ev is not None:
            ev.synchronize()
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024), dtype=torch.int32).pin_memory()
        if ev is None:
            ev = torch.cuda.Event()
        self._stages[i] = [buf, ev]
        return buf, ev

    def feed(self, tokens: torch.Tensor) -> None:
        """Keeps the token chosen for each sequence of the last step on the device (int32 [entries], in
        the order of that step's entries), where a following step(..., fed=True) finds it."""
        from .. import kernels
        ctx = self._last_ctx
        if ctx is None or tokens.numel() != ctx.n_seqs:
            raise StepError("feed() takes one token for every sequence of the step before it")
        kernels.scatter_i32(self.fed_tokens, ctx.seq_slot, tokens)

    def _forward(self, ctx, fed: bool):
        if fed:
            from .. import kernels
            kernels.gather_i32(ctx.tokens, self.fed_tokens, ctx.seq_slot)
        return self.model.forward(ctx)

    def step(self, entries: List[StepEntry], fed: bool = False) -> Optional[torch.Tensor]:
        """Returns float32 logits [sum(len(e.want)), vocab] in the order of the entries and of
        their `want` lists (None if nothing is wanted).  The tensor is valid until the next step.

        fed: every entry brings one token, and that token is not the one in the entry but the one
        last given to feed() for its slot: the host can launch this step before it has seen the tokens."""
        if not entries:
            return None
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise StepError(f"a slot appears twice in one step: {slots}")
        n_new = [len(e.tokens) for e in entries]
        if min(n_new) < 1:
            raise StepError("every sequence of a step brings at least one token")
        if fed and max(n_new) != 1:
            raise StepError("a step that takes its tokens from the device brings one token per sequence")
        tokens, out_rows, base = [], [], 0
        for e, n in zip(entries, n_new):
            for t in e.tokens:
                if not fed and not (0 <= int(t) < self.spec.vocab_size):
                    raise StepError(f"token id {t} is outside the vocabulary (0..{self.spec.vocab_size - 1})")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"wanted index {w} is outside the {n} tokens of slot {e.slot}")
            tokens += [int(t) for t in e.tokens]
            out_rows += [base + int(w) for w in e.want]
            base += n
        book = self.cache.book
        if diagnostics.BOUNDS:
            wrong = book.audit()
            if wrong:
                raise StepError("the cache's books are out of order before the step: " + "; ".join(wrong[:8]))
        for s, n in zip(slots, n_new):
            if book.length(s) + n > self.spec.max_positions:
                raise StepError(f"slot {s} would reach {book.length(s) + n} positions; the model allows "
                                f"{self.spec.max_positions}")
        # reserve pages for all sequences or for none
        before = {s: [list(p) for p in book.seqs[s].pages] for s in slots}

        def give_back():
            for s in slots:
                for g, old in enumerate(before[s]):
                    for p in book.seqs[s].pages[g][len(old):]:
                        book.pools[g].give_back(p)
                    book.seqs[s].pages[g] = old

        try:
            for s, n in zip(slots, n_new):
                book.reserve(s, n)
        except CacheError:
            give_back()
            raise
        with torch.cuda.device(self.env.device):
            diagnostics.timers.start()
            graphed = self.use_graphs and max(n_new) == 1
            shape = StepContext.shape_of(self.cache, slots, n_new, out_rows, bucket=graphed)
            try:
                if graphed:
                    logits = self._graphed_step(shape, slots, n_new, tokens, out_rows, fed)
                else:
                    ctx = StepContext(self.cache, self.env.device, *shape, self.err, self.sm_count)
                    buf, ev = self._staging(ctx.meta.numel())
                    ctx.load(slots, n_new, tokens, out_rows, buf)
                    ev.record()
                    if diagnostics.BOUNDS:
                        self._audit_step(ctx, buf)
                    logits = self._forward(ctx, fed)
                    self._last_ctx = ctx
            except Exception:
                # a launch was refused (or a kernel could not be built): lengths stay as they were and the pages
                # reserved for this step go back, so the sequences can be stepped again or released
                give_back()
                raise
            for s, n in zip(slots, n_new):
                book.commit(s, n)
            self.steps_run += 1
        return logits

    def _graphed_step(self, shape, slots, n_new, tokens, out_rows, fed=False):
        shape = shape + (bool(fed),)
        entry = self._graphs.get(shape)
        if entry is None:
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            entry = [StepContext(self.cache, self.env.device, *shape[:4], self.err, self.sm_count), None, None]
            self._graphs[shape] = entry
        ctx = entry[0]
        self._last_ctx = ctx
        buf, ev = self._staging(ctx.meta.numel())
        ctx.load(slots, n_new, tokens, out_rows, buf)
        ev.record()
        if diagnostics.BOUNDS:
            self._audit_step(ctx, buf)
        if entry[1] is None:
            logits = self._forward(ctx, fed)          # the real step, uncaptured; this also loads every kernel
            from ..kernels import ops
            n0 = ops.launch_count()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    captured = self._forward(ctx, fed)    # recorded, not run
            except Exception:
                # The step itself has run; only its recording failed.  This shape goes on uncaptured.
                ops._launches = n0
                self._graphs.pop(shape, None)
                self.use_graphs = False
                return logits
            entry[1], entry[2] = graph, captured
            entry.append(ops.launch_count() - n0)     # kernels a replay launches
            ops._launches = n0                        # the capture itself launched nothing
            return logits
        entry[1].replay()
        from ..kernels import ops
        ops._launches += entry[3]
        self.graph_replays += 1
        return entry[2]

    def _audit_step(self, ctx: StepContext, staged: torch.Tensor) -> None:
        """The step's description as the kernels will read it (the staged host copy), checked against the
        cache: every position inside the limit, every packed token inside its sequence, every page-table entry
        that a sequence's length reaches inside its group's pool and in no other sequence's row."""
        meta = staged[:ctx.meta.numel()].numpy()
        o = ctx._offs
        tok_seq, tok_pos, starts, lens = (meta[o[i]:o[i + 1]] for i in (1, 2, 3, 4))
        wrong = []
        B, T = ctx.n_seqs, ctx.n_tokens
        if starts[0] != 0 or starts[B] != T or (starts[1:] <= starts[:-1]).any():
            wrong.append(f"sequence starts {starts.tolist()} do not partition {T} tokens")
        if T and (tok_pos.min() < 0 or tok_pos.max() >= self.position_limit):
            wrong.append(f"positions {int(tok_pos.min())}..{int(tok_pos.max())} outside 0..{self.position_limit - 1}")
        if T and (tok_seq.min() < 0 or tok_seq.max() >= B):
            wrong.append("a token names a sequence outside the batch")
        for g, w in enumerate(ctx.widths):
            table = meta[o[7 + g]:o[8 + g]].reshape(B, w)
            ring, seen = self.cache.rings[g], set()
            for b in range(B):
                used = self.cache.book.pages_needed(g, int(lens[b]) + ctx.n_new[b])
                if used > w or (ring is not None and used > ring):
                    wrong.append(f"sequence {b} needs {used} pages of group {g}; its table row has {w}, its ring {ring}")
                    continue
                for pg in table[b, :used].tolist():
                    if not (0 <= pg < self.cache.group_pages[g]):
                        wrong.append(f"sequence {b} names page {pg} of group {g}, outside 0..{self.cache.group_pages[g] - 1}")
                    elif pg in seen:
                        wrong.append(f"page {pg} of group {g} is in two sequences' tables")
                    seen.add(pg)
        if wrong:
            raise StepError("the step's description is out of order: " + "; ".join(wrong[:8]))

    def check(self) -> None:
        """Waits for the device and raises if a kernel flagged an error since the last check."""
        from ..kernels import ops, tc_error
        code = int(self.err.item())
        self.cache.check_guards()
        ops.check_guards(self.env.device)
        if code:
            self.err.zero_()
        tc = tc_error(self.env.device)            # read and cleared
        if tc:
            raise StepError(f"a tensor-core kernel gave up a bounded wait (code {tc}); its output is not valid")
        if code:
            what = {1: "a token id outside the embedding table", 2: "a position outside the rotary table"}
            raise StepError(f"device-side check failed: {what.get(code, code)}")


def resolve_device(device) -> torch.device:
    """`device` with its index filled in ("cuda" -> the current CUDA device), so that everything keyed by
    device (kernel resources, error words) sees one spelling."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def build_engine(spec: ModelSpec, dtype: torch.dtype, device, cache_config: CacheConfig, source,
                 use_graphs: bool = True) -> Engine:
    """Builds the model of `spec`, binds its weights from `source` (see weights.loader) and
    wraps it with a cache."""
    from ..weights.loader import load_weights
    _require_cuda(torch.device(device))
    device = resolve_device(device)
    model = DecoderModel(spec, BuildEnv(dtype=dtype, device=device))
    load_weights(model, source)
    return Engine(model, cache_config, use_graphs=use_graphs)
