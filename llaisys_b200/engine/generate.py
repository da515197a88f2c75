"""The generation loop above the step function.

xsmccc/llaisys generates for one sequence: the prompt token by token, then one token per call
until max_new_tokens or the end token (python/llaisys/models/qwen2.py:234-283; its end test
skips the first generated token).  Here any number of prompts of unequal lengths are served:
as many as fit start together as a batch (their prompts in one step), then each live sequence
gets one token per step; a sequence that meets a stop token or its token limit leaves the
batch at once and its slot is given back; when a batch is done the next one starts, until no
request is left.  The stop test applies to every generated token.

The loop needs of its engine only: acquire(), release(slot), step(entries) -> logits,
`max_tokens`, `max_seqs`, `max_positions`, `page`; and of its sampler a call
(logits, keys, steps) -> token ids.  That keeps its decisions testable without a device.

With an engine that can take a step's tokens from the device (`feed`, `step(..., fed=True)`) and a
sampler that can leave its choice there (`on_device`), the loop runs one step ahead of what it
knows: the chosen tokens go from the sampler to the next step on the device, the next step is
launched at once, and the host reads the tokens of the step before while that one runs.  A
sequence that chose a stop token is found out one step late; the token of that extra step is
thrown away.  Tokens, reasons and the order of decisions are those of the plain loop.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from .engine import StepEntry


@dataclass
class Generation:
    """Result for one request: the new tokens (a stop token included) and why it ended:
    "stop", "length" (max_new_tokens) or "limit" (the model's position limit)."""
    tokens: List[int] = field(default_factory=list)
    reason: str = ""


class GenerationLoop:
    def __init__(self, engine, sampler: Callable, stop_ids: Sequence[int] = (), max_batch: Optional[int] = None):
        self.engine, self.sampler = engine, sampler
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.max_batch = max_batch
        self.batches_run = 0
        self.steps_run = 0
        self.step_marks: List[float] = []     # host time after each step's tokens arrived (for measurements)
        # one step ahead of the host's knowledge, where engine and sampler keep the tokens on the device
        self.pipelined = hasattr(engine, "feed") and hasattr(sampler, "on_device")

    # ---- admission: how many of the waiting requests start together
    def _room(self, prompt_len: int, max_new: int) -> int:
        page = self.engine.page
        n = min(prompt_len + max_new, self.engine.max_positions)
        return -(-n // page) * page

    def _admit(self, waiting: List[int], prompts, max_new: int) -> List[int]:
        batch, tokens = [], 0
        limit = min(self.engine.max_seqs, self.max_batch or self.engine.max_seqs)
        for r in waiting:
            need = self._room(len(prompts[r]), max_new)
            if batch and (tokens + need > self.engine.max_tokens or len(batch) >= limit):
                break
            if need > self.engine.max_tokens:
                raise ValueError(f"request {r} needs room for {need} tokens; the cache holds {self.engine.max_tokens}")
            batch.append(r)
            tokens += need
        return batch

    # ---- the loop
    def run(self, prompts: Sequence[Sequence[int]], max_new_tokens: int) -> List[Generation]:
        for r, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"request {r} has an empty prompt")
            if len(p) >= self.engine.max_positions and max_new_tokens > 0:
                raise ValueError(f"request {r}: a prompt of {len(p)} tokens leaves no position to generate at "
                                 f"(the model allows {self.engine.max_positions})")
        results = [Generation() for _ in prompts]
        waiting = list(range(len(prompts)))
        if max_new_tokens <= 0:
            for g in results:
                g.reason = "length"
            return results
        while waiting:
            batch = self._admit(waiting, prompts, max_new_tokens)
            waiting = waiting[len(batch):]
            self._run_batch(batch, prompts, max_new_tokens, results)
            self.batches_run += 1
        return results

    def _run_batch(self, batch: List[int], prompts, max_new: int, results: List[Generation]) -> None:
        if self.pipelined:
            return self._run_batch_ahead(batch, prompts, max_new, results)
        eng = self.engine
        slot = {r: eng.acquire() for r in batch}
        length = {r: len(prompts[r]) for r in batch}
        live = list(batch)
        try:
            entries = [StepEntry(slot[r], list(prompts[r]), [len(prompts[r]) - 1]) for r in live]
            while live:
                logits = eng.step(entries)
                self.steps_run += 1
                new = self.sampler(logits, live, [len(results[r].tokens) for r in live])
                self.step_marks.append(time.perf_counter())
                still, entries = [], []
                for r, tok in zip(live, new):
                    g = results[r]
                    g.tokens.append(int(tok))
                    length[r] += 1
                    if int(tok) in self.stop_ids:
                        g.reason = "stop"
                    elif len(g.tokens) >= max_new:
                        g.reason = "length"
                    elif length[r] >= eng.max_positions:
                        g.reason = "limit"
                    if g.reason:
                        eng.release(slot.pop(r))
                    else:
                        still.append(r)
                        entries.append(StepEntry(slot[r], [int(tok)], [0]))
                live = still
        finally:
            for s in slot.values():
                eng.release(s)

    def _settle(self, r: int, tok: int, results, length, slot, max_new: int) -> None:
        """Books one generated token of request r and ends the request where it has to end."""
        g = results[r]
        g.tokens.append(tok)
        length[r] += 1
        if tok in self.stop_ids:
            g.reason = "stop"
        elif len(g.tokens) >= max_new:
            g.reason = "length"
        elif length[r] >= self.engine.max_positions:
            g.reason = "limit"
        if g.reason:
            self.engine.release(slot.pop(r))

    def _run_batch_ahead(self, batch: List[int], prompts, max_new: int, results: List[Generation]) -> None:
        import torch
        eng = self.engine
        slot = {r: eng.acquire() for r in batch}
        length = {r: len(prompts[r]) for r in batch}
        drawn = {r: 0 for r in batch}                 # tokens chosen for r so far, the ones in flight included
        in_flight = []                                # [(requests, pinned host tokens, event)], oldest first
        hosts = [torch.empty(len(batch), dtype=torch.int32).pin_memory() for _ in range(3)]
        launched = []

        def launch(requests, entries, fed):
            logits = eng.step(entries, fed=fed) if fed else eng.step(entries)
            self.steps_run += 1
            chosen = self.sampler.on_device(logits, requests, [drawn[r] for r in requests])
            eng.feed(chosen)
            host = hosts[len(launched) % len(hosts)][:len(requests)]      # free again: at most two steps are in flight
            launched.append(None)
            host.copy_(chosen, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            for r in requests:
                drawn[r] += 1
            in_flight.append((list(requests), host, ev))

        try:
            launch(batch, [StepEntry(slot[r], list(prompts[r]), [len(prompts[r]) - 1]) for r in batch], False)
            while in_flight:
                # who goes on, as far as the host can tell without the tokens in flight: everyone still open whose
                # next token is neither beyond max_new nor beyond the model's positions
                last = in_flight[-1][0]
                go = [r for r in last if r in slot and drawn[r] < max_new
                      and len(prompts[r]) + drawn[r] < eng.max_positions]
                if go:
                    launch(go, [StepEntry(slot[r], [0], [0]) for r in go], True)
                # the oldest step's tokens, while the newest step runs
                requests, host, ev = in_flight.pop(0)
                ev.synchronize()
                self.step_marks.append(time.perf_counter())
                for r, tok in zip(requests, host.tolist()):
                    if r in slot:                     # else: it ended a step ago, this token is thrown away
                        self._settle(r, int(tok), results, length, slot, max_new)
        finally:
            for s in slot.values():
                eng.release(s)
