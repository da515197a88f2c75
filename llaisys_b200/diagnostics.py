"""Diagnostics that are off unless an environment variable asks for them.

  LLAISYS_LOG=info|debug   messages of the logger "llaisys_b200" on standard error (quiet otherwise; the
                           reference prints its banner and a line per token from the model code,
                           xsmccc/llaisys src/models/qwen2/qwen2.cpp:30-31, 54-56)
  LLAISYS_TIMERS=1         device time per kernel class (CUDA events around every launch of this package;
                           steps then run uncaptured, so that there are launches to time)
  LLAISYS_CANARY=1         guard words before and after every pool of the cache, every state table and the
                           tensor-core scratch; Engine.check() raises when one has changed
  LLAISYS_BOUNDS=1         before every step the host audits the cache's books (a page held twice, a page
                           outside its pool, a length that its pages cannot hold) and the step's description

None of them changes a result.  Programs set them before the package is imported; tests switch the module's
attributes instead.
"""
from __future__ import annotations

import logging
import os
import sys
from typing import Dict, List, Tuple

import torch

log = logging.getLogger("llaisys_b200")


def setup_logging(level: str | None = None) -> None:
    """Attaches one handler on standard error at the level of LLAISYS_LOG (or `level`)."""
    level = (level if level is not None else os.environ.get("LLAISYS_LOG", "")).strip().lower()
    if not level or level in ("0", "off", "quiet"):
        return
    if level not in ("info", "debug", "warning", "error"):
        raise ValueError(f"LLAISYS_LOG={level!r}: expected info or debug")
    log.setLevel(getattr(logging, level.upper()))
    if not any(getattr(h, "_llaisys", False) for h in log.handlers):
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter("[llaisys_b200] %(levelname)s %(message)s"))
        h._llaisys = True
        log.addHandler(h)
        log.propagate = False


def _flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() not in ("", "0", "off", "false")


CANARY = _flag("LLAISYS_CANARY")
BOUNDS = _flag("LLAISYS_BOUNDS")

CANARY_WORD = 0x5A5AA5A5
CANARY_WORDS = 256                          # guard length on either side: 1 KB, which keeps every alignment


class KernelTimers:
    """Device time per kernel class.  A launch's time runs from the end of the launch before it on the stream
    (or from start()) to its own end, so the classes add up to the time between start() and the last launch, and
    a launch that had to wait for its predecessor is charged only for what it added.  Work that is not this
    package's (allocations, copies of torch) falls to the launch after it."""

    def __init__(self, enabled: bool = False):
        self.enabled = enabled
        self._marks: List[Tuple[str, torch.cuda.Event]] = []
        self._totals: Dict[str, List[float]] = {}

    def start(self) -> None:
        if self.enabled:
            self.mark(None)

    def mark(self, what) -> None:
        if not self.enabled or torch.cuda.is_current_stream_capturing():
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._marks.append((what, ev))
        if len(self._marks) >= 8192:
            self._fold()

    def _fold(self) -> None:
        if not self._marks:
            return
        self._marks[-1][1].synchronize()
        for (_, before), (what, ev) in zip(self._marks, self._marks[1:]):
            if what is None:
                continue
            t = self._totals.setdefault(what, [0, 0.0])
            t[0] += 1
            t[1] += before.elapsed_time(ev)
        self._marks = self._marks[-1:]

    def report(self, reset: bool = True) -> Dict[str, Tuple[int, float]]:
        """{class: (launches, milliseconds)}, largest first."""
        self._fold()
        out = {k: (v[0], v[1]) for k, v in sorted(self._totals.items(), key=lambda kv: -kv[1][1])}
        if reset:
            self._totals = {}
            self._marks = []
        return out

    def table(self, reset: bool = True) -> str:
        rep = self.report(reset)
        total = sum(ms for _, ms in rep.values()) or 1.0
        width = max([len(k) for k in rep] + [12]) + 2
        lines = [f"{'kernel class':<{width}}{'launches':>10}{'ms':>12}{'share':>9}"]
        for k, (n, ms) in rep.items():
            lines.append(f"{k:<{width}}{n:>10}{ms:>12.3f}{100 * ms / total:>8.1f}%")
        return "\n".join(lines)


timers = KernelTimers(_flag("LLAISYS_TIMERS"))


# ---- guard words
def guarded(shape, dtype: torch.dtype, device, fill_zero: bool = True):
    """A tensor of `shape` inside a larger allocation with CANARY_WORDS guard words on either side.
    Returns (tensor, raw int32 allocation)."""
    n_bytes = 1
    for s in shape:
        n_bytes *= int(s)
    n_bytes *= torch.empty((), dtype=dtype).element_size()
    body_words = -(-n_bytes // 4)
    raw = torch.empty(2 * CANARY_WORDS + body_words, dtype=torch.int32, device=device)
    raw[:CANARY_WORDS] = CANARY_WORD
    raw[CANARY_WORDS + body_words:] = CANARY_WORD
    body = raw[CANARY_WORDS:CANARY_WORDS + body_words]
    if fill_zero:
        body.zero_()
    t = body.view(torch.uint8)[:n_bytes].view(dtype).view(*shape)
    return t, raw


def guards_intact(raw: torch.Tensor) -> bool:
    head, tail = raw[:CANARY_WORDS], raw[-CANARY_WORDS:]
    return bool((head == CANARY_WORD).all().item()) and bool((tail == CANARY_WORD).all().item())


setup_logging()

__all__ = ["log", "setup_logging", "timers", "KernelTimers", "CANARY", "BOUNDS", "guarded", "guards_intact"]
