"""Trace replay: feeds given token ids through a model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

It samples nothing and owns no model code: it drives the engine's step function, cache and
kernels, the ones generation uses.  For a step in which something is wanted it writes
OUT/<step>.f32: the logits at the wanted places, in the order of the entries and of `want`,
little-endian float32 [wanted, vocab].  After every step it prints `done <step>`.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def replay(engine, lines, out_dir: Path, emit=print) -> None:
    from .engine import StepEntry
    slots = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.acquire()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", ())))
        logits = engine.step(entries)
        if logits is not None:
            data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
            (out_dir / f"{step}.f32").write_bytes(data.tobytes())
        engine.check()
        for rid in rec.get("end", []):
            if rid in slots:
                engine.release(slots.pop(rid))
        emit(f"done {step}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=sorted(DTYPES))
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from ..cache.kv import CacheConfig
    from ..config.registry import load_config
    from ..weights.loader import FolderSource
    from .engine import build_engine

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    cfg = load_config(args.model)
    engine = build_engine(cfg.to_spec(), DTYPES[args.dtype], args.device,
                          CacheConfig(max_tokens=args.max_tokens), FolderSource(args.model))

    def emit(s):
        sys.stdout.write(s + "\n")
        sys.stdout.flush()

    replay(engine, sys.stdin, out_dir, emit)
    return 0


if __name__ == "__main__":
    sys.exit(main())
