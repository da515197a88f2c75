"""Command line in the manner of xsmccc/llaisys' test/test_infer.py (:124-140): the same option
names with the same meanings, plus what a run without network needs.

    python -m llaisys_b200.cli --model DIR --prompt "Who are you?" --max_steps 128
    python -m llaisys_b200.cli --model DIR --tokens 1,2,3 --test
    python -m llaisys_b200.cli --random-weights config.json --seed 0 --tokens 1,2,3

--test forces top_p=1, top_k=1, temperature=1 as there; that project then compares with a
library model fetched from the network, which is not possible here, so --test replays the
generated sequence through the step function as one whole prompt and requires that every
generated token is the arg-max of the logits at its place.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time


def _tokenizer(model_dir):
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model_dir, local_files_only=True)
    except Exception as e:          # no tokenizer files in the folder
        raise SystemExit(f"no tokenizer could be loaded from {model_dir} ({type(e).__name__}); "
                         f"pass token ids with --tokens") from None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llaisys_b200.cli")
    ap.add_argument("--device", default="nvidia", choices=["cpu", "nvidia"], type=str)
    ap.add_argument("--model", default=None, type=str)
    ap.add_argument("--prompt", default="Who are you?", type=str)
    ap.add_argument("--max_steps", default=128, type=int)
    ap.add_argument("--top_p", default=0.8, type=float)
    ap.add_argument("--top_k", default=50, type=int)
    ap.add_argument("--temperature", default=1.0, type=float)
    ap.add_argument("--test", action="store_true")
    ap.add_argument("--tokens", default=None, type=str, help="comma-separated prompt token ids (no tokenizer needed)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--seed", default=0, type=int)
    ap.add_argument("--random-weights", default=None, metavar="CONFIG.json",
                    help="write a model folder with seeded random weights from this configuration and run it")
    ap.add_argument("--max-tokens", default=8192, type=int, help="cache size in tokens")
    args = ap.parse_args(argv)

    if args.device == "cpu":
        raise SystemExit("llaisys_b200 has no CPU path; use --device nvidia")
    from .models import CausalLM, DeviceType
    from .engine.engine import StepEntry

    top_p, top_k, temperature = args.top_p, args.top_k, args.temperature
    if args.test:
        top_p, top_k, temperature = 1.0, 1, 1.0

    tmp = None
    model_dir = args.model
    if args.random_weights:
        from .weights.random_init import write_random_model
        tmp = tempfile.TemporaryDirectory()
        model_dir = str(write_random_model(tmp.name, json.loads(open(args.random_weights).read()), args.seed, args.dtype))
    if model_dir is None:
        raise SystemExit("give --model DIR or --random-weights CONFIG.json (there is no network to fetch a model from)")

    tok = None
    if args.tokens:
        inputs = [int(t) for t in args.tokens.replace(" ", "").split(",") if t]
    else:
        tok = _tokenizer(model_dir)
        text = tok.apply_chat_template(conversation=[{"role": "user", "content": args.prompt}],
                                       add_generation_prompt=True, tokenize=False)
        inputs = tok.encode(text)

    model = CausalLM(model_dir, DeviceType.NVIDIA, dtype=args.dtype, max_tokens=args.max_tokens, seed=args.seed)
    start = time.time()
    out = model.generate(inputs, max_new_tokens=args.max_steps, top_k=top_k, top_p=top_p, temperature=temperature)
    elapsed = time.time() - start

    print("\n=== Your Result ===\n")
    print("Tokens:")
    print(out)
    if tok is not None:
        print("\nContents:")
        print(tok.decode(out, skip_special_tokens=True))
    print(f"\nTime elapsed: {elapsed:.2f}s\n")

    if args.test:
        logits = model.logits(out[:-1])
        from . import kernels
        picks = kernels.argmax(logits).tolist()
        n = len(inputs)
        assert picks[n - 1:] == out[n:], "replayed arg-max differs from the generated tokens"
        print("\033[92mTest passed!\033[0m\n")
    if tmp:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
