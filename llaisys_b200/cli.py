"""Command line in the manner of xsmccc/llaisys' test/test_infer.py (:124-140): the same option
names with the same meanings, plus what a run without network needs.

    python -m llaisys_b200.cli --model DIR --prompt "Who are you?" --max_steps 128
    python -m llaisys_b200.cli --model DIR --tokens 1,2,3 --test
    python -m llaisys_b200.cli --random-weights config.json --seed 0 --tokens 1,2,3
    python -m llaisys_b200.cli --model DIR --batch-file prompts.txt --max_steps 32
    python -m llaisys_b200.cli --model DIR --device cpu --tokens 1,2,3 --top_k 1

--device nvidia (the default here) runs the engine; --device cpu runs the float32 CPU model of
models/cpu_model.py (greedy only, one request at a time): that is the device that project's own
model runs on.  --test forces top_p=1, top_k=1, temperature=1 as there; that project then asserts
that its tokens equal those of a second implementation (a library model fetched from the
network, test/test_infer.py:193-195).  Here the second implementation is the CPU model: in
float32 the engine's tokens must equal its tokens; in bfloat16, where two nearly equal logits may
legitimately change places, every token the engine chose must be, in the CPU model's logits at
that place, within the precision's margin of the maximum.

--batch-file names a file with one request per line: a JSON list of token ids, comma-separated
token ids, or (with a tokenizer in the model folder) text.  The requests are generated as
batches of unequal prompts through the generation loop and printed in the file's order.
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
    ap.add_argument("--device", default="nvidia", choices=["cpu", "nvidia"], type=str,
                    help="nvidia: the engine on the B200; cpu: the plain float32 CPU model (greedy, slow)")
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
    ap.add_argument("--batch-file", default=None, metavar="FILE",
                    help="one request per line (a JSON list of token ids, comma-separated ids, or text)")
    args = ap.parse_args(argv)

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

    def encode(text):
        nonlocal tok
        tok = tok or _tokenizer(model_dir)
        chat = tok.apply_chat_template(conversation=[{"role": "user", "content": text}], add_generation_prompt=True, tokenize=False)
        return tok.encode(chat)

    def ids_of(line):
        line = line.strip()
        if line.startswith("["):
            return [int(t) for t in json.loads(line)]
        if line and all(c.isdigit() or c in ", " for c in line):
            return [int(t) for t in line.replace(" ", "").split(",") if t]
        return encode(line)

    if args.batch_file:
        prompts = [ids_of(l) for l in open(args.batch_file).read().splitlines() if l.strip()]
        if not prompts:
            raise SystemExit(f"{args.batch_file} holds no request")
    elif args.tokens:
        prompts = [ids_of(args.tokens)]
    else:
        prompts = [encode(args.prompt)]

    from .config.registry import load_config
    stop_ids = list(load_config(model_dir).to_spec().stop_token_ids)
    cpu_model = None
    if args.device == "cpu" or args.test:
        from .models.cpu_model import CpuModel
        cpu_model = CpuModel.from_folder(model_dir)

    start = time.time()
    if args.device == "cpu":
        if top_k != 1:
            raise SystemExit("--device cpu generates greedily only: pass --top_k 1 (or --test)")
        outs = [cpu_model.generate(p, args.max_steps, stop_ids) for p in prompts]
    else:
        from .models import CausalLM, DeviceType
        model = CausalLM(model_dir, DeviceType.NVIDIA, dtype=args.dtype, max_tokens=args.max_tokens, seed=args.seed)
        outs = model.generate_batch(prompts, max_new_tokens=args.max_steps, top_k=top_k, top_p=top_p, temperature=temperature)
    elapsed = time.time() - start
    from .diagnostics import timers
    if timers.enabled and args.device != "cpu":
        print(timers.table(), file=sys.stderr)      # LLAISYS_TIMERS=1: device time per kernel class

    print("\n=== Your Result ===\n")
    for p, new in zip(prompts, outs):
        print("Tokens:")
        print(list(p) + list(new))
        if tok is not None:
            print("\nContents:")
            print(tok.decode(list(p) + list(new), skip_special_tokens=True))
    print(f"\nTime elapsed: {elapsed:.2f}s\n")

    if args.test and args.device != "cpu":
        import numpy as np
        layers = len(cpu_model.spec.order)
        for p, new in zip(prompts, outs):
            if args.dtype == "float32":
                want = cpu_model.generate(p, args.max_steps, stop_ids)
                assert list(new) == want, f"the engine generated {list(new)}, the CPU model {want}"
            else:
                cpu_model.reset()
                logits = cpu_model.step(list(p) + list(new)[:-1])[len(p) - 1:]
                margin = 2 * 8 * 2.0 ** -9 * (6 * layers + 2) ** 0.5 * float(np.sqrt(np.mean(logits ** 2)))
                for i, t in enumerate(new):
                    assert logits[i][t] >= logits[i].max() - margin, \
                        f"token {i} ({t}) is not a maximum of the CPU model's logits within {margin:.3g}"
        print("\033[92mTest passed!\033[0m\n")
    if tmp:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
