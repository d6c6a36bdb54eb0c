"""Command line in the manner of `spite run` (crates/spite-cli/src/main.rs:282-306):

    spite run -m MODEL_DIR -p "5 17 3" [--max-tokens 512] [--temperature 1.0] [--ctx N]

`-m/--model`, `-p/--prompt`, `--max-tokens` (default 512), `--temperature`
(default 1.0; 0 is greedy) and `--ctx` keep the reference's names, defaults and
meanings.  A prompt is a list of token ids (separated by spaces or commas)
because no tokenizer is part of this engine.  The timing lines printed to
standard error have the reference's wording (main.rs:595-628).

    spite random --config CONFIG.json --out DIR [--seed 0] [--std 0.02] [--dtype bfloat16]

writes a model folder (config.json, model.safetensors) with random weights.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from pathlib import Path


def _ids(text: str) -> list[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("the prompt must be token ids separated by spaces or commas "
                         "(this engine has no tokenizer)") from None


def cmd_run(args) -> int:
    from .api import LLM
    prompt = _ids(Path(args.prompt_file).read_text() if args.prompt_file else args.prompt)
    if not prompt:
        raise SystemExit("empty prompt")
    t0 = time.time()
    llm = LLM(args.model, dtype=args.dtype, device=args.device, ctx=args.ctx, page_size=args.page_size,
              cache_tokens=args.cache_tokens, max_batch_tokens=args.max_batch_tokens, max_requests=4)
    print(f"load time    : {time.time() - t0:.2f} s", file=sys.stderr)
    t0 = time.time()
    out = llm.generate([prompt], max_tokens=args.max_tokens, temperature=args.temperature)[0]
    secs = time.time() - t0
    print(f"generate     : {len(prompt)} prompt + {len(out)} new tokens in {secs:.2f} s "
          f"({(len(prompt) + len(out)) / max(secs, 1e-9):.2f} tok/s)", file=sys.stderr)
    print(" ".join(str(t) for t in out))
    return 0


def cmd_random(args) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict(json.loads(Path(args.config).read_text()))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_random_model(args.out, cfg, seed=args.seed, std=args.std, dtype=dtype)
    print(f"wrote {args.out}/config.json and model.safetensors", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="spite", description="B200-native Llama 4 inference engine")
    sub = ap.add_subparsers(dest="cmd", required=True)
    run = sub.add_parser("run", help="generate tokens from a single prompt and print them")
    run.add_argument("-m", "--model", required=True, metavar="DIR", help="folder with config.json and model.safetensors")
    g = run.add_mutually_exclusive_group(required=True)
    g.add_argument("-p", "--prompt", metavar="IDS", help="prompt token ids, e.g. \"5 17 3\"")
    g.add_argument("--prompt-file", metavar="FILE", help="file with the prompt's token ids")
    run.add_argument("--max-tokens", type=int, default=512, metavar="N", help="maximum tokens to generate")
    run.add_argument("--temperature", type=float, default=1.0, metavar="T",
                     help="sampling temperature; 0 = greedy (deterministic), 1 = default")
    run.add_argument("--ctx", type=int, default=None, metavar="N",
                     help="context window size; default: the model's native maximum")
    run.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    run.add_argument("--device", default="cuda:0")
    run.add_argument("--page-size", type=int, default=64)
    run.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache pool holds")
    run.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    run.set_defaults(fn=cmd_run)
    rnd = sub.add_parser("random", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    rnd.set_defaults(fn=cmd_random)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
