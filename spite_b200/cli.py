"""Command line in the manner of giveen/spite's `spite` binary.

    spite run -m MODEL_DIR -p "5 17 3" [--max-tokens 512] [--temperature 1.0] [--ctx N]

`-m/--model`, `-p/--prompt`, `--max-tokens` (default 512), `--temperature`
(default 1.0; 0 is greedy) and `--ctx` keep the names, defaults and meanings of
`spite run` (crates/spite-cli/src/main.rs:282-306).  A prompt is a list of token
ids (separated by spaces or commas) because no tokenizer is part of this engine.
The timing lines printed to standard error have the reference's wording
(main.rs:595-628), and the seed of the sampler is its constant (main.rs:606)
unless `--sample-seed` says otherwise.  Engine options: `--dtype`, `--page-size`,
`--num-pages`, `--max-batch-tokens`, `--max-requests`.  Instead of a model folder,
`--random CONFIG.json [--seed N]` runs a model with random weights.

    spite bench -m MODEL_DIR [--n-prompt 512] [--n-tokens 512] [--n-runs 5] [--json]

prefill and decode rates and the time to the first token, options and report after
`spite-bench` (crates/spite-bench/src/main.rs:22-84,269-332,364-372).

    spite random --config CONFIG.json --out DIR [--seed 0] [--std 0.02] [--dtype bfloat16]

writes a model folder (config.json, model.safetensors) with random weights.

    spite replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl

is `bin/trace_run`: given token ids in, logits out, nothing sampled.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import tempfile
import time
from pathlib import Path

DTYPES = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32"}


def _ids(text: str) -> list[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("the prompt must be token ids separated by spaces or commas "
                         "(this engine has no tokenizer)") from None


def _need_gpu(device: str):
    """One line and exit code 2 where there is no CUDA device: the engine has no other backend."""
    import torch
    if not device.startswith("cuda") or not torch.cuda.is_available():
        print(f"spite: no CUDA device for --device {device}: this engine runs on an NVIDIA B200 (sm_100a) only",
              file=sys.stderr)
        raise SystemExit(2)


def _model_folder(args, stack) -> Path:
    """The folder to load: `--model`, or a temporary one with random weights for `--random`."""
    if args.model:
        return Path(args.model)
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict(json.loads(Path(args.random).read_text()))
    folder = Path(stack.enter_context(tempfile.TemporaryDirectory(prefix="spite_random_")))
    write_random_model(folder, cfg, seed=args.seed, std=args.std, dtype=torch.bfloat16)
    return folder


def _prompt(args, vocab: int) -> list[int]:
    if args.prompt_file:
        ids = _ids(Path(args.prompt_file).read_text())
    elif args.prompt_len is not None:
        import torch
        if args.prompt_len < 1:
            raise SystemExit("--prompt-len must be positive")
        g = torch.Generator().manual_seed(args.seed)
        ids = torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist()
    else:
        ids = _ids(args.prompt)
    if not ids:
        raise SystemExit("empty prompt")
    bad = [t for t in ids if not 0 <= t < vocab]
    if bad:
        raise SystemExit(f"token id {bad[0]} is outside the model's vocabulary of {vocab}")
    return ids


def _llm(args, folder):
    from .api import LLM
    cache_tokens = args.num_pages * args.page_size if args.num_pages else None
    return LLM(folder, dtype=DTYPES[args.dtype], device=args.device, ctx=args.ctx, page_size=args.page_size,
               cache_tokens=cache_tokens, max_batch_tokens=args.max_batch_tokens, max_requests=args.max_requests)


def cmd_run(args) -> int:
    import contextlib
    from .sampling.sampler import DEFAULT_SEED
    _need_gpu(args.device)
    with contextlib.ExitStack() as stack:
        folder = _model_folder(args, stack)
        t0 = time.time()
        llm = _llm(args, folder)
        print(f"load time    : {time.time() - t0:.2f} s", file=sys.stderr)
        prompt = _prompt(args, llm.model.plan.vocab_size)
        t0 = time.time()
        seed = DEFAULT_SEED if args.sample_seed is None else args.sample_seed
        out = llm.generate([prompt], max_tokens=args.max_tokens, temperature=args.temperature, seed=seed)[0]
        secs = time.time() - t0
    print(f"generate     : {len(prompt)} prompt + {len(out)} new tokens in {secs:.2f} s "
          f"({(len(prompt) + len(out)) / max(secs, 1e-9):.2f} tok/s)", file=sys.stderr)
    print(" ".join(str(t) for t in out))
    return 0


def cmd_bench(args) -> int:
    """Per run: one prompt of `--n-prompt` tokens run whole (its time is the time to the first token),
    then `--n-tokens` greedy decode steps; rates are totals over the runs (spite-bench/src/main.rs:269-332)."""
    import contextlib
    import torch
    from .engine.executor import StepEntry
    _need_gpu(args.device)
    with contextlib.ExitStack() as stack:
        folder = _model_folder(args, stack)
        llm = _llm(args, folder)
        eng, vocab = llm.engine, llm.model.plan.vocab_size
        g = torch.Generator().manual_seed(args.seed)
        prompt = torch.randint(0, vocab, (args.n_prompt,), generator=g).tolist()
        if args.n_prompt + args.n_tokens > eng.max_positions:
            raise SystemExit(f"--n-prompt + --n-tokens exceed the context of {eng.max_positions}")
        prefill_s = decode_s = 0.0
        for run in range(args.n_runs + 1):                        # the first run warms up and is not counted
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            logits = eng.step([StepEntry("bench", prompt, [len(prompt) - 1])])
            tok = llm.sampler.greedy_on_device(logits)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            for _ in range(args.n_tokens):
                logits = eng.step([StepEntry("bench", [0], [0])], device_tokens=tok)
                tok = llm.sampler.greedy_on_device(logits)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            eng.finish("bench")
            eng.check()
            if run:
                prefill_s += t1 - t0
                decode_s += t2 - t1
        result = {"label": f"{folder.name if args.model else Path(args.random).name} [{args.device}, {DTYPES[args.dtype]}]",
                  "tps": args.n_runs * args.n_tokens / max(decode_s, 1e-9),
                  "decode_tps": args.n_runs * args.n_tokens / max(decode_s, 1e-9),
                  "prefill_tps": args.n_runs * args.n_prompt / max(prefill_s, 1e-9),
                  "ttft_ms": 1e3 * prefill_s / max(args.n_runs, 1),
                  "peak_mem_mib": torch.cuda.max_memory_allocated() / 2 ** 20, "n_runs": args.n_runs}
    if args.json:
        print(json.dumps(result, indent=2))
    else:
        print(f"{result['label']}\n  prefill {result['prefill_tps']:10.1f} tok/s   ttft {result['ttft_ms']:8.2f} ms\n"
              f"  decode  {result['decode_tps']:10.1f} tok/s   peak memory {result['peak_mem_mib']:.0f} MiB   "
              f"({args.n_runs} runs)")
    return 0


def cmd_random(args) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict(json.loads(Path(args.config).read_text()))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[DTYPES[args.dtype]]
    write_random_model(args.out, cfg, seed=args.seed, std=args.std, dtype=dtype)
    print(f"wrote {args.out}/config.json and model.safetensors", file=sys.stderr)
    return 0


def cmd_replay(args) -> int:
    from .engine import trace
    _need_gpu(args.device)
    return trace.main(["--model", args.model, "--dtype", DTYPES[args.dtype], "--out", args.out,
                       "--max-tokens", str(args.max_tokens), "--page-size", str(args.page_size),
                       "--device", args.device])


def _model_options(p, required=True):
    g = p.add_mutually_exclusive_group(required=required)
    g.add_argument("-m", "--model", metavar="DIR", help="folder with config.json and model.safetensors")
    g.add_argument("--random", metavar="CONFIG.json", help="run a model with random weights made from this configuration")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights and of --prompt-len's tokens")
    p.add_argument("--std", type=float, default=0.02, help="standard deviation of the random weights")


def _engine_options(p):
    p.add_argument("--ctx", type=int, default=None, metavar="N",
                   help="context window size; default: the model's native maximum")
    p.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    p.add_argument("--num-pages", type=int, default=None, help="pages of the cache pool (of every layer group)")
    p.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    p.add_argument("--max-requests", type=int, default=4, help="requests that may be live at a time")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="spite", description="B200-native Llama 4 inference engine")
    sub = ap.add_subparsers(dest="cmd", required=True)

    run = sub.add_parser("run", help="generate tokens from a single prompt and print them")
    _model_options(run)
    g = run.add_mutually_exclusive_group(required=True)
    g.add_argument("-p", "--prompt", "--prompt-ids", dest="prompt", metavar="IDS", help="prompt token ids, e.g. \"5 17 3\"")
    g.add_argument("--prompt-file", metavar="FILE", help="file with the prompt's token ids")
    g.add_argument("--prompt-len", type=int, metavar="N", help="a prompt of N random token ids (from --seed)")
    run.add_argument("--max-tokens", type=int, default=512, metavar="N", help="maximum tokens to generate")
    run.add_argument("--temperature", type=float, default=1.0, metavar="T",
                     help="sampling temperature; 0 = greedy (deterministic), 1 = default")
    run.add_argument("--sample-seed", type=int, default=None, metavar="S", help="seed of the sampler's generator")
    _engine_options(run)
    run.set_defaults(fn=cmd_run)

    bench = sub.add_parser("bench", help="prefill and decode rates of one request")
    _model_options(bench)
    bench.add_argument("--n-tokens", type=int, default=512, help="decode tokens per run")
    bench.add_argument("--n-runs", type=int, default=5, help="benchmark runs (results averaged)")
    bench.add_argument("--n-prompt", type=int, default=512, help="prompt tokens for the prefill rate")
    bench.add_argument("--json", action="store_true", help="emit the result as JSON")
    _engine_options(bench)
    bench.set_defaults(fn=cmd_bench)

    rnd = sub.add_parser("random", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    rnd.set_defaults(fn=cmd_random)

    rep = sub.add_parser("replay", help="feed given token ids step by step and write logits (bin/trace_run)")
    rep.add_argument("--model", required=True)
    rep.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    rep.add_argument("--out", required=True)
    rep.add_argument("--max-tokens", type=int, required=True)
    rep.add_argument("--page-size", type=int, default=64)
    rep.add_argument("--device", default="cuda:0")
    rep.set_defaults(fn=cmd_replay)

    args = ap.parse_args(argv)
    for name in ("max_tokens", "max_requests", "max_batch_tokens", "page_size", "n_tokens", "n_runs", "n_prompt"):
        v = getattr(args, name, None)
        if v is not None and v < (0 if name == "max_tokens" and args.cmd == "run" else 1):
            ap.error(f"--{name.replace('_', '-')} must be positive")
    if getattr(args, "num_pages", None) is not None and args.num_pages < 1:
        ap.error("--num-pages must be positive")
    from .config import ConfigError
    from .kernels.api import KernelError
    from .weights import WeightError
    try:
        return args.fn(args)
    except (ConfigError, WeightError, KernelError, FileNotFoundError) as e:
        print(f"spite: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
