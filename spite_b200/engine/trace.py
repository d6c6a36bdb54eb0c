"""Trace replay: feed given token ids through a model step by step and write
the logits.  Nothing is sampled.  The replay drives the same `Model`, `Engine`,
cache and kernels that generation uses; it has no forward pass, cache or loader
of its own.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: `<out>/<step>.f32` (little-endian float32 [wanted, vocab]) for steps in
which something is wanted, and a line `done <step>` after every step.

Counterparts in giveen/spite: tools/verify/llama_logits.c:23-73 and
crates/spite-models/examples/dump_logits.rs:15-53 (raw ids in, one forward per
position, `[n_tok, vocab]` float32 out).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .executor import Engine, StepEntry
from .model import Model


def replay(engine: Engine, lines, out_dir: Path, log=sys.stdout):
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in rec.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                engine.check()                 # the logits are here: did every kernel of the step finish its work?
                data.tofile(out_dir / f"{step}.f32")
        for req in rec.get("end", []):
            if engine.is_live(req):
                engine.finish(req)
        print(f"done {step}", file=log, flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size < 1 or 64 % args.page_size:
        ap.error("--page-size must divide 64")
    model = Model.from_folder(args.model, dtype=args.dtype, device=args.device)
    engine = Engine(model, cache_tokens=args.max_tokens, page_size=args.page_size, max_requests=8)
    replay(engine, sys.stdin, Path(args.out))
    return 0
