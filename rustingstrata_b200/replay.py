"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the
same :class:`~rustingstrata_b200.engine.ModelRunner` generation uses and calls its step
function with exactly the entries of each input line.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

(``--random-config FILE --weights-seed S`` instead of ``--model`` draws the weights on the device: the same
values ``init-random`` writes for that configuration and seed, for sizes not worth a file.)

Input: one JSON object per line on standard input,
``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}``.
For a step with wanted places it writes ``<out>/<step>.f32``: little-endian float32
logits [wanted, vocab] in the order of the entries and of ``want``.  After every step it
prints ``done <step>``; when its input ends it prints what the page pools did (pages handed out, of which had
been used before) to standard error.  The reference's nearest tools are ``score`` (teacher-forced
ids → argmax and top-5, src/main.rs:1050-1084) and ``force_tokens``
(src/gpu_model.rs:2871); a logits dump is this engine's own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default=None, help="folder with config.json and model.safetensors")
    ap.add_argument("--random-config", default=None,
                    help="instead of --model: a config.json whose model is drawn on the device from --weights-seed")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--weights-std", type=float, default=0.02)
    ap.add_argument("--weights-norm-std", type=float, default=0.0)
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    if (args.model is None) == (args.random_config is None):
        ap.error("give --model DIR, or --random-config config.json")

    from .config import EngineConfig
    from .engine import ModelRunner, StepEntry

    os.makedirs(args.out, exist_ok=True)
    page = args.page_size
    pool_tokens = (args.max_tokens + page - 1) // page * page
    eng = EngineConfig(dtype=args.dtype, page_size=page, num_pages=pool_tokens // page, max_seqs=8,
                       max_batch_tokens=max(pool_tokens, 64), max_logit_rows=max(pool_tokens, 64))
    print(f"[trace_run] loading {args.model or args.random_config} ({args.dtype}, {pool_tokens // page} pages of "
          f"{page})", file=sys.stderr, flush=True)
    if args.model is not None:
        runner = ModelRunner.from_dir(args.model, eng)
    else:
        with open(args.random_config) as f:
            runner = ModelRunner.from_random(json.load(f), eng, seed=args.weights_seed, std=args.weights_std,
                                             norm_std=args.weights_norm_std)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            runner.check_status()
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            runner.release(rid)
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    runner.cache.check()
    for g, pool in enumerate(runner.cache.pools):
        print(f"[trace_run] pool {g}: pages {pool.num_pages} allocations {pool.allocations} reuses {pool.reuses} "
              f"held_at_end {pool.num_pages - pool.n_free}", file=sys.stderr, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
