"""Command line in the reference's manner: ``generate``, ``bench``, ``score``, plus ``replay`` and
``init-random``.

Reference flags kept with their names and meanings (src/main.rs:22-104,960-1013,857-866):
``--model``, ``-n``, ``--ctx`` (cache size in tokens), ``--chunk`` (prefill portion),
``--temp``, ``--top-k``, ``--top-p``, ``--seed``, the penalty flags, ``--pp``, ``--tg``,
``--reps``, ``--json-out``, ``--input``.  There is no tokenizer here: ``--prompt`` takes
token ids ("1,2,3" or "-" for standard input), ``--prompt-len N`` draws N random ids.
Lines printed follow the reference: ``prompt N tok X tok/s | gen M tok Y tok/s``
(src/main.rs:1147) and ``pp N: prefill mean (min-max) tok/s | tg K: decode ... tok/s``
(src/main.rs:1232).
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _engine_flags(ap):
    ap.add_argument("--model", default=None, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--random-weights", action="store_true",
                    help="no model folder: draw the weights on the device from --config and --weights-seed")
    ap.add_argument("--config", default=None, help="config.json of the architecture (with --random-weights)")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--weights-std", type=float, default=0.02, help="spread of the drawn matrices (with --random-weights)")
    ap.add_argument("--weights-norm-std", type=float, default=0.0, help="spread of the drawn norm scales around 1")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--ctx", type=int, default=4096, help="cache size in tokens")
    ap.add_argument("--chunk", type=int, default=None, help="prefill portion in tokens [default: the token budget]")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--parallel", type=int, default=64, help="most live requests")
    ap.add_argument("--temp", type=float, default=0.0, help="sampling temperature; 0 is greedy")
    ap.add_argument("--top-k", type=int, default=0, help="sample only from the K most likely tokens (0 = all)")
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--penalty-last-n", type=int, default=64)
    ap.add_argument("--dry-multiplier", type=float, default=0.0)
    ap.add_argument("--dry-base", type=float, default=1.75)
    ap.add_argument("--dry-allowed-length", type=int, default=2)
    ap.add_argument("--seed", type=int, default=None, help="random seed for sampling [default: from the clock]")


def _sampling(args):
    from .sampling import SamplingParams
    seed = args.seed if args.seed is not None else time.time_ns()
    return SamplingParams(temp=args.temp, top_k=args.top_k, top_p=args.top_p, seed=seed,
                          presence_penalty=args.presence_penalty, frequency_penalty=args.frequency_penalty,
                          repeat_penalty=args.repeat_penalty, penalty_last_n=args.penalty_last_n,
                          dry_multiplier=args.dry_multiplier, dry_base=args.dry_base,
                          dry_allowed_length=args.dry_allowed_length)


def _make_engine(args, ctx=None, max_seqs=None):
    from .engine import Engine
    ctx = ctx or args.ctx
    from .dtypes import engine_dtype_name
    dtype = engine_dtype_name(args.dtype)
    kw = dict(dtype=dtype, page_size=args.page_size, max_tokens=ctx, max_batch_tokens=min(max(ctx, 64), 8192),
              max_seqs=max_seqs or args.parallel, prefill_chunk=args.chunk)
    if args.random_weights:
        if not args.config:
            raise SystemExit("--random-weights needs --config config.json")
        with open(args.config) as f:
            return Engine(json.load(f), random_seed=args.weights_seed, random_std=args.weights_std,
                          random_norm_std=args.weights_norm_std, **kw)
    if not args.model:
        raise SystemExit("give --model DIR, or --random-weights --config config.json")
    return Engine(args.model, **kw)


def _prompt_ids(args, vocab):
    import numpy as np
    if args.prompt_len:
        return np.random.default_rng(args.prompt_seed).integers(0, vocab, size=args.prompt_len).tolist()
    text = sys.stdin.read() if args.prompt == "-" else args.prompt
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(args):
    eng = _make_engine(args, max_seqs=1)
    ids = _prompt_ids(args, eng.runner.vocab_size)
    import torch
    from .engine import StepEntry
    sp = _sampling(args)
    n = min(args.n, eng.runner.max_positions - len(ids), args.ctx - len(ids))
    if n <= 0:
        raise SystemExit(f"context full ({len(ids)} tokens; raise --ctx)")
    rid = eng.add_request(ids, n, sp, eos_ids=args.eos or ())
    t0 = time.perf_counter()
    done = []
    eng.lookahead = False                  # the prompt's time must not hold the first decode step launched behind it
    while not eng.scheduler.running or eng.scheduler.running[0].prefilling:
        done += eng.step()
        if done:
            break
    torch.cuda.synchronize()
    eng.lookahead = True
    t1 = time.perf_counter()
    while eng.has_work():
        done += eng.step()
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    out = done[0].generated
    print(" ".join(str(t) for t in out))
    gen_rate = (len(out) - 1) / (t2 - t1) if len(out) > 1 else 0.0
    print(f"prompt {len(ids)} tok {len(ids) / (t1 - t0):.1f} tok/s | gen {len(out)} tok {gen_rate:.1f} tok/s", file=sys.stderr)
    return 0


def _stat(d):
    return f"{d['mean']:.1f} ({d['min']:.1f}-{d['max']:.1f})"


def cmd_bench(args):
    pps = [int(x) for x in args.pp.split(",")]
    ctx = max(args.ctx, (max(pps) + args.tg + 1) * args.batch)
    eng = _make_engine(args, ctx=ctx, max_seqs=max(args.batch, 1))
    results = []
    for n in pps:
        rec = eng.bench([n], args.tg, args.reps, args.batch)[0]
        print(f"pp {n:6d}: prefill {_stat(rec['prefill_tok_s'])} tok/s | tg {args.tg}: decode {_stat(rec['decode_tok_s'])} tok/s")
        rf = rec["roofline"]
        print(f"          prefill {rf['prefill']['achieved']:.1f} TFLOP/s = {rf['prefill']['frac']:.3f} of the tensor peak | decode "
              f"{rf['decode']['achieved']:.0f} GB/s = {rf['decode']['frac']:.3f} of the HBM peak ({rf['decode']['peaks']} peaks)")
        results.append(rec)
    if args.json_out:
        rec = {"schema": "rustingstrata_b200.bench.v1", "model": args.model or args.config, "dtype": args.dtype, "ctx": ctx, "tg": args.tg,
               "reps": args.reps, "unix_time": int(time.time()), "results": results}
        with open(args.json_out, "w") as f:
            f.write(json.dumps(rec) + "\n")
    return 0


def cmd_score(args):
    """Teacher-forced ids → argmax and top-5 log-probabilities per position (src/main.rs:1050-1084)."""
    import numpy as np
    from .engine import StepEntry
    text = sys.stdin.read() if args.input == "-" else open(args.input).read()
    rec = json.loads(text)
    prompt, cont = [int(t) for t in rec["prompt"]], [int(t) for t in rec["continuation"]]
    if not prompt:
        raise SystemExit("score: empty prompt")
    eng = _make_engine(args, ctx=max(args.ctx, len(prompt) + len(cont)), max_seqs=1)
    toks = prompt + cont
    want = list(range(len(prompt) - 1, len(toks) - 1)) if cont else [len(prompt) - 1]
    logits = eng.step_raw([StepEntry("s", toks if cont else prompt, want)]).cpu().numpy().astype(np.float64)
    eng.runner.check_status()
    lse = np.log(np.exp(logits - logits.max(1, keepdims=True)).sum(1, keepdims=True)) + logits.max(1, keepdims=True)
    lp = logits - lse
    top = np.argsort(-lp, axis=1, kind="stable")[:, :5]
    print(json.dumps({"argmax": [int(r[0]) for r in top],
                      "top5": [[(int(i), float(lp[k, i])) for i in r] for k, r in enumerate(top)]}))
    return 0


def cmd_init_random(args):
    from .models import manifest_for
    from .weights import write_random_model
    with open(args.config) as f:
        cfg = json.load(f)
    m = manifest_for(cfg)

    def progress(i, n, name):
        if i % 50 == 0 or i == n:
            print(f"[init-random] {i}/{n} tensors", file=sys.stderr, flush=True)
    write_random_model(args.out, cfg, m, args.seed, std=args.std, norm_std=args.norm_std, store_dtype=args.store_dtype,
                       progress=progress)
    print(args.out)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":          # everything behind the word belongs to trace replay's own parser
        from .replay import main as replay_main
        return replay_main(argv[1:])
    ap = argparse.ArgumentParser(prog="rustingstrata_b200", description="B200 inference engine for the Qwen3 dense decoder")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generation (greedy unless --temp)")
    _engine_flags(g)
    g.add_argument("--prompt", "--prompt-ids", dest="prompt", default="",
                   help='prompt token ids, e.g. "1,2,3" ("-" reads standard input)')
    g.add_argument("--prompt-len", type=int, default=0, help="draw this many random prompt ids instead")
    g.add_argument("--prompt-seed", type=int, default=0)
    g.add_argument("-n", type=int, default=32, help="tokens to generate")
    g.add_argument("--eos", type=int, action="append", help="token id that ends the generation (repeatable)")
    g.set_defaults(fn=cmd_generate)
    b = sub.add_parser("bench", help="timed prefill of --pp tokens, then timed greedy decode of --tg")
    _engine_flags(b)
    b.add_argument("--pp", default="512,4096")
    b.add_argument("--tg", type=int, default=128)
    b.add_argument("--reps", type=int, default=3)
    b.add_argument("--batch", type=int, default=1, help="requests decoded together")
    b.add_argument("--json-out", default=None)
    b.set_defaults(fn=cmd_bench)
    s = sub.add_parser("score", help='teacher-force {"prompt":[ids],"continuation":[ids]}')
    _engine_flags(s)
    s.add_argument("--input", default="-")
    s.set_defaults(fn=cmd_score)
    sub.add_parser("replay", help="trace replay (same as bin/trace_run; its options follow the word)")
    i = sub.add_parser("init-random", help="write a model folder with random weights from a config.json and a seed")
    i.add_argument("--config", required=True)
    i.add_argument("--out", required=True)
    i.add_argument("--seed", type=int, default=0)
    i.add_argument("--std", type=float, default=0.02)
    i.add_argument("--norm-std", type=float, default=0.0)
    i.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    i.set_defaults(fn=cmd_init_random)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
