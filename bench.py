#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B sizes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]
    python bench.py --workload 14b-mixed | 32b-long          (the two further measured workloads, one line each)

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 (a "step" is one
decode step of the whole batch, timed on the device with CUDA events); ``e2e`` is the
same through the Python entry point with host token ids in and out every step;
``prefill`` is one 2,048-token prompt; ``roofline`` relates the decode step's bytes
(every weight it uses once plus the cache of the live requests) to the HBM peak;
``points`` holds decode at batch 1 and 64 (``points_roofline``: each point's time per step
and fraction of the HBM peak).  Peaks come from MEASURED_PEAKS.json beside this file when
present, else from the fallback figures of this pool.

``--marginal``: instead of the benchmark line, what each kernel family costs INSIDE the captured decode step (batch
``--batch``, prompts of ``--prompt-len`` tokens): the step is timed whole and again with that family's launches left out
(the results are then wrong, only the clock is read).  The difference is what the family adds to the step with all the
overlap between neighbouring kernels that programmatic dependent launch gives, which a kernel timed alone cannot show.
``--marginal-prefill``: the same for the step that runs one whole prompt of ``--prompt-len`` tokens.

``--workload 14b-mixed``: Qwen3-14B layer sizes, 32 requests with prompts of 128 to 4,096
random tokens, all present at the start, run by the engine's scheduler with portions of 512
prompt tokens beside the decoding requests' tokens, 256 tokens each at temperature 0.7,
context 8,192: total tokens per second, time to first token, and what the steps held.
``--workload 32b-long``: Qwen3-32B layer sizes, 8 requests with 12,000-token prompts, then 256
greedy tokens each, context 16,384: decode tokens per second, its fraction of the HBM peak,
and the share of the step that is spent on the long cache (against the same step at 16 keys).

The reference (a Rust crate) cannot be installed here: ``--impl reference`` says so.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the benchmark configuration (Qwen3-8B)
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
    "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 12288, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 40960,
    "tie_word_embeddings": False, "use_sliding_window": False, "torch_dtype": "bfloat16",
}
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
CONTEXT = 4096          # tokens per request the cache is sized for
PROMPT = 2048           # tokens each request holds before decoding is timed


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run this many of the configuration's layers (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--workload", default="headline", choices=["headline", "14b-mixed", "32b-long"])
    ap.add_argument("--marginal", action="store_true", help="marginal cost of each kernel family inside the decode step")
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="with --marginal: tokens each request holds")
    ap.add_argument("--marginal-prefill", action="store_true",
                    help="marginal cost of each kernel family inside the step that runs one whole prompt of --prompt-len tokens")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust crate (no setup.py/pyproject.toml; "
                          "no cargo or rustc in this image): pip cannot install it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.marginal_prefill:
        return marginal_costs_prefill(args)
    if args.marginal:
        return marginal_costs(args)
    if args.workload == "14b-mixed":
        return mixed_workload(args)
    if args.workload == "32b-long":
        return long_context_workload(args)

    import numpy as np
    import torch
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.engine import roofline
    from rustingstrata_b200.sampling import SamplingParams

    pk = roofline.peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    cfg = dict(QWEN3_8B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    max_batch = max(args.batch, 1 if args.no_points else 64)
    eng = Engine(cfg, dtype="bfloat16", random_seed=0, page_size=16, max_tokens=max_batch * CONTEXT,
                 max_batch_tokens=PROMPT, max_seqs=max_batch)
    runner = eng.runner
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    wbytes = roofline.weight_bytes(runner.model)
    clocks = ClockSampler()

    def prefill_requests(n):
        """Admits n requests and runs their 2,048-token prompts, one prompt per step."""
        rids = []
        for _ in range(n):
            rids.append(eng.add_request(rng.integers(0, V, size=PROMPT).tolist(), CONTEXT - PROMPT, SamplingParams()))
        while eng.scheduler.waiting or any(r.prefilling for r in eng.scheduler.running):
            eng.step()
        return rids

    def finish_all():
        eng.drain()
        for r in list(eng.scheduler.running):
            eng.scheduler.running.remove(r)
            runner.release(r.rid)
            eng._samplers.pop(r.rid, None)

    def time_decode(n, steps, warmup):
        """Device-timed decode of n requests; returns (ms per step, e2e ms per step, launches per step, kv tokens)."""
        prefill_requests(n)
        for _ in range(warmup):
            eng.step()
        kv_tokens = sum(runner.length(r.rid) for r in eng.scheduler.running)
        # kernels of this package that run inside the timed region: its steps are graph replays, whose kernel nodes the
        # runner counted at capture (the warm-up steps of the device-timed loop, launched from Python, are not timed)
        ms = eng.decode_steps_device_timed(steps, warmup=3)
        launches = eng.kernels_in_timed_steps / steps
        # end to end through Engine.step: every step's inputs go up from pinned host memory and its chosen ids come
        # back to the host.  The engine launches a step while the one before it still runs, so the region starts and
        # ends with nothing under way: `steps` calls, then the step the last call launched ahead is taken in too.
        eng.drain()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()
        done_steps = steps + (1 if eng._flight is not None else 0)
        eng.drain()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1000 / done_steps
        finish_all()
        return ms, e2e_ms, launches, kv_tokens

    # ---- prefill of one 2,048-token prompt (warm-up runs first)
    for _ in range(2):
        prefill_requests(1)
        finish_all()
    clocks.start()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rid_prompt = rng.integers(0, V, size=PROMPT).tolist()
    eng.add_request(rid_prompt, CONTEXT - PROMPT, SamplingParams())
    eng.lookahead = False                      # the timed step is the prompt alone, not the first decode step behind it
    ev0.record()
    eng.step()
    ev1.record()
    eng.lookahead = True
    torch.cuda.synchronize()
    prefill_ms = ev0.elapsed_time(ev1)
    finish_all()
    pf_flops = roofline.step_flops(runner.model, [PROMPT], [PROMPT], 1)
    prefill = {"value": PROMPT / prefill_ms * 1000, "tokens": PROMPT, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1000) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode at the headline batch
    ms, e2e_ms, launches, kv_tokens = time_decode(args.batch, args.steps, args.warmup)
    points, points_roofline = {}, {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _, pkv = time_decode(b, max(64, args.steps), args.warmup)
            points[f"decode_b{b}"] = b / pms * 1000
            pr = roofline.decode_roofline(runner.model, runner.kv_bytes_per_token, pkv, pms, pk)
            points_roofline[f"decode_b{b}"] = {"ms_per_step": pms, "steps": max(64, args.steps), "achieved": pr["achieved"],
                                               "frac": pr["frac"]}
    clk = clocks.stop()

    step_bytes = wbytes + kv_tokens * runner.kv_bytes_per_token
    achieved = step_bytes / (ms / 1000) / 1e9
    value = args.batch / ms * 1000
    rec = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B sizes, bf16, random weights, 2,048-token prompts)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "qwen3-8b-sizes", "layers": n_layers, "layers_of_config": full_layers,
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": 16, "parallelism": "single-gpu",
                   "weights": "random N(0,0.02) bf16", "l2": "inputs larger than L2 (weights + cache)",
                   "peaks": pk["source"]},
        "e2e": {"value": args.batch / e2e_ms * 1000, "unit": "tok/s", "h2d_bytes_per_step": eng.h2d_bytes_last_step,
                "d2h_bytes_per_step": eng.d2h_bytes_last_step},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "points_roofline": points_roofline,
        "clocks": clk,
    }
    print(json.dumps(rec))
    return 0


def marginal_costs(args) -> int:
    """Times the captured decode step whole, then with one kernel family's launches left out at a time."""
    import numpy as np
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.kernels import ops
    from rustingstrata_b200.sampling import SamplingParams
    cfg = dict(QWEN3_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    L, B, S = cfg["num_hidden_layers"], args.batch, args.prompt_len
    eng = Engine(cfg, dtype="bfloat16", random_seed=0, page_size=16, max_tokens=B * CONTEXT, max_batch_tokens=PROMPT, max_seqs=B)
    rng = np.random.default_rng(0)
    for _ in range(B):
        eng.add_request(rng.integers(0, cfg["vocab_size"], size=S).tolist(), CONTEXT - S, SamplingParams())
    while eng.scheduler.waiting or any(r.prefilling for r in eng.scheduler.running):
        eng.step()

    def timed():
        eng.runner._graphs.clear()                       # the step is captured anew, without the launches that are off
        return eng.decode_steps_device_timed(max(args.steps, 32), warmup=4)
    for _ in range(3):
        timed()                                          # until the clocks have settled under the power cap
    whole = timed()
    out = {"batch": B, "prompt_len": S, "layers": L, "ms_per_step": whole, "us_per_layer": whole / L * 1000, "marginal_us_per_layer": {},
           "marginal_us_per_step": {}}
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    families = [("attention_decode (+ merge)", "attention_decode", None), ("qk_norm_rope_kv", "qk_norm_rope_kv", None),
                ("gate/up product", "linear_swiglu", None), ("row norms (+ owed sums)", "rmsnorm", None),
                ("qkv product", "linear", (qkv, H)), ("output product", "linear", (H, cfg["num_attention_heads"] * cfg["head_dim"])),
                ("down product", "linear", (H, I)), ("output head", "linear", (cfg["vocab_size"], H))]
    for label, fn_name, shape in families:
        real = getattr(ops, fn_name)
        if shape is None:
            setattr(ops, fn_name, lambda *a, **k: None)
        else:
            setattr(ops, fn_name, lambda a, w, *r, _real=real, _shape=shape, **k: None if tuple(w.shape) == _shape else _real(a, w, *r, **k))
        try:
            t = timed()
        finally:
            setattr(ops, fn_name, real)
        again = timed()                                  # the whole step once more: clocks drift under a long load
        per_step = ((whole + again) / 2 - t) * 1000
        whole = again
        key = "marginal_us_per_step" if label == "output head" else "marginal_us_per_layer"
        out[key][label] = per_step if label == "output head" else per_step / L
    out["ms_per_step_at_the_end"] = whole
    print(json.dumps(out))
    return 0


def marginal_costs_prefill(args) -> int:
    """Times the step that runs one whole prompt, then the same step with one kernel family's launches left out."""
    import numpy as np
    import torch
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.kernels import ops
    from rustingstrata_b200.sampling import SamplingParams
    cfg = dict(QWEN3_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    L, S = cfg["num_hidden_layers"], args.prompt_len
    eng = Engine(cfg, dtype="bfloat16", random_seed=0, page_size=16, max_tokens=2 * S + 64, max_batch_tokens=S, max_seqs=2)
    eng.lookahead = False
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["vocab_size"], size=S).tolist()

    def once():
        rid = eng.add_request(prompt, 1, SamplingParams())
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        eng.step()
        ev1.record()
        torch.cuda.synchronize()
        eng.drain()
        for r in list(eng.scheduler.running):
            eng.scheduler.running.remove(r)
            eng.runner.release(r.rid)
            eng._samplers.pop(r.rid, None)
        return ev0.elapsed_time(ev1)

    def timed():
        return float(np.median([once() for _ in range(max(5, args.steps // 8))]))
    for _ in range(3):
        timed()
    whole = timed()
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    out = {"prompt_len": S, "layers": L, "ms_per_step": whole, "us_per_layer": whole / L * 1000, "marginal_us_per_layer": {},
           "marginal_us_per_step": {}}
    families = [("attention of the portion", "attention_prefill", None), ("qk_norm_rope_kv", "qk_norm_rope_kv", None),
                ("gate/up product", "linear_swiglu", None), ("row norms (+ owed sums)", "rmsnorm", None),
                ("qkv product", "linear", (qkv, H)), ("output product", "linear", (H, cfg["num_attention_heads"] * cfg["head_dim"])),
                ("down product", "linear", (H, I)), ("output head", "linear", (cfg["vocab_size"], H))]
    for label, fn_name, shape in families:
        real = getattr(ops, fn_name)
        if shape is None:
            setattr(ops, fn_name, lambda *a, **k: None)
        else:
            setattr(ops, fn_name, lambda a, w, *r, _real=real, _shape=shape, **k: None if tuple(w.shape) == _shape else _real(a, w, *r, **k))
        try:
            t = timed()
        finally:
            setattr(ops, fn_name, real)
        again = timed()
        per_step = ((whole + again) / 2 - t) * 1000
        whole = again
        key = "marginal_us_per_step" if label == "output head" else "marginal_us_per_layer"
        out[key][label] = per_step if label == "output head" else per_step / L
    out["ms_per_step_at_the_end"] = whole
    print(json.dumps(out))
    return 0


def _flat_config(name, cfg, n_layers, full_layers, **more):
    out = {"model": name, "layers": n_layers, "layers_of_config": full_layers, "hidden": cfg["hidden_size"],
           "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": 16,
           "parallelism": "single-gpu", "weights": "random N(0,0.02) bf16"}
    out.update(more)
    return out


def mixed_workload(args) -> int:
    """Qwen3-14B layer sizes: 32 requests, prompts U[128, 4096], portions of 512 beside decode tokens, 256 tokens each
    at temperature 0.7, context 8,192, all through the engine's own scheduler and entry point."""
    import numpy as np
    import torch
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.engine import roofline
    from rustingstrata_b200.sampling import SamplingParams
    cfg = dict(QWEN3_14B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_req, ctx, chunk, n_new = 32, 8192, 512, 256
    pk = roofline.peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    eng = Engine(cfg, dtype="bfloat16", random_seed=0, page_size=16, max_tokens=n_req * ctx, max_batch_tokens=chunk + n_req,
                 max_seqs=n_req, prefill_chunk=chunk)
    rng = np.random.default_rng(1)
    V = cfg["vocab_size"]

    def run(seed):
        lens = rng.integers(128, 4097, size=n_req)
        rids = [eng.add_request(rng.integers(0, V, size=int(n)).tolist(), n_new, SamplingParams(temp=0.7, seed=seed + i))
                for i, n in enumerate(lens)]
        first, steps = {}, []
        launch = eng._launch

        def spy(batch, prev):
            steps.append((sum(len(s.tokens) for s in batch if len(s.tokens) > 1 or s.request.prefilling),
                          sum(1 for s in batch if len(s.tokens) == 1 and not s.request.prefilling)))
            return launch(batch, prev)
        eng._launch = spy
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        generated = 0
        while eng.has_work():
            eng.step()
            now = time.perf_counter()
            for r in eng.scheduler.running:
                if r.generated and r.rid not in first:
                    first[r.rid] = now - t0
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        eng._launch = launch
        eng.runner.check_status()
        for rid in rids:
            first.setdefault(rid, wall)
        generated = n_req * n_new
        return wall, generated, int(lens.sum()), sorted(first.values()), steps

    run(100)                                   # warm-up: every kernel shape and graph of the workload has run once
    clocks = ClockSampler()
    clocks.start()
    wall, generated, prompt_tokens, ttft, steps = run(200)
    clk = clocks.stop()
    pre = [p for p, d in steps]
    dec = [d for p, d in steps]
    mix = {"steps": len(steps), "steps_with_prompt_tokens": sum(1 for p in pre if p), "steps_decode_only": sum(1 for p in pre if not p),
           "steps_mixed": sum(1 for p, d in steps if p and d), "prompt_tokens_per_step_mean": float(np.mean([p for p in pre if p] or [0])),
           "decode_tokens_per_step_mean": float(np.mean(dec)), "decode_tokens_per_step_max": int(max(dec))}
    rec = {"metric": "total generated tok/s, continuous batch of 32 (Qwen3-14B sizes, bf16, random weights)",
           "value": generated / wall, "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
           "data": "synthetic", "workload": "14b-mixed", "wall_s": wall, "generated_tokens": generated,
           "prompt_tokens": prompt_tokens, "all_tokens_per_s": (generated + prompt_tokens) / wall,
           "ttft_s": {"mean": float(np.mean(ttft)), "max": float(ttft[-1]), "min": float(ttft[0])},
           "step_mix": mix, "preemptions": eng.scheduler.preemptions,
           "config": _flat_config("qwen3-14b-sizes", cfg, cfg["num_hidden_layers"], full_layers, requests=n_req, seq_len=ctx,
                                  prompt_len="U[128,4096]", chunk=chunk, new_tokens=n_new, temperature=0.7,
                                  peaks=pk["source"]),
           "clocks": clk}
    print(json.dumps(rec))
    return 0


def long_context_workload(args) -> int:
    """Qwen3-32B layer sizes: 8 requests with 12,000-token prompts, then 256 greedy tokens each, context 16,384."""
    import numpy as np
    import torch
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.engine import roofline
    from rustingstrata_b200.sampling import SamplingParams
    cfg = dict(QWEN3_32B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_req, ctx, prompt, n_new = 8, 16384, 12000, 256
    pk = roofline.peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    eng = Engine(cfg, dtype="bfloat16", random_seed=0, page_size=16, max_tokens=n_req * ctx, max_batch_tokens=2048,
                 max_seqs=n_req)
    runner = eng.runner
    rng = np.random.default_rng(2)
    V = cfg["vocab_size"]

    def prefill(n_tokens):
        for _ in range(n_req):
            eng.add_request(rng.integers(0, V, size=n_tokens).tolist(), ctx - n_tokens, SamplingParams())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while eng.scheduler.waiting or any(r.prefilling for r in eng.scheduler.running):
            eng.step()
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    def finish_all():
        eng.drain()
        for r in list(eng.scheduler.running):
            eng.scheduler.running.remove(r)
            runner.release(r.rid)
            eng._samplers.pop(r.rid, None)

    # the same decode step with next to no cache: what is left of the step when attention has nothing to read
    prefill(16)
    short_ms = eng.decode_steps_device_timed(64, warmup=8)
    finish_all()
    clocks = ClockSampler()
    clocks.start()
    prefill_s = prefill(prompt)
    for _ in range(args.warmup):
        eng.step()
    kv0 = sum(runner.length(r.rid) for r in eng.scheduler.running)
    steps = n_new - args.warmup - 8
    ms = eng.decode_steps_device_timed(steps, warmup=3)
    kv1 = sum(runner.length(r.rid) for r in eng.scheduler.running)
    clk = clocks.stop()
    runner.check_status()
    roof = roofline.decode_roofline(runner.model, runner.kv_bytes_per_token, (kv0 + kv1) / 2.0, ms, pk)
    kv_bytes = (kv0 + kv1) / 2.0 * runner.kv_bytes_per_token
    rec = {"metric": "decode tok/s at batch 8 after 12,000-token prompts (Qwen3-32B sizes, bf16, random weights)",
           "value": n_req / ms * 1000, "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
           "data": "synthetic", "workload": "32b-long", "steps": steps, "ms_per_step": ms,
           "roofline": {k: roof[k] for k in ("bound", "achieved", "peak", "unit", "frac")},
           "kv_share_of_bytes": kv_bytes / roof["bytes_per_step"],
           "ms_per_step_at_16_keys": short_ms, "long_cache_share_of_step": (ms - short_ms) / ms,
           "long_cache_gbs": kv_bytes / ((ms - short_ms) / 1000) / 1e9 if ms > short_ms else None,
           "prefill": {"tokens": n_req * prompt, "s": prefill_s, "value": n_req * prompt / prefill_s},
           "config": _flat_config("qwen3-32b-sizes", cfg, cfg["num_hidden_layers"], full_layers, global_batch=n_req,
                                  seq_len=ctx, prompt_len=prompt, new_tokens=n_new, peaks=pk["source"]),
           "clocks": clk}
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
