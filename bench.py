#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B sizes with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 (a "step" is one
decode step of the whole batch, timed on the device with CUDA events); ``e2e`` is the
same through the Python entry point with host token ids in and out every step;
``prefill`` is one 2,048-token prompt; ``roofline`` relates the decode step's bytes
(every weight it uses once plus the cache of the live requests) to the HBM peak;
``points`` holds decode at batch 1 and 64.  Peaks come from MEASURED_PEAKS.json beside
this file when present, else from the fallback figures of this pool.

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
CONTEXT = 4096          # tokens per request the cache is sized for
PROMPT = 2048           # tokens each request holds before decoding is timed
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


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


def weight_bytes(runner) -> int:
    """Bytes of every weight one decode step reads once (the token table only through the rows it gathers)."""
    seen, total = set(), 0
    for part in runner.model.parts():
        for v in vars(part).values():
            if hasattr(v, "data_ptr") and hasattr(v, "element_size") and v.data_ptr() not in seen and v.dim() >= 1:
                if part is runner.model.embedding and part.weight is not runner.model.head.weight:
                    continue
                seen.add(v.data_ptr())
                total += v.numel() * v.element_size()
    return total


def step_flops(cfg, n_layers, tokens, kv_tokens_sum) -> float:
    """Multiply-add flops of a step: projections of every token, causal attention, the head on one row."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_tok = 2 * (H * (q + 2 * kv) + q * H + 3 * H * I)
    attn = 4 * q * kv_tokens_sum
    return n_layers * (per_tok * tokens + attn) + 2 * H * cfg["vocab_size"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run this many of the configuration's layers (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
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

    import numpy as np
    import torch
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.kernels import ops
    from rustingstrata_b200.sampling import SamplingParams

    pk = peaks()
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
    wbytes = weight_bytes(runner)
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
    pf_flops = step_flops(cfg, n_layers, PROMPT, PROMPT * (PROMPT + 1) / 2)
    prefill = {"value": PROMPT / prefill_ms * 1000, "tokens": PROMPT, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1000) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode at the headline batch
    ms, e2e_ms, launches, kv_tokens = time_decode(args.batch, args.steps, args.warmup)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _, _ = time_decode(b, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = b / pms * 1000
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
        "clocks": clk,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
