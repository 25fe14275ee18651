"""What a step has to move and to compute, against the device's peaks.

The reference's bench prints tokens per second and keeps per-step host timings
(src/main.rs:792-840,1192-1265; src/gpu_model.rs:1416-1434); its kernel tests report
achieved bandwidth (tests/kernels.rs:271-331).  Here every timed run can be set
against a roofline: a decode step is bound by the bytes it must read (every weight it
uses once, and the cache of the live requests), a prompt step by its multiply-adds on
the tensor cores.  The counts come from the model's parts, not from an architecture's
formula, so they hold for any arrangement of parts.

Peaks: ``MEASURED_PEAKS.json`` (keys ``hbm_gbs``, ``bf16_tflops``,
``bf16_tflops_sustained``) in the working directory or beside the package, if a
measurement of this machine was left there; else the figures of an earlier measurement
of the same kind of device, marked "fallback".
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Sequence

import numpy as np

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
_PKG_PARENT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks(path: Optional[str] = None) -> Dict:
    cands = [path] if path else [os.path.join(os.getcwd(), "MEASURED_PEAKS.json"), os.path.join(_PKG_PARENT, "MEASURED_PEAKS.json")]
    for p in cands:
        if p and os.path.isfile(p):
            try:
                with open(p) as f:
                    d = json.load(f)
            except (OSError, ValueError):
                continue
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
    return dict(FALLBACK_PEAKS, source="fallback")


def _tensors(part):
    for v in vars(part).values():
        if hasattr(v, "data_ptr") and hasattr(v, "element_size") and v.dim() >= 1:
            yield v


def weight_bytes(model) -> int:
    """Bytes of every weight one step reads once: all tensors of all parts, each once; the token table only when it is
    also the output head (a step gathers a few rows of it otherwise)."""
    seen, total = set(), 0
    head_ptrs = {t.data_ptr() for t in _tensors(model.head)}
    for part in model.parts():
        for t in _tensors(part):
            if part is model.embedding and t.data_ptr() not in head_ptrs:
                continue
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def flops_per_token(model) -> float:
    """Multiply-add flops of the projections one token passes through: twice the elements of every matrix of every
    part between the embedding and the head, once per time its layer is in the run order."""
    def of_block(b):
        n = 0
        for p in b.parts.values():
            n += sum(2 * t.numel() for t in _tensors(p) if t.dim() == 2)
        return n
    return float(sum(of_block(model.blocks[c.layer]) for c in model.calls))


def head_flops_per_row(model) -> float:
    return float(sum(2 * t.numel() for t in _tensors(model.head) if t.dim() == 2))


def mixing_flops(model, q_lens: Sequence[int], kv_lens: Sequence[int]) -> float:
    """Flops the mixers spend on looking at other tokens (attention scores and weighted sums), as each mixer counts them
    itself (``Mixer.mixing_flops``; a mixer that says nothing counts as none)."""
    total = 0.0
    for c in model.calls:
        for m in model.blocks[c.layer].mixers().values():
            fn = getattr(m, "mixing_flops", None)
            if fn is not None:
                total += float(fn(np.asarray(q_lens), np.asarray(kv_lens)))
    return total


def step_flops(model, q_lens: Sequence[int], kv_lens: Sequence[int], n_logit_rows: int) -> float:
    return (flops_per_token(model) * float(np.sum(q_lens)) + mixing_flops(model, q_lens, kv_lens)
            + head_flops_per_row(model) * n_logit_rows)


def decode_roofline(model, kv_bytes_per_token: int, kv_tokens: float, ms_per_step: float, pk: Optional[Dict] = None) -> Dict:
    """The decode step as a stream of bytes: weights once plus the live requests' cache, over the measured time."""
    pk = pk or peaks()
    nbytes = weight_bytes(model) + kv_tokens * kv_bytes_per_token
    achieved = nbytes / (ms_per_step / 1000) / 1e9
    return {"bound": "hbm", "bytes_per_step": int(nbytes), "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}


def prefill_roofline(model, q_lens, kv_lens, n_logit_rows: int, ms: float, pk: Optional[Dict] = None,
                     dtype: str = "bfloat16") -> Dict:
    """A prompt step as multiply-adds on the tensor cores (the 32-bit engine runs on CUDA cores; its fraction of the
    bfloat16 tensor peak is given all the same, for scale)."""
    pk = pk or peaks()
    flops = step_flops(model, q_lens, kv_lens, n_logit_rows)
    achieved = flops / (ms / 1000) / 1e12
    return {"bound": "tensor", "flops": flops, "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
            "frac": achieved / pk["bf16_tflops"], "peaks": pk["source"], "dtype": dtype}
