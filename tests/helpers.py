"""Shared helpers of the test suite: the tiny configurations, model folders, trace replay, error measure."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations of the architecture that differ in every size and option, a third with sizes that
# are no power of two anywhere (head size 48, 5 query heads on 1 kv head, odd widths), and a fourth whose
# head size, group and page size are ones the tcgen05/TMA attention kernels take, so that those kernels
# (and not only their CUDA-core stand-ins) run inside the engine under test.
TINY = {
    "A": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 256, "hidden_size": 64,
                "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
                "intermediate_size": 160, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
                "max_position_embeddings": 384, "tie_word_embeddings": True, "use_sliding_window": False,
                "torch_dtype": "bfloat16"},
        seed=0, std=0.08, norm_std=0.0, page_size=4),
    "B": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 515, "hidden_size": 96,
                "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
                "intermediate_size": 250, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
                "max_position_embeddings": 512, "tie_word_embeddings": False, "use_sliding_window": True,
                "sliding_window": 24, "layer_types": ["full_attention", "sliding_attention", "full_attention"],
                "torch_dtype": "bfloat16"},
        seed=1, std=0.08, norm_std=0.1, page_size=16),
    "C": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 301, "hidden_size": 80,
                "num_hidden_layers": 2, "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48,
                "intermediate_size": 136, "rms_norm_eps": 3e-6, "rope_theta": 50000.0,
                "max_position_embeddings": 320, "tie_word_embeddings": False, "use_sliding_window": True,
                "sliding_window": 40, "max_window_layers": 1, "torch_dtype": "bfloat16"},
        seed=2, std=0.1, norm_std=0.05, page_size=8),
    "D": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 777, "hidden_size": 128,
                "num_hidden_layers": 3, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64,
                "intermediate_size": 328, "rms_norm_eps": 2e-6, "rope_theta": 500000.0,
                "max_position_embeddings": 640, "tie_word_embeddings": False, "use_sliding_window": True,
                "sliding_window": 150, "layer_types": ["full_attention", "sliding_attention", "full_attention"],
                "torch_dtype": "bfloat16"},
        seed=3, std=0.06, norm_std=0.05, page_size=16),
    # head size 128 with four query heads on one kv head (the benchmark model's head shape) and room for thousands
    # of positions: long sequences inside the engine, attention splits counted in dozens
    "E": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 1000, "hidden_size": 256,
                "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128,
                "intermediate_size": 384, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
                "max_position_embeddings": 4096, "tie_word_embeddings": False, "use_sliding_window": False,
                "torch_dtype": "bfloat16"},
        seed=4, std=0.05, norm_std=0.05, page_size=16),
}

# Tolerances, as max |difference| / max |reference logit| over the compared rows.  The 32-bit engine
# differs from the float64 plain implementation by float32 rounding only; the bfloat16 engine rounds
# activations, cache and projections to 8 bits of mantissa (2^-8 = 3.9e-3 per rounding).
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def make_model_dir(path: str, name: str) -> str:
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.weights import write_random_model
    t = TINY[name]
    write_random_model(path, t["config"], manifest_for(t["config"]), t["seed"], std=t["std"], norm_std=t["norm_std"])
    return path


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - ref)) / np.max(np.abs(ref)))


def random_tokens(vocab: int, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


class TraceResult(dict):
    """{step: float32 array [wanted, vocab]}; ``pools``: what trace_run reported about each page pool at its end."""
    pools: list


def run_trace(model_dir: str, dtype: str, steps, max_tokens: int, page_size: int = 16, timeout: int = 600,
              random_config=None, weights_seed: int = 0, weights_std: float = 0.02, weights_norm_std: float = 0.0):
    """Runs bin/trace_run on ``steps`` (list of dicts) and returns the logits it wrote, per step.  ``model_dir`` is a
    model folder, or None with ``random_config`` (a config mapping) for weights drawn on the device."""
    import re
    import shutil
    out = tempfile.mkdtemp(prefix="trace_out_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--dtype", dtype, "--out", out,
           "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    if model_dir is not None:
        cmd += ["--model", model_dir]
        with open(os.path.join(model_dir, "config.json")) as f:
            vocab = json.load(f)["vocab_size"]
    else:
        cfg_path = os.path.join(out, "random_config.json")
        with open(cfg_path, "w") as f:
            json.dump(dict(random_config), f)
        cmd += ["--random-config", cfg_path, "--weights-seed", str(weights_seed), "--weights-std", str(weights_std),
                "--weights-norm-std", str(weights_norm_std)]
        vocab = random_config["vocab_size"]
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    if r.returncode != 0:
        shutil.rmtree(out, ignore_errors=True)
        raise RuntimeError(f"trace_run failed ({r.returncode}):\n{r.stderr[-4000:]}")
    done = [ln for ln in r.stdout.splitlines() if ln.startswith("done ")]
    assert [ln.split()[1] for ln in done] == [str(s["step"]) for s in steps], "trace_run did not acknowledge every step"
    res = TraceResult()
    res.pools = [{k: int(v) for k, v in re.findall(r"(pages|allocations|reuses|held_at_end) (\d+)", ln)}
                 for ln in r.stderr.splitlines() if ln.startswith("[trace_run] pool ")]
    for s in steps:
        p = os.path.join(out, f"{s['step']}.f32")
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        if wanted:
            res[s["step"]] = np.fromfile(p, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not os.path.exists(p), f"step {s['step']} wanted nothing but wrote a file"
    shutil.rmtree(out, ignore_errors=True)
    return res
