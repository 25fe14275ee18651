"""The command line, run as a user runs it (``python -m rustingstrata_b200 <subcommand>``), on a tiny model:
init-random, generate, score, bench and replay, compared with the plain implementation where they print numbers.
Reference manner of the subcommands: src/main.rs:1085-1155 (generate), :1050-1084 (score), :1192-1265 (bench)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen3 as P
from helpers import ROOT, TINY, random_tokens

pytestmark = pytest.mark.gpu


def cli(*args, stdin=None, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "rustingstrata_b200", *map(str, args)], input=stdin, capture_output=True,
                       text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, f"{args}: exit {r.returncode}\n{r.stderr[-3000:]}"
    return r.stdout, r.stderr


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    """A model folder written by ``init-random`` from Tiny B's configuration."""
    base = tmp_path_factory.mktemp("cli")
    t = TINY["B"]
    cfg_path = base / "config.json"
    cfg_path.write_text(json.dumps(t["config"]))
    out, _ = cli("init-random", "--config", cfg_path, "--out", base / "model", "--seed", t["seed"], "--std", t["std"],
                 "--norm-std", t["norm_std"])
    assert out.strip() == str(base / "model")
    assert sorted(os.listdir(base / "model")) == ["config.json", "model.safetensors"]
    return str(base / "model"), str(cfg_path)


def test_init_random_writes_the_model_the_library_call_writes(folder, tiny_models):
    a = open(os.path.join(folder[0], "model.safetensors"), "rb").read()
    b = open(os.path.join(tiny_models["B"], "model.safetensors"), "rb").read()
    assert a == b


def test_generate_greedy_equals_the_plain_implementation(folder):
    cfg, w = P.read_model(folder[0])
    prompt = random_tokens(cfg["vocab_size"], 23, 8)
    out, err = cli("generate", "--model", folder[0], "--dtype", "fp32", "--prompt", ",".join(map(str, prompt)), "-n", 9,
                   "--ctx", 256)
    assert [int(t) for t in out.split()] == P.greedy_generate(cfg, w, prompt, 9)
    assert err.strip().splitlines()[-1].startswith("prompt 23 tok ") and " | gen 9 tok " in err      # the reference's line
    # ids on standard input, an end-of-sequence id that stops the generation early
    want = P.greedy_generate(cfg, w, prompt, 9)
    out, _ = cli("generate", "--model", folder[0], "--dtype", "float32", "--prompt", "-", "-n", 9, "--ctx", 256, "--eos", want[4],
                 stdin=" ".join(map(str, prompt)))
    assert [int(t) for t in out.split()] == want[:want.index(want[4])]


def test_generate_with_random_weights_and_sampling_options(folder):
    # no folder: the model is drawn on the device from the configuration and a seed; the same seed gives the same tokens
    args = ("generate", "--random-weights", "--config", folder[1], "--weights-seed", 5, "--prompt-len", 30, "-n", 6, "--ctx", 256,
            "--temp", 0.9, "--top-k", 20, "--top-p", 0.95, "--seed", 3, "--repeat-penalty", 1.1)
    a, _ = cli(*args)
    b, _ = cli(*args)
    assert a == b and len(a.split()) == 6 and all(0 <= int(t) < 515 for t in a.split())
    c, _ = cli(*args[:-2], "--seed", 4, "--repeat-penalty", 1.1)
    assert len(c.split()) == 6
    # the folder written from the same seed is the same model: greedy tokens agree between the two ways
    t = TINY["B"]
    g1, _ = cli("generate", "--model", folder[0], "--dtype", "fp32", "--prompt-len", 12, "-n", 5, "--ctx", 256)
    g2, _ = cli("generate", "--random-weights", "--config", folder[1], "--weights-seed", t["seed"], "--weights-std", t["std"],
                "--weights-norm-std", t["norm_std"], "--dtype", "fp32", "--prompt-len", 12, "-n", 5, "--ctx", 256)
    assert g1 == g2


def test_score_gives_argmax_and_top5_log_probabilities(folder):
    cfg, w = P.read_model(folder[0])
    prompt, cont = random_tokens(cfg["vocab_size"], 17, 1), random_tokens(cfg["vocab_size"], 6, 2)
    out, _ = cli("score", "--model", folder[0], "--dtype", "fp32", "--ctx", 256, stdin=json.dumps({"prompt": prompt, "continuation": cont}))
    rec = json.loads(out)
    logits = P.forward_logits(cfg, w, prompt + cont)[len(prompt) - 1: len(prompt) + len(cont) - 1]
    lp = logits - np.log(np.exp(logits - logits.max(1, keepdims=True)).sum(1, keepdims=True)) - logits.max(1, keepdims=True)
    assert len(rec["argmax"]) == len(rec["top5"]) == len(cont)
    assert rec["argmax"] == [int(i) for i in np.argmax(logits, axis=1)]
    for k, row in enumerate(rec["top5"]):
        ids = [i for i, _ in row]
        assert ids == [int(i) for i in np.argsort(-lp[k], kind="stable")[:5]]
        assert np.allclose([v for _, v in row], lp[k][ids], atol=2e-5)


def test_bench_prints_the_reference_line_and_a_record(folder, tmp_path):
    rec_path = tmp_path / "bench.json"
    out, _ = cli("bench", "--model", folder[0], "--pp", "20,130", "--tg", 6, "--reps", 2, "--batch", 2, "--json-out", rec_path)
    lines = [ln for ln in out.splitlines() if ln.startswith("pp ")]
    assert len(lines) == 2 and "prefill" in lines[0] and "| tg 6: decode" in lines[0] and "tok/s" in lines[0]
    rec = json.loads(rec_path.read_text())
    assert rec["schema"] == "rustingstrata_b200.bench.v1" and rec["tg"] == 6 and rec["reps"] == 2
    assert [r["pp"] for r in rec["results"]] == [20, 130]
    for r in rec["results"]:
        assert r["batch"] == 2
        for k in ("prefill_tok_s", "decode_tok_s"):
            assert 0 < r[k]["min"] <= r[k]["mean"] <= r[k]["max"]
        # what the step had to move and to compute, against the device's peaks
        roof = r["roofline"]
        assert roof["decode"]["bound"] == "hbm" and roof["decode"]["bytes_per_step"] > 0 and 0 < roof["decode"]["frac"] < 1.5
        assert roof["prefill"]["bound"] == "tensor" and roof["prefill"]["flops"] > 0 and 0 < roof["prefill"]["frac"] < 1.5


def test_replay_subcommand_is_trace_run(folder, tmp_path):
    cfg, w = P.read_model(folder[0])
    toks = random_tokens(cfg["vocab_size"], 12, 4)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:], "want": [0, 4]}], "end": ["a"]}]
    out, err = cli("replay", "--model", folder[0], "--dtype", "float32", "--out", tmp_path / "o", "--max-tokens", 64,
                   stdin="".join(json.dumps(s) + "\n" for s in steps))
    assert out.split() == ["done", "0", "done", "1"] and "reuses" in err
    ref = P.forward_logits(cfg, w, toks)
    got = np.fromfile(tmp_path / "o" / "1.f32", dtype="<f4").reshape(2, -1)
    assert np.max(np.abs(got - ref[[7, 11]])) / np.max(np.abs(ref)) < 1e-5
