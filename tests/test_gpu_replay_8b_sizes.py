"""Trace replay at the layer sizes of Qwen3-8B (2 of its 36 layers), against the plain implementation.

The widths are the real ones - hidden 4,096, 32 query heads on 8 key/value heads of 128, feed-forward 12,288,
vocabulary 151,936, untied head, pages of 16 - so that the kernels run in the shapes the benchmark times: the
tiled tcgen05 product and the tcgen05 attention on portions of more than 128 tokens, the stream-K tcgen05 product
on portions of 9 to 128, the few-rows product and the TMA-fed decode attention on single tokens, the output head
over 151,936 rows, and captured decode steps on both sides of 1,024 and of 2,048 keys.  Only the depth is cut (2
layers, named here and in the configuration below): a full-depth model would take the plain implementation
minutes per request.

The weights are drawn on the device from a seed (``trace_run --random-config``); the test draws the same values
with the same generator for the plain side (``tests/test_random_weights.py`` shows host and device agree to the
bit).  The plain side is ``plain_qwen3``: float64, whole sequences, no cache; the matrices stay float32 in memory
and are widened one at a time where they are used.  All of a row's 151,936 logits are compared.
"""
import random

import numpy as np
import pytest

import plain_qwen3 as P
from helpers import TOL, random_tokens, run_trace

pytestmark = pytest.mark.gpu

LAYERS, LAYERS_OF_MODEL = 2, 36
CONFIG = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
          "num_hidden_layers": LAYERS, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
          "intermediate_size": 12288, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 40960,
          "tie_word_embeddings": False, "use_sliding_window": False, "torch_dtype": "bfloat16"}
SEED, STD, PAGE = 7, 0.02, 16
LENGTHS = {"a": 2070, "b": 1045, "c": 300, "d": 150}       # a's and b's last 32 tokens cross 2,048 and 1,024 keys
PORTIONS = [150, 9, 2, 128, 33, 2, 64, 200, 17, 5, 100, 3]


def round64(n):
    return (n + 63) // 64 * 64


def drawn_weights():
    """name → float32 array, drawn on the device by the engine's generator (bfloat16 values) and copied back."""
    import torch
    from rustingstrata_b200.kernels import ops
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.weights.random_init import normal_table, scale_shift, tensor_key
    table = torch.from_numpy(normal_table().copy()).cuda()
    out = {}
    for name, need in manifest_for(CONFIG).items():
        scale, shift = scale_shift(need, STD, 0.0)
        t = torch.empty(need.shape, dtype=torch.bfloat16, device="cuda")
        ops.fill_random(t, tensor_key(SEED, name), table, scale, shift)
        out[name] = t.float().cpu().numpy()
        del t
    torch.cuda.empty_cache()
    return out


def plain_rows(w, tokens, rows):
    """float64 logits of the whole sequence at ``rows`` (the layers run on every position, the head on these)."""
    cfg = CONFIG
    positions = np.arange(len(tokens))
    x = P.embed(tokens, w).astype(np.float64)
    for il in range(cfg["num_hidden_layers"]):
        x = P.block(x, w, il, cfg, positions, None)
    return P.head(x[np.asarray(rows)], w, cfg)


class Trace:
    def __init__(self):
        self.steps, self.rows = [], {}

    def add(self, entries, end=()):
        k = len(self.steps)
        self.steps.append({"step": k, "entries": [{"id": r, "tokens": t, "want": list(wt)} for r, _, t, wt in entries],
                           "end": list(end)})
        rows = [(r, s + i) for r, s, _, wt in entries for i in wt]
        if rows:
            self.rows[k] = rows


def build(tokens):
    tr, parts = Trace(), {}
    wanted = {r: set() for r in tokens}

    def want(rid, start, n, places):
        places = [p for p in places if 0 <= p < n]
        wanted[rid].update(start + p for p in places)
        return places
    # 1. whole: the first rows, the rows around the tile edges of the kernels, and the last rows
    s0 = 0
    for rid, t in tokens.items():
        n = len(t)
        places = sorted({0, 1, 2, 15, 16, 127, 128, 129, n // 2, n - 3, n - 2, n - 1})
        tr.add([(rid, 0, t, want(rid, 0, n, places))], end=[rid])
    parts["whole"] = range(s0, len(tr.steps))
    # 2. most of it in one step, the last 32 one by one (captured decode steps; a crosses 2,048 keys, b 1,024)
    s0 = len(tr.steps)
    for rid, t in tokens.items():
        n = len(t) - 32
        tr.add([(rid, 0, t[:n], want(rid, 0, n, [n - 1]))])
        for i in range(n, len(t)):
            tr.add([(rid, i, [t[i]], want(rid, i, 1, [0]))], end=[rid] if i == len(t) - 1 else [])
    parts["tail32"] = range(s0, len(tr.steps))
    # 3. portions of changing size: above 128 tokens, 9 to 128, and down to two
    s0 = len(tr.steps)
    for rid, t in tokens.items():
        pos = k = 0
        while pos < len(t):
            n = min(PORTIONS[k % len(PORTIONS)], len(t) - pos)
            k += 1
            tr.add([(rid, pos, t[pos:pos + n], want(rid, pos, n, [0, n - 1]))], end=[rid] if pos + n == len(t) else [])
            pos += n
    parts["portions"] = range(s0, len(tr.steps))
    # 4. mixed: every request twice (a second copy under another name, so that eight requests pass through), up to
    #    four live, portions of some beside single tokens of others, in a pool that holds less than half of them
    s0 = len(tr.steps)
    rng = random.Random(99)
    copies = {f"{rid}{j}": rid for j in (1, 2) for rid in tokens}
    pool = round64(LENGTHS["a"]) + round64(LENGTHS["b"]) + round64(LENGTHS["c"]) + round64(LENGTHS["d"])
    waiting, live, pos, held, peak = list(copies), [], {}, 0, 0
    while waiting or live:
        for name in list(waiting):
            if len(live) < 4 and held + round64(len(tokens[copies[name]])) <= pool:
                waiting.remove(name)
                live.append(name)
                pos[name] = 0
                held += round64(len(tokens[copies[name]]))
        peak = max(peak, held)
        chosen = [r for r in live if rng.random() < 0.8] or [live[0]]
        entries, ended = [], []
        for name in chosen:
            rid = copies[name]
            t = tokens[rid]
            left = len(t) - pos[name]
            single = left <= 12
            n = 1 if single else min(rng.choice([2, 7, 40, 130, 300, 700]), left - 12)
            places = want(rid, pos[name], n, [0] if single else rng.choice([[n - 1], [0, n - 1], []]))
            entries.append((name, pos[name], t[pos[name]:pos[name] + n], places))
            pos[name] += n
            if pos[name] == len(t):
                ended.append(name)
        tr.add(entries, end=ended)
        for name in ended:
            live.remove(name)
            held -= round64(len(tokens[copies[name]]))
    parts["mixed"] = range(s0, len(tr.steps))
    # rows of the mixed cutting are named by the copy: map them back to the request
    for k in parts["mixed"]:
        if k in tr.rows:
            tr.rows[k] = [(copies[name], p) for name, p in tr.rows[k]]
    return tr, parts, pool, {r: sorted(v) for r, v in wanted.items()}


_STATE = {}


def state():
    if not _STATE:
        tokens = {rid: random_tokens(CONFIG["vocab_size"], n, 500 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
        tr, parts, pool, wanted = build(tokens)
        w = drawn_weights()
        ref = {}
        for rid, t in tokens.items():
            rows = wanted[rid]
            logits = plain_rows(w, t, rows)
            ref[rid] = ({p: logits[i] for i, p in enumerate(rows)}, float(np.max(np.abs(logits))))
        del w
        _STATE.update(tokens=tokens, trace=tr, parts=parts, pool=pool, ref=ref, got={})
    return _STATE


def replay(dtype):
    st = state()
    if dtype not in st["got"]:
        st["got"][dtype] = run_trace(None, dtype, st["trace"].steps, st["pool"], page_size=PAGE, timeout=1500,
                                     random_config=CONFIG, weights_seed=SEED, weights_std=STD)
    return st["got"][dtype]


@pytest.mark.parametrize("cutting", ["whole", "tail32", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_at_8b_layer_sizes_matches_plain(dtype, cutting):
    st = state()
    got = replay(dtype)
    tr = st["trace"]
    worst, n_rows, wrong_argmax = (0.0, None), 0, 0
    for k in st["parts"][cutting]:
        if k not in tr.rows:
            continue
        assert got[k].shape == (len(tr.rows[k]), CONFIG["vocab_size"])
        for row, (rid, p) in zip(got[k], tr.rows[k]):
            ref, scale = st["ref"][rid]
            err = float(np.max(np.abs(row.astype(np.float64) - ref[p])) / scale)
            n_rows += 1
            wrong_argmax += int(np.argmax(row) != np.argmax(ref[p]))
            if err > worst[0]:
                worst = (err, (k, rid, p))
            assert err <= TOL[dtype], (f"{LAYERS} of {LAYERS_OF_MODEL} layers, {dtype}, {cutting}: step {k} request {rid} "
                                       f"position {p}: error {err:.3e}")
    assert n_rows >= 40
    if dtype == "float32":
        assert wrong_argmax == 0
    print(f"8B layer sizes ({LAYERS} of {LAYERS_OF_MODEL} layers) {dtype} {cutting}: {n_rows} rows, worst {worst[0]:.3e} "
          f"at {worst[1]}, arg-max differs in {wrong_argmax}")


def test_the_mixed_cutting_at_8b_sizes_used_pages_again():
    st = state()
    got = replay("float32")
    assert 2 * st["pool"] <= 2 * sum(round64(n) for n in LENGTHS.values())
    for pool in got.pools:
        assert pool["reuses"] > 0 and pool["allocations"] > pool["pages"] and pool["held_at_end"] == 0, pool


def test_a_whole_prompt_gives_the_same_bits_whatever_ran_before():
    """At the layer sizes of Qwen3-8B (2 layers, a smaller vocabulary): a prompt run whole, again and again, between
    other prompts that leave other keys and values in the pages it is given.  The logits of its first run equal those
    of the later ones to the bit.  A kernel that reads what the step itself has not finished writing (a wait that
    lets it through too early) shows here: the first run then sees the other prompt's leftovers, the later ones see
    a copy of what they are about to write."""
    import torch
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.engine import StepEntry
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 4096, "hidden_size": 4096,
           "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
           "intermediate_size": 12288, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 40960,
           "tie_word_embeddings": False, "use_sliding_window": False, "torch_dtype": "bfloat16"}
    eng = Engine(cfg, dtype="bfloat16", random_seed=7, max_tokens=4096, max_batch_tokens=2304)
    rng = np.random.default_rng(1)
    for n in (1045, 300, 150, 300, 2070, 300):
        toks = rng.integers(0, cfg["vocab_size"], n).tolist()
        places = sorted({0, 1, 127, 128, 129, n // 2, n - 2, n - 1})
        first = None
        for _ in range(3):
            rows = eng.step_raw([StepEntry("x", toks, places)]).float().cpu()
            eng.release("x")
            if first is None:
                first = rows
            assert torch.equal(rows, first), f"{n} tokens: a later run differs from the first"
        assert torch.isfinite(first).all()
    eng.runner.check_status()
