"""The two tiny workloads exactly as the benchmark description states them (the other tests use variants of
them that are harder on the kernels: wider weights so that logits spread, sizes that are no power of two, a
sliding-window layer, longer sequences).

Tiny A: 2 layers, hidden 64, 4 query heads on 2 key/value heads of 16, feed-forward 160, vocabulary 256,
rope_theta 10,000, eps 1e-6, tied embeddings, full attention, 128 positions; weights N(0, 0.02) from seed 0, norm
weights 1.0; pages of 4; four requests with prompts of 1, 7, 16 and 33 tokens, 8 greedy tokens each; run with whole
prompts, token by token, in portions of 5 tokens, and as one mixed batch.

Tiny B: 3 layers, hidden 96, 6 query heads on 2 key/value heads of 32 (query width 192), feed-forward 256,
vocabulary 512, rope_theta 1,000,000, eps 1e-5, untied head, full attention, 256 positions; weights N(0, 0.02) from
seed 1, norm weights 1 + N(0, 0.1); pages of 16; six requests with prompts of 3 to 120 tokens arriving over time,
12 tokens each at temperature 0.8 from fixed sampler seeds.
"""
import numpy as np
import pytest

import plain_qwen3 as P
from helpers import TOL, random_tokens

pytestmark = pytest.mark.gpu

STATED = {
    "A": dict(config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 256, "hidden_size": 64,
                      "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
                      "intermediate_size": 160, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 128,
                      "tie_word_embeddings": True, "use_sliding_window": False, "torch_dtype": "bfloat16"},
              seed=0, std=0.02, norm_std=0.0, page_size=4),
    "B": dict(config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 512, "hidden_size": 96,
                      "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
                      "intermediate_size": 256, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "max_position_embeddings": 256,
                      "tie_word_embeddings": False, "use_sliding_window": False, "torch_dtype": "bfloat16"},
              seed=1, std=0.02, norm_std=0.1, page_size=16),
}


@pytest.fixture(scope="module")
def stated_models(tmp_path_factory):
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.weights import write_random_model
    base = tmp_path_factory.mktemp("stated")
    out = {}
    for name, t in STATED.items():
        out[name] = str(base / name)
        write_random_model(out[name], t["config"], manifest_for(t["config"]), t["seed"], std=t["std"], norm_std=t["norm_std"])
    return out


def engine(stated_models, name, dtype, **kw):
    from rustingstrata_b200 import Engine
    kw.setdefault("max_tokens", 512)
    kw.setdefault("max_batch_tokens", 128)
    kw.setdefault("max_seqs", 8)
    return Engine(stated_models[name], dtype=dtype, page_size=STATED[name]["page_size"], **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_a_as_stated_in_every_cutting(stated_models, dtype):
    from rustingstrata_b200.engine import StepEntry
    cfg, w = P.read_model(stated_models["A"])
    prompts = [random_tokens(256, n, 900 + n) for n in (1, 7, 16, 33)]
    want = [P.greedy_generate(cfg, w, p, 8) for p in prompts]
    full = [p + g for p, g in zip(prompts, want)]
    ref = [P.forward_logits(cfg, w, t) for t in full]

    # generation through the entry point: the four requests as one mixed batch (prompts beside decoding requests)
    eng = engine(stated_models, "A", dtype, max_batch_tokens=24, prefill_chunk=5)
    outs = eng.generate(prompts, max_new_tokens=8)
    if dtype == "float32":
        assert outs == want
    eng = engine(stated_models, "A", dtype)
    # teacher-forced logits of prompt + the plain continuation, cut three ways
    def check(rows, i, first):
        err = np.max(np.abs(rows - ref[i][first:first + len(rows)])) / np.max(np.abs(ref[i]))
        assert err <= TOL[dtype], f"request {i} from {first}: {err:.3e}"
    for i, t in enumerate(full):                              # whole
        check(eng.step_raw([StepEntry(("w", i), t, list(range(len(t))))]).cpu().numpy(), i, 0)
        eng.release(("w", i))
    for i, t in enumerate(full):                              # token by token
        for k, tok in enumerate(t):
            check(eng.step_raw([StepEntry(("t", i), [tok], [0])]).cpu().numpy(), i, k)
        eng.release(("t", i))
    for i, t in enumerate(full):                              # portions of 5
        for a in range(0, len(t), 5):
            n = min(5, len(t) - a)
            check(eng.step_raw([StepEntry(("c", i), t[a:a + n], list(range(n)))]).cpu().numpy(), i, a)
        eng.release(("c", i))
    # one mixed batch per step: all four requests together, each advancing by its own stride
    pos, strides = [0, 0, 0, 0], [1, 3, 5, 9]
    while any(pos[i] < len(full[i]) for i in range(4)):
        live = [i for i in range(4) if pos[i] < len(full[i])]
        ns = [min(strides[i], len(full[i]) - pos[i]) for i in live]
        rows = eng.step_raw([StepEntry(("m", i), full[i][pos[i]:pos[i] + n], list(range(n))) for i, n in zip(live, ns)]).cpu().numpy()
        at = 0
        for i, n in zip(live, ns):
            check(rows[at:at + n], i, pos[i])
            at += n
            pos[i] += n
    eng.runner.check_status()


def plain_temperature_draw(row, temp, u):
    """The device's draw restated in float64: weights exp((l - max) / temp), none for tokens 20 or more below the best,
    walked in token order until the running sum passes u * total.  Returns (token, distance of the target from the
    nearest boundary as a share of the total)."""
    x = (row - row.max()) / temp
    wgt = np.where(x > -20.0, np.exp(x), 0.0)
    acc = np.cumsum(wgt)
    target = u * acc[-1]
    tok = int(np.searchsorted(acc, target, side="right"))
    return tok, float(np.min(np.abs(acc - target)) / acc[-1])


def test_tiny_b_as_stated_staggered_arrivals_and_temperature(stated_models):
    from rustingstrata_b200.sampling import SamplingParams
    from rustingstrata_b200.sampling.sampler import XorShift64, seed_state
    cfg, w = P.read_model(stated_models["B"])
    lens = [3, 120, 47, 88, 19, 64]
    prompts = [random_tokens(512, n, 700 + n) for n in lens]

    def run(dtype, budget, chunk):
        eng = engine(stated_models, "B", dtype, max_batch_tokens=budget, prefill_chunk=chunk, max_tokens=1024)
        rids = [eng.add_request(p, 12, SamplingParams(temp=0.8, seed=40 + i), arrival=3 * i) for i, p in enumerate(prompts)]
        done = {}
        while eng.has_work():
            for r in eng.step():
                done[r.rid] = list(r.generated)
        eng.runner.check_status()
        eng.runner.cache.check()
        return [done[r] for r in rids]
    outs = run("float32", 48, 16)
    assert outs == run("float32", 256, None)                   # the same draws however the work is cut
    assert all(len(o) == 12 for o in outs)
    # every token is the draw the plain logits give for the request's own stream of uniforms
    for i, (p, o) in enumerate(zip(prompts, outs)):
        rng = XorShift64(seed_state(40 + i))
        logits = P.forward_logits(cfg, w, p + o)
        for k, t in enumerate(o):
            tok, margin = plain_temperature_draw(logits[len(p) - 1 + k], 0.8, rng.uniform())
            assert t == tok or margin < 1e-5, f"request {i} token {k}: engine {t}, plain {tok} (margin {margin:.1e})"
    # bfloat16: the same workload runs to the end; its tokens are draws from slightly different logits
    assert all(len(o) == 12 for o in run("bfloat16", 48, 16))
