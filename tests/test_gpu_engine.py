"""Generation through the Python entry point and the scheduler, long decoding, the first tokens of a
sequence, and what happens when pages run out - compared with the plain implementation."""
import numpy as np
import pytest

import plain_qwen3 as P
from helpers import TINY, TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu


def engine(tiny_models, name, dtype, **kw):
    from rustingstrata_b200 import Engine
    kw.setdefault("page_size", TINY[name]["page_size"])
    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_batch_tokens", 256)
    kw.setdefault("max_seqs", 8)
    return Engine(tiny_models[name], dtype=dtype, **kw)


def teacher_forced_ok(cfg, w, prompt, generated, dtype):
    """Every generated token is the plain implementation's argmax given the tokens before it, or a
    near-tie within the engine's tolerance (bfloat16 may flip such a tie; the 32-bit engine must not)."""
    logits = P.forward_logits(cfg, w, list(prompt) + list(generated))
    for i, t in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        best = int(np.argmax(row))
        if t != best:
            margin = (row[best] - row[t]) / np.max(np.abs(logits))
            assert dtype == "bfloat16" and margin < 2 * TOL[dtype], f"token {i}: {t} vs argmax {best}, margin {margin:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_greedy_generation_through_the_entry_point(tiny_models, name, dtype):
    cfg, w = P.read_model(tiny_models[name])
    eng = engine(tiny_models, name, dtype)
    prompts = [random_tokens(cfg["vocab_size"], n, 50 + n) for n in (1, 7, 16, 33)]
    outs = eng.generate(prompts, max_new_tokens=8)
    assert [len(o) for o in outs] == [8] * 4
    for p, o in zip(prompts, outs):
        if dtype == "float32":
            assert o == P.greedy_generate(cfg, w, p, 8)
        teacher_forced_ok(cfg, w, p, o, dtype)
    single = eng.generate(prompts[2], max_new_tokens=8)            # one prompt in, one list out
    assert single == outs[2]
    eng.runner.cache.check()
    assert all(eng.runner.cache.n_free(g) == eng.runner.num_pages for g in range(len(eng.runner.cache.groups)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tiny_models, dtype):
    """A sequence fed one token at a time from its very first token for 300 positions."""
    from rustingstrata_b200.engine import StepEntry
    cfg, w = P.read_model(tiny_models["A"])
    eng = engine(tiny_models, "A", dtype)
    toks = random_tokens(cfg["vocab_size"], 300, 77)
    ref = P.forward_logits(cfg, w, toks)
    worst = 0.0
    for i, t in enumerate(toks):
        row = eng.step_raw([StepEntry("x", [t], [0])]).cpu().numpy()[0]
        err = float(np.max(np.abs(row - ref[i])) / np.max(np.abs(ref)))
        assert err <= TOL[dtype], f"position {i}: {err:.3e}"
        worst = max(worst, err)
    eng.runner.check_status()
    eng.release("x")


def test_tensor_core_attention_inside_the_engine(tiny_models):
    """The bfloat16 engine on a configuration the tcgen05 prefill and TMA decode attention kernels take: a
    long prompt in uneven portions, then decoding across several 128-key splits and past the window's edge,
    two requests side by side, every row against the plain implementation."""
    from rustingstrata_b200.engine import StepEntry
    from rustingstrata_b200.kernels import ops
    c = TINY["D"]["config"]
    n_q, n_kv, hd, page = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], TINY["D"]["page_size"]
    import torch
    assert ops.attention_prefill_kernel(torch.bfloat16, n_q, n_kv, hd, page) == "tc"
    assert ops.attention_decode_fast_ok(torch.bfloat16, n_q, n_kv, hd, page)
    cfg, w = P.read_model(tiny_models["D"])
    eng = engine(tiny_models, "D", "bfloat16", max_tokens=1536, max_batch_tokens=512)
    toks = {"x": random_tokens(cfg["vocab_size"], 430, 5), "y": random_tokens(cfg["vocab_size"], 300, 6)}
    ref = {k: P.forward_logits(cfg, w, t) for k, t in toks.items()}
    scale = {k: np.max(np.abs(r)) for k, r in ref.items()}
    pos = {"x": 0, "y": 0}
    worst = 0.0

    def feed(entries):
        # the engine returns at most 64 rows a step: the last 30 of each portion
        nonlocal worst
        first = {k: max(0, n - 30) for k, n in entries}
        rows = eng.step_raw([StepEntry(k, toks[k][pos[k]:pos[k] + n], list(range(first[k], n))) for k, n in entries]).cpu().numpy()
        at = 0
        for k, n in entries:
            m = n - first[k]
            lo = pos[k] + first[k]
            err = float(np.max(np.abs(rows[at:at + m] - ref[k][lo:lo + m])) / scale[k])
            assert err <= TOL["bfloat16"], f"{k} at {lo}..{lo + m}: {err:.3e}"
            worst = max(worst, err)
            at += m
            pos[k] += n

    feed([("x", 201)])
    feed([("x", 130), ("y", 137)])
    feed([("x", 1), ("y", 100)])
    for _ in range(60):
        feed([("x", 1), ("y", 1)])
    eng.runner.check_status()
    eng.release("x")
    eng.release("y")
    eng.runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32"])
def test_preemption_recomputes_and_gives_the_same_tokens(tiny_models, dtype):
    """With too few pages for all requests, some are preempted and recomputed; greedy output is unchanged."""
    cfg, w = P.read_model(tiny_models["A"])
    prompts = [random_tokens(cfg["vocab_size"], n, 200 + n) for n in (30, 25, 41, 12)]
    roomy = engine(tiny_models, "A", dtype).generate(prompts, max_new_tokens=40)
    tight = engine(tiny_models, "A", dtype, num_pages=40, max_tokens=0)       # 160 tokens for 4 x ~70
    outs = tight.generate(prompts, max_new_tokens=40)
    assert tight.scheduler.preemptions > 0
    assert outs == roomy
    for p, o in zip(prompts, outs):
        assert o == P.greedy_generate(cfg, w, p, 40)
    tight.runner.cache.check()
    assert tight.runner.cache.pools[0].reuses > 0


def test_chunked_prefill_with_staggered_arrivals_and_temperature(tiny_models):
    """Configuration B's workload: prompts of 3-120 tokens arriving over time, a small token budget so
    prompts are cut into portions beside decoding requests, temperature 0.8 with a fixed sampler seed."""
    from rustingstrata_b200.sampling import SamplingParams
    cfg, w = P.read_model(tiny_models["B"])
    lens = [3, 120, 47, 88, 19, 64]

    def run(budget, chunk):
        eng = engine(tiny_models, "B", "float32", max_batch_tokens=budget, prefill_chunk=chunk)
        rids = [eng.add_request(random_tokens(cfg["vocab_size"], n, 300 + n), 12, SamplingParams(temp=0.8, seed=9 + i),
                                arrival=2 * i) for i, n in enumerate(lens)]
        done = {}
        batches = []                                         # per step: (request, tokens in the step)
        launch = eng._launch

        def spy(batch, prev):
            batches.append([(s.request.rid, len(s.tokens)) for s in batch])
            return launch(batch, prev)
        eng._launch = spy
        while eng.has_work():
            for r in eng.step():
                done[r.rid] = r.generated
        return [done[r] for r in rids], eng, batches
    a, eng_a, steps_a = run(32, 16)
    b, _, steps_b = run(256, None)
    assert a == b and all(len(x) == 12 for x in a)           # the cut of the work does not change the draws
    # the small budget really cut prompts and ran their portions beside other requests' single tokens
    mixed = [st for st in steps_a if any(n > 1 for _, n in st) and any(n == 1 for _, n in st)]
    assert len(mixed) >= 5, steps_a
    flat = sum(steps_a, [])
    assert any(sum(1 for rid, n in flat if rid == r and n > 1) >= 3 for r in {rid for rid, _ in flat})   # a prompt in 3+ portions
    assert max(sum(n for _, n in st) for st in steps_a) <= 32 and max(n for st in steps_a for _, n in st) <= 16
    assert max(n for st in steps_b for _, n in st) == 120    # the roomy engine took the longest prompt whole
    c, _, _ = run(32, 16)
    assert c == a                                            # same seeds, same tokens
    eng_a.runner.cache.check()


def test_sampling_with_cuts_goes_through_the_host_sampler(tiny_models):
    from rustingstrata_b200.sampling import Sampler, SamplingParams
    cfg, w = P.read_model(tiny_models["A"])
    eng = engine(tiny_models, "A", "float32")
    p = random_tokens(cfg["vocab_size"], 10, 1)
    out = eng.generate(p, max_new_tokens=6, temperature=0.7, top_k=5, top_p=0.9, seed=4)
    # replay the same choice from the plain implementation's logits with the host sampler
    smp = Sampler(SamplingParams(temp=0.7, top_k=5, top_p=0.9, seed=4))
    toks = list(p)
    for t in out:
        row = P.forward_logits(cfg, w, toks)[-1].astype(np.float32)
        ids, _ = smp.candidates(row)
        assert t in ids.tolist() and len(ids) <= 5
        smp.note(t)
        toks.append(t)


def test_greedy_choice_sees_the_penalties(tiny_models):
    """Greedy generation with a repeat penalty, a presence penalty and DRY: the penalties change the logits before
    the arg-max (src/ops.rs:220-227), so the tokens are those of the host sampler on the plain logits, and they
    differ from plain greedy tokens."""
    from rustingstrata_b200.sampling import Sampler, SamplingParams
    cfg, w = P.read_model(tiny_models["A"])
    eng = engine(tiny_models, "A", "float32")
    p = random_tokens(cfg["vocab_size"], 12, 3)
    opts = dict(repeat_penalty=1.8, presence_penalty=0.4, dry_multiplier=0.8)
    out = eng.generate(p, max_new_tokens=24, temperature=0.0, **opts)
    smp = Sampler(SamplingParams(temp=0.0, **opts))
    toks = list(p)
    for i, t in enumerate(out):
        row = P.forward_logits(cfg, w, toks)[-1].astype(np.float32)
        assert t == smp.pick(row), f"token {i}"
        toks.append(t)
    assert out != eng.generate(p, max_new_tokens=24, temperature=0.0)
    assert len(set(out)) == len(out)                         # a penalty this strong never repeats a token here


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_long_request_beside_short_ones_in_decode_steps(tiny_models, dtype):
    """Steps of single tokens only (the ones the engine captures and replays) with one request at about 3,000 keys
    beside seven at 20 to 40: the long one's splits outnumber the others' a hundred to one and its count crosses a
    bucket of the captured launch shape (3,072 keys = 24 splits) on the way.  Every row against the plain
    implementation."""
    from rustingstrata_b200.engine import StepEntry
    cfg, w = P.read_model(tiny_models["E"])
    eng = engine(tiny_models, "E", dtype, max_tokens=3072 + 64 + 7 * 80, max_batch_tokens=512, max_seqs=8)
    n_steps, long_prompt = 40, 3050
    toks = {"long": random_tokens(cfg["vocab_size"], long_prompt + n_steps, 1)}
    for i in range(7):
        toks[f"s{i}"] = random_tokens(cfg["vocab_size"], 20 + 3 * i + n_steps, 10 + i)
    ref = {k: P.forward_logits(cfg, w, t) for k, t in toks.items()}
    scale = {k: np.max(np.abs(r)) for k, r in ref.items()}
    for k, t in toks.items():                                  # prompts, in portions of at most 512 tokens
        n = len(t) - n_steps
        for a in range(0, n, 512):
            eng.step_raw([StepEntry(k, t[a:min(a + 512, n)], [])])
    assert eng.runner.length("long") == long_prompt
    order = list(toks)
    worst, replays0 = 0.0, eng.runner.graph_replays
    for j in range(n_steps):
        rows = eng.step_raw([StepEntry(k, [toks[k][len(toks[k]) - n_steps + j]], [0]) for k in order]).cpu().numpy()
        for row, k in zip(rows, order):
            pos = len(toks[k]) - n_steps + j
            err = float(np.max(np.abs(row - ref[k][pos])) / scale[k])
            assert err <= TOL[dtype], f"step {j} request {k} position {pos}: {err:.3e}"
            worst = max(worst, err)
    eng.runner.check_status()
    assert eng.runner.length("long") == long_prompt + n_steps > 3072
    assert eng.runner.graph_replays - replays0 >= n_steps - 6          # captured and replayed, on both sides of the bucket
    print(f"{dtype}: worst {worst:.3e}")


def test_a_wait_that_runs_out_becomes_a_step_error_and_the_engine_goes_on(tiny_models):
    """Every wait inside the tensor-core kernels is bounded.  A probe kernel built with a 2 ms limit waits on a barrier
    nobody arrives at, with the runner's status word: the wait gives up, the kernel ends, the status bit turns into a
    StepError at the next check, and the very next step on the same context runs and is right."""
    from rustingstrata_b200.engine import StepEntry, StepError
    from rustingstrata_b200.kernels import ops
    cfg, w = P.read_model(tiny_models["D"])
    eng = engine(tiny_models, "D", "bfloat16")
    toks = random_tokens(cfg["vocab_size"], 40, 8)
    ref = P.forward_logits(cfg, w, toks)
    eng.step_raw([StepEntry("x", toks[:30], [])])
    eng.runner.check_status()
    res = ops.wait_probe(eng.runner.status)
    assert not res["satisfied"] and res["limit_us"] == 2000 and 2000 <= res["waited_us"] < 200_000, res
    with pytest.raises(StepError, match="bounded wait"):
        eng.runner.check_status()
    eng.runner.check_status()                                  # the word was cleared: one report per event
    rows = eng.step_raw([StepEntry("x", toks[30:], list(range(10)))]).cpu().numpy()
    eng.runner.check_status()
    assert rel_err(rows, ref[30:]) <= TOL["bfloat16"]
    eng.release("x")


def test_step_errors_leave_the_cache_untouched(tiny_models):
    from rustingstrata_b200.cache import OutOfPages
    from rustingstrata_b200.engine import StepEntry, StepError
    eng = engine(tiny_models, "A", "float32", num_pages=8, max_tokens=0)      # 32 tokens
    r = eng.runner
    r.step([StepEntry("a", list(range(10)), [9])])
    free = r.cache.n_free(0)
    with pytest.raises(OutOfPages):
        r.step([StepEntry("a", [1], [0]), StepEntry("b", list(range(30)), [])])
    assert r.cache.n_free(0) == free and r.length("a") == 10 and not r.cache.is_live("b")
    with pytest.raises(StepError, match="vocabulary"):
        r.step([StepEntry("a", [256], [0])])
    with pytest.raises(StepError, match="wanted place"):
        r.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(StepError, match="once"):
        r.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    assert r.length("a") == 10
    r.cache.check()
    out = r.step([StepEntry("a", [5], [0])])
    assert out.shape == (1, 256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(tiny_models, dtype):
    """While a step runs, the engine launches the next one with the chosen ids staying on the device.  The tokens
    are those of an engine that waits for every step, with greedy and with temperature sampling, when requests end
    by length at different times, when one ends by an end-of-sequence token the engine could not foresee, and
    when a request arrives in the middle."""
    from rustingstrata_b200.sampling import SamplingParams
    cfg, w = P.read_model(tiny_models["B"])
    prompts = [random_tokens(cfg["vocab_size"], n, 300 + n) for n in (5, 17, 9, 30)]
    plans = [(12, 0.0), (25, 0.8), (7, 0.0), (18, 1.3)]

    def run(lookahead, eos=()):
        eng = engine(tiny_models, "B", dtype)
        eng.lookahead = lookahead
        rids = [eng.add_request(p, n, SamplingParams(temp=t, seed=11 + i), eos_ids=eos)
                for i, (p, (n, t)) in enumerate(zip(prompts[:3], plans[:3]))]
        out, steps = {}, 0
        while eng.has_work():
            for r in eng.step():
                out[r.rid] = (list(r.generated), r.finish_reason)
            steps += 1
            if steps == 6:                                       # a late arrival
                rids.append(eng.add_request(prompts[3], plans[3][0], SamplingParams(temp=plans[3][1], seed=99), eos_ids=eos))
        eng.runner.check_status()
        eng.runner.cache.check()
        assert all(eng.runner.cache.n_free(g) == eng.runner.num_pages for g in range(len(eng.runner.cache.groups)))
        return [out[r] for r in rids], eng.steps_launched_ahead

    slow, n0 = run(False)
    fast, n1 = run(True)
    assert n0 == 0 and n1 > 20
    assert fast == slow
    assert [len(g) for g, _ in slow] == [12, 25, 7, 18]
    # an end-of-sequence token in the middle of the longest request
    eos = (slow[1][0][10],)
    slow_e, _ = run(False, eos)
    fast_e, n2 = run(True, eos)
    assert fast_e == slow_e and n2 > 5
    assert slow_e[1][1] == "eos" and len(slow_e[1][0]) <= 10


def test_sums_left_to_the_next_norm_change_no_bit(tiny_models, monkeypatch):
    """In steps of up to 128 tokens the output and down projections leave the adding-up of their shared tiles to the
    norm that reads the residual stream next.  Fewer kernels run, and the tokens are the same as with every product
    finishing itself."""
    from rustingstrata_b200.kernels import ops
    cfg, w = P.read_model(tiny_models["D"])
    prompts = [random_tokens(cfg["vocab_size"], n, 70 + n) for n in (3, 12, 20)]

    def run():
        eng = engine(tiny_models, "D", "bfloat16")
        n0 = ops.launch_count()
        outs = eng.generate(prompts, max_new_tokens=12)
        n = ops.launch_count() - n0
        eng.runner.check_status()
        return outs, n

    with_owed, n_owed = run()
    monkeypatch.setattr(ops, "DEFER_SUMS", False)
    without, n_plain = run()
    assert with_owed == without
    assert n_owed < n_plain


def test_bench_method_of_the_entry_point(tiny_models):
    eng = engine(tiny_models, "D", "bfloat16")
    recs = eng.bench(pp=[20, 130], tg=6, reps=2, batch=3)
    assert [r["pp"] for r in recs] == [20, 130] and all(r["batch"] == 3 and r["tg"] == 6 for r in recs)
    for r in recs:
        for k in ("prefill_tok_s", "decode_tok_s"):
            assert 0 < r[k]["min"] <= r[k]["mean"] <= r[k]["max"]
    assert not eng.has_work()
    eng.runner.cache.check()


def test_the_32_bit_engine_loads_only_the_library_it_needs(tiny_models):
    """A float32 engine in a fresh process generates without loading (so, in a fresh checkout, without compiling) the
    library of bfloat16 tensor-core kernels."""
    import subprocess
    import sys
    from helpers import ROOT
    code = (f"import sys; sys.path.insert(0, {ROOT!r})\n"
            "from rustingstrata_b200 import Engine\n"
            "from rustingstrata_b200.kernels import build\n"
            f"eng = Engine({tiny_models['A']!r}, dtype='float32', page_size=4, max_tokens=128, max_batch_tokens=32, max_seqs=2)\n"
            "print(eng.generate([1, 2, 3], max_new_tokens=4))\n"
            "print('LOADED', sorted(build._LOADED))\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "LOADED ['core']" in r.stdout, r.stdout
