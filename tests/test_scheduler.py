"""The scheduler's decisions, driven without a model: the 'model' here picks token ids by a rule (no GPU)."""
import pytest

from rustingstrata_b200.cache import CacheManager, GroupNeed
from rustingstrata_b200.engine.scheduler import Request, RequestRejected, Scheduler


def make(num_pages=16, page_size=4, budget=16, max_seqs=4, chunk=None, windows=(None,), max_positions=1000):
    cache = CacheManager([GroupNeed(w) for w in windows], page_size, num_pages, max_seqs)
    return cache, Scheduler(cache, budget, max_seqs, max_positions, chunk)


def run_step(cache, sched, pick=lambda req: 1000 + len(req.generated)):
    """What the engine does around a step, with the model replaced by ``pick``."""
    batch = sched.schedule()
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
    for s in batch:
        cache.commit(s.request.rid, len(s.tokens))
    cache.check()
    done = sched.advance(batch, {s.request.rid: pick(s.request) for s in batch if s.samples})
    cache.check()
    return batch, done


def test_prompt_is_cut_into_portions_under_the_token_budget():
    cache, sched = make(num_pages=32, budget=8)
    sched.add(Request("a", list(range(19)), 3))
    sizes, samples = [], []
    for _ in range(3):
        batch, _ = run_step(cache, sched)
        sizes.append([len(s.tokens) for s in batch])
        samples.append([s.samples for s in batch])
    assert sizes == [[8], [8], [3]] and samples == [[False], [False], [True]]
    batch, _ = run_step(cache, sched)
    assert [(s.tokens, s.samples) for s in batch] == [([1000], True)]      # decoding the first generated token


def test_decodes_go_first_and_portions_fill_the_rest():
    cache, sched = make(num_pages=64, budget=8)
    sched.add(Request("a", [1, 2, 3], 10))
    run_step(cache, sched)                                   # a: whole prompt, first token chosen
    sched.add(Request("b", list(range(20)), 2))
    batch, _ = run_step(cache, sched)
    assert [(s.request.rid, len(s.tokens)) for s in batch] == [("a", 1), ("b", 7)]
    batch, _ = run_step(cache, sched)
    assert [(s.request.rid, len(s.tokens)) for s in batch] == [("a", 1), ("b", 7)]
    batch, _ = run_step(cache, sched)
    assert [(s.request.rid, len(s.tokens), s.samples) for s in batch] == [("a", 1, True), ("b", 6, True)]


def test_prefill_chunk_caps_a_portion():
    cache, sched = make(num_pages=64, budget=16, chunk=5)
    sched.add(Request("a", list(range(12)), 1))
    assert [len(s.tokens) for s in run_step(cache, sched)[0]] == [5]


def test_requests_are_admitted_in_arrival_order_and_by_free_slots():
    cache, sched = make(num_pages=64, budget=64, max_seqs=2)
    for rid in "abc":
        sched.add(Request(rid, [1, 2, 3, 4], 2))
    batch, _ = run_step(cache, sched)
    assert [s.request.rid for s in batch] == ["a", "b"]       # two slots
    _, done = run_step(cache, sched)                          # a and b reach their two tokens
    assert sorted(r.rid for r in done) == ["a", "b"] and all(r.finish_reason == "length" for r in done)
    batch, _ = run_step(cache, sched)
    assert [s.request.rid for s in batch] == ["c"]


def test_staggered_arrivals_wait_for_their_step():
    cache, sched = make(num_pages=64, budget=64)
    sched.add(Request("a", [1, 2], 8, arrival=0))
    sched.add(Request("b", [3, 4], 8, arrival=2))
    seen = []
    for _ in range(4):
        batch, _ = run_step(cache, sched)
        seen.append([s.request.rid for s in batch])
    assert seen == [["a"], ["a"], ["a", "b"], ["a", "b"]]


def test_admission_needs_room_for_the_whole_prompt_and_a_decode_page():
    cache, sched = make(num_pages=6, page_size=4, budget=64)
    sched.add(Request("a", list(range(12)), 4))               # 3 pages + 1
    sched.add(Request("b", list(range(9)), 4))                # 3 pages + 1 > what is left
    batch, _ = run_step(cache, sched)
    assert [s.request.rid for s in batch] == ["a"]
    assert [r.rid for r in sched.waiting] == ["b"]
    for _ in range(3):
        run_step(cache, sched)
    assert not cache.is_live("a")                             # a finished and gave its pages back
    batch, _ = run_step(cache, sched)
    assert [s.request.rid for s in batch] == ["b"]


def test_eos_finishes_and_frees():
    cache, sched = make()
    sched.add(Request("a", [1, 2, 3], 50, eos_ids=(7,)))
    run_step(cache, sched, pick=lambda r: 5)
    _, done = run_step(cache, sched, pick=lambda r: 7)
    assert done[0].finish_reason == "eos" and done[0].generated == [5] and cache.n_free(0) == 16


def test_context_limit_finishes():
    cache, sched = make(max_positions=6)
    sched.add(Request("a", [1, 2, 3], 3))
    for _ in range(3):
        _, done = run_step(cache, sched)
    assert done and done[0].finish_reason in ("length", "context") and len(done[0].generated) == 3


def test_requests_that_can_never_fit_are_rejected():
    cache, sched = make(num_pages=4, page_size=4, max_positions=100)
    with pytest.raises(RequestRejected, match="context full"):
        sched.add(Request("a", list(range(10)), 10))          # 20 tokens > 16 the cache holds
    with pytest.raises(RequestRejected, match="positions"):
        sched.add(Request("b", list(range(60)), 50))
    with pytest.raises(RequestRejected, match="empty"):
        sched.add(Request("c", [], 5))
    with pytest.raises(RequestRejected, match="max_new_tokens"):
        sched.add(Request("d", [1], 0))


def test_when_pages_run_out_the_newest_request_is_preempted_and_recomputed():
    cache, sched = make(num_pages=6, page_size=4, budget=64)
    sched.add(Request("a", list(range(7)), 12))               # 2 pages + decode page = 3 to be admitted
    sched.add(Request("b", list(range(6)), 12))               # the same
    batch, _ = run_step(cache, sched)
    assert [s.request.rid for s in batch] == ["a", "b"]
    preempted_at = None
    for step in range(40):
        batch, done = run_step(cache, sched)
        if sched.preemptions and preempted_at is None:
            preempted_at = step
            b = next(r for r in sched.waiting if r.rid == "b")
            assert b.computed == 0 and b.preemptions == 1 and len(b.generated) > 0
            assert not cache.is_live("b")                     # its pages went back
        if not sched.has_work():
            break
    assert preempted_at is not None and not sched.has_work()
    assert cache.n_free(0) == 6
    cache.check()


def test_preempted_request_resumes_with_its_generated_tokens_as_prompt():
    cache, sched = make(num_pages=6, page_size=4, budget=64)
    a, b = Request("a", list(range(7)), 12), Request("b", list(range(6)), 12)
    sched.add(a)
    sched.add(b)
    fed = {"a": [], "b": []}
    while sched.has_work():
        batch = sched.schedule()
        for s in batch:
            cache.reserve(s.request.rid, len(s.tokens))
            cache.commit(s.request.rid, len(s.tokens))
            fed[s.request.rid].append(list(s.tokens))
        sched.advance(batch, {s.request.rid: 1000 + len(s.request.generated) for s in batch if s.samples})
    assert b.preemptions >= 1 and len(a.generated) == 12 and len(b.generated) == 12
    # after the preemption, b was fed prompt + everything it had generated, as one recomputed prompt
    recompute = [t for t in fed["b"] if len(t) > 1][-1]
    assert recompute[:6] == list(range(6)) and recompute[6:] == b.generated[: len(recompute) - 6]


def test_a_lone_request_is_never_preempted_and_never_deadlocks():
    cache, sched = make(num_pages=4, page_size=4, budget=64)
    sched.add(Request("a", list(range(5)), 11))               # exactly the 16 tokens the cache holds
    steps = 0
    while sched.has_work():
        run_step(cache, sched)
        steps += 1
        assert steps < 40
    assert sched.preemptions == 0 and cache.n_free(0) == 4


# ------------------------------------------------------------------ the step after the one in flight
def _decoding(n_req=3, pages=64, max_new=8, eos=()):
    from rustingstrata_b200.cache import CacheManager, GroupNeed
    from rustingstrata_b200.engine.scheduler import Request, Scheduler
    cache = CacheManager([GroupNeed(None)], page_size=4, num_pages=pages, max_seqs=8)
    sch = Scheduler(cache, max_batch_tokens=64, max_seqs=8, max_positions=256)
    for i in range(n_req):
        sch.add(Request(rid=i, prompt=[1, 2, 3, 4, 5][: 3 + i % 3], max_new_tokens=max_new, eos_ids=tuple(eos)))
    return cache, sch


def _run(cache, sch, batch, token=7):
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    return sch.advance(batch, {s.request.rid: token for s in batch if s.samples})


def test_lookahead_is_the_batch_schedule_would_build():
    cache, sch = _decoding()
    batch = sch.schedule()                                     # the three prompts, whole
    for s in batch:                                            # what the runner's step does on the host
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    ahead = sch.lookahead(batch)
    assert ahead is not None and [s.request.rid for s in ahead] == [0, 1, 2]
    assert all(s.tokens == [-1] and s.samples for s in ahead)
    sch.advance(batch, {0: 7, 1: 7, 2: 7})
    real = sch.schedule()
    assert [s.request.rid for s in real] == [s.request.rid for s in ahead] and all(len(s.tokens) == 1 for s in real)


def test_lookahead_waits_when_it_cannot_know():
    from rustingstrata_b200.engine.scheduler import Request
    cache, sch = _decoding()
    batch = sch.schedule()
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    sch.add(Request(rid=9, prompt=[1, 2], max_new_tokens=4))   # somebody waits: admission comes first
    assert sch.lookahead(batch) is None
    sch.waiting.clear()
    assert sch.lookahead(batch[:2]) is None                    # a running request that is not in the batch
    assert sch.lookahead([]) is None


def test_lookahead_with_a_portion_that_does_not_end_the_prompt():
    from rustingstrata_b200.cache import CacheManager, GroupNeed
    from rustingstrata_b200.engine.scheduler import Request, Scheduler
    cache = CacheManager([GroupNeed(None)], page_size=4, num_pages=64, max_seqs=4)
    sch = Scheduler(cache, max_batch_tokens=64, max_seqs=4, max_positions=256, prefill_chunk=4)
    sch.add(Request(rid=0, prompt=list(range(1, 11)), max_new_tokens=4))
    batch = sch.schedule()
    assert not batch[0].samples
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    assert sch.lookahead(batch) is None                        # still prefilling after this step


def test_lookahead_leaves_out_requests_that_end_by_length_and_stops_when_pages_run_out():
    cache, sch = _decoding(n_req=2, pages=64, max_new=2)
    batch = sch.schedule()
    _run(cache, sch, batch)                                    # one token generated each
    batch = sch.schedule()
    for s in batch:
        cache.reserve(s.request.rid, 1)
        cache.commit(s.request.rid, 1)
    assert sch.lookahead(batch) is None                        # both end with this step: nothing to launch
    # pages: two requests hold one full page each and one page is free: the fifth tokens of both do not fit
    from rustingstrata_b200.cache import CacheManager, GroupNeed
    from rustingstrata_b200.engine.scheduler import Request, Scheduler
    cache = CacheManager([GroupNeed(None)], page_size=4, num_pages=3, max_seqs=4)
    sch = Scheduler(cache, max_batch_tokens=64, max_seqs=4, max_positions=256)
    for i in range(2):
        sch.add(Request(rid=i, prompt=[1, 2, 3], max_new_tokens=6))
    batch = sch.schedule()
    assert len(batch) == 2                                     # both prompts: one page each, one page stays free
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    ahead = sch.lookahead(batch)                               # their fourth tokens go into the pages they hold
    assert ahead is not None and len(ahead) == 2
    sch.advance(batch, {0: 7, 1: 7})
    batch = sch.schedule()
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    assert cache.n_free(0) == 1
    assert sch.lookahead(batch) is None                        # both need a new page and one is free: schedule() decides


# ------------------------------------------------------------------ progress: no state in which schedule() returns nothing for ever
def _drain(cache, sched, limit=2000):
    """Runs to the end; every schedule() call with work to do and nobody arriving later must return a batch."""
    steps = 0
    while sched.has_work():
        future = any(r.arrival > sched.step_index for r in sched.waiting)
        batch, _ = run_step(cache, sched)
        assert batch or future, "schedule() returned nothing although requests could run"
        steps += 1
        assert steps < limit, "the scheduler does not finish"
    return steps


def test_two_prompts_cut_into_portions_do_not_starve_each_other():
    """Portions smaller than the budget: the second prompt must not be admitted on the strength of pages the first
    one has yet to take (pool of 10 pages of 4, portions of 8, prompts of 30 and 20 tokens)."""
    cache, sched = make(num_pages=10, page_size=4, budget=64, chunk=8)
    a, b = Request("a", list(range(30)), 2), Request("b", list(range(20)), 2)
    sched.add(a)
    sched.add(b)
    batch, _ = run_step(cache, sched)
    assert [s.request.rid for s in batch] == ["a"]             # a's 8 pages + 1 are spoken for: b waits
    _drain(cache, sched)
    assert len(a.generated) == 2 and len(b.generated) == 2 and sched.preemptions == 0
    assert cache.n_free(0) == 10


def test_a_prompt_that_fills_the_last_page_is_admitted():
    """What add() accepts must be admissible: 38 + 2 tokens are exactly the pool's 10 pages of 4."""
    cache, sched = make(num_pages=10, page_size=4, budget=64)
    a = Request("a", list(range(38)), 2)
    sched.add(a)
    batch, _ = run_step(cache, sched)
    assert [len(s.tokens) for s in batch] == [38]
    _drain(cache, sched)
    assert len(a.generated) == 2 and cache.n_free(0) == 10


def test_prefilling_requests_that_block_each_other_are_untangled_by_preemption():
    """Two requests that are both in the middle of their prompts and hold all pages between them (a state admission
    avoids, forced here by hand): the newest yields, the oldest goes on, both finish."""
    cache, sched = make(num_pages=10, page_size=4, budget=64, chunk=8)
    a, b = Request("a", list(range(30)), 2), Request("b", list(range(20)), 2)
    for r, n in ((a, 24), (b, 16)):
        cache.admit(r.rid)
        cache.reserve(r.rid, n)
        cache.commit(r.rid, n)
        r.computed = n
        sched.running.append(r)
    assert cache.n_free(0) == 0
    batch = sched.schedule()
    assert [s.request.rid for s in batch] == ["a"] and sched.preemptions == 1 and b.computed == 0
    for s in batch:
        cache.reserve(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid, len(s.tokens))
    sched.advance(batch, {s.request.rid: 1000 for s in batch if s.samples})
    _drain(cache, sched)
    assert len(a.generated) == 2 and len(b.generated) == 2 and cache.n_free(0) == 10


def test_a_running_request_that_can_never_go_on_raises_instead_of_spinning():
    from rustingstrata_b200.engine.scheduler import SchedulerStuck
    cache, sched = make(num_pages=2, page_size=4, budget=64)
    a = Request("a", list(range(6)), 2)
    cache.admit("a")
    sched.running.append(a)
    cache.admit("thief")                                      # pages held by something the scheduler does not know
    cache.reserve("thief", 8)
    with pytest.raises(SchedulerStuck, match="cannot take a token"):
        sched.schedule()


@pytest.mark.parametrize("seed", range(12))
def test_random_workloads_always_finish(seed):
    """Random prompts, lengths, arrivals, portion sizes, budgets and pool sizes (windowed groups too): every request
    ends with all its tokens, no page is lost, and schedule() never returns nothing while somebody could run."""
    import random
    rng = random.Random(seed)
    page = rng.choice([2, 4, 16])
    pages = rng.randint(6, 40)
    windows = rng.choice([(None,), (None,), (None, 3 * page), (None, page + 1)])
    budget = rng.choice([4, 8, 32, 256])
    chunk = rng.choice([None, 3, 8, 17])
    cache, sched = make(num_pages=pages, page_size=page, budget=budget, max_seqs=rng.randint(1, 5), chunk=chunk,
                        windows=windows, max_positions=10_000)
    reqs = []
    for i in range(rng.randint(3, 12)):
        total = rng.randint(2, pages * page)
        n_new = rng.randint(1, total - 1)
        r = Request(i, list(range(total - n_new)), n_new, arrival=rng.randint(0, 20))
        sched.add(r)
        reqs.append(r)
    _drain(cache, sched)
    assert all(len(r.generated) == r.max_new_tokens and r.finished for r in reqs)
    assert all(cache.n_free(g) == pages for g in range(len(windows)))
    cache.check()
