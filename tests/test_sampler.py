"""The host sampler against the reference's algorithm (src/ops.rs:118-323; tests/ops.rs:36-72) (no GPU)."""
import numpy as np
import pytest

from rustingstrata_b200.sampling import Sampler, SamplingError, SamplingParams, XorShift64, seed_state


def test_xorshift_sequence_and_seed_mix():
    # computed by hand from the recurrence x ^= x<<13; x ^= x>>7; x ^= x<<17 on 64 bits, state 1
    r = XorShift64(1)
    r.uniform()
    assert r.state == 0x40822041
    assert seed_state(0) == 1 and seed_state(1) == (0x9E3779B97F4A7C15 | 1) and seed_state(2) & 1 == 1
    u = [XorShift64(seed_state(7)).uniform() for _ in range(1)]
    assert 0.0 <= u[0] < 1.0
    r = XorShift64(seed_state(3))
    xs = [r.uniform() for _ in range(2000)]
    assert 0.45 < np.mean(xs) < 0.55 and min(xs) >= 0 and max(xs) < 1


def test_greedy_first_index_on_ties_and_non_finite_error():
    s = Sampler(SamplingParams())
    assert s.pick(np.array([0.5, 2.0, 2.0, -1.0], np.float32)) == 1
    with pytest.raises(SamplingError):
        Sampler(SamplingParams()).pick(np.array([np.nan, np.nan], np.float32))
    with pytest.raises(SamplingError):
        Sampler(SamplingParams(temp=1.0)).pick(np.array([np.nan, np.inf], np.float32))


def test_temperature_frequencies_follow_softmax():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], np.float32))
    s = Sampler(SamplingParams(temp=1.0, seed=11))
    n = 20000
    counts = np.bincount([s.pick(logits) for _ in range(n)], minlength=4) / n
    np.testing.assert_allclose(counts, [0.5, 0.3, 0.15, 0.05], atol=0.012)
    s2 = Sampler(SamplingParams(temp=0.5, seed=11))
    c2 = np.bincount([s2.pick(logits) for _ in range(n)], minlength=4) / n
    want = np.array([0.25, 0.09, 0.0225, 0.0025]) / 0.365
    np.testing.assert_allclose(c2, want, atol=0.012)


def test_top_k_and_top_p_cut_the_sorted_candidates():
    logits = np.log(np.array([0.1, 0.4, 0.2, 0.3], np.float32))
    ids, w = Sampler(SamplingParams(temp=1.0, top_k=2)).candidates(logits)
    assert ids.tolist() == [1, 3]
    ids, _ = Sampler(SamplingParams(temp=1.0, top_p=0.65)).candidates(logits)
    assert ids.tolist() == [1, 3]                                  # 0.4 + 0.3 >= 0.65
    ids, _ = Sampler(SamplingParams(temp=1.0, top_p=0.75)).candidates(logits)
    assert ids.tolist() == [1, 3, 2]
    ids, _ = Sampler(SamplingParams(temp=1.0, top_k=3, top_p=0.5)).candidates(logits)
    assert ids.tolist() == [1, 3]                                  # top_p of the mass left after top_k (0.9)
    ids, _ = Sampler(SamplingParams(temp=1.0)).candidates(np.array([1.0, 1.0, 1.0], np.float32))
    assert ids.tolist() == [0, 1, 2]                               # ties by id
    s = Sampler(SamplingParams(temp=1.0, top_k=1, seed=5))
    assert {s.pick(logits) for _ in range(50)} == {1}


def test_far_tokens_are_dropped_before_the_draw():
    logits = np.array([0.0, -5.0, -20.0, -25.0, np.nan], np.float32)
    ids, _ = Sampler(SamplingParams(temp=1.0)).candidates(logits)
    assert ids.tolist() == [0, 1]                                  # scaled logit must be above -20
    ids, _ = Sampler(SamplingParams(temp=2.0)).candidates(logits)
    assert ids.tolist() == [0, 1, 2, 3]


def test_same_seed_same_tokens():
    logits = np.random.default_rng(0).standard_normal(300).astype(np.float32)
    a = Sampler(SamplingParams(temp=0.8, seed=42))
    b = Sampler(SamplingParams(temp=0.8, seed=42))
    c = Sampler(SamplingParams(temp=0.8, seed=43))
    ta, tb, tc = ([s.pick(logits) for _ in range(40)] for s in (a, b, c))
    assert ta == tb and ta != tc


def test_presence_frequency_and_repeat_penalties():
    logits = np.array([2.0, 1.9, -1.0], np.float32)
    s = Sampler(SamplingParams(temp=1.0, top_k=1, presence_penalty=0.5, seed=1))
    assert [s.pick(logits) for _ in range(3)] == [0, 1, 0]         # 2.0 → 1.5 after one use; then 1.9 → 1.4
    s = Sampler(SamplingParams(temp=1.0, top_k=1, frequency_penalty=0.2, seed=1))
    assert [s.pick(logits) for _ in range(4)] == [0, 1, 0, 1]
    s = Sampler(SamplingParams(temp=1.0, top_k=1, repeat_penalty=2.0, penalty_last_n=1, seed=1))
    assert [s.pick(logits) for _ in range(3)] == [0, 1, 0]         # only the last token is penalised
    neg = np.array([-1.0, -1.5], np.float32)
    s = Sampler(SamplingParams(temp=1.0, top_k=1, repeat_penalty=2.0, penalty_last_n=-1, seed=1))
    assert [s.pick(neg) for _ in range(2)] == [0, 1]               # negative logits are multiplied


def test_dry_penalises_the_token_that_would_extend_a_repeat():
    s = Sampler(SamplingParams(temp=1.0, dry_multiplier=1.0, dry_base=2.0, dry_allowed_length=2))
    for t in [5, 6, 7, 9, 5, 6]:
        s.note(t)
    pen = dict(s._dry_penalties())
    assert pen == {7: 1.0}                                         # "5 6" seen before, followed by 7; length 2 = allowed
    s.note(7)
    assert dict(s._dry_penalties()) == {9: 2.0}                    # match of length 3 → mult * base^(3-2)


def test_penalties_need_the_host_sampler_also_for_greedy():
    """The reference applies the penalties before the arg-max of temp <= 0 (src/ops.rs:220-227)."""
    assert not SamplingParams().needs_host() and not SamplingParams(temp=0.7).needs_host()
    assert not SamplingParams(temp=0.0, top_k=5, top_p=0.5).needs_host()        # cuts mean nothing to an arg-max
    assert SamplingParams(temp=0.7, top_k=5).needs_host() and SamplingParams(temp=0.7, top_p=0.9).needs_host()
    for opts in (dict(repeat_penalty=1.3), dict(presence_penalty=0.1), dict(frequency_penalty=0.1), dict(dry_multiplier=0.5)):
        assert SamplingParams(temp=0.0, **opts).needs_host() and SamplingParams(temp=0.9, **opts).needs_host()
    s = Sampler(SamplingParams(temp=0.0, repeat_penalty=2.0))
    row = np.array([0.0, 3.0, 2.9, 1.0], dtype=np.float32)
    assert s.pick(row) == 1 and s.pick(row) == 2 and s.pick(row) == 1          # 3.0/2 < 2.9, then 2.9/2 < 3.0/2
