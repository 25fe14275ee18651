"""Token choice after the logits: the reference's sampler on the host, and its device twin.

Reference ``Sampler`` (src/ops.rs:118-323): greedy when ``temp`` is 0 (first index of
the largest logit; a best logit that is not finite is an error), else weights
exp((l - max)/temp) with tokens 20 or more below the best dropped, candidates sorted
by weight descending then id ascending, cut to ``top_k`` (0 = all), then to the
smallest prefix whose mass reaches ``top_p`` times the total; a uniform u from
xorshift64 (shifts 13, 7, 17; the top 24 bits) picks the first candidate at which
u * total minus the running weights goes negative.  Before that, the reply-token
penalties: repeat (llama.cpp ``repeat_penalty`` over the last ``last_n`` reply
tokens), presence and frequency (OpenAI), and DRY.  The seed becomes the state
``seed * 0x9e3779b97f4a7c15 | 1`` (src/main.rs:635-638).

:class:`Sampler` is that algorithm on a float32 numpy row.  The engine uses the device
kernels (argmax; temperature draw by token id order) when no cut or penalty is set, and
this class on logits copied to the host otherwise.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

NON_FINITE = "the forward pass produced NaN or infinite logits"
_MASK = (1 << 64) - 1
DRY_WINDOW = 4096
DRY_MAX_MATCH = 64


class SamplingError(RuntimeError):
    pass


def seed_state(seed: int) -> int:
    """A non-zero xorshift64 state from a seed (src/main.rs:635-638)."""
    return ((seed * 0x9E3779B97F4A7C15) & _MASK) | 1


@dataclass
class SamplingParams:
    """Options by the reference's flag names (src/main.rs:72-104): --temp, --top-k, --top-p, --seed,
    --presence-penalty, --frequency-penalty, --repeat-penalty, --penalty-last-n, --dry-multiplier,
    --dry-base, --dry-allowed-length."""
    temp: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repeat_penalty: float = 1.0
    penalty_last_n: int = 64
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2

    def has_penalties(self) -> bool:
        return (self.presence_penalty != 0 or self.frequency_penalty != 0 or self.repeat_penalty != 1.0
                or self.dry_multiplier > 0)

    def needs_host(self) -> bool:
        """Whether the choice needs the host sampler: the penalties change the logits before any choice, the greedy
        one included (src/ops.rs:220-227), and the top-k/top-p cuts need the sorted candidates."""
        if self.has_penalties():
            return True
        return self.temp > 0 and (self.top_k > 0 or self.top_p < 1.0)


class XorShift64:
    def __init__(self, state: int):
        self.state = state & _MASK
        if self.state == 0:
            raise ValueError("xorshift64 state must not be 0")

    def uniform(self) -> float:
        """Uniform in [0, 1) from the top 24 bits (src/ops.rs:317-322)."""
        s = self.state
        s ^= (s << 13) & _MASK
        s ^= s >> 7
        s ^= (s << 17) & _MASK
        self.state = s
        return float(np.float32(s >> 40) / np.float32(1 << 24))


class Sampler:
    def __init__(self, params: SamplingParams):
        self.p = params
        self.rng = XorShift64(seed_state(params.seed))
        self.seen: Dict[int, int] = {}
        self.hist: List[int] = []

    # -------------------------------------------------------------- penalties (src/ops.rs:165-207)
    def _dry_penalties(self) -> List[Tuple[int, float]]:
        p = self.p
        h = self.hist[-DRY_WINDOW:]
        n = len(h)
        if p.dry_multiplier <= 0 or n < 2:
            return []
        last = h[-1]
        best: Dict[int, int] = {}
        for i in range(n - 1):
            if h[i] != last:
                continue
            ln = 1
            while ln < DRY_MAX_MATCH and ln <= i and h[i - ln] == h[n - 1 - ln]:
                ln += 1
            best[h[i + 1]] = max(best.get(h[i + 1], 0), ln)
        allowed = max(p.dry_allowed_length, 1)
        return [(t, p.dry_multiplier * p.dry_base ** (ln - allowed)) for t, ln in best.items() if ln >= allowed]

    def _penalized(self, logits: np.ndarray) -> np.ndarray:
        p = self.p
        rep = bool(self.seen) and (p.presence_penalty != 0 or p.frequency_penalty != 0)
        dry = self._dry_penalties()
        if p.repeat_penalty == 1.0:
            n = 0
        else:
            n = len(self.hist) if p.penalty_last_n < 0 else p.penalty_last_n
        last = sorted(set(self.hist[len(self.hist) - min(n, len(self.hist)):])) if n else []
        if not rep and not dry and not last:
            return logits
        l = logits.astype(np.float32, copy=True)
        for t in last:
            if 0 <= t < l.size:
                l[t] = l[t] / np.float32(p.repeat_penalty) if l[t] > 0 else l[t] * np.float32(p.repeat_penalty)
        if rep:
            for t, c in self.seen.items():
                if 0 <= t < l.size:
                    l[t] -= np.float32(p.presence_penalty + p.frequency_penalty * c)
        for t, pen in dry:
            if 0 <= t < l.size:
                l[t] -= np.float32(pen)
        return l

    def note(self, t: int) -> None:
        self.seen[t] = self.seen.get(t, 0) + 1
        self.hist.append(t)

    # -------------------------------------------------------------- candidates and draw (src/ops.rs:281-314)
    def candidates(self, logits: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
        """(token ids, weights) the draw chooses from, most likely first."""
        p = self.p
        l = np.asarray(logits, dtype=np.float32)
        finite = np.isfinite(l)
        if not finite.any():
            return np.zeros(0, np.int64), np.zeros(0, np.float32)
        m = np.max(np.where(np.isnan(l), -np.inf, l))
        x = (l - np.float32(m)) / np.float32(p.temp)
        keep = np.nonzero((x > -20.0) & ~np.isnan(x))[0]
        w = np.exp(x[keep]).astype(np.float32)
        order = np.lexsort((keep, -w))              # weight descending, id ascending
        ids, w = keep[order], w[order]
        if p.top_k > 0:
            ids, w = ids[: p.top_k], w[: p.top_k]
        total = np.float32(0)
        for v in w:                                 # float32 running sums, as the reference
            total += v
        acc, n = np.float32(0), len(w)
        goal = np.float32(p.top_p) * total
        for j, v in enumerate(w):
            acc += v
            if acc >= goal:
                n = j + 1
                break
        return ids[:n], w[:n]

    def draw(self, ids: np.ndarray, w: np.ndarray) -> int:
        if len(ids) == 0:
            raise SamplingError(NON_FINITE)
        total = np.float32(0)
        for v in w:
            total += v
        r = np.float32(self.rng.uniform()) * total
        for i, v in zip(ids, w):
            r -= v
            if r < 0:
                return int(i)
        return int(ids[-1])

    def pick(self, logits: np.ndarray) -> int:
        l = self._penalized(np.asarray(logits, dtype=np.float32))
        if self.p.temp <= 0:
            i = int(np.argmax(np.where(np.isnan(l), -np.inf, l)))     # first index on ties
            if not np.isfinite(l[i]):
                raise SamplingError(NON_FINITE)
        else:
            i = self.draw(*self.candidates(l))
        self.note(i)
        return i
