"""Trace replay through bin/trace_run, compared with the plain implementation.

The same requests are replayed whole, with the last 32 tokens decoded one by one, in
portions of changing size (down to two tokens), and mixed (up to four live requests,
portions of some beside single tokens of others, with so few pages that pages are used
again), in 32-bit and in bfloat16.  Every logits row is compared with the plain
implementation's row for that request and position.
"""
import json
import os
import random

import numpy as np
import pytest

import plain_qwen3 as P
from helpers import TINY, TOL, random_tokens, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = [100, 75, 130, 61, 33, 90]            # all above 32; none a multiple of a page
PORTIONS = [7, 2, 13, 2, 5, 3, 29, 2, 16, 4, 11, 2]


def round64(n):
    return (n + 63) // 64 * 64


class Trace:
    """Builds steps and remembers which (request, position) each written row is."""

    def __init__(self):
        self.steps, self.rows = [], {}

    def add(self, entries, end=()):
        k = len(self.steps)
        rows = []
        ents = []
        for rid, start, toks, want in entries:
            ents.append({"id": rid, "tokens": toks, "want": want})
            rows += [(rid, start + w) for w in want]
        self.steps.append({"step": k, "entries": ents, "end": list(end)})
        if rows:
            self.rows[k] = rows
        return k


def build_trace(tokens):
    """tokens: {rid: list}.  Returns (Trace, {cutting name: set of steps}, max live tokens)."""
    tr = Trace()
    parts = {}
    four = list(tokens)[:4]
    # 1. each request alone and whole
    s0 = len(tr.steps)
    for rid in four:
        t = tokens[rid]
        tr.add([(rid, 0, t, list(range(len(t))))], end=[rid])
    parts["whole"] = range(s0, len(tr.steps))
    # 2. most of it in one step, the last 32 tokens one by one
    s0 = len(tr.steps)
    for rid in four:
        t = tokens[rid]
        n = len(t) - 32
        tr.add([(rid, 0, t[:n], [n - 1])])
        for i in range(n, len(t)):
            tr.add([(rid, i, [t[i]], [0])], end=[rid] if i == len(t) - 1 else [])
    parts["tail32"] = range(s0, len(tr.steps))
    # 3. portions of changing size, down to two tokens
    s0 = len(tr.steps)
    for rid in four:
        t = tokens[rid]
        pos, k = 0, 0
        while pos < len(t):
            n = min(PORTIONS[k % len(PORTIONS)], len(t) - pos)
            k += 1
            last = pos + n == len(t)
            tr.add([(rid, pos, t[pos:pos + n], list(range(n)))], end=[rid] if last else [])
            pos += n
    parts["portions"] = range(s0, len(tr.steps))
    # 4. mixed: up to four live, portions beside single tokens, requests left out of steps, few pages
    s0 = len(tr.steps)
    rng = random.Random(1234)
    pool = 384                                    # tokens; the six requests need 704 in all
    waiting = list(tokens)
    live, pos, held = [], {}, 0
    peak = 0
    while waiting or live:
        for rid in list(waiting):                 # the first waiting requests that still fit the pool
            if len(live) < 4 and held + round64(len(tokens[rid])) <= pool:
                waiting.remove(rid)
                live.append(rid)
                pos[rid] = 0
                held += round64(len(tokens[rid]))
        peak = max(peak, held)
        chosen = [r for r in live if rng.random() < 0.75] or [live[0]]
        entries, ended = [], []
        for rid in chosen:
            t = tokens[rid]
            left = len(t) - pos[rid]
            decode_phase = left <= 20
            n = 1 if decode_phase else min(rng.choice([2, 3, 5, 9, 17, 31]), left - 20)
            want = [0] if decode_phase else rng.choice([list(range(n)), [n - 1], []])
            entries.append((rid, pos[rid], t[pos[rid]:pos[rid] + n], want))
            pos[rid] += n
            if pos[rid] == len(t):
                ended.append(rid)
        tr.add(entries, end=ended)
        for rid in ended:
            live.remove(rid)
            held -= round64(len(tokens[rid]))
    parts["mixed"] = range(s0, len(tr.steps))
    return tr, parts, max(peak, max(round64(len(t)) for t in tokens.values()))


_CACHE = {}


def replayed(tiny_models, name, dtype):
    key = (name, dtype)
    if key not in _CACHE:
        cfg, w = P.read_model(tiny_models[name])
        tokens = {f"r{i}": random_tokens(cfg["vocab_size"], n, 100 + i) for i, n in enumerate(LENGTHS)}
        ref = {rid: P.forward_logits(cfg, w, t) for rid, t in tokens.items()}
        tr, parts, max_tokens = build_trace(tokens)
        got = run_trace(tiny_models[name], dtype, tr.steps, max_tokens, page_size=TINY[name]["page_size"])
        _CACHE[key] = (tr, parts, got, ref, max_tokens, tokens)
    return _CACHE[key]


@pytest.mark.parametrize("cutting", ["whole", "tail32", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_matches_plain(tiny_models, name, dtype, cutting):
    tr, parts, got, ref, _, _ = replayed(tiny_models, name, dtype)
    worst, n_rows = (0.0, None), 0
    for k in parts[cutting]:
        if k not in tr.rows:
            continue
        assert got[k].shape[0] == len(tr.rows[k])
        for row, (rid, p) in zip(got[k], tr.rows[k]):
            scale = np.max(np.abs(ref[rid]))
            err = float(np.max(np.abs(row.astype(np.float64) - ref[rid][p])) / scale)
            n_rows += 1
            if err > worst[0]:
                worst = (err, (k, rid, p))
            # the first wrong row is what to look at: its step, request and position
            assert err <= TOL[dtype], f"{name} {dtype} {cutting}: step {k} request {rid} position {p}: error {err:.3e}"
    assert n_rows > 0
    print(f"{name} {dtype} {cutting}: {n_rows} rows, worst {worst[0]:.3e} at {worst[1]}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_replay_uses_pages_again(tiny_models, name):
    """The mixed cutting runs 704 tokens of requests through a pool of at most 384: the pools say at the end of the
    replay that pages were handed out more often than there are pages, that some had been used before, and that
    every page came back."""
    tr, parts, got, _, max_tokens, tokens = replayed(tiny_models, name, "float32")
    assert max_tokens <= 384 < sum(round64(len(t)) for t in tokens.values())
    assert got.pools, "trace_run reported nothing about its page pools"
    for pool in got.pools:
        assert pool["pages"] * TINY[name]["page_size"] <= 384
        assert pool["allocations"] > pool["pages"] and pool["reuses"] > 0 and pool["held_at_end"] == 0, pool
    live_peak = 0
    live = set()
    for k in parts["mixed"]:
        s = tr.steps[k]
        live |= {e["id"] for e in s["entries"]}
        live_peak = max(live_peak, len(live))
        live -= set(s["end"])
    assert live_peak == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_agree_with_each_other(tiny_models, dtype):
    """The same position reached by different cuttings gives the same logits beyond rounding."""
    tr, parts, got, ref, _, _ = replayed(tiny_models, "B", dtype)
    by_pos = {}
    for cutting, steps in parts.items():
        for k in steps:
            for row, key in zip(got.get(k, []), tr.rows.get(k, [])):
                by_pos.setdefault(key, {})[cutting] = row
    pairs = 0
    for key, rows in by_pos.items():
        if "whole" not in rows:
            continue
        for cutting, row in rows.items():
            scale = np.max(np.abs(ref[key[0]]))
            assert np.max(np.abs(row - rows["whole"])) / scale <= 2 * TOL[dtype], (key, cutting)
            pairs += 1
    assert pairs > 500
