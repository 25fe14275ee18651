"""The attention part's per-step plan against the size of its workspace, on the host (no GPU).

A step of single tokens may hold one very long sequence beside many short ones.  Whatever lengths fit the cache
pool and the number of live requests, the plan's work lists must fit the workspace the part declared at build
time, and the launcher's own size check must accept them - also in the form a captured step uses, where the
number of splits launched per sequence is rounded up to a bucket.
"""
import numpy as np
import pytest
import torch

from rustingstrata_b200.kernels import ops
from rustingstrata_b200.parts import HostBatch, PartSpec, Runtime
from rustingstrata_b200.parts.attention import SPLIT_BUCKET, SPLIT_KEYS, PagedAttention, decode_splits


def make_part(pool_tokens, max_seqs, n_heads=8, n_kv=2, hd=32, window=None, page_size=16):
    rt = Runtime(torch.bfloat16, torch.device("cpu"), max_batch_tokens=256, max_seqs=max_seqs, max_logit_rows=max_seqs,
                 page_size=page_size, max_positions=1 << 20, pool_tokens=pool_tokens)
    spec = PartSpec("paged_attention", {"hidden": 64, "n_heads": n_heads, "n_kv_heads": n_kv, "head_dim": hd,
                                        "qk_norm": False, "window": window},
                    {k: k for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
    att = PagedAttention(spec, rt)
    att.q_per_cta = 4                  # what the kernel library would say; the plan of single tokens does not use it
    return att, rt


def host_batch(kv_lens, q_lens, page_size, bucketed):
    kv_lens, q_lens = np.asarray(kv_lens, np.int32), np.asarray(q_lens, np.int32)
    q_start = np.zeros(len(kv_lens) + 1, np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    return HostBatch(n_tokens=int(q_lens.sum()), n_seqs=len(kv_lens), q_lens=q_lens, kv_lens=kv_lens, q_start=q_start,
                     state_slots=np.arange(len(kv_lens), dtype=np.int32), first_step=np.zeros(len(kv_lens), np.int32),
                     page_size=page_size, max_blocks=[int(-(-kv_lens.max() // page_size))], bucketed=bucketed)


def workspace_of(att, rt):
    rows, width, dt = rt._wanted[f"attn_partial:{torch.float32}"]
    return torch.empty(rows * width, dtype=dt, device="meta")


def lengths_that_fit(rng, pool_tokens, max_seqs, page_size):
    """Random lengths whose pages fit the pool, skewed: often one sequence takes most of it."""
    n = int(rng.integers(1, max_seqs + 1))
    pages = pool_tokens // page_size
    if pages < n:
        n = pages
    share = rng.dirichlet(np.full(n, rng.choice([0.05, 0.3, 1.0, 5.0])))
    p = np.maximum(1, np.floor(share * pages).astype(np.int64))
    while p.sum() > pages:
        p[np.argmax(p)] -= 1
    kv = p * page_size - rng.integers(0, page_size, size=n)
    return np.maximum(1, kv).astype(np.int32)


@pytest.mark.parametrize("bucketed", [False, True])
@pytest.mark.parametrize("pool_tokens,max_seqs", [(4096, 64), (4096, 2), (32 * 4096, 32), (256, 4), (64 * 4096, 64)])
def test_plan_of_single_tokens_fits_the_workspace(pool_tokens, max_seqs, bucketed):
    att, rt = make_part(pool_tokens, max_seqs)
    ws = workspace_of(att, rt)
    rng = np.random.default_rng(pool_tokens + max_seqs)
    for _ in range(200):
        kv = lengths_that_fit(rng, pool_tokens, max_seqs, rt.page_size)
        plan = att.build_plan(host_batch(kv, np.ones_like(kv), rt.page_size, bucketed))
        assert int(plan["split_start"][-1]) <= att.partial_slots
        slots = ops._partial_slots(ws, plan["total_splits"], att.n_heads, att.hd, "test")      # the launcher's check
        assert slots >= int(plan["split_start"][-1])
        assert plan["max_splits"] >= int(decode_splits(kv, 0).max())
        if bucketed:
            assert plan["max_splits"] % SPLIT_BUCKET == 0


def test_the_cases_that_used_to_be_refused():
    """One sequence of 2,049 keys beside 63 short ones in a 4,096-token pool; 4,000 and 10 keys with two slots; one of
    12,000 beside 31 of 300 in a pool of 32 x 4,096 (all fit their pools)."""
    for pool, max_seqs, kv in ((4096, 64, [2049] + [30] * 63), (4096, 2, [4000, 10]),
                               (32 * 4096, 32, [12000] + [300] * 31), (64 * 4096, 64, [40000] + [100] * 63)):
        att, rt = make_part(pool, max_seqs)
        plan = att.build_plan(host_batch(kv, [1] * len(kv), 16, True))
        ops._partial_slots(workspace_of(att, rt), plan["total_splits"], att.n_heads, att.hd, "test")


def test_a_window_counts_the_splits_it_straddles():
    att, rt = make_part(pool_tokens=1024, max_seqs=8, window=200)
    rng = np.random.default_rng(5)
    for _ in range(200):
        n = int(rng.integers(1, 9))
        kv = rng.integers(1, 100_000, size=n).astype(np.int32)      # a window group holds the window, whatever the length
        plan = att.build_plan(host_batch(kv, np.ones_like(kv), 16, True))
        assert int(plan["split_start"][-1]) <= att.partial_slots
        assert int(np.diff(plan["split_start"]).max()) <= 200 // SPLIT_KEYS + 2


def test_a_step_beyond_the_pool_is_refused_with_a_sentence():
    att, rt = make_part(pool_tokens=256, max_seqs=2)
    with pytest.raises(ValueError, match="more keys than the cache pool holds"):
        att.build_plan(host_batch([4000, 4000], [1, 1], 16, False))


def test_launcher_names_both_numbers_when_the_workspace_is_too_small():
    with pytest.raises(ops.KernelError, match="need .* float32 values of partial workspace, 100 were given"):
        ops._partial_slots(torch.empty(100, device="meta"), 5, 8, 32, "attention")
