"""The decode-attention entry point that takes no workspace, called through its exported C symbol.

Some hosts of this library cannot request device memory when they call it (a plug-in inside another
runtime's memory budget, a loop that forbids allocator calls after start-up), so they cannot give the
split-KV attention kernel its workspace.  ``rs_attention_decode_noalloc`` keeps that workspace in an
array inside the library instead.  This test loads the shared library with ctypes, calls the symbol
twice in a row on different inputs, and compares each result with the ordinary entry point's (which
is given a workspace tensor), then checks that a request beyond the array's stated size is refused
with a readable reason.  It lives in a file that pytest collects last, so a run that stops at the
first failure has already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_long, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SPLIT = 128


def load():
    from rustingstrata_b200.kernels.build import compile_library
    lib = ctypes.CDLL(compile_library("core"))
    fn = lib.rs_attention_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_int, c_void_p,
                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int,
                   c_void_p, c_void_p]
    lib.rs_attention_decode_noalloc_error.restype = ctypes.c_char_p
    lib.rs_attention_decode_noalloc_capacity.restype = c_long
    return lib


def problem(seed, dtype, n_q, n_kv, hd, page, kv_lens, window):
    g = torch.Generator().manual_seed(seed)
    S = len(kv_lens)
    width = max((n + page - 1) // page for n in kv_lens)
    n_pages = S * width + 2
    table = torch.randperm(n_pages, generator=g)[: S * width].reshape(S, width).to(torch.int32).to(DEV)
    cache = torch.randn(n_pages, 2, n_kv, page, hd, generator=g).to(dtype).to(DEV)
    q = torch.randn(S, n_q * hd, generator=g).to(dtype).to(DEV)
    kv = np.asarray(kv_lens, np.int32)
    lo = np.maximum(0, kv - window) if window else np.zeros_like(kv)
    splits = (kv + SPLIT - 1) // SPLIT - lo // SPLIT
    start = np.zeros(S + 1, np.int32)
    start[1:] = np.cumsum(splits)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    return dict(q=q, cache=cache, table=table, q_start=d(np.arange(S + 1)), kv_len=d(kv), work=d(np.arange(S)),
                split_start=d(start), max_splits=int(splits.max()), total=int(start[-1]), S=S)


def call_noalloc(lib, pr, out, n_q, n_kv, hd, page, window, status):
    code = {torch.float32: 0, torch.bfloat16: 1}[pr["q"].dtype]
    p = lambda t: c_void_p(t.data_ptr())  # noqa: E731
    return lib.rs_attention_decode_noalloc(
        p(pr["q"]), pr["q"].stride(0), p(out), out.stride(0), code, p(pr["cache"]), pr["cache"].stride(0),
        pr["cache"].shape[0], page, p(pr["table"]), pr["table"].stride(0), p(pr["q_start"]), p(pr["kv_len"]), p(pr["work"]),
        pr["S"], n_q, n_kv, hd, window, 1.0 / math.sqrt(hd), SPLIT, pr["max_splits"], p(pr["split_start"]), pr["total"],
        p(status), c_void_p(torch.cuda.current_stream().cuda_stream))


def call_ordinary(pr, out, n_q, n_kv, hd, page, window, status):
    from rustingstrata_b200.kernels import ops
    partial = torch.empty(ops.attention_partial_floats(pr["total"], n_q, hd), device=DEV)
    ops.attention_simt(pr["q"], out, pr["cache"], pr["table"], pr["q_start"], pr["kv_len"], pr["work"], pr["S"], n_q, n_kv,
                       hd, page, window, 1.0 / math.sqrt(hd), True, status, split_keys=SPLIT, max_splits=pr["max_splits"],
                       split_start=pr["split_start"], total_splits=pr["total"], partial=partial)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(dtype):
    lib = load()
    torch.cuda.set_device(0)
    n_q, n_kv, hd, page = 8, 2, 64, 16
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # the second call is smaller than the first and has a window: it must not see what the first left behind
    for seed, kv_lens, window in ((1, [700, 129, 1, 300], 0), (2, [260, 90], 100)):
        pr = problem(seed, dtype, n_q, n_kv, hd, page, kv_lens, window)
        got = torch.zeros(pr["S"], n_q * hd, device=DEV, dtype=dtype)
        want = torch.zeros_like(got)
        rc = call_noalloc(lib, pr, got, n_q, n_kv, hd, page, window, status)
        assert rc == 0, lib.rs_attention_decode_noalloc_error().decode()
        call_ordinary(pr, want, n_q, n_kv, hd, page, window, status)
        torch.cuda.synchronize()
        assert status.item() == 0
        err = (got.double() - want.double()).abs().max().item() / want.double().abs().max().item()
        assert err <= (3e-6 if dtype == torch.float32 else 1.5e-2), err     # the kernel tests' tolerances
        assert torch.equal(got, want)          # same kernels, same order of sums: in fact identical


def test_requests_beyond_the_built_in_workspace_are_refused():
    lib = load()
    cap = lib.rs_attention_decode_noalloc_capacity()
    assert cap == 2 * 1024 * 1024
    n_q, n_kv, hd, page = 32, 8, 128, 16
    pr = problem(3, torch.bfloat16, n_q, n_kv, hd, page, [200], 0)
    pr["total"] = cap // (n_q * (hd + 2)) + 1                   # one split more than fits
    out = torch.zeros(1, n_q * hd, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = call_noalloc(lib, pr, out, n_q, n_kv, hd, page, 0, status)
    msg = lib.rs_attention_decode_noalloc_error().decode()
    assert rc == -2 and str(cap) in msg and "needs" in msg
    assert torch.all(out == 0)                                   # refused before anything ran
    pr["total"] = 2
    assert call_noalloc(lib, pr, out, n_q, n_kv, 24, page, 0, status) == -3      # head size the kernels refuse
    assert "multiple of 16" in lib.rs_attention_decode_noalloc_error().decode()


def test_a_split_list_that_points_beyond_the_workspace_is_flagged_not_written():
    """The function sees total_splits only; the first slot of each sequence lies in device memory.  A list that
    disagrees with total_splits (a slot beyond what the array holds for this shape) is caught by the kernels: the
    sequence's result is left alone and a status bit is set.  Nothing is written outside the array."""
    from rustingstrata_b200.kernels import ops
    lib = load()
    n_q, n_kv, hd, page = 8, 2, 64, 16
    pr = problem(4, torch.float32, n_q, n_kv, hd, page, [200, 300], 0)
    slots = lib.rs_attention_decode_noalloc_capacity() // (n_q * (hd + 2))
    good = torch.zeros(2, n_q * hd, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert call_noalloc(lib, pr, good, n_q, n_kv, hd, page, 0, status) == 0
    start = pr["split_start"].cpu().numpy().copy()
    start[1] = slots - 1                                       # the second sequence's splits would end past the array
    pr["split_start"] = torch.from_numpy(start).to(DEV)
    out = torch.full((2, n_q * hd), 7.0, device=DEV)
    assert call_noalloc(lib, pr, out, n_q, n_kv, hd, page, 0, status) == 0
    torch.cuda.synchronize()
    assert status.item() == ops.STATUS_BAD_PLAN
    assert torch.equal(out[0], good[0]) and torch.all(out[1] == 7.0)
    status.zero_()
