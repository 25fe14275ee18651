"""Times one kernel alone at a given shape, for profiling and tuning.

    python -m rustingstrata_b200.kernels.microbench KERNEL [--m M] [--n N] [--k K] [--batch B] [--ctx S] ...

KERNEL: skinny | mid | gemm | chain | decode_attention | prefill_attention | rmsnorm | qk_norm_rope | sample.
``chain``: the run of few-rows products between two attention calls of a decode step (output projection, norm, gate/up,
down projection, norm, next QKV; --k = hidden size, --n = feed-forward size, heads from --heads/--kv-heads/--head-dim)
as separate kernels and as one chained kernel.
The launches are captured in a CUDA graph and the replay is timed with CUDA events, so the figure is
device time per launch without host overhead; weights (or caches) rotate over buffers larger than the
L2 cache so every launch reads from HBM.  With ``--once`` it launches the kernel a few times without a
graph (what a profiler wants).  Prints one line: microseconds, and TB/s or TFLOP/s of the algorithmic
bytes or flops.
"""
from __future__ import annotations

import argparse
import math
import sys

import numpy as np
import torch

from . import ops

DEV = "cuda:0"


def timed(fn, n_bufs: int, iters: int, once: bool) -> float:
    for i in range(3):
        fn(i % n_bufs)
    torch.cuda.synchronize()
    if once:
        return float("nan")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i % n_bufs)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1000.0


def bench_linear(kind: str, M: int, N: int, K: int, epilogue: str, bn: int, iters: int, once: bool, then_norm: str = ""):
    nb = max(2, int(400e6 / (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(nb)]
    rows = max(M, 128)
    a = torch.randn(rows, K, device=DEV).to(torch.bfloat16)
    kw = {}
    if epilogue == "bf16":
        out = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16)
    elif epilogue == "f32":
        out = torch.zeros(rows, N, device=DEV)
    elif epilogue == "add":
        out, kw = torch.zeros(rows, N, device=DEV), dict(accumulate=True)
    else:
        out, kw = torch.zeros(rows, N // 2, device=DEV, dtype=torch.bfloat16), dict(swiglu=True)
    if kind in ("skinny", "mid") and then_norm:
        # the product into the residual stream and the row norm behind it: as two kernels and a small one between
        # them ("apart"), or with the norm adding up the product's shared tiles ("owed")
        nw = torch.ones(N, device=DEV, dtype=torch.bfloat16)
        h = torch.empty(rows, N, device=DEV, dtype=torch.bfloat16)

        def both(i):
            product = ops.skinny_gemm_bf16 if kind == "skinny" else ops.mid_gemm_bf16
            owed = product(a, ws[i], out, M, accumulate=True, defer=then_norm == "owed")
            ops.rmsnorm(out, nw, 1e-6, h, n_rows=M, pending=owed)
        us = timed(both, nb, iters, once)
        epilogue = f"add then norm ({then_norm})"
    elif kind == "skinny":
        us = timed(lambda i: ops.skinny_gemm_bf16(a, ws[i], out, M, **kw), nb, iters, once)
    elif kind == "mid":
        us = timed(lambda i: ops.mid_gemm_bf16(a, ws[i], out, M, **kw), nb, iters, once)
    else:
        us = timed(lambda i: ops.gemm_bf16_tc(a, ws[i], out, M, bn=bn, **kw), nb, iters, once)
    print(f"{kind} M={M} N={N} K={K} {epilogue}: {us:.1f} us, weights {N * K * 2 / us / 1e6:.2f} TB/s, "
          f"{2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")


def paged_problem(B: int, S: int, q_len: int, n_q: int, n_kv: int, hd: int, page: int, n_bufs: int):
    width = (S + page - 1) // page
    n_pages = B * width
    caches = [torch.randn(n_pages, 2, n_kv, page, hd, device=DEV).to(torch.bfloat16) for _ in range(n_bufs)]
    table = torch.randperm(n_pages, device=DEV).to(torch.int32).reshape(B, width)
    q = torch.randn(B * q_len, n_q * hd, device=DEV).to(torch.bfloat16)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    common = dict(q=q, out=torch.zeros_like(q), block_table=table, q_start=d(np.arange(B + 1) * q_len),
                  kv_len=d(np.full(B, S)), n_q=n_q, n_kv=n_kv, head_dim=hd, page_size=page, window=0,
                  scale=1 / math.sqrt(hd), status=torch.zeros(1, dtype=torch.int32, device=DEV))
    return caches, common, d


def bench_decode_attention(B, S, n_q, n_kv, hd, page, iters, once):
    from ..parts.attention import SPLIT_KEYS, decode_splits
    nb = max(1, min(8, int(400e6 / (B * S * n_kv * hd * 4)) + 1))
    caches, common, d = paged_problem(B, S, 1, n_q, n_kv, hd, page, nb)
    sp = decode_splits(np.full(B, S, np.int32), 0)
    ss = np.zeros(B + 1, np.int32)
    ss[1:] = np.cumsum(sp)
    partial = torch.empty(ops.attention_partial_floats(int(ss[-1]), n_q, hd), device=DEV)
    args = dict(work=d(np.arange(B)), n_work=B, split_keys=SPLIT_KEYS, max_splits=int(sp.max()), split_start=d(ss),
                total_splits=int(ss[-1]), partial=partial, **common)
    if ops.attention_decode_fast_ok(torch.bfloat16, n_q, n_kv, hd, page):
        # the list of items is built once per step and serves all its layers: not part of a layer's time
        args["items"] = torch.empty(int(ss[-1]) * n_kv, dtype=torch.int32, device=DEV)
        ops.attention_decode_items(args["split_start"], B, n_kv, args["max_splits"], args["items"])
    us = timed(lambda i: ops.attention_decode(cache=caches[i], **args), nb, iters, once)
    byts = B * S * n_kv * hd * 2 * 2
    print(f"decode_attention B={B} S={S} heads {n_q}/{n_kv} hd={hd} page={page}: {us:.1f} us, cache {byts / us / 1e6:.2f} TB/s, "
          f"{ops.attention_decode_loads_per_page()} TMA load(s) per page")


def bench_prefill_attention(S, n_q, n_kv, hd, page, iters, once, force=""):
    caches, common, d = paged_problem(1, S, S, n_q, n_kv, hd, page, 1)
    qpc = ops.attention_prefill_q_per_cta(torch.bfloat16, n_q, n_kv, hd, page, force)
    tiles = np.array([(0, o) for o in range(0, S, qpc)][::-1], np.int32).reshape(-1)     # longest first, as the mixer plans
    args = dict(work=d(tiles), n_work=len(tiles) // 2, **common)
    us = timed(lambda i: ops.attention_prefill(cache=caches[0], force=force, **args), 1, iters, once)
    kind = ops.attention_prefill_kernel(torch.bfloat16, n_q, n_kv, hd, page, force)
    print(f"prefill_attention [{kind}] S={S} heads {n_q}/{n_kv} hd={hd} page={page}: {us:.1f} us, {4.0 * n_q * hd * S * S / 2 / us / 1e6:.1f} "
          f"TFLOP/s (causal half counted)")


def bench_chain(M: int, hidden: int, inter: int, n_q: int, n_kv: int, hd: int, iters: int):
    """One layer's products at M rows: the kernels one by one against the chained kernel, each timed as a graph of
    `iters` runs; the layer's weights (larger than L2 at real sizes) are read from HBM every time."""
    g = torch.Generator(device=DEV).manual_seed(0)
    r = lambda *s: torch.randn(*s, device=DEV, generator=g)  # noqa: E731
    Q, KV = n_q * hd, n_kv * hd
    t = dict(attn=r(8, Q).to(torch.bfloat16), wo=(r(hidden, Q) * 0.03).to(torch.bfloat16), res=r(8, hidden),
             n1=torch.ones(hidden, device=DEV, dtype=torch.bfloat16), wgu=(r(2 * inter, hidden) * 0.03).to(torch.bfloat16),
             wd=(r(hidden, inter) * 0.03).to(torch.bfloat16), n2=torch.ones(hidden, device=DEV, dtype=torch.bfloat16),
             wqkv=(r(Q + 2 * KV, hidden) * 0.03).to(torch.bfloat16),
             h=torch.zeros(8, hidden, device=DEV, dtype=torch.bfloat16), act=torch.zeros(8, inter, device=DEV, dtype=torch.bfloat16),
             h2=torch.zeros(8, hidden, device=DEV, dtype=torch.bfloat16), qkv=torch.zeros(8, Q + 2 * KV, device=DEV, dtype=torch.bfloat16))
    st = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run(chained: bool, norms: bool):
        if chained:
            ops.begin_chain(st)
        owed = ops.linear(t["attn"], t["wo"], t["res"], M, accumulate=True, status=st, may_defer=norms)
        if norms:
            ops.rmsnorm(t["res"], t["n1"], 1e-6, t["h"], n_rows=M, pending=owed)
        ops.linear_swiglu(t["h"], t["wgu"], t["act"], M, status=st)
        owed = ops.linear(t["act"], t["wd"], t["res"], M, accumulate=True, status=st, may_defer=norms)
        if norms:
            ops.rmsnorm(t["res"], t["n2"], 1e-6, t["h2"], n_rows=M, pending=owed)
        ops.linear(t["h2"], t["wqkv"], t["qkv"], M, status=st)
        if chained:
            ops.end_chain()
    mb = sum(t[k].numel() * 2 for k in ("wo", "wgu", "wd", "wqkv")) / 1e6
    for name, norms in (("four products", False), ("products and the two norms between them", True)):
        a = timed(lambda i: run(False, norms), 1, iters, False)
        b = timed(lambda i: run(True, norms), 1, iters, False)
        print(f"chain M={M} hidden={hidden} ffn={inter} ({mb:.0f} MB of weights): {name}: separate kernels {a:.1f} us "
              f"({mb / a / 1e6 * 1e6:.2f} TB/s), chained {b:.1f} us ({mb / b / 1e6 * 1e6:.2f} TB/s)")
    assert st.item() == 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("kernel", choices=["skinny", "mid", "gemm", "chain", "decode_attention", "prefill_attention", "rmsnorm", "qk_norm_rope",
                                       "sample"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--epilogue", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--force", default="", help="prefill_attention: tc | mma | simt instead of the default choice")
    ap.add_argument("--then-norm", default="", choices=["", "apart", "owed"],
                    help="skinny or mid with --epilogue add: time the product together with the RMSNorm of its rows")
    ap.add_argument("--once", action="store_true", help="a few plain launches, no graph and no timing (for profilers)")
    a = ap.parse_args(argv)
    if a.kernel in ("skinny", "mid", "gemm"):
        bench_linear(a.kernel, a.m, a.n, a.k, a.epilogue, a.bn, a.iters, a.once, a.then_norm)
    elif a.kernel == "chain":
        bench_chain(a.m, a.k, a.n, a.heads, a.kv_heads, a.head_dim, min(a.iters, 20))
    elif a.kernel == "decode_attention":
        bench_decode_attention(a.batch, a.ctx, a.heads, a.kv_heads, a.head_dim, a.page_size, a.iters, a.once)
    elif a.kernel == "prefill_attention":
        bench_prefill_attention(a.ctx, a.heads, a.kv_heads, a.head_dim, a.page_size, a.iters, a.once, a.force)
    elif a.kernel == "rmsnorm":
        x = torch.randn(a.m, a.k, device=DEV)
        w = torch.ones(a.k, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(a.m, a.k, device=DEV, dtype=torch.bfloat16)
        print(f"rmsnorm rows={a.m} width={a.k}: {timed(lambda i: ops.rmsnorm(x, w, 1e-6, o), 1, a.iters, a.once):.1f} us")
    elif a.kernel == "qk_norm_rope":
        T, nq, nkv, hd = a.m, a.heads, a.kv_heads, a.head_dim
        qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
        w = torch.ones(hd, device=DEV, dtype=torch.bfloat16)
        cs = torch.randn(4096, hd, device=DEV)
        pos = torch.full((T,), 100, dtype=torch.int32, device=DEV)
        sq = torch.arange(T, dtype=torch.int32, device=DEV)
        tb = torch.arange(T * 8, dtype=torch.int32, device=DEV).reshape(T, 8)
        cache = torch.zeros(T * 8, 2, nkv, 16, hd, device=DEV, dtype=torch.bfloat16)
        st = torch.zeros(1, dtype=torch.int32, device=DEV)
        us = timed(lambda i: ops.qk_norm_rope_kv(qkv, T, nq, nkv, hd, w, w, 1e-6, cs, hd, pos, sq, tb, 16, cache, True, st), 1,
                   a.iters, a.once)
        print(f"qk_norm_rope tokens={T}: {us:.1f} us")
    else:
        lg = torch.randn(a.m, a.vocab, device=DEV)
        o = torch.zeros(a.m, dtype=torch.int32, device=DEV)
        st = torch.zeros(1, dtype=torch.int32, device=DEV)
        print(f"sample rows={a.m} vocab={a.vocab}: {timed(lambda i: ops.sample(lg, a.m, o, st), 1, a.iters, a.once):.1f} us")
    return 0


if __name__ == "__main__":
    sys.exit(main())
