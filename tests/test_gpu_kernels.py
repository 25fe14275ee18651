"""Each CUDA kernel alone against a plain reference of the same operation, at sizes other than the
engine's tiny configurations: widths and vocabularies that are no power of two, head sizes in steps
of 16, any number of heads and groups, several page sizes."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from rustingstrata_b200.kernels import ops as o
    return o


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def tol(dtype, f32=2e-6, bf16=1e-2):
    return f32 if dtype == torch.float32 else bf16


def close(got, want, rel):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= rel, f"relative error {err:.3e} > {rel:.1e}"


# ------------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    V, H, T = 1003, 72, 37
    table = torch.randn(V, H, device=DEV).to(dtype)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    ids[0], ids[1] = 0, V - 1
    out = torch.empty(T, H, device=DEV)
    st = status()
    ops().embed(table, ids, out, st)
    assert torch.equal(out, table[ids.long()].float()) and st.item() == 0
    ids[3] = V
    ops().embed(table, ids, out, st)
    assert st.item() & ops().STATUS_BAD_TOKEN          # flagged, not a fault


# ------------------------------------------------------------------------------- RMSNorm
@pytest.mark.parametrize("n", [48, 100, 1000, 4096, 5120])
@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("w_dtype", DTYPES)
def test_rmsnorm(n, out_dtype, w_dtype):
    rows, eps = 13, 1e-5
    x = torch.randn(rows, n, device=DEV) * 3
    w = (1 + 0.1 * torch.randn(n, device=DEV)).to(w_dtype)
    out = torch.empty(rows, n, device=DEV, dtype=out_dtype)
    ops().rmsnorm(x, w, eps, out)
    xd = x.double()
    want = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps) * w.double()
    close(out, want, tol(out_dtype, 1e-6, 5e-3))


def test_rmsnorm_gathers_rows_and_respects_strides():
    n = 200
    big = torch.randn(9, 256, device=DEV)
    x = big[:, :n]                                        # row stride 256
    w = torch.ones(n, device=DEV)
    rows = torch.tensor([7, 2, 2, 0], dtype=torch.int32, device=DEV)
    out = torch.full((6, n), 7.0, device=DEV)
    ops().rmsnorm(x, w, 1e-6, out, rows=rows, n_rows=4)
    xd = x.double()[rows.long()]
    close(out[:4], xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-6), 1e-6)
    assert torch.all(out[4:] == 7.0)                      # rows beyond n_rows untouched


# ------------------------------------------------------------------------------- matrix product
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 130, 77), (67, 250, 96), (130, 515, 200), (3, 1003, 4096)])
@pytest.mark.parametrize("a_dt,w_dt,o_dt", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                            (torch.bfloat16, torch.bfloat16, torch.float32),
                                            (torch.bfloat16, torch.float32, torch.bfloat16)])
def test_linear_simt(M, N, K, a_dt, w_dt, o_dt):
    a = torch.randn(M + 2, K, device=DEV).to(a_dt)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(w_dt)
    out = torch.full((M + 2, N), 5.0, device=DEV, dtype=o_dt)
    ops().linear_simt(a, w, out, M)
    want = a[:M].double() @ w.double().T
    # float32 running sum over K terms: rounding grows like sqrt(K) * 2^-24 of the terms' size
    f32_tol = 4 * math.sqrt(K) * 2.0 ** -24
    close(out[:M], want, tol(o_dt, f32_tol, 6e-3))
    assert torch.all(out[M:] == 5.0)
    if o_dt == torch.float32:
        base = torch.randn(M + 2, N, device=DEV)
        acc = base.clone()
        ops().linear_simt(a, w, acc, M, accumulate=True)
        close(acc[:M], base[:M].double() + want, f32_tol)


def test_linear_row_result_does_not_depend_on_the_batch():
    """Row 3 of a 50-row product equals the same row computed alone, bit for bit."""
    K, N = 300, 130
    a = torch.randn(50, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    full = torch.empty(50, N, device=DEV)
    one = torch.empty(1, N, device=DEV)
    ops().linear_simt(a, w, full, 50)
    ops().linear_simt(a[3:4].contiguous(), w, one, 1)
    assert torch.equal(full[3], one[0])


# ------------------------------------------------------------------------------- SiLU * up
@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    rows, I = 11, 250
    gu = (torch.randn(rows, 2 * I, device=DEV) * 4).to(dtype)
    out = torch.empty(rows, I, device=DEV, dtype=dtype)
    ops().silu_mul(gu, out, rows)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    close(out, g / (1 + torch.exp(-g)) * u, tol(dtype, 1e-6, 5e-3))


# ------------------------------------------------------------------------------- QK-norm + RoPE + cache write
def rope_table(n_pos, n_rot, base):
    i = np.arange(n_rot // 2, dtype=np.float64)
    th = np.arange(n_pos, dtype=np.float64)[:, None] * np.power(np.float64(np.float32(base)), -2.0 * i / n_rot)[None]
    return torch.from_numpy(np.concatenate([np.cos(th), np.sin(th)], 1).astype(np.float32)).to(DEV)


def ref_norm_rope(x, w, eps, pos, n_rot, base):
    """x [T, heads, hd] float64; per-head RMSNorm then NEOX rotation (src/ops.rs:3-7,36-45)."""
    if w is not None:
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
    half = n_rot // 2
    tab = rope_table(int(pos.max()) + 1, n_rot, base).double().cpu()[pos.long().cpu()]
    c, s = tab[:, None, :half], tab[:, None, half:]
    a, b = x[..., :half], x[..., half:n_rot]
    return torch.cat([a * c - b * s, a * s + b * c, x[..., n_rot:]], -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd,n_rot,page", [(4, 2, 16, 16, 4), (5, 1, 48, 48, 8), (6, 3, 80, 64, 5),
                                                  (8, 8, 128, 128, 16), (2, 1, 256, 256, 16)])
def test_qk_norm_rope_kv_write(dtype, n_q, n_kv, hd, n_rot, page):
    o = ops()
    eps, base = 1e-5, 12345.0
    q_lens, starts = [5, 1, 9], [3, 40, 0]                # three sequences at different positions
    T = sum(q_lens)
    n_pages = 40
    positions = torch.tensor([s + i for n, s in zip(q_lens, starts) for i in range(n)], dtype=torch.int32, device=DEV)
    seq_of = torch.tensor([k for k, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    width = max((s + n + page - 1) // page for n, s in zip(q_lens, starts))
    perm = torch.randperm(n_pages)[: 3 * width].reshape(3, width).to(torch.int32)
    table = perm.to(DEV)
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV).to(dtype)
    src = qkv.clone()
    qw = (1 + 0.2 * torch.randn(hd, device=DEV)).to(dtype)
    kw = (1 + 0.2 * torch.randn(hd, device=DEV)).to(dtype)
    cache = torch.zeros(n_pages, 2, n_kv, page, hd, device=DEV, dtype=dtype)
    st = status()
    o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, qw, kw, eps, rope_table(64, n_rot, base), n_rot, positions, seq_of,
                      table, page, cache, True, st)
    assert st.item() == 0
    s64 = src.double().cpu()
    q_ref = ref_norm_rope(s64[:, : n_q * hd].reshape(T, n_q, hd), qw.cpu(), eps, positions, n_rot, base)
    k_ref = ref_norm_rope(s64[:, n_q * hd:(n_q + n_kv) * hd].reshape(T, n_kv, hd), kw.cpu(), eps, positions, n_rot, base)
    v_ref = s64[:, (n_q + n_kv) * hd:].reshape(T, n_kv, hd)
    close(qkv[:, : n_q * hd].reshape(T, n_q, hd), q_ref, tol(dtype, 2e-6, 8e-3))
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(T):
        pos, sq = int(positions[t]), int(seq_of[t])
        pg = int(perm[sq, pos // page])
        written[pg, pos % page] = True
        close(cache[pg, 0, :, pos % page], k_ref[t], tol(dtype, 2e-6, 8e-3))
        assert torch.equal(cache[pg, 1, :, pos % page].cpu(), src[t, (n_q + n_kv) * hd:].reshape(n_kv, hd).cpu())
    untouched = cache.cpu().permute(0, 3, 1, 2, 4)[~written]
    assert torch.all(untouched == 0)                       # nothing outside the tokens' own slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd,n_rot,page", [(4, 2, 16, 16, 4), (8, 2, 128, 128, 16), (6, 3, 80, 64, 5)])
def test_rotation_follows_the_named_position_stream(dtype, n_q, n_kv, hd, n_rot, page):
    """A token carries three position values; the cache place is stream 0 whatever stream the rotation follows.  A
    stream value outside the rotation table is flagged, and that token is left alone."""
    o = ops()
    eps, base, T, n_pages = 1e-5, 777.0, 11, 8
    place = torch.arange(20, 20 + T, dtype=torch.int32)
    streams = torch.stack([place, (place * 7) % 50, 49 - torch.arange(T, dtype=torch.int32)], dim=1).contiguous()
    seq_of = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.randperm(n_pages)[None, : (20 + T + page - 1) // page + 1].to(torch.int32)
    src = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV).to(dtype)
    qw = (1 + 0.2 * torch.randn(hd, device=DEV)).to(dtype)
    kw = (1 + 0.2 * torch.randn(hd, device=DEV)).to(dtype)
    n_pages = int(table.max()) + 1
    for stream in (0, 1, 2):
        qkv = src.clone()
        cache = torch.zeros(n_pages, 2, n_kv, page, hd, device=DEV, dtype=dtype)
        st = status()
        o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, qw, kw, eps, rope_table(50, n_rot, base), n_rot, streams.to(DEV), seq_of,
                          table.to(DEV), page, cache, True, st, stream=stream)
        assert st.item() == 0
        s64 = src.double().cpu()
        q_ref = ref_norm_rope(s64[:, : n_q * hd].reshape(T, n_q, hd), qw.cpu(), eps, streams[:, stream], n_rot, base)
        k_ref = ref_norm_rope(s64[:, n_q * hd:(n_q + n_kv) * hd].reshape(T, n_kv, hd), kw.cpu(), eps, streams[:, stream], n_rot, base)
        close(qkv[:, : n_q * hd].reshape(T, n_q, hd), q_ref, tol(dtype, 2e-6, 8e-3))
        for t in range(T):
            pos = int(place[t])
            close(cache[int(table[0, pos // page]), 0, :, pos % page], k_ref[t], tol(dtype, 2e-6, 8e-3))
    bad = streams.clone()
    bad[3, 1] = 50                                            # one row beyond the table of 50
    qkv = src.clone()
    st = status()
    o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, qw, kw, eps, rope_table(50, n_rot, base), n_rot, bad.to(DEV), seq_of,
                      table.to(DEV), page, torch.zeros(n_pages, 2, n_kv, page, hd, device=DEV, dtype=dtype), True, st, stream=1)
    assert st.item() == o.STATUS_BAD_PLAN
    assert torch.equal(qkv[3, : n_q * hd], src[3, : n_q * hd]) and not torch.equal(qkv[4], src[4])
    with pytest.raises(o.KernelError, match="stream"):
        o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, qw, kw, eps, rope_table(50, n_rot, base), n_rot, streams.to(DEV), seq_of,
                          table.to(DEV), page, torch.zeros(n_pages, 2, n_kv, page, hd, device=DEV, dtype=dtype), True, st, stream=3)


def test_qk_without_norm_without_rope_and_without_kv():
    o = ops()
    T, n_q, n_kv, hd, page = 4, 2, 1, 32, 4
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV)
    src = qkv.clone()
    cache = torch.zeros(4, 2, n_kv, page, hd, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.tensor([[2]], dtype=torch.int32, device=DEV)
    o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, None, None, 0.0, None, 0, pos, seq, table, page, cache, False, status())
    assert torch.equal(qkv, src) and torch.all(cache == 0)          # a reader of another call's cache writes nothing
    o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, None, None, 0.0, None, 0, pos, seq, table, page, cache, True, status())
    assert torch.equal(cache[2, 0, 0], src[:, n_q * hd:(n_q + 1) * hd]) and torch.equal(cache[2, 1, 0], src[:, -hd:])
    bad = torch.tensor([[9]], dtype=torch.int32, device=DEV)
    st = status()
    o.qk_norm_rope_kv(qkv, T, n_q, n_kv, hd, None, None, 0.0, None, 0, pos, seq, bad, page, cache, True, st)
    assert st.item() & o.STATUS_BAD_PAGE                            # flagged, not a fault


# ------------------------------------------------------------------------------- attention
def ref_attention(q, keys, vals, q_pos, n_kv, window, scale):
    """q [nq, hd] at position q_pos over keys/vals [L, nkv, hd] (float64): src/model.rs:778-791."""
    nq = q.shape[0]
    lo = max(0, q_pos - window + 1) if window else 0
    out = torch.zeros_like(q)
    for h in range(nq):
        g = h // (nq // n_kv)
        s = (keys[lo:q_pos + 1, g] @ q[h]) * scale
        p = torch.softmax(s, 0)
        out[h] = p @ vals[lo:q_pos + 1, g]
    return out


def run_attention(dtype, n_q, n_kv, hd, page, seqs, window=0, scale=None, boost=None, force_simt=False, prefill=""):
    """seqs: list of (kv_len, q_len).  Builds a shuffled paged cache, runs the kernels the mixer would
    run (split form for one query, tile form otherwise) and returns (got, want) [T, n_q, hd]."""
    o = ops()
    scale = scale or 1.0 / math.sqrt(hd)
    S = len(seqs)
    T = sum(q for _, q in seqs)
    width = max((kv + page - 1) // page for kv, _ in seqs)
    n_pages = S * width + 3
    perm = torch.randperm(n_pages)[: S * width].reshape(S, width).to(torch.int32)
    cache = torch.zeros(n_pages, 2, n_kv, page, hd, device=DEV, dtype=dtype)
    keys, vals = [], []
    for s, (kv, _) in enumerate(seqs):
        k = torch.randn(kv, n_kv, hd).to(dtype)
        v = torch.randn(kv, n_kv, hd).to(dtype)
        if boost is not None:
            boost(s, k)
        keys.append(k.double())
        vals.append(v.double())
        for p in range(kv):
            cache[perm[s, p // page], 0, :, p % page] = k[p].to(DEV)
            cache[perm[s, p // page], 1, :, p % page] = v[p].to(DEV)
    q = torch.randn(T, n_q * hd).to(dtype)
    if boost is not None:
        boost(None, q.view(T, n_q, hd))
    qd = q.to(DEV)
    out = torch.zeros(T, n_q * hd, device=DEV, dtype=dtype)
    q_lens = np.array([ql for _, ql in seqs], np.int32)
    kv_lens = np.array([kv for kv, _ in seqs], np.int32)
    q_start = np.zeros(S + 1, np.int32)
    q_start[1:] = np.cumsum(q_lens)
    from rustingstrata_b200.parts.attention import SPLIT_KEYS, decode_splits
    prefill = "simt" if force_simt else prefill
    qpc = o.attention_prefill_q_per_cta(dtype, n_q, n_kv, hd, page, prefill)
    dec = np.nonzero(q_lens == 1)[0].astype(np.int32)
    tiles = [(s, off) for s in np.nonzero(q_lens != 1)[0] for off in range(0, q_lens[s], qpc)]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    st = status()
    common = dict(q=qd, out=out, cache=cache, block_table=perm.to(DEV), q_start=dev(q_start), kv_len=dev(kv_lens),
                  n_q=n_q, n_kv=n_kv, head_dim=hd, page_size=page, window=window, scale=scale, status=st)
    if tiles:
        o.attention_prefill(work=dev(np.array(tiles).reshape(-1)), n_work=len(tiles), force=prefill, **common)
    if len(dec):
        splits = decode_splits(kv_lens[dec], window)
        ss = np.zeros(len(dec) + 1, np.int32)
        ss[1:] = np.cumsum(splits)
        partial = torch.empty(o.attention_partial_floats(int(ss[-1]), n_q, hd), device=DEV)
        o.attention_decode(work=dev(dec), n_work=len(dec), split_keys=SPLIT_KEYS, max_splits=int(splits.max()),
                           split_start=dev(ss), total_splits=int(ss[-1]), partial=partial, force_simt=force_simt, **common)
    assert st.item() == 0
    want = torch.zeros(T, n_q, hd, dtype=torch.float64)
    for s, (kv, ql) in enumerate(seqs):
        for i in range(ql):
            t = q_start[s] + i
            want[t] = ref_attention(q[t].double().view(n_q, hd), keys[s], vals[s], kv - ql + i, n_kv, window, scale)
    return out.view(T, n_q, hd), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd,page", [(4, 2, 16, 4), (5, 1, 48, 8), (6, 2, 80, 5), (8, 2, 128, 16),
                                              (32, 8, 128, 16), (3, 3, 256, 16), (40, 2, 64, 16)])
def test_attention_portions_and_single_queries(dtype, n_q, n_kv, hd, page):
    seqs = [(37, 37), (300, 1), (65, 20), (1, 1), (129, 1), (200, 33), (128, 2)]
    got, want = run_attention(dtype, n_q, n_kv, hd, page, seqs)
    close(got, want, tol(dtype, 3e-6, 1.5e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 32, 100, 129])
def test_attention_window_edge(dtype, window):
    seqs = [(150, 150), (300, 1), (140, 31), (window, 1), (window + 1, 1), (257, 1)]
    got, want = run_attention(dtype, 4, 2, 32, 8, seqs, window=window)
    close(got, want, tol(dtype, 3e-6, 1.5e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 127, 128, 255, 511, 600])
def test_attention_finds_a_far_key_among_hundreds(dtype, far):
    """One key far back is made to dominate: the output must be (nearly) that key's value, so a kernel that
    skips a page, a split or a tile edge is caught even though random scores would hide it."""
    hd = 64

    def boost(s, t):
        if s is None:
            t[:, :, 0] = 6.0                  # every query points along dim 0
        else:
            t[:, :, 0] = 0.0
            t[far, :, 0] = 40.0               # only key `far` answers
    seqs = [(700, 1), (700, 64), (far + 1, 1)]
    got, want = run_attention(dtype, 4, 2, hd, 16, seqs, boost=boost)
    close(got, want, tol(dtype, 3e-6, 1.5e-2))
    assert (got[0].double().cpu() - want[0]).abs().max() < 0.05


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window", [116, 128, 100, 77])
@pytest.mark.parametrize("inside", [True, False])
def test_window_edge_in_the_tensor_core_kernels(hd, window, inside):
    """The tcgen05 portion kernel and the TMA-fed single-query kernel (head 64/128, pages of 16, bfloat16) with one key
    that answers every query, placed on the oldest position a window still shows (it must carry the result) or one
    before it (it must not be seen at all).  The lengths put that edge on a boundary between 128-key splits and between
    pages (500 keys, window 116: key 384), on a page boundary only (window 100: key 400), and inside a page."""
    o = ops()
    n_q, n_kv, page = 8, 2, 16
    assert o.attention_prefill_kernel(torch.bfloat16, n_q, n_kv, hd, page) == "tc"
    assert o.attention_decode_fast_ok(torch.bfloat16, n_q, n_kv, hd, page)
    # (keys, queries): single queries at three lengths, and a portion whose queries straddle the marked key's edge
    seqs = [(500, 1), (1024 + window, 1), (window + 7, 1), (700, 64), (300, 150)]
    edge = [kv - ql - window + 1 if ql > 1 else kv - window for kv, ql in seqs]       # oldest key the first query sees
    marked = [e + (20 if ql > 1 else 0) - (0 if inside else 1) for e, (kv, ql) in zip(edge, seqs)]

    def boost(s, t):
        if s is None:
            t[:, :, 0] = 6.0
        else:
            t[:, :, 0] = 0.0
            t[marked[s], :, 0] = 40.0
    got, want = run_attention(torch.bfloat16, n_q, n_kv, hd, page, seqs, window=window, boost=boost)
    close(got, want, 1.5e-2)
    # the construction bites: for the single queries the marked key either is the answer or is not there
    starts = np.cumsum([0] + [ql for _, ql in seqs])
    for s, (kv, ql) in enumerate(seqs[:3]):
        w = want[starts[s]]
        assert (got[starts[s]].double().cpu() - w).abs().max() < 0.05
    # in a portion, the marked key is seen by the first queries and has left the window of the later ones
    for s in (3, 4):
        kv, ql = seqs[s]
        first_pos = kv - ql
        sees = [marked[s] > first_pos + i - window and marked[s] <= first_pos + i for i in range(ql)]
        assert any(sees) and not all(sees)


@pytest.mark.parametrize("n_q,n_kv,hd,page", [(8, 2, 128, 16), (32, 8, 128, 16), (16, 1, 64, 8), (9, 1, 64, 16), (3, 3, 128, 32),
                                              (4, 1, 64, 128), (12, 4, 64, 64), (16, 1, 128, 8)])
@pytest.mark.parametrize("window", [0, 100])
def test_decode_tensor_core_kernel_agrees_with_the_cuda_core_kernel(n_q, n_kv, hd, page, window):
    from rustingstrata_b200.kernels import ops as o
    assert o.attention_decode_fast_ok(torch.bfloat16, n_q, n_kv, hd, page)
    assert not o.attention_decode_fast_ok(torch.float32, n_q, n_kv, hd, page)
    assert not o.attention_decode_fast_ok(torch.bfloat16, 34, 2, 64, 16) and not o.attention_decode_fast_ok(torch.bfloat16, 4, 2, 48, 16)
    assert not o.attention_decode_fast_ok(torch.bfloat16, 4, 2, 64, 4) and not o.attention_decode_fast_ok(torch.bfloat16, 4, 2, 64, 24)
    seqs = [(1, 1), (127, 1), (128, 1), (129, 1), (300, 1), (1000, 1), (16, 1), (2048, 1)]
    torch.manual_seed(3)
    fast, want = run_attention(torch.bfloat16, n_q, n_kv, hd, page, seqs, window=window)
    torch.manual_seed(3)
    slow, _ = run_attention(torch.bfloat16, n_q, n_kv, hd, page, seqs, window=window, force_simt=True)
    close(fast, want, 1.5e-2)
    close(fast, slow.double().cpu(), 1.5e-2)


def test_decode_item_list_names_every_live_split_once():
    """The list the tensor-core decode kernel walks: sequence w owns the ids from split_start[w] * n_kv, split fastest,
    then kv head; splits beyond a sequence's own (the launch shape is rounded up) leave no entry."""
    o = ops()
    n_kv, splits = 3, np.array([4, 1, 0, 7, 2], np.int32)
    start = np.zeros(len(splits) + 1, np.int32)
    start[1:] = np.cumsum(splits)
    items = torch.full((int(start[-1]) * n_kv + 5,), -1, dtype=torch.int32, device=DEV)
    o.attention_decode_items(torch.from_numpy(start).to(DEV), len(splits), n_kv, 16, items)
    got = items.cpu().numpy()
    want = [(w << 20) | (h << 12) | s for w, n in enumerate(splits) for h in range(n_kv) for s in range(n)]
    assert got[:len(want)].tolist() == want and (got[len(want):] == -1).all()
    with pytest.raises(Exception, match="int32"):
        o.attention_decode_items(torch.from_numpy(start).to(DEV), len(splits), n_kv, 16, items.float())


def test_decode_result_of_a_long_sequence_does_not_depend_on_the_batch_around_it():
    """A 5,000-key sequence alone (the merge kernel runs four threads per head dim) and beside 150 short ones (one
    thread per head dim, and its items land on other CTAs): the same bits."""
    from rustingstrata_b200.parts.attention import SPLIT_KEYS, decode_splits
    o = ops()
    n_q, n_kv, hd, page, long_kv = 8, 2, 64, 16, 5000
    g = torch.Generator().manual_seed(11)
    width = (long_kv + page - 1) // page
    n_pages = width + 150 * 2
    cache = (torch.randn(n_pages, 2, n_kv, page, hd, generator=g)).to(torch.bfloat16).to(DEV)
    q_all = torch.randn(151, n_q * hd, generator=g).to(torch.bfloat16).to(DEV)
    table = torch.zeros(151, width, dtype=torch.int32)
    table[0] = torch.arange(width, dtype=torch.int32)
    for s in range(1, 151):
        table[s, :2] = torch.tensor([width + 2 * (s - 1), width + 2 * (s - 1) + 1], dtype=torch.int32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    outs = []
    for n in (1, 151):
        kv_lens = np.array([long_kv] + [20] * (n - 1), np.int32)
        splits = decode_splits(kv_lens, 0)
        ss = np.zeros(n + 1, np.int32)
        ss[1:] = np.cumsum(splits)
        out = torch.zeros(n, n_q * hd, device=DEV, dtype=torch.bfloat16)
        st = status()
        o.attention_decode(q=q_all[:n].contiguous(), out=out, cache=cache, block_table=table[:n].contiguous().to(DEV),
                           q_start=dev(np.arange(n + 1)), kv_len=dev(kv_lens), work=dev(np.arange(n)), n_work=n, n_q=n_q,
                           n_kv=n_kv, head_dim=hd, page_size=page, window=0, scale=1 / math.sqrt(hd), status=st,
                           split_keys=SPLIT_KEYS, max_splits=int(splits.max()), split_start=dev(ss), total_splits=int(ss[-1]),
                           partial=torch.empty(o.attention_partial_floats(int(ss[-1]), n_q, hd), device=DEV))
        assert st.item() == 0
        outs.append(out[0].clone())
    assert torch.equal(outs[0], outs[1])
    k = cache[:width, 0].permute(0, 2, 1, 3).reshape(width * page, n_kv, hd)[:long_kv].double().cpu()
    v = cache[:width, 1].permute(0, 2, 1, 3).reshape(width * page, n_kv, hd)[:long_kv].double().cpu()
    want = ref_attention(q_all[0].double().cpu().view(n_q, hd), k, v, long_kv - 1, n_kv, 0, 1 / math.sqrt(hd))
    close(outs[0].view(1, n_q, hd), want.view(1, n_q, hd), 1.5e-2)


@pytest.mark.parametrize("n_q,n_kv,hd,page", [(8, 2, 128, 16), (32, 8, 128, 16), (6, 2, 32, 4), (16, 1, 64, 8), (3, 3, 96, 16),
                                              (10, 2, 64, 16), (40, 1, 64, 16)])
@pytest.mark.parametrize("window", [0, 70])
def test_prefill_tensor_core_kernel_agrees_with_the_cuda_core_kernel(n_q, n_kv, hd, page, window):
    from rustingstrata_b200.kernels import ops as o
    assert o.attention_prefill_fast_ok(torch.bfloat16, n_q, n_kv, hd) and not o.attention_prefill_fast_ok(torch.float32, n_q, n_kv, hd)
    seqs = [(37, 37), (300, 2), (65, 20), (64, 64), (129, 128), (200, 33), (128, 2), (700, 257), (2, 2), (1000, 3)]
    torch.manual_seed(4)
    fast, want = run_attention(torch.bfloat16, n_q, n_kv, hd, page, seqs, window=window, prefill="mma")
    torch.manual_seed(4)
    slow, _ = run_attention(torch.bfloat16, n_q, n_kv, hd, page, seqs, window=window, force_simt=True)
    close(fast, want, 1.5e-2)
    close(fast, slow.double().cpu(), 1.5e-2)


@pytest.mark.parametrize("n_q,n_kv,hd,page", [(8, 2, 128, 16), (32, 8, 128, 16), (16, 1, 64, 8), (10, 2, 64, 16), (3, 3, 128, 32),
                                              (4, 1, 64, 128)])
@pytest.mark.parametrize("window", [0, 70, 200])
def test_prefill_tcgen05_kernel(n_q, n_kv, hd, page, window):
    from rustingstrata_b200.kernels import ops as o
    assert o.attention_prefill_kernel(torch.bfloat16, n_q, n_kv, hd, page) == "tc"
    assert o.attention_prefill_kernel(torch.bfloat16, n_q, n_kv, hd, 4) == "mma"
    assert o.attention_prefill_kernel(torch.float32, n_q, n_kv, hd, page) == "simt"
    seqs = [(37, 37), (300, 2), (65, 20), (128, 128), (129, 128), (200, 33), (256, 2), (700, 257), (2, 2), (1000, 3), (513, 200)]
    torch.manual_seed(6)
    fast, want = run_attention(torch.bfloat16, n_q, n_kv, hd, page, seqs, window=window, prefill="tc")
    close(fast, want, 1.5e-2)


@pytest.mark.parametrize("prefill", ["tc", "mma", "simt"])
def test_prefill_when_every_block_of_keys_raises_the_maximum(prefill):
    """Scores that grow with the key's position (by more than 2^8 per 128 keys): the running maximum moves at every
    block, so the accumulated result is rescaled every time, in the kernels that keep it in tensor memory too."""
    hd = 128
    scale = 1.0 / math.sqrt(hd)

    def boost(s, t):
        if s is None:
            t[:, :, 0] = 1.0 / scale                      # queries: the first dim picks the keys' ramp up
        else:
            t[:, :, 0] = 0.1 * torch.arange(t.shape[0], dtype=torch.float32).to(t.dtype)[:, None]
    torch.manual_seed(11)
    seqs = [(700, 257), (1500, 300), (129, 129)]
    fast, want = run_attention(torch.bfloat16, 8, 2, hd, 16, seqs, boost=boost, prefill=prefill)
    close(fast, want, 1.5e-2)


def test_prefill_tcgen05_kernel_beyond_the_items_it_keeps_in_shared_memory():
    """A portion so long that a persistent CTA walks more items than it describes up front in shared memory (64): the
    later ones are worked out when they are met.  Against the mma.sync kernel on the same 40,000 tokens."""
    o = ops()
    n_q, n_kv, hd, page, T = 32, 8, 128, 16, 40000
    torch.manual_seed(0)
    width = (T + page - 1) // page
    perm = torch.randperm(width + 3)[:width].reshape(1, width).to(torch.int32).to(DEV)
    cache = (torch.randn(width + 3, 2, n_kv, page, hd, device=DEV) * 0.5).to(torch.bfloat16)
    q = (torch.randn(T, n_q * hd, device=DEV) * 0.5).to(torch.bfloat16)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    st, outs = status(), {}
    for force in ("tc", "mma"):
        qpc = o.attention_prefill_q_per_cta(torch.bfloat16, n_q, n_kv, hd, page, force)
        tiles = sorted(((0, off) for off in range(0, T, qpc)), key=lambda t: -t[1])
        if force == "tc":
            assert len(tiles) * n_kv > 64 * torch.cuda.get_device_properties(0).multi_processor_count
        out = torch.zeros(T, n_q * hd, device=DEV, dtype=torch.bfloat16)
        o.attention_prefill(q=q, out=out, cache=cache, block_table=perm, q_start=dev(np.array([0, T])), kv_len=dev(np.array([T])),
                            n_q=n_q, n_kv=n_kv, head_dim=hd, page_size=page, window=0, scale=1 / math.sqrt(hd), status=st,
                            work=dev(np.array(tiles).reshape(-1)), n_work=len(tiles), force=force)
        outs[force] = out.float()
    assert st.item() == 0
    close(outs["tc"], outs["mma"].double().cpu(), 1.5e-2)


def test_attention_refuses_unsupported_sizes():
    from rustingstrata_b200.kernels.ops import KernelError
    with pytest.raises(KernelError, match="head size"):
        run_attention(torch.float32, 2, 1, 24, 4, [(5, 5)])
    with pytest.raises(KernelError, match="multiple"):
        run_attention(torch.float32, 3, 2, 32, 4, [(5, 5)])


# ------------------------------------------------------------------------------- sampling
def test_argmax_first_index_on_ties_and_non_finite():
    o = ops()
    V = 151_937
    logits = torch.randn(5, V, device=DEV)
    logits[0, 77] = logits[0, 90_001] = 50.0
    logits[1, V - 1] = 60.0
    logits[2, 0] = 60.0
    logits[3, 5] = float("nan")
    logits[3, 1000] = 70.0
    logits[4, :] = float("nan")
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    st = status()
    o.sample(logits, 5, out, st)
    assert out.tolist() == [77, V - 1, 0, 1000, -1]
    assert st.item() & o.STATUS_NON_FINITE


def test_temperature_draw_distribution_and_edges():
    o = ops()
    p = torch.tensor([0.5, 0.3, 0.15, 0.05])
    V, R = 1003, 20000
    logits = torch.full((R, V), -1e9, device=DEV)
    ids = [3, 400, 401, 1002]
    for i, pr in zip(ids, p):
        logits[:, i] = math.log(pr)
    temps = torch.ones(R, device=DEV)
    u = torch.rand(R, device=DEV)
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    o.sample(logits, R, out, status(), temps, u)
    counts = torch.bincount(out.long().cpu(), minlength=V)[ids].double() / R
    assert torch.all((counts - p.double()).abs() < 0.012), counts
    # inverse CDF in id order: u just below/above the first boundary
    u2 = torch.tensor([0.0, 0.4999, 0.5001, 0.7999, 0.8001, 0.9499, 0.9501, 0.999999], device=DEV)
    out2 = torch.zeros(8, dtype=torch.int32, device=DEV)
    o.sample(logits[:8].contiguous(), 8, out2, status(), temps[:8].contiguous(), u2)
    assert out2.tolist() == [3, 3, 400, 400, 401, 401, 1002, 1002]
    # temperature sharpens; rows with temp 0 are greedy
    temps3 = torch.tensor([0.0, 0.25], device=DEV)
    u3 = torch.tensor([0.9, 0.9], device=DEV)
    out3 = torch.zeros(2, dtype=torch.int32, device=DEV)
    o.sample(logits[:2].contiguous(), 2, out3, status(), temps3, u3)
    assert out3.tolist() == [3, 400]          # p^4 normalised: 0.5^4 / sum = 0.877 < 0.9 → second token


# ------------------------------------------------------------------------------- ids of the next step, on the device
@pytest.mark.parametrize("n", [1, 7, 128, 129, 1000])
def test_gather_of_chosen_ids(n):
    o = ops()
    g = torch.Generator().manual_seed(n)
    src = torch.randint(0, 1 << 20, (1500,), generator=g, dtype=torch.int32)
    idx = torch.randint(0, 1500, (n,), generator=g, dtype=torch.int32)
    dst = torch.full((n + 3,), -5, dtype=torch.int32, device=DEV)
    o.gather_i32(dst, src.to(DEV), idx.to(DEV), n)
    assert torch.equal(dst[:n].cpu(), src[idx.long()]) and torch.all(dst[n:] == -5)
    with pytest.raises(o.KernelError):
        o.gather_i32(dst, src.to(DEV).float(), idx.to(DEV), n)
