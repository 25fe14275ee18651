"""The chained decode kernel (csrc/decode_chain.cu): the products of a small decode step and the row norms between them
as one persistent kernel whose CTAs meet at barriers across the grid.  Its arithmetic is that of the separate kernels,
so everything here is compared bit for bit with the same operations launched one by one, and against float64."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def layer_ops(o, t, M, chained):
    """The decode step's run of products between two attention calls, on the tensors in t: output projection into the
    residual stream, norm, gate/up with SiLU, down projection into the stream, norm, the next layer's QKV projection."""
    if chained:
        o.begin_chain(t["status"])
    try:
        owed = o.linear(t["attn"], t["wo"], t["res"], M, accumulate=True, status=t["status"], may_defer=True)
        o.rmsnorm(t["res"], t["n1"], 1e-6, t["h"], n_rows=M, pending=owed)
        o.linear_swiglu(t["h"], t["wgu"], t["act"], M, status=t["status"])
        owed = o.linear(t["act"], t["wd"], t["res"], M, accumulate=True, status=t["status"], may_defer=True)
        o.rmsnorm(t["res"], t["n2"], 1e-6, t["h2"], n_rows=M, pending=owed)
        o.linear(t["h2"], t["wqkv"], t["qkv"], M, status=t["status"])
    finally:
        return o.end_chain() if chained else 0


def make(M, H, Q, KV, I, seed, norm_dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    t = dict(attn=r(8, Q).to(torch.bfloat16), wo=(r(H, Q) * 0.03).to(torch.bfloat16), res=r(8, H),
             n1=(1 + 0.1 * r(H)).to(norm_dtype), wgu=(r(2 * I, H) * 0.03).to(torch.bfloat16),
             wd=(r(H, I) * 0.03).to(torch.bfloat16), n2=(1 + 0.1 * r(H)).to(norm_dtype),
             wqkv=(r(Q + 2 * KV, H) * 0.03).to(torch.bfloat16))
    t = {k: v.to(DEV) for k, v in t.items()}
    t.update(h=torch.zeros(8, H, device=DEV, dtype=torch.bfloat16), act=torch.zeros(8, I, device=DEV, dtype=torch.bfloat16),
             h2=torch.zeros(8, H, device=DEV, dtype=torch.bfloat16), qkv=torch.zeros(8, Q + 2 * KV, device=DEV, dtype=torch.bfloat16),
             status=torch.zeros(1, dtype=torch.int32, device=DEV))
    return t


def reference(t, M):
    f = lambda k: t[k][:M].double().cpu() if t[k].dim() == 2 and t[k].shape[0] == 8 and k in ("attn", "res") else t[k].double().cpu()  # noqa: E731
    res = f("res") + f("attn") @ f("wo").T
    norm = lambda x, w: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w  # noqa: E731
    h = norm(res, f("n1")).to(torch.bfloat16).double()
    gu = h @ f("wgu").T
    act = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]).to(torch.bfloat16).double()
    res2 = res + act @ f("wd").T
    h2 = norm(res2, f("n2")).to(torch.bfloat16).double()
    return res2, h2 @ f("wqkv").T


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("H,Q,KV,I", [(4096, 4096, 1024, 12288), (128, 512, 128, 328), (1024, 768, 256, 2816), (5120, 5120, 1024, 1000)])
def test_chain_equals_the_separate_kernels_bit_for_bit(M, H, Q, KV, I):
    from rustingstrata_b200.kernels import ops as o
    a, b = make(M, H, Q, KV, I, 5), make(M, H, Q, KV, I, 5)
    assert layer_ops(o, a, M, chained=False) == 0
    n = layer_ops(o, b, M, chained=True)
    torch.cuda.synchronize()
    assert n == 1                                             # the whole run left as one kernel
    assert a["status"].item() == 0 and b["status"].item() == 0
    for k in ("res", "h", "act", "h2", "qkv"):
        assert torch.equal(a[k][:M], b[k][:M]), k
        assert torch.equal(b[k][M:], make(M, H, Q, KV, I, 5)[k][M:]), f"{k}: rows beyond M were touched"
    res2, qkv = reference(b, M)
    # `res` in the reference starts from the tensors before the chain ran: rebuild them
    src = make(M, H, Q, KV, I, 5)
    res2, qkv = reference(src, M)
    assert rel_err(b["res"][:M].double().cpu().numpy(), res2.numpy()) < 2e-2
    assert rel_err(b["qkv"][:M].double().cpu().numpy(), qkv.numpy()) < 3e-2


def test_chain_with_float32_norm_weights_and_repeated_launches():
    """Norm weights stored in 32 bits; the same chain launched fifty times in a row (its barrier words count up and
    reset every time) gives the same bits every time."""
    from rustingstrata_b200.kernels import ops as o
    M, shape = 5, (1024, 768, 256, 2816)
    want = make(M, *shape, 9, norm_dtype=torch.float32)
    layer_ops(o, want, M, chained=False)
    for _ in range(50):
        t = make(M, *shape, 9, norm_dtype=torch.float32)
        assert layer_ops(o, t, M, chained=True) == 1
        for k in ("res", "h2", "qkv"):
            assert torch.equal(t[k], want[k]), k
    assert t["status"].item() == 0


def test_what_the_chain_does_not_take_runs_as_before():
    """Nine rows, a gathered norm, float32 activations: the launchers fall back to the separate kernels inside an open
    chain, in order, and the result is the same."""
    from rustingstrata_b200.kernels import ops as o
    t = make(8, 1024, 768, 256, 2816, 3)
    big = {k: (torch.cat([v, v[:1]]) if v.dim() == 2 and v.shape[0] == 8 else v) for k, v in t.items()}     # nine rows
    want = {k: v.clone() for k, v in big.items()}
    st = big["status"]
    o.linear(want["attn"], want["wo"], want["res"], 9, accumulate=True, status=st)
    o.rmsnorm(want["res"], want["n1"], 1e-6, want["h"], n_rows=9)
    o.begin_chain(st)
    o.linear(big["attn"], big["wo"], big["res"], 9, accumulate=True, status=st)        # nine rows: not chained
    o.rmsnorm(big["res"], big["n1"], 1e-6, big["h"], n_rows=9)
    assert o.end_chain() == 0
    assert torch.equal(big["res"], want["res"]) and torch.equal(big["h"], want["h"])
    # a product of 8 rows, then a norm of gathered rows (not chained: the chain is flushed first, then the norm runs)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    a, b = make(8, 1024, 768, 256, 2816, 4), make(8, 1024, 768, 256, 2816, 4)
    o.linear(a["attn"], a["wo"], a["res"], 8, accumulate=True, status=a["status"])
    o.rmsnorm(a["res"], a["n1"], 1e-6, a["h"], rows=rows, n_rows=3)
    o.begin_chain(b["status"])
    o.linear(b["attn"], b["wo"], b["res"], 8, accumulate=True, status=b["status"], may_defer=True)
    o.rmsnorm(b["res"], b["n1"], 1e-6, b["h"], rows=rows, n_rows=3)
    assert o.end_chain() == 1
    assert torch.equal(a["res"], b["res"]) and torch.equal(a["h"], b["h"])


@pytest.mark.parametrize("name", ["D", "E"])
def test_engine_gives_the_same_logits_with_and_without_the_chain(tiny_models, name, monkeypatch):
    """Decode steps of one to eight requests through the engine, chained and not: identical logits, every row against
    the plain implementation; the chained engine launches fewer kernels."""
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.engine import StepEntry
    from rustingstrata_b200.kernels import ops
    cfg, w = P.read_model(tiny_models[name])
    toks = {f"r{i}": random_tokens(cfg["vocab_size"], 30 + 11 * i, 40 + i) for i in range(8)}
    ref = {k: P.forward_logits(cfg, w, t) for k, t in toks.items()}

    def run(chained):
        monkeypatch.setattr(ops, "CHAIN_DECODE", chained)
        eng = Engine(tiny_models[name], dtype="bfloat16", page_size=TINY[name]["page_size"], max_tokens=2048,
                     max_batch_tokens=256, max_seqs=8)
        out = []
        for k, t in toks.items():
            eng.step_raw([StepEntry(k, t[:-12], [])])
        n0 = ops.launch_count()
        at = {k: len(t) - 12 for k, t in toks.items()}           # the next token of each request
        for j in range(12):
            live = list(toks)[: 8 - (j % 3) * 3] if j < 9 else list(toks)[:1]       # 8, 5, 2 requests, then one alone
            live = [k for k in live if at[k] < len(toks[k])]
            rows = eng.step_raw([StepEntry(k, [toks[k][at[k]]], [0]) for k in live])
            out.append(([(k, at[k]) for k in live], rows.clone()))
            for k in live:
                at[k] += 1
        eng.runner.check_status()
        return out, ops.launch_count() - n0 + eng.runner.kernels_replayed, eng.runner.chain_kernels

    plain, n_plain, c0 = run(False)
    chained, n_chained, c1 = run(True)
    assert c0 == 0 and c1 > 0 and n_chained < n_plain
    for j, ((live, a), (_, b)) in enumerate(zip(plain, chained)):
        assert torch.equal(a, b), f"step {j}"
        for row, (k, pos) in zip(b.cpu().numpy(), live):
            assert np.max(np.abs(row - ref[k][pos])) / np.max(np.abs(ref[k])) <= TOL["bfloat16"], (j, k)
