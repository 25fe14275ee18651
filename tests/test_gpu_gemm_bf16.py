"""The bfloat16 tensor-core matrix products (tcgen05 kernel and streaming skinny kernel) against a float64
product of the same bfloat16 inputs, over many shapes: sizes that are no multiple of any tile, every
epilogue, several tiles per CTA, tile widths 64/128/256."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from rustingstrata_b200.kernels import ops as o
    return o


def make(M, N, K, cap=None, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    a = torch.randn(cap or M, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    return a, w


def err(got, want):
    return ((got.double() - want).abs().max() / want.abs().max()).item()


def silu_mul(x):
    g, u = x[:, 0::2], x[:, 1::2]
    return g / (1 + torch.exp(-g)) * u


SHAPES = [(128, 256, 64), (128, 128, 128), (129, 136, 72), (300, 520, 200), (2048, 1024, 4096), (257, 6144, 4096),
          (40, 4096, 1024), (1000, 1000, 1000), (33, 24, 8), (512, 8192, 512)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bn", [0, 64, 128, 144, 176, 240, 256])
def test_tcgen05_gemm_store_and_accumulate(M, N, K, bn):
    o = ops()
    a, w = make(M, N, K, cap=M + 5)
    want = a[:M].double() @ w.double().T
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M + 5, N), 3.0, device=DEV, dtype=torch.bfloat16)
    o.gemm_bf16_tc(a, w, out, M, status=st, bn=bn)
    assert err(out[:M], want) < 6e-3 and torch.all(out[M:] == 3.0)
    f = torch.full((M + 5, N), 3.0, device=DEV)
    o.gemm_bf16_tc(a, w, f, M, status=st, bn=bn)
    assert err(f[:M], want) < 1e-5 and torch.all(f[M:] == 3.0)
    base = torch.randn(M + 5, N, device=DEV)
    acc = base.clone()
    o.gemm_bf16_tc(a, w, acc, M, accumulate=True, status=st, bn=bn)
    assert err(acc[:M], base[:M].double() + want) < 1e-5 and torch.equal(acc[M:], base[M:])
    assert st.item() == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (2048, 2048, 1024), (77, 24576, 4096)])
@pytest.mark.parametrize("max_ctas", [1, 3, 0])
def test_tcgen05_gemm_swiglu_and_several_tiles_per_cta(M, N, K, max_ctas):
    if max_ctas == 1 and M * N > 2048 * 2048:
        pytest.skip("one CTA for a large product is only slow")
    o = ops()
    a, w = make(M, N, K, seed=1)
    want = silu_mul(a.double() @ w.double().T)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(M, N // 2, device=DEV, dtype=torch.bfloat16)
    o.gemm_bf16_tc(a, w, out, M, swiglu=True, status=st, max_ctas=max_ctas)
    assert err(out, want) < 8e-3 and st.item() == 0
    f = torch.zeros(M, N, device=DEV)
    o.gemm_bf16_tc(a, w, f, M, status=st, max_ctas=max_ctas, bn=128)
    assert err(f, a.double() @ w.double().T) < 1e-5 and st.item() == 0


@pytest.mark.parametrize("M,N,K,bn,max_ctas", [(300, 1280, 512, 256, 9), (640, 1024, 1024, 128, 12), (200, 2000, 200, 64, 20),
                                               (2048, 4096, 1024, 0, 0), (1000, 2304, 448, 256, 11), (257, 1536, 4096, 256, 5)])
def test_tcgen05_gemm_float32_accumulate_several_tiles_per_cta_same_bits_every_run(M, N, K, bn, max_ctas):
    """A float32 += over tile counts that do not fill the last wave of CTAs, against the float64 product, and the same
    bits run after run (the additions to C go through the TMA unit; each element belongs to one tile)."""
    o = ops()
    a, w = make(M, N, K, cap=M + 3, seed=4)
    want = a[:M].double() @ w.double().T
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    base = torch.randn(M + 3, N, device=DEV)
    first = None
    for _ in range(6):
        acc = base.clone()
        o.gemm_bf16_tc(a, w, acc, M, accumulate=True, status=st, bn=bn, max_ctas=max_ctas)
        assert err(acc[:M], base[:M].double() + want) < 1e-5 and torch.equal(acc[M:], base[M:])
        if first is None:
            first = acc
        assert torch.equal(acc, first)
    assert st.item() == 0


@pytest.mark.parametrize("bn", [144, 208, 224, 240])
def test_tcgen05_gemm_tile_widths_between_128_and_256_with_the_fused_epilogue(bn):
    """Tiles whose width is not a multiple of the 32-column epilogue step: the last step of a tile must not write
    into the next tile's columns (gate/up pairs included), with several tiles per CTA."""
    o = ops()
    for (M, N, K) in ((300, 1000, 200), (2048, 4096, 512)):
        a, w = make(M, N, K, seed=2)
        full = a.double() @ w.double().T
        st = torch.zeros(1, dtype=torch.int32, device=DEV)
        sw = torch.zeros(M, N // 2, device=DEV, dtype=torch.bfloat16)
        o.gemm_bf16_tc(a, w, sw, M, swiglu=True, status=st, bn=bn, max_ctas=5)
        assert err(sw, silu_mul(full)) < 8e-3
        base = torch.randn(M, N, device=DEV)
        acc = base.clone()
        o.gemm_bf16_tc(a, w, acc, M, accumulate=True, status=st, bn=bn, max_ctas=5)
        assert err(acc, base.double() + full) < 1e-5 and st.item() == 0


def test_tcgen05_gemm_strided_views_and_unaligned_output():
    o = ops()
    big_a = torch.randn(200, 512 + 64, device=DEV).to(torch.bfloat16)
    a = big_a[:, 64:]                                   # row pitch 576, pointer offset 128 bytes
    w = (torch.randn(300, 512, device=DEV) / 22).to(torch.bfloat16)
    big_o = torch.zeros(200, 300 + 3, device=DEV)
    out = big_o[:, 3:]                                  # rows not 16-byte aligned: scalar stores
    o.gemm_bf16_tc(a, w, out, 150)
    assert err(out[:150], a[:150].double() @ w.double().T) < 1e-5 and torch.all(big_o[:, :3] == 0) and torch.all(out[150:] == 0)


def test_refused_shapes_say_why_and_linear_falls_back():
    o = ops()
    a = torch.randn(64, 250, device=DEV).to(torch.bfloat16)          # K = 250: rows are not 16-byte aligned
    w = torch.randn(96, 250, device=DEV).to(torch.bfloat16)
    out = torch.zeros(64, 96, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(o.KernelError, match="16-byte aligned"):
        o.gemm_bf16_tc(a, w, out, 64)
    with pytest.raises(o.KernelError, match="16-byte aligned"):
        o.skinny_gemm_bf16(a, w, out, 4)
    o.linear(a, w, out, 64)                                           # the CUDA-core kernel takes it
    assert err(out, a.double() @ w.double().T) < 6e-3
    a32 = torch.randn(64, 256, device=DEV)
    assert not o.tensor_core_shape_ok(a32, torch.randn(96, 256, device=DEV))


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 31, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(64, 64), (100, 72), (4096, 4096), (6144, 4096), (1000, 1000), (24576, 4096),
                                 (4096, 12288), (151936, 256), (70, 8)])
def test_streaming_skinny_kernel(M, N, K):
    o = ops()
    a, w = make(M, N, K, cap=M + 2, seed=M)
    want = a[:M].double() @ w.double().T
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M + 2, N), 3.0, device=DEV, dtype=torch.bfloat16)
    o.skinny_gemm_bf16(a, w, out, M, status=st)
    assert err(out[:M], want) < 6e-3 and torch.all(out[M:] == 3.0)
    f = torch.full((M + 2, N), 3.0, device=DEV)
    o.skinny_gemm_bf16(a, w, f, M, status=st)
    assert err(f[:M], want) < 1e-5
    base = torch.randn(M + 2, N, device=DEV)
    acc = base.clone()
    o.skinny_gemm_bf16(a, w, acc, M, accumulate=True, status=st)
    assert err(acc[:M], base[:M].double() + want) < 1e-5 and torch.equal(acc[M:], base[M:])
    if N % 2 == 0:
        sw = torch.zeros(M + 2, N // 2, device=DEV, dtype=torch.bfloat16)
        o.skinny_gemm_bf16(a, w, sw, M, swiglu=True, status=st)
        assert err(sw[:M], silu_mul(want)) < 8e-3 and torch.all(sw[M:] == 0)
    assert st.item() == 0


@pytest.mark.parametrize("max_ctas", [1, 2, 3, 7, 50, 147])
def test_streaming_skinny_kernel_any_split_of_the_work(max_ctas):
    """However the units are dealt to CTAs (row tiles shared by 2..many CTAs, CTAs spanning several tiles),
    the result is the same product, and the same bits on a second run."""
    o = ops()
    for (M, N, K) in ((8, 320, 1024), (64, 200, 4096), (3, 4096, 640)):
        a, w = make(M, N, K, seed=7)
        want = a.double() @ w.double().T
        f1 = torch.zeros(M, N, device=DEV)
        f2 = torch.zeros(M, N, device=DEV)
        o.skinny_gemm_bf16(a, w, f1, M, max_ctas=max_ctas)
        o.skinny_gemm_bf16(a, w, f2, M, max_ctas=max_ctas)
        assert err(f1, want) < 1e-5 and torch.equal(f1, f2)


@pytest.mark.parametrize("M", [1, 2, 5, 8])
@pytest.mark.parametrize("max_ctas", [0, 1, 3, 50, 147])
@pytest.mark.parametrize("N,K", [(4096, 4096), (4096, 12288), (1000, 1000), (100, 72), (5120, 640), (8192, 256), (64, 2048)])
@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32])
def test_product_that_leaves_its_last_sum_to_the_norm(M, max_ctas, N, K, w_dtype):
    """x += a W^T with the shared tiles left in the workspace, then one kernel that adds them and norms the rows:
    the same bits, in x and in the normed rows, as the product that finishes itself followed by the row norm.
    Tiles shared by two to many CTAs, tiles owned whole, widths that end inside a tile."""
    o = ops()
    a, w = make(M, N, K, cap=M + 2, seed=M + N)
    base = torch.randn(M + 2, N, device=DEV)
    nw = (1 + 0.1 * torch.randn(N, device=DEV)).to(w_dtype)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    x1, x2, x3 = base.clone(), base.clone(), base.clone()
    h1 = torch.full((M + 2, N), 3.0, device=DEV, dtype=torch.bfloat16)
    h2 = h1.clone()
    assert o.skinny_gemm_bf16(a, w, x1, M, accumulate=True, status=st, max_ctas=max_ctas) is None
    o.rmsnorm(x1, nw, 1e-6, h1, n_rows=M)
    owed = o.skinny_gemm_bf16(a, w, x2, M, accumulate=True, status=st, max_ctas=max_ctas, defer=True)
    o.rmsnorm(x2, nw, 1e-6, h2, n_rows=M, pending=owed)
    assert owed.done and torch.equal(x1, x2) and torch.equal(h1, h2) and torch.all(h2[M:] == 3.0)
    owed = o.skinny_gemm_bf16(a, w, x3, M, accumulate=True, status=st, max_ctas=max_ctas, defer=True)
    owed.finish()
    owed.finish()                                           # a second call does nothing
    assert torch.equal(x1, x3) and st.item() == 0


@pytest.mark.parametrize("M", [1, 9, 16, 33, 64, 100, 128])
@pytest.mark.parametrize("max_ctas", [0, 3, 50])
@pytest.mark.parametrize("N,K", [(4096, 4096), (4096, 12288), (1000, 1000), (100, 72), (5120, 640), (128, 2048)])
def test_stream_k_tcgen05_product_that_leaves_its_last_sum_to_the_norm(M, max_ctas, N, K):
    """The same for the product of up to 128 rows: its shared tiles (128 rows of W, partials of 16 to 128 rows) are
    added by the norm, one CTA per row; x and the normed rows are the bits of product, finishing kernel and norm in turn."""
    o = ops()
    a, w = make(M, N, K, cap=M + 2, seed=M + N)
    base = torch.randn(M + 2, N, device=DEV)
    nw = (1 + 0.1 * torch.randn(N, device=DEV)).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    x1, x2, x3 = base.clone(), base.clone(), base.clone()
    h1 = torch.full((M + 2, N), 3.0, device=DEV, dtype=torch.bfloat16)
    h2 = h1.clone()
    assert o.mid_gemm_bf16(a, w, x1, M, accumulate=True, status=st, max_ctas=max_ctas) is None
    o.rmsnorm(x1, nw, 1e-6, h1, n_rows=M)
    owed = o.mid_gemm_bf16(a, w, x2, M, accumulate=True, status=st, max_ctas=max_ctas, defer=True)
    o.rmsnorm(x2, nw, 1e-6, h2, n_rows=M, pending=owed)
    assert owed.done and torch.equal(x1, x2) and torch.equal(h1, h2) and torch.all(h2[M:] == 3.0)
    owed = o.mid_gemm_bf16(a, w, x3, M, accumulate=True, status=st, max_ctas=max_ctas, defer=True)
    owed.finish()
    assert torch.equal(x1, x3) and torch.equal(x3[M:], base[M:]) and st.item() == 0
    with pytest.raises(o.KernelError):
        o.mid_gemm_bf16(a, w, torch.zeros(M, N, device=DEV, dtype=torch.bfloat16), M, defer=True)


def test_owed_sum_is_finished_first_when_the_norm_cannot_take_it():
    """Other rows than the product's (a gather), another buffer, a float32 output: the sum is added by its own kernel
    and the plain norm runs."""
    o = ops()
    M, N, K = 4, 4096, 1024
    a, w = make(M, N, K, seed=3)
    base = torch.randn(M, N, device=DEV)
    nw = torch.ones(N, device=DEV, dtype=torch.bfloat16)
    want_x = base.clone()
    o.skinny_gemm_bf16(a, w, want_x, M, accumulate=True)
    rows = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    for kind in ("gather", "f32", "fewer"):
        x = base.clone()
        owed = o.skinny_gemm_bf16(a, w, x, M, accumulate=True, defer=True)
        if kind == "gather":
            h, want = torch.empty(2, N, device=DEV, dtype=torch.bfloat16), torch.empty(2, N, device=DEV, dtype=torch.bfloat16)
            o.rmsnorm(x, nw, 1e-6, h, rows=rows, n_rows=2, pending=owed)
            o.rmsnorm(want_x, nw, 1e-6, want, rows=rows, n_rows=2)
        elif kind == "f32":
            h, want = torch.empty(M, N, device=DEV), torch.empty(M, N, device=DEV)
            o.rmsnorm(x, nw, 1e-6, h, pending=owed)
            o.rmsnorm(want_x, nw, 1e-6, want)
        else:
            h, want = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16), torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
            o.rmsnorm(x, nw, 1e-6, h, n_rows=2, pending=owed)
            o.rmsnorm(want_x, nw, 1e-6, want, n_rows=2)
        assert owed.done and torch.equal(x, want_x) and torch.equal(h, want)
    with pytest.raises(o.KernelError):
        o.skinny_gemm_bf16(a, w, torch.zeros(M, N, device=DEV, dtype=torch.bfloat16), M, defer=True)


@pytest.mark.parametrize("M", [1, 17, 33, 40, 64, 65, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 128), (100, 72), (4096, 4096), (6144, 4096), (1000, 1000), (24576, 4096),
                                 (4096, 12288), (151936, 256), (70, 8), (130, 136)])
def test_stream_k_tcgen05_kernel(M, N, K):
    """The stream-K tcgen05 kernel (the engine's choice for 17 to 128 rows): every epilogue, rows beyond M untouched, widths and depths that end inside a
    tile, tiles finished by one CTA and tiles pieced together from several."""
    o = ops()
    a, w = make(M, N, K, cap=M + 2, seed=M)
    want = a[:M].double() @ w.double().T
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M + 2, N), 3.0, device=DEV, dtype=torch.bfloat16)
    o.mid_gemm_bf16(a, w, out, M, status=st)
    assert err(out[:M], want) < 6e-3 and torch.all(out[M:] == 3.0)
    f = torch.full((M + 2, N), 3.0, device=DEV)
    o.mid_gemm_bf16(a, w, f, M, status=st)
    assert err(f[:M], want) < 1e-5 and torch.all(f[M:] == 3.0)
    base = torch.randn(M + 2, N, device=DEV)
    acc = base.clone()
    o.mid_gemm_bf16(a, w, acc, M, accumulate=True, status=st)
    assert err(acc[:M], base[:M].double() + want) < 1e-5 and torch.equal(acc[M:], base[M:])
    if N % 2 == 0:
        sw = torch.zeros(M + 2, N // 2, device=DEV, dtype=torch.bfloat16)
        o.mid_gemm_bf16(a, w, sw, M, swiglu=True, status=st)
        assert err(sw[:M], silu_mul(want)) < 8e-3 and torch.all(sw[M:] == 0)
    assert st.item() == 0


@pytest.mark.parametrize("max_ctas", [1, 2, 3, 7, 50, 147])
def test_stream_k_tcgen05_kernel_any_split_of_the_work(max_ctas):
    o = ops()
    for (M, N, K) in ((40, 320, 1024), (64, 200, 4096), (128, 4096, 640), (100, 515, 2056)):
        a, w = make(M, N, K, seed=7)
        want = a.double() @ w.double().T
        f1 = torch.zeros(M, N, device=DEV)
        f2 = torch.zeros(M, N, device=DEV)
        o.mid_gemm_bf16(a, w, f1, M, max_ctas=max_ctas)
        o.mid_gemm_bf16(a, w, f2, M, max_ctas=max_ctas)
        assert err(f1, want) < 1e-5 and torch.equal(f1, f2)
        sw = torch.zeros(M, N // 2, device=DEV, dtype=torch.bfloat16)
        if N % 2 == 0:
            o.mid_gemm_bf16(a, w, sw, M, swiglu=True, max_ctas=max_ctas)
            assert err(sw, silu_mul(want)) < 8e-3


def test_stream_k_tcgen05_rows_do_not_depend_on_the_batch():
    o = ops()
    a, w = make(64, 2048, 4096, seed=5)
    g = torch.zeros(64, 2048, device=DEV)
    o.mid_gemm_bf16(a, w, g, 64)
    part = torch.zeros(40, 2048, device=DEV)
    o.mid_gemm_bf16(a[10:50].contiguous(), w, part, 40)
    assert torch.equal(part, g[10:50])                   # same k order whatever the batch
    t = torch.zeros(64, 2048, device=DEV)
    o.gemm_bf16_tc(a, w, t, 64)
    assert err(g, t.double()) < 2e-5


def test_skinny_and_tcgen05_agree_and_rows_do_not_depend_on_the_batch():
    o = ops()
    a, w = make(32, 2048, 4096, seed=5)
    g = torch.zeros(32, 2048, device=DEV)
    t = torch.zeros(32, 2048, device=DEV)
    o.skinny_gemm_bf16(a, w, g, 32)
    o.gemm_bf16_tc(a, w, t, 32)
    assert err(g, t.double()) < 2e-5                    # each is within 1e-5 of the exact product
    one = torch.zeros(1, 2048, device=DEV)
    o.skinny_gemm_bf16(a[5:6].contiguous(), w, one, 1)
    assert torch.equal(one[0], g[5])                     # same k order whatever the batch
