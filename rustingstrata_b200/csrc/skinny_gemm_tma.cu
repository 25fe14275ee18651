// Skinny bfloat16 matrix product for decode batches (M <= 64 rows of activations), built around one job:
// stream the weight W[N, K] from HBM exactly once at full bandwidth.
//
//   C[m, n] (=|+=) sum_k A[m, k] * W[n, k]
//
// Persistent CTAs, one per SM.  The product is cut into units of (64 rows of W) x (128 of k); the units, in
// row-tile-major order, are dealt to the CTAs in equal contiguous shares ("stream-K"), so every SM reads the
// same number of bytes whatever N and K are.  In a CTA
//   warp 4 (one elected lane) - producer: for each unit two TMA loads of 64 x 64 tiles of W (16 KiB) and two
//                               of the matching [rows of A] x 64 tiles, 128-byte swizzle, into a ring of stages
//                               that keeps well over 100 KiB in flight per SM independent of the math.  The
//                               kernel is launched so that it may start while its predecessor still runs:
//                               the producer fills the whole ring with W (which no kernel writes) at once and
//                               asks for the A tiles only after the predecessor has finished;
//   warps 0-3                 - consumers: each owns 16 of the unit's 64 rows; 16-byte shared-memory reads feed
//                               mma.sync m16n8k16 (W rows are the 16-row operand, up to eight groups of 8
//                               activation rows the 8-column operand).  W and A are read with the same
//                               lane-to-k assignment, so no shuffle is needed: the sum over k does not care
//                               in which order k is visited.
// A row tile whose k range is shared by several CTAs is completed by a second, small kernel launched behind this one
// (skinny_reduce_kernel): each contributor writes its float32 partial (same thread-to-element mapping everywhere) to
// a workspace and is done, so every CTA of the product does the same amount of work and none lags behind adding up
// a tile; the small kernel adds the partials in CTA order, which the shape alone fixes, and applies the epilogue.
// Epilogues: store bf16 | store f32 | f32 += (residual add) | SiLU(gate)*up over interleaved rows of W.
// Waits on mbarriers are bounded (tma_helpers.cuh).
//
// Reference counterpart: gemv_bf16 / gemvn_bf16 (src/cuda/kernels.cu:307-329,826-853): one warp per row on CUDA
// cores, each weight read once for up to 4 inputs.
#include "skinny_tile.cuh"

namespace {
using namespace rs_skinny;

template <int NT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const SkinnyParams p) {
    constexpr int MP = 8 * NT;                               // activation rows per stage
    constexpr int X_BOX_BYTES = MP * BOX_K * 2;                 // >= 1024: every tile stays 1024-byte aligned
    constexpr int X_BYTES = X_BOX_BYTES * BOXES;
    constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const int stages = p.stages;
    const uint32_t bar0 = base + stages * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (base - raw) + stages * STAGE_BYTES + 16 * stages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = (p.K + TILE_K - 1) / TILE_K;
    const int tiles = (p.N + TILE_N - 1) / TILE_N;
    const int U = tiles * KB, G = gridDim.x;
    const int u0 = first_unit(blockIdx.x, U, G), u1 = first_unit(blockIdx.x + 1, U, G);

    auto load_w = [&](int s, int tile, int kb) {
        const uint32_t dst = base + s * STAGE_BYTES;
#pragma unroll
        for (int b = 0; b < BOXES; ++b)
            tma_load_2d(dst + b * W_BOX_BYTES, &map_w, kb * TILE_K + b * BOX_K, tile * TILE_N, full_bar(s));
    };
    auto load_x = [&](int s, int kb) {
        const uint32_t dst = base + s * STAGE_BYTES + W_BYTES;
#pragma unroll
        for (int b = 0; b < BOXES; ++b)
            tma_load_2d(dst + b * X_BOX_BYTES, &map_a, kb * TILE_K + b * BOX_K, 0, full_bar(s));
    };
    // The producer's lane sets the barriers up itself and starts the first ring of weights (which no kernel writes)
    // before the CTA meets, so that the loads are on their way while the other warps are still arriving.
    const int ahead = min(stages, u1 - u0);
    if (warp == CONSUMER_WARPS && lane == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), CONSUMER_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
        int tile = u0 / KB, kb = u0 % KB;
        for (int i = 0; i < ahead; ++i) {
            mbar_expect_tx(full_bar(i), W_BYTES + X_BYTES);
            load_w(i, tile, kb);
            if (++kb == KB) { kb = 0; ++tile; }
        }
    }
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int tile = (u0 + ahead) / KB, kb = (u0 + ahead) % KB;          // the next unit whose weights are to be asked for
            pdl_wait();                                                   // the kernel that writes A is done
            for (int i = 0, kx = u0 % KB; i < ahead; ++i) {
                load_x(i, kx);
                if (++kx == KB) kx = 0;
            }
            int s = ahead == stages ? 0 : ahead; uint32_t phase = ahead == stages ? 1u : 0u;
            for (int u = u0 + ahead; u < u1; ++u) {
                if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status)) break;
                mbar_expect_tx(full_bar(s), W_BYTES + X_BYTES);
                load_w(s, tile, kb);
                load_x(s, kb);
                if (++s == stages) { s = 0; phase ^= 1u; }
                if (++kb == KB) { kb = 0; ++tile; }
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        const int g = lane >> 2, t = lane & 3;
        pdl_wait();                                            // C and the workspace belong to earlier kernels until now
        float acc[NT][4], acc2[NT][4];                         // one set per box: two independent MMA chains
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
            acc2[j][0] = acc2[j][1] = acc2[j][2] = acc2[j][3] = 0.f;
        }
        int s = 0; uint32_t phase = 0;
        bool ok = true;
        int seg_start = u0;                                    // first unit of the current tile segment
        int tile = u0 / KB, kb = u0 % KB;
        // A warp whose wait ran out keeps walking its units without touching them, so that the consumers' named
        // barrier below always finds all four warps.
        for (int u = u0; u < u1; ++u) {
            if (ok) ok = mbar_wait(full_bar(s), phase, abort_flag, p.status);
            const uint32_t wst = base + s * STAGE_BYTES, xst = wst + W_BYTES;
            if (ok) {
                consume_unit<NT>(wst, xst, warp, g, t, acc, acc2);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
            }
            if (++s == stages) { s = 0; phase ^= 1u; }

            if (kb == KB - 1 || u == u1 - 1) {
                // ---- the CTA's share of this row tile ends here
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) { acc[j][i] += acc2[j][i]; acc2[j][i] = 0.f; }
                const int tile_first = tile * KB;
                const bool whole = seg_start == tile_first && kb == KB - 1;
                if (whole) {
                    if (ok) store_tile<NT, EPI>(p, acc, tile, warp, g, t);
                } else {
                    // shared with other CTAs: my float32 partial goes to the workspace; skinny_reduce_kernel adds them up
                    const int slot = (u0 >= tile_first) ? 0 : 1;            // 0: the tile my range starts in
                    store_partial<NT>(p.workspace, blockIdx.x, slot, warp, g, t, acc);
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
                seg_start = u + 1;
            }
            if (++kb == KB) { kb = 0; ++tile; }
        }
    }
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);          // let loads already issued land
    }
    __syncthreads();
}

// Adds up the partials of the row tiles that several CTAs of skinny_gemm_kernel shared and applies the epilogue: one CTA
// per CTA boundary of the product; it acts if its boundary is the first one inside a tile.  The partials are added in
// CTA order, which the shape alone fixes.  G is the grid of the product.
template <int NT, int EPI>
__global__ void __launch_bounds__(CONSUMER_WARPS * 32) skinny_reduce_kernel(const SkinnyParams p, int G) {
    pdl_launch_dependents();
    // who shares which tile follows from the shape alone: worked out while the product is still running
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const SharedTile st = shared_tile_of_boundary(blockIdx.x + 1, p.N, p.K, G);
    pdl_wait();                                                // every CTA waits, so that this grid never ends before the product
    if (!st.acts) return;
    finish_shared_tile<NT, EPI>(p, st, G, warp, g, t);
}

template <int NT> constexpr int stage_bytes() { return W_BYTES + 8 * NT * TILE_K * 2; }

// CTAs of the product: one per SM, at most max_ctas (if positive), at most one per unit of work
long grid_of(int N, int K, int max_ctas) {
    const long U = (long)((N + TILE_N - 1) / TILE_N) * ((K + TILE_K - 1) / TILE_K);
    long grid = rs_tma::sm_count();
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    return grid > U ? U : grid;
}

template <int NT, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, SkinnyParams p, int max_ctas, bool defer, cudaStream_t s) {
    constexpr int SB = stage_bytes<NT>();
    int stages = SMEM_BUDGET / SB;
    if (stages > 24) stages = 24;
    const int smem = stages * SB + 1024 + 16 * stages + 64;
    auto kern = skinny_gemm_kernel<NT, EPI>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    p.stages = stages;
    const long grid = grid_of(p.N, p.K, max_ctas);
    int rc = rs_launch_pdl(kern, dim3((unsigned)grid), dim3(THREADS), (size_t)smem, s, mw, ma, p);
    if (rc != 0 || grid < 2 || defer) return rc;
    return rs_launch_pdl(skinny_reduce_kernel<NT, EPI>, dim3((unsigned)(grid - 1)), dim3(CONSUMER_WARPS * 32), 0, s, p, (int)grid);
}

template <int NT>
int launch_epi(int epi, const CUtensorMap& mw, const CUtensorMap& ma, const SkinnyParams& p, int max_ctas, bool defer, cudaStream_t s) {
    switch (epi) {
        case EPI_STORE_BF16: return launch<NT, EPI_STORE_BF16>(mw, ma, p, max_ctas, defer, s);
        case EPI_STORE_F32: return launch<NT, EPI_STORE_F32>(mw, ma, p, max_ctas, defer, s);
        case EPI_ADD_F32: return launch<NT, EPI_ADD_F32>(mw, ma, p, max_ctas, defer, s);
        case EPI_SWIGLU_BF16: return launch<NT, EPI_SWIGLU_BF16>(mw, ma, p, max_ctas, defer, s);
    }
    return (int)cudaErrorInvalidValue;
}
}  // namespace

RS_EXPORT int rs_skinny_gemm_max_rows() { return 64; }

// float32 values of workspace a launch needs (for any M <= 64).
RS_EXPORT long rs_skinny_gemm_workspace_floats() { return (long)rs_tma::sm_count() * 2 * CONSUMER_WARPS * 8 * 4 * 32; }

// C[M, N] (=|+=) A[M, K] . W[N, K]^T for M <= 64, bf16 inputs; same epilogue codes as rs_gemm_bf16_tc.  a_rows is the
// row capacity of A's buffer.  workspace as sized above.  Launches that share a workspace must not overlap on the GPU.
// defer != 0 (f32 += epilogue, M <= 8 only): the tiles that several CTAs share stay unfinished in the workspace until
// rs_skinny_finish or rs_skinny_finish_rmsnorm is launched with the same C, shape, workspace and max_ctas; no other
// product may use the workspace in between.
RS_EXPORT int rs_skinny_gemm_bf16(const void* A, long lda, long a_rows, const void* W, long ldw, void* C, long ldc, int M,
                                  int N, int K, int epi, float* workspace, int max_ctas, int defer, int* status,
                                  void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || K % 8 || lda % 8 || ldw % 8 || ((long)A & 15) || ((long)W & 15) || a_rows < M ||
        workspace == nullptr)
        return (int)cudaErrorInvalidValue;
    if (epi == EPI_SWIGLU_BF16 && (N & 1)) return (int)cudaErrorInvalidValue;
    if (defer && (epi != EPI_ADD_F32 || M > 8)) return (int)cudaErrorInvalidValue;
    const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
    CUtensorMap mw, ma;
    int rc = rs_tma::get_map(W, N, K, ldw, TILE_N, &mw);
    if (rc) return rc;
    rc = rs_tma::get_map(A, a_rows, K, lda, 8 * nt, &ma);
    if (rc) return rc;
    SkinnyParams p;
    p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.stages = 0; p.workspace = workspace;
    p.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    switch (nt) {
        case 1: return launch_epi<1>(epi, mw, ma, p, max_ctas, defer != 0, s);
        case 2: return launch_epi<2>(epi, mw, ma, p, max_ctas, false, s);
        case 4: return launch_epi<4>(epi, mw, ma, p, max_ctas, false, s);
        default: return launch_epi<8>(epi, mw, ma, p, max_ctas, false, s);
    }
}

// Finishes a deferred product: C += the partials of the shared tiles.
RS_EXPORT int rs_skinny_finish(void* C, long ldc, int M, int N, int K, float* workspace, int max_ctas, void* stream) {
    if (M <= 0 || M > 8 || N <= 0 || K <= 0 || workspace == nullptr) return (int)cudaErrorInvalidValue;
    SkinnyParams p;
    p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.stages = 0; p.workspace = workspace; p.status = nullptr;
    const long grid = grid_of(N, K, max_ctas);
    if (grid < 2) return 0;
    return rs_launch_pdl(skinny_reduce_kernel<1, EPI_ADD_F32>, dim3((unsigned)(grid - 1)), dim3(CONSUMER_WARPS * 32), 0,
                         (cudaStream_t)stream, p, (int)grid);
}

namespace rs_streamk {
// RMSNorm of the rows of C straight after a product with the f32 += epilogue whose shared tiles were left unfinished:
// one CTA per row does what the product's small finishing kernel and the row norm would do one after the other, with
// the same arithmetic in the same order (partials in CTA order, then added to C; the sum of squares by thread-strided
// float4 partials and a tree), so the bits are those of the two kernels.  It saves a kernel boundary and a round trip
// to memory between two small dependent kernels.  Rows of up to 512 * 4 * VPT values.
// C[M, N] float32 with row pitch ldc; workspace, N, K, G, L: the product's; w: the norm's weights (float32 or bfloat16).
template <int VPT>
__global__ void __launch_bounds__(512) finish_rmsnorm_kernel(float* C, long ldc, int N, int K, const float* workspace, int G,
                                                             const Layout L, const void* __restrict__ w, int w_dt, float eps,
                                                             __nv_bfloat16* __restrict__ out, long out_stride) {
    constexpr int MAX_TILES = 512 * 4 * VPT / 64;              // tiles are at least 64 wide
    __shared__ float scratch[33];
    __shared__ int2 sharers[MAX_TILES];                        // per row tile: first and last CTA of the product that worked on it
    pdl_launch_dependents();
    // Nothing before the wait reads what the product wrote: who shared which tile follows from the shape, and the
    // norm's weights are the model's.  So this part runs while the product is still at work.
    const int m = blockIdx.x;
    const int KB = (K + L.tile_k - 1) / L.tile_k;
    const int n_tiles = (N + L.tile_n - 1) / L.tile_n;
    const int U = n_tiles * KB;
    const int per_cta = U / G, extra = U % G;                  // the first `extra` CTAs take one unit more
    for (int tile = threadIdx.x; tile < n_tiles; tile += 512) sharers[tile] = sharers_of_tile(tile, KB, U, G);
    const int n4 = N >> 2;
    float wv[VPT][4];
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = threadIdx.x + u * 512;
        wv[u][0] = wv[u][1] = wv[u][2] = wv[u][3] = 0.f;
        if (idx < n4) {
            if (w_dt == RS_F32) {
                const float4 f = reinterpret_cast<const float4*>(w)[idx];
                wv[u][0] = f.x; wv[u][1] = f.y; wv[u][2] = f.z; wv[u][3] = f.w;
            } else {
                const uint2 h = reinterpret_cast<const uint2*>(w)[idx];
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&h.x), b = *reinterpret_cast<const __nv_bfloat162*>(&h.y);
                wv[u][0] = __low2float(a); wv[u][1] = __high2float(a); wv[u][2] = __low2float(b); wv[u][3] = __high2float(b);
            }
        }
    }
    __syncthreads();
    pdl_wait();
    float* xr = C + (size_t)m * ldc;
    float4 v[VPT];
    OwedBatch part[VPT];
    int2 sh[VPT];
    // every load first: the row's values and the first four contributors' partials of each of this thread's columns
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = threadIdx.x + u * 512;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        sh[u] = make_int2(0, 0);
        if (idx < n4) {
            v[u] = ld_dep(reinterpret_cast<const float4*>(xr) + idx);
            sh[u] = sharers[idx * 4 / L.tile_n];
            if (sh[u].x != sh[u].y) owed_begin4(part[u], workspace, L, m, idx * 4, KB, per_cta, extra, sh[u].x, sh[u].y);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = threadIdx.x + u * 512;
        if (idx < n4 && sh[u].x != sh[u].y) {
            const float4 acc = owed_end4(part[u], workspace, L, m, idx * 4, KB, per_cta, extra, sh[u].x, sh[u].y);
            v[u].x += acc.x; v[u].y += acc.y; v[u].z += acc.z; v[u].w += acc.w;
            reinterpret_cast<float4*>(xr)[idx] = v[u];
        }
        ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss); ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float sc = 1.0f / sqrtf(ss / (float)N + eps);
    __nv_bfloat16* o = out + (size_t)m * out_stride;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = threadIdx.x + u * 512;
        if (idx < n4) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x * sc * wv[u][0], v[u].y * sc * wv[u][1]);
            const __nv_bfloat162 hi2 = __floats2bfloat162_rn(v[u].z * sc * wv[u][2], v[u].w * sc * wv[u][3]);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi2);
            reinterpret_cast<uint2*>(o)[idx] = pk;
        }
    }
}

bool finish_rmsnorm_supported(const void* C, long ldc, int N, const void* w, const void* out, long out_stride) {
    return N > 0 && N % 4 == 0 && N <= 512 * 4 * 4 && ldc % 4 == 0 && out_stride % 4 == 0 && ((long)C & 15) == 0 &&
           ((long)out & 7) == 0 && ((long)w & 15) == 0;
}

int launch_finish_rmsnorm(void* C, long ldc, int M, int N, int K, const float* workspace, int G, Layout L, const void* w,
                                 int w_dt, float eps, void* out, long out_stride, cudaStream_t s) {
    if (M <= 0 || M > L.rows_padded || K <= 0 || workspace == nullptr || G < 1 || (w_dt != RS_F32 && w_dt != RS_BF16) ||
        L.tile_n < 64 || L.tile_n % 4 || !finish_rmsnorm_supported(C, ldc, N, w, out, out_stride))
        return (int)cudaErrorInvalidValue;
    float* c = (float*)C;
    auto* o = (__nv_bfloat16*)out;
    if (N <= 512 * 4) return rs_launch_pdl(finish_rmsnorm_kernel<1>, dim3(M), dim3(512), 0, s, c, ldc, N, K, workspace, G, L, w, w_dt, eps, o, out_stride);
    if (N <= 512 * 8) return rs_launch_pdl(finish_rmsnorm_kernel<2>, dim3(M), dim3(512), 0, s, c, ldc, N, K, workspace, G, L, w, w_dt, eps, o, out_stride);
    return rs_launch_pdl(finish_rmsnorm_kernel<4>, dim3(M), dim3(512), 0, s, c, ldc, N, K, workspace, G, L, w, w_dt, eps, o, out_stride);
}
}  // namespace rs_streamk

// Whether rs_skinny_finish_rmsnorm takes a row of this width with these pitches and pointers.
RS_EXPORT int rs_skinny_finish_rmsnorm_supported(const void* C, long ldc, int N, const void* w, const void* out, long out_stride) {
    return rs_streamk::finish_rmsnorm_supported(C, ldc, N, w, out, out_stride) ? 1 : 0;
}

// Finishes a deferred product and writes out[m] = RMSNorm(C[m]) * w as bfloat16, in one kernel.
RS_EXPORT int rs_skinny_finish_rmsnorm(void* C, long ldc, int M, int N, int K, float* workspace, int max_ctas, const void* w,
                                       int w_dt, float eps, void* out, long out_stride, void* stream) {
    if (M > 8) return (int)cudaErrorInvalidValue;
    const rs_streamk::Layout L = {TILE_N, TILE_K, 8};
    return rs_streamk::launch_finish_rmsnorm(C, ldc, M, N, K, workspace, (int)grid_of(N, K, max_ctas), L, w, w_dt, eps, out, out_stride,
                                             (cudaStream_t)stream);
}

// Turns programmatic dependent launch on or off for every kernel of this library (default on).
RS_EXPORT void rs_bf16_set_pdl(int on) { rs_pdl_switch() = on ? 1 : 0; }
