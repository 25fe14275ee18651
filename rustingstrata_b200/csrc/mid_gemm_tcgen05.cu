// bfloat16 matrix product for up to 128 rows of activations (the engine uses it from 9 rows: larger decode batches,
// short prompt portions) on the
// 5th-generation tensor cores, built like the skinny kernel around one job: stream the weight W[N, K] from HBM
// exactly once, with every SM reading the same number of bytes.
//
//   C[m, n] (=|+=) sum_k A[m, k] * W[n, k]
//
// The operands are swapped with respect to the large-M kernel: 128 rows of W are the M side of tcgen05.mma and
// the (padded: 16, 32, 64 or 128) rows of A its N side, so a tile of the accumulator in tensor memory is [128 rows of W] x [MP rows
// of A] and no tensor-core row is wasted on padding.  The product is cut into units of (128 rows of W) x (128 of
// k); the units, in row-tile-major order, are dealt to the persistent CTAs (one per SM) in equal contiguous
// shares ("stream-K").  In a CTA
//   warp 0 (one lane) - TMA producer: per unit two 128 x 64 boxes of W and two MP x 64 boxes of A, 128-byte
//                       swizzle, into a ring of stages; started before its predecessor has finished (programmatic
//                       dependent launch), it fills the ring with W, which no kernel writes, and asks for A only
//                       once the predecessor is done;
//   warp 1 (one lane) - issues tcgen05.mma (M = 128, N = MP, K = 16; eight per unit), accumulator double
//                       buffered in tensor memory, tcgen05.commit frees the stage;
//   warps 2-5         - epilogue: tcgen05.ld of their 32 accumulator lanes (one row of W per thread).  A row tile
//                       whose k range this CTA covers alone is finished at once; otherwise the float32 partial
//                       goes to a workspace and the CTA is done with it.
// A second, small kernel launched behind this one (mid_reduce_kernel) adds the partials of every shared tile in CTA
// order (fixed by the shape alone) and applies the epilogue, so that every CTA of the product does the same work and
// none stays behind adding up a tile.  Nobody waits for anybody.
// Epilogues: store bf16 | store f32 | f32 += (residual add) | SiLU(gate)*up over interleaved rows of W.
// Every wait on an mbarrier is bounded (tma_helpers.cuh).
//
// Reference counterpart: gemvn_bf16 / gemm_bf16 (src/cuda/kernels.cu:826-853,1062-1231); the reference has no
// kernel of its own for this range of rows.
#include "tma_helpers.cuh"
#include "stream_k_partials.cuh"

namespace {
constexpr int TILE_N = 128;                // rows of W per unit = M of the MMA
constexpr int BOX_K = 64;                  // 64 bf16 = 128 bytes = one swizzle row
constexpr int BOXES = 2;
constexpr int TILE_K = BOX_K * BOXES;      // k per unit
constexpr int UMMA_K = 16;
constexpr int W_BOX_BYTES = TILE_N * BOX_K * 2;
constexpr int W_BYTES = W_BOX_BYTES * BOXES;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

enum Epilogue : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3 };

struct MidParams {
    void* C; long ldc;
    int M, N, K;
    int stages;
    int vec_ok;                // rows of C allow 16-byte (f32) / 8-byte (bf16) access at every fourth column
    float* workspace;          // [grid][2][MP][128] float32 partials
    int* status;
};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart; descriptor version 1, layout 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// f32 accumulator, bf16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

using rs_streamk::first_unit;
using rs_streamk::cta_of_unit;

// one finished value of C: row m of A, row n of W (all 32 lanes of a warp call this together, n consecutive)
template <int EPI>
__device__ __forceinline__ void store_value(const MidParams& p, float v, int m, int n) {
    if (EPI == EPI_SWIGLU_BF16) {
        // rows of W alternate gate, up: the even lane of a pair writes
        const float up = __shfl_xor_sync(0xffffffffu, v, 1);
        if ((n & 1) == 0 && n + 1 < p.N)
            ((__nv_bfloat16*)p.C)[(size_t)m * p.ldc + (n >> 1)] = __float2bfloat16_rn(silu_mul_fast(v, up));
    } else if (n < p.N) {
        const size_t o = (size_t)m * p.ldc + n;
        if (EPI == EPI_STORE_BF16) ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(v);
        else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = v;
        else ((float*)p.C)[o] += v;
    }
}

// four finished values of C: row m of A, rows n0 .. n0 + 3 of W (n0 a multiple of 4); `old` holds what C had there
// (read by the caller ahead of time) when the epilogue accumulates
template <int EPI>
__device__ __forceinline__ void store_four(const MidParams& p, float4 v, float4 old, int m, int n0) {
    if (EPI == EPI_SWIGLU_BF16) {
        __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)m * p.ldc + (n0 >> 1);
        const float a = silu_mul_fast(v.x, v.y), b = silu_mul_fast(v.z, v.w);
        if (p.vec_ok && n0 + 3 < p.N) {
            *reinterpret_cast<__nv_bfloat162*>(out) = __floats2bfloat162_rn(a, b);
        } else {
            if (n0 + 1 < p.N) out[0] = __float2bfloat16_rn(a);
            if (n0 + 3 < p.N) out[1] = __float2bfloat16_rn(b);
        }
    } else if (p.vec_ok && n0 + 3 < p.N) {
        const size_t o = (size_t)m * p.ldc + n0;
        if (EPI == EPI_STORE_BF16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            *reinterpret_cast<uint2*>((__nv_bfloat16*)p.C + o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        } else if (EPI == EPI_STORE_F32) {
            *reinterpret_cast<float4*>((float*)p.C + o) = v;
        } else {
            *reinterpret_cast<float4*>((float*)p.C + o) = make_float4(old.x + v.x, old.y + v.y, old.z + v.z, old.w + v.w);
        }
    } else {
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (n0 + i < p.N) {
                const size_t o = (size_t)m * p.ldc + n0 + i;
                if (EPI == EPI_STORE_BF16) ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(e[i]);
                else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = e[i];
                else ((float*)p.C)[o] += e[i];
            }
        }
    }
}

template <int MP, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
mid_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const MidParams p) {
    constexpr int X_BOX_BYTES = MP * BOX_K * 2;
    constexpr int X_BYTES = X_BOX_BYTES * BOXES;
    constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = 2 * MP < 64 ? 64 : 2 * MP;     // the epilogue reads 32 columns at a time
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw);
    const int stages = p.stages;
    // barriers: full[stages], empty[stages], tmem_full[2], tmem_empty[2]; then tensor-memory base, abort flag
    const uint32_t bar0 = base + stages * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * stages + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * stages + 2 + b); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aligned + (size_t)stages * STAGE_BYTES + 8 * (2 * stages + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = (p.K + TILE_K - 1) / TILE_K;
    const int tiles = (p.N + TILE_N - 1) / TILE_N;
    const int U = tiles * KB, G = gridDim.x;
    const int u0 = first_unit(blockIdx.x, U, G), u1 = first_unit(blockIdx.x + 1, U, G);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            pdl_launch_dependents();
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
            // fill the ring with weights before waiting for the kernel that writes A
            const int ahead = min(stages, u1 - u0);
            int tile = u0 / KB, kb = u0 % KB;
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(full_bar(i), STAGE_BYTES);
                load_w(i, tile, kb);
                if (++kb == KB) { kb = 0; ++tile; }
            }
            pdl_wait();
            kb = u0 % KB;
            for (int i = 0; i < ahead; ++i) {
                load_x(i, kb);
                if (++kb == KB) kb = 0;
            }
            int s = ahead == stages ? 0 : ahead; uint32_t phase = ahead == stages ? 1u : 0u;
            for (int u = u0 + ahead; u < u1; ++u) {
                if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status)) break;
                mbar_expect_tx(full_bar(s), STAGE_BYTES);
                load_w(s, tile, kb);
                load_x(s, kb);
                if (++s == stages) { s = 0; phase ^= 1u; }
                if (++kb == KB) { kb = 0; ++tile; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer: one accumulator per tile segment
        if (lane == 0) {
            const uint32_t idesc = make_idesc(TILE_N, MP);
            int s = 0; uint32_t phase = 0;
            int seg = 0;
            bool ok = true;
            int u = u0;
            while (u < u1 && ok) {
                const int kb0 = u % KB;
                const int seg_end = min(u1, u - kb0 + KB);                 // first unit after this segment
                const int buf = seg & 1;
                if (!mbar_wait(tempty_bar(buf), ((seg >> 1) & 1) ^ 1u, abort_flag, p.status)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * MP;
                for (int i = 0; u < seg_end; ++u, ++i) {
                    if (!mbar_wait(full_bar(s), phase, abort_flag, p.status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t wst = base + s * STAGE_BYTES, xst = wst + W_BYTES;
#pragma unroll
                    for (int b = 0; b < BOXES; ++b) {
                        const uint64_t dw = make_smem_desc(wst + b * W_BOX_BYTES), dx = make_smem_desc(xst + b * X_BOX_BYTES);
#pragma unroll
                        for (int k = 0; k < BOX_K / UMMA_K; ++k)    // 32 bytes (>> 4 = 2) per K = 16 inside the swizzle row
                            umma_bf16(d_tmem, dw + 2u * k, dx + 2u * k, idesc, (i | b | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));                       // stage free once these MMAs have read it
                    if (++s == stages) { s = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(tfull_bar(buf));                 // the segment's accumulator is complete
                ++seg;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps 2..5: thread = one row of W
        const int quarter = warp & 3;                                // tensor-memory lanes [32 * quarter, +32)
        const int nl = quarter * 32 + lane;                          // row of W within the tile
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        pdl_wait();                                                  // C and the workspace belong to earlier kernels until now
        bool ok = true;
        int seg = 0;
        int u = u0;
        while (u < u1) {
            const int tile = u / KB, kb0 = u % KB;
            const int seg_end = min(u1, u - kb0 + KB);
            const bool whole = kb0 == 0 && seg_end == u - kb0 + KB;
            const int buf = seg & 1;
            const int n = tile * TILE_N + nl;
            const int tile_first = tile * KB;
            const int slot = (u0 >= tile_first) ? 0 : 1;             // 0: the tile my range starts in
            if (ok) ok = mbar_wait(tfull_bar(buf), (seg >> 1) & 1, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);                        // the loads below are warp-wide
            if (ok) {
                tc_fence_after();
                float* mine = p.workspace + ((size_t)blockIdx.x * 2 + slot) * MP * TILE_N;
#pragma unroll 1
                for (int c = 0; c < MP; c += 32) {
                    if (c >= p.M) break;
                    uint32_t r[32];
                    tmem_ld32(lane_base + buf * MP + c, r);
                    tmem_ld_wait();
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c + j < p.M) store_value<EPI>(p, __uint_as_float(r[j]), c + j, n);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c + j < p.M) __stcg(mine + (size_t)(c + j) * TILE_N + nl, __uint_as_float(r[j]));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(buf));         // the accumulator may be overwritten
            }
            u = seg_end;
            ++seg;
        }
    }
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);      // let loads already issued land
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Finishes the row tiles that several CTAs of mid_gemm_kernel shared: one CTA per CTA boundary of the product (G its
// grid); it acts if its boundary is the first one inside a tile.  The contributors' float32 partials ([row of A][128] per
// CTA and slot) are added in CTA order, which the shape alone fixes, and the epilogue is applied.  Who shares which tile
// is worked out before the wait for the product; for every four positions of a thread the first two contributors'
// values and what C holds are asked for together.
template <int MP, int EPI>
__global__ void __launch_bounds__(256) mid_reduce_kernel(const MidParams p, int G) {
    pdl_launch_dependents();
    const int KB = (p.K + TILE_K - 1) / TILE_K;
    const int U = ((p.N + TILE_N - 1) / TILE_N) * KB;
    const int b = blockIdx.x + 1;                              // boundary between CTA b - 1 and CTA b
    const int ub = first_unit(b, U, G);
    const int tile = ub / KB, tile_first = tile * KB;
    // on a tile's edge nobody shares because of this boundary; if an earlier boundary lies in the tile, its CTA acts
    const bool acts = ub % KB != 0 && first_unit(b - 1, U, G) <= tile_first;
    const int c_first = b - 1, c_last = acts ? cta_of_unit(tile_first + KB - 1, U, G) : b - 1;
    const int per_cta = U / G, extra = U % G;
    auto partial_of = [&](int c) {                             // contributor c's partial of this tile
        const int cslot = (c * per_cta + min(c, extra) >= tile_first) ? 0 : 1;
        return reinterpret_cast<const float4*>(p.workspace + ((size_t)c * 2 + cslot) * MP * TILE_N);
    };
    pdl_wait();                                                // every CTA waits, so that this grid never ends before the product
    if (!acts) return;
    const float4* first = partial_of(c_first);
    const float4* second = partial_of(c_first + 1);            // a shared tile has at least two contributors
    const int per = p.M * (TILE_N / 4);                        // float4 positions of the tile
    constexpr int Q = 4;
#pragma unroll 1
    for (int i0 = threadIdx.x; i0 < per; i0 += Q * 256) {
        float4 acc[Q], nxt[Q], old[Q];
#pragma unroll
        for (int q = 0; q < Q; ++q) {
            const int i = i0 + q * 256;
            old[q] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < per) {
                acc[q] = ld_dep(first + i);
                nxt[q] = ld_dep(second + i);
                const int m = i / (TILE_N / 4), n0 = tile * TILE_N + (i % (TILE_N / 4)) * 4;
                if (EPI == EPI_ADD_F32 && p.vec_ok && n0 + 3 < p.N)
                    old[q] = ld_dep(reinterpret_cast<const float4*>((const float*)p.C + (size_t)m * p.ldc + n0));
            }
        }
#pragma unroll
        for (int q = 0; q < Q; ++q)
            if (i0 + q * 256 < per) { acc[q].x += nxt[q].x; acc[q].y += nxt[q].y; acc[q].z += nxt[q].z; acc[q].w += nxt[q].w; }
        for (int c = c_first + 2; c <= c_last; ++c) {
            const float4* more = partial_of(c);
#pragma unroll
            for (int q = 0; q < Q; ++q)
                if (i0 + q * 256 < per) nxt[q] = ld_dep(more + i0 + q * 256);
#pragma unroll
            for (int q = 0; q < Q; ++q)
                if (i0 + q * 256 < per) { acc[q].x += nxt[q].x; acc[q].y += nxt[q].y; acc[q].z += nxt[q].z; acc[q].w += nxt[q].w; }
        }
#pragma unroll
        for (int q = 0; q < Q; ++q) {
            const int i = i0 + q * 256;
            if (i < per) store_four<EPI>(p, acc[q], old[q], i / (TILE_N / 4), tile * TILE_N + (i % (TILE_N / 4)) * 4);
        }
    }
}

// CTAs of the product: one per SM, at most max_ctas (if positive), at most one per unit of work
long grid_of(int N, int K, int max_ctas) {
    const long U = (long)((N + TILE_N - 1) / TILE_N) * ((K + TILE_K - 1) / TILE_K);
    long grid = rs_tma::sm_count();
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    return grid > U ? U : grid;
}
int padded_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }

template <int MP, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, MidParams p, int max_ctas, bool defer, cudaStream_t s) {
    constexpr int SB = W_BYTES + MP * TILE_K * 2;
    constexpr int stages = SMEM_BUDGET / SB;
    constexpr int smem = stages * SB + 1024 + 8 * (2 * stages + 5) + 64;
    auto kern = mid_gemm_kernel<MP, EPI>;
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
    return rs_launch_pdl(mid_reduce_kernel<MP, EPI>, dim3((unsigned)(grid - 1)), dim3(256), 0, s, p, (int)grid);
}

template <int MP>
int launch_epi(int epi, const CUtensorMap& mw, const CUtensorMap& ma, const MidParams& p, int max_ctas, bool defer, cudaStream_t s) {
    switch (epi) {
        case EPI_STORE_BF16: return launch<MP, EPI_STORE_BF16>(mw, ma, p, max_ctas, defer, s);
        case EPI_STORE_F32: return launch<MP, EPI_STORE_F32>(mw, ma, p, max_ctas, defer, s);
        case EPI_ADD_F32: return launch<MP, EPI_ADD_F32>(mw, ma, p, max_ctas, defer, s);
        case EPI_SWIGLU_BF16: return launch<MP, EPI_SWIGLU_BF16>(mw, ma, p, max_ctas, defer, s);
    }
    return (int)cudaErrorInvalidValue;
}
}  // namespace

RS_EXPORT int rs_mid_gemm_max_rows() { return 128; }

// float32 values of workspace a launch needs (for any M <= 128).
RS_EXPORT long rs_mid_gemm_workspace_floats() { return (long)rs_tma::sm_count() * 2 * 128 * TILE_N; }

// C[M, N] (=|+=) A[M, K] . W[N, K]^T for M <= 128, bf16 inputs; same epilogue codes as rs_gemm_bf16_tc.  a_rows is the
// row capacity of A's buffer.  workspace as sized above.  Launches that share a workspace must not overlap on the GPU.
// defer != 0 (f32 += epilogue only): the tiles that several CTAs share stay unfinished in the workspace until
// rs_mid_finish or rs_mid_finish_rmsnorm is launched with the same C, shape, workspace and max_ctas; no other product
// of this kind may run in between.
RS_EXPORT int rs_mid_gemm_bf16(const void* A, long lda, long a_rows, const void* W, long ldw, void* C, long ldc, int M, int N,
                               int K, int epi, float* workspace, int max_ctas, int defer, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128 || K <= 0 || K % 8 || lda % 8 || ldw % 8 || ((long)A & 15) || ((long)W & 15) || a_rows < M ||
        workspace == nullptr)
        return (int)cudaErrorInvalidValue;
    if (epi == EPI_SWIGLU_BF16 && (N & 1)) return (int)cudaErrorInvalidValue;
    if (defer && epi != EPI_ADD_F32) return (int)cudaErrorInvalidValue;
    const int mp = padded_rows(M);
    CUtensorMap mw, ma;
    int rc = rs_tma::get_map(W, N, K, ldw, TILE_N, &mw);
    if (rc) return rc;
    rc = rs_tma::get_map(A, a_rows, K, lda, mp, &ma);
    if (rc) return rc;
    MidParams p;
    p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.stages = 0; p.workspace = workspace;
    p.status = status;
    const int out_elem = (epi == EPI_STORE_BF16 || epi == EPI_SWIGLU_BF16) ? 2 : 4;
    p.vec_ok = (((long)C & 15) == 0 && (ldc * out_elem) % 16 == 0) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (mp == 16) return launch_epi<16>(epi, mw, ma, p, max_ctas, defer != 0, s);
    if (mp == 32) return launch_epi<32>(epi, mw, ma, p, max_ctas, defer != 0, s);
    if (mp == 64) return launch_epi<64>(epi, mw, ma, p, max_ctas, defer != 0, s);
    return launch_epi<128>(epi, mw, ma, p, max_ctas, defer != 0, s);
}

// Finishes a deferred product: C += the partials of the shared tiles.
RS_EXPORT int rs_mid_finish(void* C, long ldc, int M, int N, int K, float* workspace, int max_ctas, void* stream) {
    if (M <= 0 || M > 128 || N <= 0 || K <= 0 || workspace == nullptr) return (int)cudaErrorInvalidValue;
    MidParams p;
    p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.stages = 0; p.workspace = workspace; p.status = nullptr;
    p.vec_ok = (((long)C & 15) == 0 && (ldc * 4) % 16 == 0) ? 1 : 0;
    const long grid = grid_of(N, K, max_ctas);
    if (grid < 2) return 0;
    const dim3 g((unsigned)(grid - 1)), b(256);
    cudaStream_t s = (cudaStream_t)stream;
    switch (padded_rows(M)) {
        case 16: return rs_launch_pdl(mid_reduce_kernel<16, EPI_ADD_F32>, g, b, 0, s, p, (int)grid);
        case 32: return rs_launch_pdl(mid_reduce_kernel<32, EPI_ADD_F32>, g, b, 0, s, p, (int)grid);
        case 64: return rs_launch_pdl(mid_reduce_kernel<64, EPI_ADD_F32>, g, b, 0, s, p, (int)grid);
        default: return rs_launch_pdl(mid_reduce_kernel<128, EPI_ADD_F32>, g, b, 0, s, p, (int)grid);
    }
}

// Finishes a deferred product and writes out[m] = RMSNorm(C[m]) * w as bfloat16, in one kernel (one CTA per row).
RS_EXPORT int rs_mid_finish_rmsnorm(void* C, long ldc, int M, int N, int K, float* workspace, int max_ctas, const void* w,
                                    int w_dt, float eps, void* out, long out_stride, void* stream) {
    if (M <= 0 || M > 128) return (int)cudaErrorInvalidValue;
    const rs_streamk::Layout L = {TILE_N, TILE_K, padded_rows(M)};
    return rs_streamk::launch_finish_rmsnorm(C, ldc, M, N, K, workspace, (int)grid_of(N, K, max_ctas), L, w, w_dt, eps, out, out_stride,
                                             (cudaStream_t)stream);
}
