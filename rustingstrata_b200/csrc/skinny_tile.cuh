// What the few-rows product (skinny_gemm_tma.cu) and the chained decode kernel (decode_chain.cu) share: the shape of a
// unit of work, the consumers' arithmetic on one unit, where a finished value goes (the four epilogues), and how the
// partial sums of a row tile that several CTAs shared are added up.  Both kernels go through these functions, so a row
// of the product has the same bits whichever of them computed it.
#pragma once
#include "tma_helpers.cuh"
#include "mma_helpers.cuh"
#include "stream_k_partials.cuh"

namespace rs_skinny {
using rs_streamk::first_unit;
using rs_streamk::cta_of_unit;
constexpr int TILE_N = 64;                 // rows of W per unit
constexpr int BOX_K = 64;                  // k per TMA box (one 128-byte swizzle row)
constexpr int BOXES = 2;                   // boxes per unit
constexpr int TILE_K = BOX_K * BOXES;      // k per unit
constexpr int W_BOX_BYTES = TILE_N * BOX_K * 2;
constexpr int W_BYTES = W_BOX_BYTES * BOXES;
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int SMEM_BUDGET = 200 * 1024;

enum Epilogue : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3 };

struct SkinnyParams {
    void* C; long ldc;
    int M, N, K;
    int stages;
    float* workspace;          // [grid][2][8 NT activation rows][TILE_N] float32 partials
    int* status;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <int NT, int EPI>
__device__ __forceinline__ void store_tile(const SkinnyParams& p, const float (&acc)[NT][4], int tile, int warp, int g, int t) {
    const int na = tile * TILE_N + 16 * warp + g, nb = na + 8;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int m0 = 8 * j + 2 * t;
        if (EPI == EPI_SWIGLU_BF16) {
            // rows of W alternate gate, up: lanes g and g ^ 1 hold a pair; the even one writes
            float partner[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) partner[i] = __shfl_xor_sync(0xffffffffu, acc[j][i], 4);
            if ((g & 1) == 0) {
                __nv_bfloat16* out = (__nv_bfloat16*)p.C;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = m0 + (i & 1), n = (i >> 1) ? nb : na;
                    if (m < p.M && n + 1 < p.N) {
                        const float gate = acc[j][i], up = partner[i];
                        out[(size_t)m * p.ldc + (n >> 1)] = __float2bfloat16_rn(silu_mul_fast(gate, up));
                    }
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = m0 + (i & 1), n = (i >> 1) ? nb : na;
                if (m < p.M && n < p.N) {
                    const size_t o = (size_t)m * p.ldc + n;
                    if (EPI == EPI_STORE_BF16) ((__nv_bfloat16*)p.C)[o] = __float2bfloat16_rn(acc[j][i]);
                    else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = acc[j][i];
                    else ((float*)p.C)[o] = __ldcg((const float*)p.C + o) + acc[j][i];   // from L2: another CTA of the same kernel may have written it
                }
            }
        }
    }
}


// The consumers' work on one unit in shared memory (W tile at wst, activation tile at xst, both as TMA left them with the
// 128-byte swizzle): warp `warp` of four owns rows 16 * warp .. + 15 of the unit's 64 rows of W; lane (g, t) as in
// mma.sync.  acc takes the first 64 of k, acc2 the second: two independent MMA chains.
template <int NT>
__device__ __forceinline__ void consume_unit(uint32_t wst, uint32_t xst, int warp, int g, int t, float (&acc)[NT][4],
                                             float (&acc2)[NT][4]) {
    constexpr int X_BOX_BYTES = 8 * NT * BOX_K * 2;
#pragma unroll
    for (int b = 0; b < BOXES; ++b) {
        const uint32_t row_a = wst + b * W_BOX_BYTES + (16 * warp + g) * 128, row_b = row_a + 8 * 128;
        const uint32_t xb = xst + b * X_BOX_BYTES;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            // lane t takes the 16-byte chunks 2t and 2t+1 of the row (the same for W and A, whatever g is:
            // the k slots of the MMA pair lane (g, t) of one operand with lane (g', t) of the other);
            // with the swizzle the 8 lanes of a quarter-warp then fall into 8 different bank groups
            const uint32_t chunk = (uint32_t)(((2 * t + half) ^ g) << 4);
            const uint4 wa = lds128(row_a + chunk), wb = lds128(row_b + chunk);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 x = lds128(xb + (8 * j + g) * 128 + chunk);
                const uint32_t a0[4] = {wa.x, wb.x, wa.y, wb.y}, a1[4] = {wa.z, wb.z, wa.w, wb.w};
                if (b == 0) { mma16816(acc[j], a0, x.x, x.y); mma16816(acc[j], a1, x.z, x.w); }
                else { mma16816(acc2[j], a0, x.x, x.y); mma16816(acc2[j], a1, x.z, x.w); }
            }
        }
    }
}

// A CTA's float32 partial of a row tile it shares with other CTAs: slot 0 for the tile its range starts in, 1 for the
// tile it ends in.
template <int NT>
__device__ __forceinline__ void store_partial(float* workspace, int cta, int slot, int warp, int g, int t, const float (&acc)[NT][4]) {
    float* mine = workspace + ((size_t)cta * 2 + slot) * (8 * NT * TILE_N) + 16 * warp + g;
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) __stcg(mine + (8 * j + 2 * t + (i & 1)) * TILE_N + 8 * (i >> 1), acc[j][i]);
}

// Which row tile the boundary between CTA b - 1 and CTA b of a product with G CTAs finishes, if any: it acts if the
// boundary lies inside a tile and no earlier boundary does.
struct SharedTile { bool acts; int tile, tile_first, c_first, c_last; };
__device__ __forceinline__ SharedTile shared_tile_of_boundary(int b, int N, int K, int G) {
    const int KB = (K + TILE_K - 1) / TILE_K;
    const int U = ((N + TILE_N - 1) / TILE_N) * KB;
    const int ub = first_unit(b, U, G);
    SharedTile st;
    st.tile = ub / KB; st.tile_first = st.tile * KB;
    st.acts = ub % KB != 0 && first_unit(b - 1, U, G) <= st.tile_first;
    st.c_first = b - 1;
    st.c_last = st.acts ? cta_of_unit(st.tile_first + KB - 1, U, G) : b - 1;
    return st;
}

// Adds the partials of a shared row tile in CTA order (fixed by the shape alone) and applies the epilogue; the 128
// threads of four warps, laid out as the consumers of the product.
template <int NT, int EPI>
__device__ __forceinline__ void finish_shared_tile(const SkinnyParams& p, const SharedTile& st, int G, int warp, int g, int t) {
    const int KB = (p.K + TILE_K - 1) / TILE_K;
    const int U = ((p.N + TILE_N - 1) / TILE_N) * KB;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
    constexpr int CH = NT == 1 ? 4 : (NT == 2 ? 2 : 1);       // contributors whose loads are in flight together
    for (int c0 = st.c_first; c0 <= st.c_last; c0 += CH) {
        float v[CH][NT][4];
#pragma unroll
        for (int cc = 0; cc < CH; ++cc) {
            const int c = min(c0 + cc, st.c_last);
            const int cslot = (first_unit(c, U, G) >= st.tile_first) ? 0 : 1;
            const float* src = p.workspace + ((size_t)c * 2 + cslot) * (8 * NT * TILE_N) + 16 * warp + g;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) v[cc][j][i] = ld_dep(src + (8 * j + 2 * t + (i & 1)) * TILE_N + 8 * (i >> 1));
        }
#pragma unroll
        for (int cc = 0; cc < CH; ++cc)
            if (c0 + cc <= st.c_last) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[j][i] += v[cc][j][i];
            }
    }
    store_tile<NT, EPI>(p, acc, st.tile, warp, g, t);
}
}  // namespace rs_skinny
