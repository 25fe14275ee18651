// How the two streaming ("stream-K") products deal their work to CTAs and where they leave the float32 partial sums of
// a row tile that several CTAs shared: the product for few rows (skinny_gemm_tma.cu: tiles of 64 rows of W, units 128
// of k deep, partials of 8 rows) and the tcgen05 product for up to 128 rows (mid_gemm_tcgen05.cu: tiles of 128 rows,
// units 128 deep, partials of 16, 32, 64 or 128 rows).  The products, the small kernels that add the partials up and
// the row norm that adds them while it reads a product's output all go by these rules.
//
// Work: units of tile_n rows of W x tile_k of k, numbered tile by tile (a tile's KB = ceil(K / tile_k) units are
// consecutive), dealt to G CTAs as evenly as possible: the first U % G CTAs take one unit more.  A tile whose units lie
// in one CTA is stored by that CTA.  Every CTA that holds only part of a tile writes its partial to
//   workspace[((cta * 2 + slot) * rows_padded + m) * tile_n + (n - tile * tile_n)],
// slot 0 for the tile its range starts in, slot 1 for the tile its range ends in (a range has at most one shared tile
// at either end).  The sum of a shared tile is taken in CTA order, then the epilogue is applied: that order is the
// shape's alone.
#pragma once
#include "common.cuh"

namespace rs_streamk {
struct Layout { int tile_n, tile_k, rows_padded; };

// first unit of CTA c when U units are dealt to G CTAs as evenly as possible
__host__ __device__ __forceinline__ int first_unit(int c, int U, int G) { return c * (U / G) + (c < U % G ? c : U % G); }
__host__ __device__ __forceinline__ int cta_of_unit(int u, int U, int G) {
    const int base = U / G, rem = U % G;
    return u < rem * (base + 1) ? u / (base + 1) : rem + (u - rem * (base + 1)) / base;
}

// First and last CTA that worked on a row tile (equal: the tile was stored whole).
__device__ __forceinline__ int2 sharers_of_tile(int tile, int KB, int U, int G) {
    return make_int2(cta_of_unit(tile * KB, U, G), cta_of_unit(tile * KB + KB - 1, U, G));
}

// Sum of the partials of row m, columns [n0, n0 + 4) (n0 a multiple of 4), of a tile shared by CTAs c_first..c_last,
// from zero in CTA order.  per_cta = U / G, extra = U % G.  Reads through L2.  In two steps, so that a caller with
// several such sums to take can have all their loads in flight before it waits for any: owed_begin4 asks for the first
// OWED_BATCH contributors' values (a tile rarely has more), owed_end4 adds them up and fetches what is left.
constexpr int OWED_BATCH = 4;
struct OwedBatch { float4 q[OWED_BATCH]; };

__device__ __forceinline__ const float4* owed_addr(const float* workspace, const Layout& L, int m, int n0, int KB, int per_cta,
                                                   int extra, int c) {
    const int tile = n0 / L.tile_n, r = n0 % L.tile_n;
    const int cslot = (c * per_cta + min(c, extra) >= tile * KB) ? 0 : 1;                  // first_unit(c) without the division
    return reinterpret_cast<const float4*>(workspace + (((size_t)c * 2 + cslot) * L.rows_padded + m) * L.tile_n + r);
}

__device__ __forceinline__ void owed_begin4(OwedBatch& b, const float* workspace, const Layout& L, int m, int n0, int KB, int per_cta,
                                            int extra, int c_first, int c_last) {
#pragma unroll
    for (int cc = 0; cc < OWED_BATCH; ++cc)
        b.q[cc] = __ldcg(owed_addr(workspace, L, m, n0, KB, per_cta, extra, min(c_first + cc, c_last)));
}

__device__ __forceinline__ float4 owed_end4(const OwedBatch& b, const float* workspace, const Layout& L, int m, int n0, int KB,
                                            int per_cta, int extra, int c_first, int c_last) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int cc = 0; cc < OWED_BATCH; ++cc)
        if (c_first + cc <= c_last) { acc.x += b.q[cc].x; acc.y += b.q[cc].y; acc.z += b.q[cc].z; acc.w += b.q[cc].w; }
    for (int c0 = c_first + OWED_BATCH; c0 <= c_last; c0 += OWED_BATCH) {
        OwedBatch more;
        owed_begin4(more, workspace, L, m, n0, KB, per_cta, extra, c0, c_last);
#pragma unroll
        for (int cc = 0; cc < OWED_BATCH; ++cc)
            if (c0 + cc <= c_last) { acc.x += more.q[cc].x; acc.y += more.q[cc].y; acc.z += more.q[cc].z; acc.w += more.q[cc].w; }
    }
    return acc;
}

// Whether launch_finish_rmsnorm takes a row of this width with these pitches and pointers.
bool finish_rmsnorm_supported(const void* C, long ldc, int N, const void* w, const void* out, long out_stride);

// RMSNorm of the M rows of C straight after a product with the f32 += epilogue whose shared tiles were left unfinished
// (workspace, N, K, G, L: the product's), one CTA per row: out[m] = RMSNorm(C[m] + partials) * w as bfloat16, and C[m]
// made whole.  Defined once, in skinny_gemm_tma.cu, for both products.
int launch_finish_rmsnorm(void* C, long ldc, int M, int N, int K, const float* workspace, int G, Layout L, const void* w, int w_dt,
                          float eps, void* out, long out_stride, cudaStream_t s);
}  // namespace rs_streamk
