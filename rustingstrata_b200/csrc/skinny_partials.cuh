// How the streaming product for few rows (skinny_gemm_tma.cu) deals its work to CTAs and where it leaves the float32
// partial sums of a row tile that several CTAs shared.  The product itself, the small kernel that adds the partials up
// and a kernel that adds them while it reads the product's output (the row norm behind a product into the residual
// stream) all go by these rules.
//
// Work: units of TILE_N rows of W x TILE_K of k, numbered tile by tile (a tile's KB = ceil(K / TILE_K) units are
// consecutive), dealt to G CTAs as evenly as possible: the first U % G CTAs take one unit more.  A tile whose units lie
// in one CTA is stored by that CTA.  Every CTA that holds only part of a tile writes its partial to
//   workspace[(cta * 2 + slot) * rows_padded * TILE_N + m * TILE_N + (n - tile * TILE_N)],
// slot 0 for the tile its range starts in, slot 1 for the tile its range ends in (a range has at most one shared tile
// at either end), rows_padded = 8 for up to 8 rows.
// The sum of a shared tile is taken from zero in CTA order, then the epilogue is applied: that order is the shape's alone.
#pragma once

namespace rs_skinny {
constexpr int TILE_N = 64;                 // rows of W per unit
constexpr int TILE_K = 128;                // k per unit

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

// Sum of the partials of row m (< 8), columns [n0, n0 + 4) (n0 a multiple of 4), of a tile shared by CTAs
// c_first..c_last, from zero in CTA order.  per_cta = U / G, extra = U % G.  Reads through L2.  In two steps, so that a
// caller with several such sums to take can have all their loads in flight before it waits for any:
// owed_begin4 asks for the first OWED_BATCH contributors' values (a tile rarely has more), owed_end4 adds them up and
// fetches what is left.
constexpr int OWED_BATCH = 4;
struct OwedBatch { float4 q[OWED_BATCH]; };

__device__ __forceinline__ const float4* owed_addr(const float* workspace, int m, int n0, int KB, int per_cta, int extra, int c) {
    const int tile = n0 / TILE_N, r = n0 % TILE_N;
    const int cslot = (c * per_cta + min(c, extra) >= tile * KB) ? 0 : 1;                  // first_unit(c) without the division
    return reinterpret_cast<const float4*>(workspace + ((size_t)c * 2 + cslot) * (8 * TILE_N) + m * TILE_N + r);
}

__device__ __forceinline__ void owed_begin4(OwedBatch& b, const float* workspace, int m, int n0, int KB, int per_cta, int extra,
                                            int c_first, int c_last) {
#pragma unroll
    for (int cc = 0; cc < OWED_BATCH; ++cc)
        b.q[cc] = __ldcg(owed_addr(workspace, m, n0, KB, per_cta, extra, min(c_first + cc, c_last)));
}

__device__ __forceinline__ float4 owed_end4(const OwedBatch& b, const float* workspace, int m, int n0, int KB, int per_cta, int extra,
                                            int c_first, int c_last) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int cc = 0; cc < OWED_BATCH; ++cc)
        if (c_first + cc <= c_last) { acc.x += b.q[cc].x; acc.y += b.q[cc].y; acc.z += b.q[cc].z; acc.w += b.q[cc].w; }
    for (int c0 = c_first + OWED_BATCH; c0 <= c_last; c0 += OWED_BATCH) {
        OwedBatch more;
        owed_begin4(more, workspace, m, n0, KB, per_cta, extra, c0, c_last);
#pragma unroll
        for (int cc = 0; cc < OWED_BATCH; ++cc)
            if (c0 + cc <= c_last) { acc.x += more.q[cc].x; acc.y += more.q[cc].y; acc.z += more.q[cc].z; acc.w += more.q[cc].w; }
    }
    return acc;
}
}  // namespace rs_skinny
