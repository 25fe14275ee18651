// Token choice on the device, one CTA per row of float32 logits: argmax (greedy) and
// temperature sampling.
//
// Reference: greedy = first index of the largest logit (src/ops.rs:110-112; device
// argmax_part/argmax_rows src/cuda/kernels.cu:1574-1588); a best logit that is not
// finite is an error (src/ops.rs:223-226).  Sampling (host-side in the reference,
// src/ops.rs:281-314): weights exp((l - max)/temp), tokens whose scaled logit is 20 or
// more below the best are dropped, a uniform u in [0,1) picks the first candidate whose
// running sum exceeds u * total.  The reference walks candidates sorted by weight; this
// kernel walks them by token id, which draws from the same distribution.  The top-k and
// top-p cuts need that sorted order and are done by the host sampler.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 1024;

struct ArgPair { float v; int i; };

__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
    // larger value wins, lower index on ties; a NaN never displaces a number
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgPair block_argmax(const float* __restrict__ row, int V, ArgPair* sh) {
    ArgPair best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += THREADS) best = better(best, ArgPair{ld_dep(row + i), i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sh[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (threadIdx.x == 0) sh[0] = best;
    }
    __syncthreads();
    return sh[0];
}

// temps[r] <= 0 (or temps == nullptr): argmax.  Else inverse-CDF draw with uniforms[r].
// out[r] = token id, or -1 with RS_STATUS_NON_FINITE set when the best logit is not finite.
__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, long stride, int V,
                                                         const float* __restrict__ temps,
                                                         const float* __restrict__ uniforms, int* __restrict__ out,
                                                         int* __restrict__ status) {
    __shared__ ArgPair sha[32];
    __shared__ float warp_tot[32];
    __shared__ float total_sh;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * stride;
    const ArgPair best = block_argmax(row, V, sha);
    if (best.i == 0x7fffffff || !(fabsf(best.v) < INFINITY)) {
        if (threadIdx.x == 0) { out[r] = -1; atomicOr(status, RS_STATUS_NON_FINITE); }
        return;
    }
    const float temp = temps ? temps[r] : 0.f;
    if (temp <= 0.f) {
        if (threadIdx.x == 0) out[r] = best.i;
        return;
    }
    const float inv_temp = 1.0f / temp, mx = best.v;
    // each thread owns a contiguous range of ids, so ranges are in id order across the block
    const int per = (V + THREADS - 1) / THREADS;
    const int lo = threadIdx.x * per, hi = min(V, lo + per);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float x = (ld_dep(row + i) - mx) * inv_temp;
        mine += (x > -20.0f) ? expf(x) : 0.f;
    }
    // exclusive prefix over threads: warp scan, then scan of warp totals
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = warp_tot[lane], wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        warp_tot[lane] = wi - w;                      // exclusive prefix of warp totals
        if (lane == 31) total_sh = wi;
    }
    __syncthreads();
    const float before = warp_tot[warp] + (incl - mine);
    const float target = uniforms[r] * total_sh;
    if (threadIdx.x == 0) out[r] = best.i;            // fallback if rounding leaves no range containing target
    __syncthreads();
    if (mine > 0.f && target >= before && target < before + mine) {
        float acc = before;
        int pick = -1, last = -1;
        for (int i = lo; i < hi; ++i) {
            const float x = (ld_dep(row + i) - mx) * inv_temp;
            const float w = (x > -20.0f) ? expf(x) : 0.f;
            if (w > 0.f) {
                last = i;
                acc += w;
                if (target < acc) { pick = i; break; }
            }
        }
        out[r] = pick >= 0 ? pick : last;
    }
}
}  // namespace

RS_EXPORT int rs_sample(const float* logits, long stride, int rows, int V, const float* temps, const float* uniforms,
                        int* out, int* status, void* stream) {
    if (rows <= 0) return 0;
    return rs_launch_pdl(sample_kernel, dim3(rows), dim3(THREADS), 0, (cudaStream_t)stream, logits, stride, V, temps, uniforms,
                         out, status);
}
