// Skinny bfloat16 matrix product for decode batches (M <= 32 rows of activations):
//   C[m, n] (=|+=) sum_k A[m, k] * W[n, k]
// The work is reading W once from HBM, so the kernel is organised around that stream: a CTA owns 16
// consecutive rows of W; its 8 warps take interleaved 32-wide slices of K, each lane loading 16 contiguous
// bytes of two rows per slice (the CTA reads 512 contiguous bytes of every row at a time), with several
// slices in flight.  The products run on the tensor cores as mma.sync m16n8k16 with W as the 16-row operand
// and up to four groups of 8 activation rows as the 8-column operand; because both operands are loaded with
// the same lane-to-k assignment, the 16-byte loads feed the fragments without a shuffle (the sum over k does
// not care in which order k is visited).  Warps' partial sums meet in shared memory and are added in warp
// order, so the result does not depend on timing.  Accumulation is float32.
//
// Reference counterpart: gemv_bf16 / gemvn_bf16 (src/cuda/kernels.cu:307-329,826-853): one warp per row on
// CUDA cores, each weight read once for up to 4 inputs.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int ROWS = 16;       // rows of W per CTA
constexpr int KC = 32;         // k per warp slice

enum Epilogue : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3 };

__device__ __forceinline__ void mma_bf16_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <int NT, int EPI>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(const __nv_bfloat16* __restrict__ A, long lda,
                                                          const __nv_bfloat16* __restrict__ W, long ldw, void* C,
                                                          long ldc, int M, int N, int K) {
    __shared__ float part[WARPS][ROWS][8 * NT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * ROWS;
    const int rowa = r0 + g, rowb = r0 + g + 8;
    const __nv_bfloat16* wa = W + (size_t)rowa * ldw + 8 * t;
    const __nv_bfloat16* wb = W + (size_t)rowb * ldw + 8 * t;
    const bool oka = rowa < N, okb = rowb < N;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const int n_slices = (K + KC - 1) / KC;
    constexpr int UNROLL = 4;
    for (int s0 = warp; s0 < n_slices; s0 += WARPS * UNROLL) {
        uint4 va[UNROLL], vb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (s0 + u * WARPS) * KC + 8 * t;
            const bool in = k < K;                                   // K is a multiple of 8: a lane's 8 values are all in or all out
            va[u] = (in && oka) ? ld_stream16(wa + (size_t)(s0 + u * WARPS) * KC) : make_uint4(0, 0, 0, 0);
            vb[u] = (in && okb) ? ld_stream16(wb + (size_t)(s0 + u * WARPS) * KC) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (s0 + u * WARPS) * KC + 8 * t;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int m = 8 * j + g;
                uint4 x = make_uint4(0, 0, 0, 0);
                if (m < M && k < K) x = __ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda + k));
                mma_bf16_16816(acc[j], va[u].x, vb[u].x, va[u].y, vb[u].y, x.x, x.y);
                mma_bf16_16816(acc[j], va[u].z, vb[u].z, va[u].w, vb[u].w, x.z, x.w);
            }
        }
    }
    // fragment → shared: d0,d1 = (row g, cols 2t, 2t+1); d2,d3 = (row g+8, same cols)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        part[warp][g][8 * j + 2 * t] = acc[j][0];
        part[warp][g][8 * j + 2 * t + 1] = acc[j][1];
        part[warp][g + 8][8 * j + 2 * t] = acc[j][2];
        part[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    if (EPI == EPI_SWIGLU_BF16) {
        // rows alternate gate, up: out[m, (r0 + 2i) / 2] = silu(gate) * up
        for (int idx = threadIdx.x; idx < (ROWS / 2) * 8 * NT; idx += WARPS * 32) {
            const int i = idx % (ROWS / 2), m = idx / (ROWS / 2);
            if (m >= M || r0 + 2 * i + 1 >= N) continue;
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) { gsum += part[w][2 * i][m]; usum += part[w][2 * i + 1][m]; }
            ((__nv_bfloat16*)C)[(size_t)m * ldc + (r0 >> 1) + i] = __float2bfloat16_rn(gsum / (1.0f + __expf(-gsum)) * usum);
        }
    } else {
        for (int idx = threadIdx.x; idx < ROWS * 8 * NT; idx += WARPS * 32) {
            const int r = idx % ROWS, m = idx / ROWS;
            if (m >= M || r0 + r >= N) continue;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) sum += part[w][r][m];
            const size_t o = (size_t)m * ldc + r0 + r;
            if (EPI == EPI_STORE_BF16) ((__nv_bfloat16*)C)[o] = __float2bfloat16_rn(sum);
            else if (EPI == EPI_STORE_F32) ((float*)C)[o] = sum;
            else ((float*)C)[o] += sum;
        }
    }
}

template <int NT>
int launch_nt(int epi, const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int N, int K,
              cudaStream_t s) {
    const dim3 grid((N + ROWS - 1) / ROWS), block(WARPS * 32);
    const __nv_bfloat16* a = (const __nv_bfloat16*)A;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    switch (epi) {
        case EPI_STORE_BF16: gemv_kernel<NT, EPI_STORE_BF16><<<grid, block, 0, s>>>(a, lda, w, ldw, C, ldc, M, N, K); break;
        case EPI_STORE_F32: gemv_kernel<NT, EPI_STORE_F32><<<grid, block, 0, s>>>(a, lda, w, ldw, C, ldc, M, N, K); break;
        case EPI_ADD_F32: gemv_kernel<NT, EPI_ADD_F32><<<grid, block, 0, s>>>(a, lda, w, ldw, C, ldc, M, N, K); break;
        case EPI_SWIGLU_BF16: gemv_kernel<NT, EPI_SWIGLU_BF16><<<grid, block, 0, s>>>(a, lda, w, ldw, C, ldc, M, N, K); break;
        default: return (int)cudaErrorInvalidValue;
    }
    return rs_launch_result();
}
}  // namespace

RS_EXPORT int rs_gemv_bf16_max_rows() { return 32; }

// Same contract as rs_gemm_bf16_tc for M <= 32.  Needs K, lda, ldw multiples of 8 and 16-byte aligned A and W.
RS_EXPORT int rs_gemv_bf16(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int N, int K,
                           int epi, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 32 || K <= 0 || K % 8 || lda % 8 || ldw % 8 || ((long)A & 15) || ((long)W & 15)) return (int)cudaErrorInvalidValue;
    if (epi == EPI_SWIGLU_BF16 && (N & 1)) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (M <= 8) return launch_nt<1>(epi, A, lda, W, ldw, C, ldc, M, N, K, s);
    if (M <= 16) return launch_nt<2>(epi, A, lda, W, ldw, C, ldc, M, N, K, s);
    if (M <= 24) return launch_nt<3>(epi, A, lda, W, ldw, C, ldc, M, N, K, s);
    return launch_nt<4>(epi, A, lda, W, ldw, C, ldc, M, N, K, s);
}
