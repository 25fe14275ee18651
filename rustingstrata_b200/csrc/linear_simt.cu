// Plain CUDA-core matrix product for every element-type combination:
//   out[m, n] (=|+=) sum_k A[m, k] * W[n, k]
// A: activations [M, K] (float32 or bfloat16), W: weight [N, K] row-major as stored in
// the checkpoint (float32 or bfloat16), out: float32 or bfloat16.  Products and sums are
// float32 FMAs (no TF32, no tensor cores), and each output element accumulates k in
// ascending order whatever M is, so a row's result does not depend on the batch it is in.
// This is the matrix product of the 32-bit engine and the fallback of the bfloat16
// engine for shapes its tensor-core kernels refuse.
//
// Reference counterpart: gemm_f32/gemm_bf16 (src/cuda/kernels.cu:1062-1231), whose
// epilogue modes 0 (store), 2 (y += result) are kept; mode 1 (SiLU*mul) is a kernel of
// its own in the 32-bit engine.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

template <typename TA, typename TW, typename TO, bool ACCUMULATE>
__global__ void __launch_bounds__(256) linear_simt_kernel(const TA* __restrict__ A, long lda, const TW* __restrict__ W,
                                                          long ldw, TO* __restrict__ out, long ldo, int M, int N,
                                                          int K) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;          // tx → n, ty → m
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread; consecutive threads walk k (contiguous)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? to_f32<TA>(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32<TW>(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            TO* o = out + (size_t)gm * ldo + gn;
            if (ACCUMULATE) *o = from_f32<TO>(to_f32<TO>(*o) + acc[i][j]);
            else *o = from_f32<TO>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TO>
int launch(const void* A, long lda, const void* W, long ldw, void* out, long ldo, int M, int N, int K, int accumulate,
           cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (accumulate)
        linear_simt_kernel<TA, TW, TO, true><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, ldw, (TO*)out, ldo, M, N, K);
    else
        linear_simt_kernel<TA, TW, TO, false><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, ldw, (TO*)out, ldo, M, N, K);
    return rs_launch_result();
}
}  // namespace

RS_EXPORT int rs_linear_simt(const void* A, int a_dt, long lda, const void* W, int w_dt, long ldw, void* out,
                             int out_dt, long ldo, int M, int N, int K, int accumulate, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RS_CASE(a, w, o, TA, TW, TO) \
    if (a_dt == a && w_dt == w && out_dt == o) return launch<TA, TW, TO>(A, lda, W, ldw, out, ldo, M, N, K, accumulate, s);
    RS_CASE(RS_F32, RS_F32, RS_F32, float, float, float)
    RS_CASE(RS_BF16, RS_BF16, RS_BF16, bf, bf, bf)
    RS_CASE(RS_BF16, RS_BF16, RS_F32, bf, bf, float)
    RS_CASE(RS_BF16, RS_F32, RS_BF16, bf, float, bf)
    RS_CASE(RS_BF16, RS_F32, RS_F32, bf, float, float)
    RS_CASE(RS_F32, RS_BF16, RS_F32, float, bf, float)
    RS_CASE(RS_F32, RS_F32, RS_BF16, float, float, bf)
    RS_CASE(RS_F32, RS_BF16, RS_BF16, float, bf, bf)
#undef RS_CASE
    return (int)cudaErrorInvalidValue;
}
