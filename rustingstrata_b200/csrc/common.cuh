// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes and
// the CUDA stream to launch on, and returns the cudaError_t of the launch (0 = ok).
// Element types are passed as small integer codes so one symbol serves the 32-bit
// and the bfloat16 engine.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define RS_EXPORT extern "C" __attribute__((visibility("default")))

enum RsDtype : int { RS_F32 = 0, RS_BF16 = 1 };

// status bits written by kernels that detect a bad input instead of faulting
enum RsStatus : int {
    RS_STATUS_BAD_TOKEN = 1,      // token id outside the vocabulary
    RS_STATUS_BAD_PAGE = 2,       // block table entry outside the pool where a live key was expected
    RS_STATUS_WAIT_EXPIRED = 4,   // a bounded wait on a barrier gave up
    RS_STATUS_NON_FINITE = 8,     // a row of logits holds no finite maximum
    RS_STATUS_BAD_PLAN = 16,      // a work list points outside a workspace (partial-result slot beyond its capacity)
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// load element i of an array whose element type is only known at run time
__device__ __forceinline__ float load_any(const void* p, int dt, size_t i) {
    return dt == RS_F32 ? reinterpret_cast<const float*>(p)[i]
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// 2^x on the special-function unit (ex2.approx.ftz): one instruction, no range branches.  Its relative error
// (2^-22) is far below the bfloat16 rounding of the probabilities it feeds; exp2f() compiles to branchy code.
// SiLU(gate) * up of the bfloat16 products' epilogues.  The quotient is taken with the fast reciprocal (2 ulp, far
// below the rounding to bfloat16 that follows): the IEEE division costs ten instructions more per value and, when
// exp(-gate) overflows, a slow path of over a hundred cycles, which showed in the products of many rows.  Every
// bfloat16 kernel uses this one function, so they agree to the bit; the 32-bit path divides exactly.
__device__ __forceinline__ float silu_mul_fast(float gate, float up) { return __fdividef(gate, 1.0f + __expf(-gate)) * up; }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

#define RS_DISPATCH_DTYPE(dt, T, ...)                                   \
    do {                                                                \
        if ((dt) == RS_F32) { using T = float; __VA_ARGS__; }           \
        else if ((dt) == RS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return (int)cudaErrorInvalidValue;                         \
    } while (0)

static inline int rs_launch_result() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch -----------------------------------------------------------------
// Kernels of the decode step are launched so that a kernel may begin (be scheduled, read weights and other
// data no earlier kernel writes) while its predecessor in the stream is still running.  The contract of every
// kernel launched with rs_launch_pdl: it executes pdl_wait() before it reads anything an earlier kernel
// produced and before it writes anything at all; after pdl_wait() every earlier kernel has completed and its
// writes are visible.  pdl_launch_dependents() lets the next kernel start being scheduled.  Launched without
// the attribute (or with the switch off) both instructions do nothing and the stream order is the usual one.
// Data written by an earlier kernel of the step must not be read through the non-coherent path (ld.global.nc,
// which the compiler may choose for `const __restrict__` pointers) nor be served from a stale L1 line: a kernel
// that started early shares its SM with kernels that ran before the data was written.  Read it from L2.
template <typename T> __device__ __forceinline__ T ld_dep(const T* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_dep_f32(const __nv_bfloat16* p) {
    return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// one switch per shared library (an inline function's static is shared by its translation units)
inline int& rs_pdl_switch() { static int on = 1; return on; }

template <typename... KArgs, typename... Args>
static inline int rs_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = rs_pdl_switch() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
