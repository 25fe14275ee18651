// bfloat16 matrix product on the 5th-generation tensor cores (sm_100a only):
//   C[m, n] (=|+=) sum_k A[m, k] * W[n, k],  A: [M, K] activations, W: [N, K] weight, both K-major.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Inside a CTA:
//   warp 0 (one elected lane)  - TMA producer: cp.async.bulk.tensor loads of a 128 x 64 tile of A and a
//                                BN x 64 tile of W per pipeline stage, 128-byte swizzle, completion on an mbarrier;
//   warp 1 (one elected lane)  - issues tcgen05.mma (M = 128, N = BN, K = 16, four per stage) with the
//                                accumulator in tensor memory, tcgen05.commit releases the stage;
//   warps 2-5                  - epilogue: tcgen05.ld of their 32 accumulator lanes, then one of
//                                  store bf16 | store f32 | f32 += (residual add) | SiLU(gate)*up on interleaved columns.
// The accumulator is double buffered in tensor memory (2 x BN columns), so the epilogue of one tile runs
// under the main loop of the next.  No cluster, no multicast: every CTA loads its own tiles.
//
// Every wait on an mbarrier is bounded (about two seconds): on expiry the kernel sets
// RS_STATUS_WAIT_EXPIRED in the status word, stops issuing work, lets copies in flight land, frees its
// tensor memory and returns, so a logic error cannot hang the device.
//
// Reference counterpart: gemm_f32/gemm_bf16 with epilogue modes 0/1/2 (src/cuda/kernels.cu:1062-1231),
// an mma.sync kernel whose inputs are rounded to f16; there is no Blackwell kernel in the reference.
#include "tma_helpers.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                    // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;      // 16 KiB
constexpr int THREADS = 192;

enum Epilogue : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3 };

template <int BN> struct Cfg {
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int OUT_STAGE_BYTES = 4 * 2 * 4096;    // results on their way out: per epilogue warp two buffers of 32 rows x 128 bytes
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, bf16 inputs, f32 accumulate
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
// shared memory -> global through the TMA unit: a plain tiled store, or an addition to what is there (done in L2)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_out_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_out_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_out_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups of
// 8 rows 1024 bytes apart (stride byte offset), leading byte offset 1 (unused for swizzled K-major),
// descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: f32 accumulator (bits 4-5 = 1), bf16 A and B (bits 7-9, 10-12 = 1), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct GemmParams {
    void* C; long ldc;
    int M, N, K;
    int vec_ok;            // C rows allow 16-byte vector access
    int bn;                // columns per tile: the template's BN, or less (a multiple of 16) in buffers sized for BN
    int out_by_tma;        // float32 results leave through shared memory and the TMA unit (map_c is valid)
    int* status;
};

template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t* r, int row, int col0, int nmax) {
    // r: 32 consecutive accumulator columns [col0, col0 + 32) of output row `row`; columns from nmax on are not this tile's
    if (row >= p.M) return;
    if (EPI == EPI_SWIGLU_BF16) {
        // columns alternate gate, up: out[row, (col0 + 2j) / 2] = silu(gate_j) * up_j
        const int half_n = nmax >> 1, oc0 = col0 >> 1;
        __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + oc0;
        if (p.vec_ok && oc0 + 16 <= half_n) {
            uint32_t packed[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
                const float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
                __nv_bfloat162 v = __floats2bfloat162_rn(silu_mul_fast(g0, u0), silu_mul_fast(g1, u1));
                packed[j] = *reinterpret_cast<uint32_t*>(&v);
            }
            reinterpret_cast<uint4*>(out)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(out)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (oc0 + j < half_n) {
                    const float g = __uint_as_float(r[2 * j]), u = __uint_as_float(r[2 * j + 1]);
                    out[j] = __float2bfloat16_rn(silu_mul_fast(g, u));
                }
            }
        }
    } else if (EPI == EPI_STORE_BF16) {
        __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + col0;
        if (p.vec_ok && col0 + 32 <= nmax) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * j]), __uint_as_float(r[8 * q + 2 * j + 1]));
                    w[j] = *reinterpret_cast<uint32_t*>(&v);
                }
                reinterpret_cast<uint4*>(out)[q] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < nmax) out[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
        }
    } else {   // float32 store or accumulate
        float* out = (float*)p.C + (size_t)row * p.ldc + col0;
        if (p.vec_ok && col0 + 32 <= nmax) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                       __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                if (EPI == EPI_ADD_F32) {
                    const float4 o = reinterpret_cast<float4*>(out)[q];
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                reinterpret_cast<float4*>(out)[q] = v;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < nmax) out[j] = (EPI == EPI_ADD_F32 ? out[j] : 0.f) + __uint_as_float(r[j]);
        }
    }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                       // swizzled tiles need 1024-byte alignment
    uint8_t* aligned = smem_raw + (base - raw);
    uint8_t* out_stage = aligned + C::STAGES * C::STAGE_BYTES;          // 1 KiB aligned: the stages are multiples of 1 KiB
    uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + C::OUT_STAGE_BYTES);
    // barrier layout: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then tmem base + abort flag
    const uint32_t bar0 = base + C::STAGES * C::STAGE_BYTES + C::OUT_STAGE_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * C::STAGES + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * C::STAGES + 2 + b); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn = p.bn;                                                // <= BN: buffers and tensor-memory columns are laid out for BN
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + bn - 1) / bn;
    const int num_tiles = tiles_m * tiles_n, num_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    // Launched with programmatic stream serialization the kernel may have come this far while its predecessor in the
    // stream is still running.  The weights are nobody's output: the producer starts the first ring of W tiles, then
    // waits for the predecessor before it touches A; the epilogue warps wait before they touch C.

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const int pre = num_kb < C::STAGES ? num_kb : C::STAGES;              // stages of the first tile started early
            {
                const int n0 = (blockIdx.x / tiles_m) * bn;
                for (int kb = 0; kb < pre; ++kb) {
                    mbar_expect_tx(full_bar(kb), A_BYTES + bn * BK * 2);
                    tma_load_2d(base + kb * C::STAGE_BYTES + A_BYTES, &map_w, kb * BK, n0, full_bar(kb));
                }
                pdl_wait();
                const int m0 = (blockIdx.x % tiles_m) * BM;
                for (int kb = 0; kb < pre; ++kb) tma_load_2d(base + kb * C::STAGE_BYTES, &map_a, kb * BK, m0, full_bar(kb));
            }
            int s = pre == C::STAGES ? 0 : pre; uint32_t phase = pre == C::STAGES ? 1u : 0u;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * bn;       // m fastest: neighbours share W
                for (int kb = t == (int)blockIdx.x ? pre : 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, p.status)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), A_BYTES + bn * BK * 2);
                    const uint32_t sa = base + s * C::STAGE_BYTES;
                    tma_load_2d(sa, &map_a, kb * BK, m0, full_bar(s));
                    tma_load_2d(sa + A_BYTES, &map_w, kb * BK, n0, full_bar(s));
                    if (++s == C::STAGES) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BM, bn);
            int s = 0; uint32_t phase = 0;
            bool ok = true;
            int local = 0;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(tempty_bar(buf), ((local >> 1) & 1) ^ 1u, abort_flag, p.status)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar(s), phase, abort_flag, p.status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + s * C::STAGE_BYTES;
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)       // advance 32 bytes (>>4 = 2) per K = 16 inside the swizzle row
                        umma_bf16(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(empty_bar(s));                   // stage free once these MMAs have read it
                    if (++s == C::STAGES) { s = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(tfull_bar(buf));             // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps 2..5
        const int quarter = warp & 3;                            // TMEM lanes [32 * quarter, +32) belong to this warp
        int local = 0;
        bool ok = true;
        // Float32 results (the residual stream) leave through shared memory: a warp writes its 32 rows x 32 columns as a
        // tile of 128-byte rows, 16-byte chunks swizzled by the row, and one lane hands the tile to the TMA unit, which
        // stores it or, for +=, adds it to what is there (each element belongs to one tile only, so it is the same single
        // addition).  Stored from the registers, every lane of an instruction touched a line of its own, and the old
        // values had to be fetched the same way first: 16 k line accesses per tile in the queue that the MMA and TMA
        // issue share.
        // bfloat16 results go the same way, two chunks (bf16 store) or four (SiLU(gate) * up: 16 results per chunk) to
        // a row of 128 bytes.
        const bool tma_out = p.out_by_tma;
        constexpr int CHUNKS_PER_ROW = (EPI == EPI_STORE_BF16) ? 2 : (EPI == EPI_SWIGLU_BF16 ? 4 : 1);
        uint8_t* my_stage = out_stage + (warp - 2) * 2 * 4096;
        uint32_t n_out = 0;
        pdl_wait();
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * bn;
            const int nmax = min(p.N, n0 + bn);
            if (!mbar_wait(tfull_bar(buf), (local >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < bn; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + c, r);
                tmem_ld_wait();
                if (tma_out) {
                    if (m0 + quarter * 32 >= p.M) continue;          // none of this warp's rows exists: nothing to send
                    // (columns from N on are sent too: they lie outside the tensor, and the TMA unit drops them)
                    const int part = (c >> 5) % CHUNKS_PER_ROW;      // which piece of the 128-byte row this chunk fills
                    uint8_t* dst = my_stage + (n_out & 1u) * 4096;
                    if (part == 0) {
                        if (lane == 0) tma_out_wait_read_1();        // the tile sent from this buffer two rows ago has been read
                        __syncwarp();
                    }
                    if (EPI == EPI_ADD_F32 || EPI == EPI_STORE_F32) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<uint4*>(dst + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    } else if (EPI == EPI_STORE_BF16) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * j]), __uint_as_float(r[8 * q + 2 * j + 1]));
                                w[j] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            *reinterpret_cast<uint4*>(dst + lane * 128 + (((part * 4 + q) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float g0 = __uint_as_float(r[16 * q + 4 * j]), u0 = __uint_as_float(r[16 * q + 4 * j + 1]);
                                const float g1 = __uint_as_float(r[16 * q + 4 * j + 2]), u1 = __uint_as_float(r[16 * q + 4 * j + 3]);
                                __nv_bfloat162 v = __floats2bfloat162_rn(silu_mul_fast(g0, u0), silu_mul_fast(g1, u1));
                                w[j] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            *reinterpret_cast<uint4*>(dst + lane * 128 + (((part * 2 + q) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                    if (part != CHUNKS_PER_ROW - 1) continue;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        // first result column of the row: accumulator column / 2 for SiLU(gate) * up
                        const int c_first = n0 + c - 32 * (CHUNKS_PER_ROW - 1);
                        const int x = EPI == EPI_SWIGLU_BF16 ? c_first >> 1 : c_first;
                        if (x < (EPI == EPI_SWIGLU_BF16 ? p.N >> 1 : p.N)) {          // else the whole row lies past the last column
                            if (EPI == EPI_ADD_F32) tma_add_2d(&map_c, smem_u32(dst), x, m0 + quarter * 32);
                            else tma_store_2d(&map_c, smem_u32(dst), x, m0 + quarter * 32);
                        }
                        tma_out_commit();
                    }
                    ++n_out;
                } else if (n0 + c < nmax) {
                    epilogue_chunk<EPI>(p, r, row, n0 + c, nmax);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
        }
        if (tma_out && lane == 0) tma_out_wait_all();            // the results are in place before the kernel ends
    }
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // give loads that were already issued time to land before the shared memory is released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
using rs_tma::get_map;
using rs_tma::sm_count;

// Tensor map of the result [M, N] (float32 or bfloat16) with row pitch ldc: boxes of 128 bytes x 32 rows, 128-byte
// swizzle.  Rows from M on and columns from N on are outside the tensor, so the TMA unit drops them.
struct CMapKey { const void* c; long ldc; int M, N, elem; };
std::vector<std::pair<CMapKey, CUtensorMap>> g_cmaps;
std::mutex g_cmaps_mutex;
int c_map(const void* Cptr, long ldc, int M, int N, int elem, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_cmaps_mutex);
    for (auto& e : g_cmaps)
        if (e.first.c == Cptr && e.first.ldc == ldc && e.first.M == M && e.first.N == N && e.first.elem == elem) { *out = e.second; return 0; }
    rs_tma::EncodeTiledFn enc = rs_tma::get_encoder();
    if (!enc) return 1;
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)ldc * elem};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elem), 32};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(Cptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1;
    if (g_cmaps.size() > 256) g_cmaps.clear();
    g_cmaps.push_back({CMapKey{Cptr, ldc, M, N, elem}, m});
    *out = m;
    return 0;
}

template <int BN, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mc, const GemmParams& p, int max_ctas, cudaStream_t s) {
    auto kern = gemm_tc_kernel<BN, EPI>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + p.bn - 1) / p.bn);
    int grid = tiles < sm_count() ? tiles : sm_count();
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    return rs_launch_pdl(kern, dim3(grid), dim3(THREADS), (size_t)Cfg<BN>::SMEM_BYTES, s, ma, mw, mc, p);
}

template <int BN>
int launch_epi(int epi, const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mc, const GemmParams& p, int max_ctas, cudaStream_t s) {
    switch (epi) {
        case EPI_STORE_BF16: return launch<BN, EPI_STORE_BF16>(ma, mw, mc, p, max_ctas, s);
        case EPI_STORE_F32: return launch<BN, EPI_STORE_F32>(ma, mw, mc, p, max_ctas, s);
        case EPI_ADD_F32: return launch<BN, EPI_ADD_F32>(ma, mw, mc, p, max_ctas, s);
        case EPI_SWIGLU_BF16: return launch<BN, EPI_SWIGLU_BF16>(ma, mw, mc, p, max_ctas, s);
    }
    return (int)cudaErrorInvalidValue;
}
}  // namespace

// Whether the tensor-core kernel takes this problem (else the caller uses the CUDA-core kernel):
// K and the row pitches must keep every row 16-byte aligned, and the pointers themselves too.
RS_EXPORT int rs_gemm_tc_supported(long a_ptr, long lda, long w_ptr, long ldw, int N, int K, int epi) {
    if (K <= 0 || N <= 0 || K % 8 || lda % 8 || ldw % 8) return 0;
    if ((a_ptr & 15) || (w_ptr & 15)) return 0;
    if (epi == EPI_SWIGLU_BF16 && (N & 1)) return 0;
    return 1;
}

// C[M, N] (=|+=) A[M, K] . W[N, K]^T with bf16 inputs.  a_rows is the row capacity of A's buffer (>= M): the
// tensor map covers the whole buffer, rows beyond M are computed and dropped.  epi: 0 bf16 store, 1 f32 store,
// 2 f32 accumulate, 3 SiLU(gate)*up over interleaved columns into a bf16 [M, N/2] output.  bn: columns per tile, 64, 128,
// a multiple of 16 from 144 to 256, or 0 to choose.  max_ctas > 0 caps the grid (tests use it to force several tiles per CTA).
RS_EXPORT int rs_gemm_bf16_tc(const void* A, long lda, long a_rows, const void* W, long ldw, void* C, long ldc, int M,
                              int N, int K, int epi, int bn, int max_ctas, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!rs_gemm_tc_supported((long)A, lda, (long)W, ldw, N, K, epi) || a_rows < M) return (int)cudaErrorInvalidValue;
    int tpl = bn;                                        // template instantiation (buffer sizes): 64, 128 or 256
    if (bn == 0) {
        // The tile width that needs the least time by a model fitted to measurements at 256 to 2,048 rows: the time is
        // the number of waves of tiles over the SMs times what a wave of that width costs (256 columns: 1, 192: 0.94,
        // 128: 0.745, 64: 0.68 - narrower tiles load the rows of A more often per flop).  Many waves always end at 256.
        // (240 or 176 columns for 4,096 or 6,144 were measured at 2,048 rows: slower than 256 by 2 to 17 %.)
        const long tm = (M + BM - 1) / BM;
        const int sms = sm_count();
        const int widths[4] = {256, 192, 128, 64};
        const double wave_cost[4] = {1.0, 0.94, 0.745, 0.68};
        double best = 0;
        for (int i = 0; i < 4; ++i) {
            const long tiles = tm * ((N + widths[i] - 1) / widths[i]);
            const double cost = (double)((tiles + sms - 1) / sms) * wave_cost[i];
            if (i == 0 || cost < best - 1e-9) { best = cost; bn = widths[i]; }
        }
        tpl = bn == 192 ? 256 : bn;
    } else if (bn > 128 && bn <= 256 && bn % 16 == 0) {
        tpl = 256;
    }
    CUtensorMap ma, mw;
    int rc = get_map(A, a_rows, K, lda, BM, &ma);
    if (rc) return rc;
    rc = get_map(W, N, K, ldw, bn, &mw);
    if (rc) return rc;
    GemmParams p;
    p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.status = status; p.bn = bn;
    const int out_elem = (epi == EPI_STORE_BF16 || epi == EPI_SWIGLU_BF16) ? 2 : 4;
    p.vec_ok = (((long)C & 15) == 0 && (ldc * out_elem) % 16 == 0) ? 1 : 0;
    // results go out through the TMA unit when a tile's columns fill whole 128-byte rows of the staging tiles
    CUtensorMap mc = ma;
    const int acc_cols_per_row = out_elem == 4 ? 32 : (epi == EPI_SWIGLU_BF16 ? 128 : 64);
    p.out_by_tma = p.vec_ok && bn % acc_cols_per_row == 0 &&
                   c_map(C, ldc, M, epi == EPI_SWIGLU_BF16 ? N / 2 : N, out_elem, &mc) == 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (tpl == 256) return launch_epi<256>(epi, ma, mw, mc, p, max_ctas, s);
    if (tpl == 128 && bn == 128) return launch_epi<128>(epi, ma, mw, mc, p, max_ctas, s);
    if (tpl == 64 && bn == 64) return launch_epi<64>(epi, ma, mw, mc, p, max_ctas, s);
    return (int)cudaErrorInvalidValue;
}
