// A chain of decode-step operations in ONE persistent kernel: the matrix products of up to 8 activation rows that
// follow one another between two attention calls, with the row norms and the adding-up of shared tiles between them.
//
// A decode step at small batch is a chain of dependent products whose time is the time to stream their weights:
//   residual += attn_out . Wo^T ;  h = RMSNorm(residual) ;  act = SiLU(h . Wg^T) * (h . Wu^T) ;  residual += act . Wd^T ;
//   h' = RMSNorm(residual) ;  qkv = h' . Wqkv^T            (then rotation, cache write and attention: other kernels)
// Launched one by one, every product pays for a kernel boundary: its CTAs can only move in when those of the product
// before have left their SMs, and then wait for their first weights to arrive, so the HBM stream stops four times a
// layer.  Here the chain is one launch of one CTA per SM.  Each CTA's producer lane walks the units of ALL products of
// the chain in order and keeps the ring of shared-memory stages full of weight tiles, across the boundaries: weights
// are nobody's output, so they may be fetched as early as a stage is free.  Only the small activation tile of a unit
// has to wait until the operation that writes it is complete on every CTA.  That point is a barrier across the grid
// (an arrival counter and a generation word in global memory, self-resetting; every wait on it is bounded).  While the
// consumers stand at a barrier, or add up a shared tile, or norm a row, the weights of the next product keep arriving.
//
// Operations (a list built by the host, the same for every CTA):
//   GEMV     C (=|+=) A[M <= 8, K] . W[N, K]^T with the epilogues of the few-rows product (skinny_tile.cuh): units of
//            64 rows x 128 of k dealt to the CTAs in equal contiguous shares; a row tile whose k range one CTA covers
//            is finished by it, a shared one leaves as float32 partials in the workspace;
//   REDUCE   the shared tiles of the GEMV before it: partials added in CTA order, epilogue applied (CTA b - 1 takes the
//            boundary between CTA b - 1 and CTA b);
//   ROWNORM  out[m] = RMSNorm(x[m]) * w as bfloat16 for the M rows of x (CTA m takes row m), adding first, if asked,
//            the partials that the GEMV before it (a float32 += into x) left for its shared tiles.
// A grid barrier follows every operation but the last.  The arithmetic of every operation, and its order, are those of
// the separate kernels (skinny_gemm_kernel, skinny_reduce_kernel, finish_rmsnorm_kernel, rmsnorm_bf16_vec_kernel), so a
// step gives the same bits whether its products run chained or one by one.
//
// The CTAs wait for one another, so all of them must be resident at once: the grid is one CTA per SM (each takes more
// than half an SM's shared memory, so no SM holds two), and the kernel before it in the stream never waits for this
// one.  Should a CTA not arrive all the same, the barrier's wait runs out (RS_WAIT_LIMIT_NS), the status word gets
// RS_STATUS_WAIT_EXPIRED and every CTA walks to its end without touching memory again: an error, never a hang.
//
// Reference counterpart: the decode layer loop of src/gpu_model.rs:3181-3328 (nine launches a layer).
#include "skinny_tile.cuh"
#include <string.h>

namespace {
using namespace rs_skinny;
using rs_streamk::Layout;
using rs_streamk::OwedBatch;
using rs_streamk::owed_begin4;
using rs_streamk::owed_end4;
using rs_streamk::sharers_of_tile;

constexpr int MAX_OPS = 12;
constexpr int MAX_GEMV = 6;
constexpr int NT = 1;                                         // up to 8 activation rows
constexpr int X_BOX_BYTES = 8 * NT * BOX_K * 2;
constexpr int X_BYTES = X_BOX_BYTES * BOXES;
constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int CHAIN_THREADS = CONSUMER_THREADS + 64;          // four consumer warps, a warp for the weights, a warp for the activations
constexpr int NORM_VIRTUAL = 512;                             // threads of the row norm kernels whose arithmetic ROWNORM repeats
constexpr int NORM_Q = NORM_VIRTUAL / CONSUMER_THREADS;       // ... each consumer thread stands for this many of them
constexpr int NORM_MAX_VPT = 4;                               // rows of up to 512 * 4 * 4 values

enum OpType : int { OP_GEMV = 0, OP_REDUCE = 1, OP_ROWNORM = 2 };

struct ChainOp {
    int type;
    int M, N, K;               // GEMV, REDUCE: the product; ROWNORM: M rows of N values, K = depth of the product that owes
    int epi;                   // GEMV, REDUCE: epilogue
    int map;                   // GEMV: which pair of tensor maps
    int owed;                  // ROWNORM: the GEMV before it left partials for x
    int w_dt;                  // ROWNORM: element type of the norm's weights
    void* C; long ldc;         // GEMV, REDUCE: output; ROWNORM: x (float32 rows)
    const void* w;             // ROWNORM: weights
    void* out; long out_stride;   // ROWNORM: bfloat16 rows
    float eps;
    int pad;
};

struct ChainParams {
    int n_ops, stages;
    float* workspace;          // partials: [grid][2][8][64] float32
    unsigned int* barrier;     // [0] arrivals at the current barrier, [1] generation
    int* status;
    ChainOp ops[MAX_OPS];
};

struct ChainMaps { CUtensorMap w[MAX_GEMV]; CUtensorMap a[MAX_GEMV]; };

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Barrier across the grid, called by the 128 consumer threads of every CTA.  bar[0] counts arrivals and is set back to
// zero by the last one, who then bumps the generation bar[1]; the others wait for the generation to move.  Returns false
// if the wait ran out or the CTA had given up already (then nothing was waited for).
__device__ __forceinline__ bool grid_barrier(unsigned int* bar, unsigned int G, volatile int* abort_flag, int* status) {
    consumer_sync();                                          // this CTA's writes of the operation are issued
    if (threadIdx.x == 0 && !*abort_flag) {
        const unsigned int gen = ld_acquire_gpu(bar + 1);     // cannot move before this CTA has arrived
        __threadfence();                                      // the CTA's writes are visible to the GPU before it counts as arrived
        if (atomicAdd(bar, 1u) == G - 1) {
            bar[0] = 0u;
            st_release_gpu(bar + 1, gen + 1u);
        } else {
            const unsigned long long t0 = global_ns();
            for (unsigned int i = 0; ld_acquire_gpu(bar + 1) == gen; ++i) {
                if ((i & 15u) == 15u && global_ns() - t0 > RS_WAIT_LIMIT_NS) {
                    *abort_flag = 1;
                    atomicOr(status, RS_STATUS_WAIT_EXPIRED);
                    break;
                }
            }
        }
        __threadfence();
    }
    consumer_sync();
    return !*abort_flag;
}

// out[m] = RMSNorm(x[m] (+ the owed partials)) * w as bfloat16 and x[m] made whole, by 128 threads with the arithmetic
// of the 512-thread row norm kernels: thread r stands for their threads r, r + 128, r + 256 and r + 384 in turn (each
// with its own running sum of squares), and the block's sum is taken over the same tree.
template <int VPT>
__device__ __forceinline__ void rownorm(const ChainOp& op, const float* workspace, int G, int m, float* scratch) {
    const int N = op.N, n4 = N >> 2;
    const Layout L = {TILE_N, TILE_K, 8};
    const int KB = (op.K + TILE_K - 1) / TILE_K;
    const int U = ((N + TILE_N - 1) / TILE_N) * KB;
    const int per_cta = op.owed ? U / G : 0, extra = op.owed ? U % G : 0;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* xr = (float*)op.C + (size_t)m * op.ldc;
    float4 v[NORM_Q][VPT];
    float ss[NORM_Q];
#pragma unroll
    for (int q = 0; q < NORM_Q; ++q) {
        OwedBatch part[VPT];
        int2 sh[VPT];
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int idx = tid + q * CONSUMER_THREADS + u * NORM_VIRTUAL;
            v[q][u] = make_float4(0.f, 0.f, 0.f, 0.f);
            sh[u] = make_int2(0, 0);
            if (idx < n4) {
                v[q][u] = ld_dep(reinterpret_cast<const float4*>(xr) + idx);
                if (op.owed) {
                    sh[u] = sharers_of_tile(idx * 4 / TILE_N, KB, U, G);
                    if (sh[u].x != sh[u].y) owed_begin4(part[u], workspace, L, m, idx * 4, KB, per_cta, extra, sh[u].x, sh[u].y);
                }
            }
        }
        float s = 0.f;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int idx = tid + q * CONSUMER_THREADS + u * NORM_VIRTUAL;
            if (idx < n4 && sh[u].x != sh[u].y) {
                const float4 acc = owed_end4(part[u], workspace, L, m, idx * 4, KB, per_cta, extra, sh[u].x, sh[u].y);
                v[q][u].x += acc.x; v[q][u].y += acc.y; v[q][u].z += acc.z; v[q][u].w += acc.w;
                reinterpret_cast<float4*>(xr)[idx] = v[q][u];
            }
            s = fmaf(v[q][u].x, v[q][u].x, s); s = fmaf(v[q][u].y, v[q][u].y, s);
            s = fmaf(v[q][u].z, v[q][u].z, s); s = fmaf(v[q][u].w, v[q][u].w, s);
        }
        ss[q] = warp_sum(s);
    }
    // the tree of block_sum over 16 warps of 32: warp sums, then one warp adds the 16
    consumer_sync();
    if (lane == 0) {
#pragma unroll
        for (int q = 0; q < NORM_Q; ++q) scratch[warp + CONSUMER_WARPS * q] = ss[q];
    }
    consumer_sync();
    if (warp == 0) {
        float t = lane < NORM_VIRTUAL / 32 ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    consumer_sync();
    const float sc = 1.0f / sqrtf(scratch[32] / (float)N + op.eps);
    __nv_bfloat16* o = (__nv_bfloat16*)op.out + (size_t)m * op.out_stride;
#pragma unroll
    for (int q = 0; q < NORM_Q; ++q)
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int idx = tid + q * CONSUMER_THREADS + u * NORM_VIRTUAL;
            if (idx < n4) {
                float w0, w1, w2, w3;
                if (op.w_dt == RS_F32) {
                    const float4 f = reinterpret_cast<const float4*>(op.w)[idx];
                    w0 = f.x; w1 = f.y; w2 = f.z; w3 = f.w;
                } else {
                    const uint2 h = reinterpret_cast<const uint2*>(op.w)[idx];
                    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&h.x), b = *reinterpret_cast<const __nv_bfloat162*>(&h.y);
                    w0 = __low2float(a); w1 = __high2float(a); w2 = __low2float(b); w3 = __high2float(b);
                }
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v[q][u].x * sc * w0, v[q][u].y * sc * w1);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(v[q][u].z * sc * w2, v[q][u].w * sc * w3);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(o)[idx] = pk;
            }
        }
}

template <int EPI>
__device__ __forceinline__ void gemv_segment_end(const SkinnyParams& sp, float (&acc)[NT][4], bool whole, bool ok, int slot, int tile,
                                                 int warp, int g, int t) {
    if (whole) {
        if (ok) store_tile<NT, EPI>(sp, acc, tile, warp, g, t);
    } else {
        store_partial<NT>(sp.workspace, blockIdx.x, slot, warp, g, t, acc);
    }
}

__global__ void __launch_bounds__(CHAIN_THREADS, 1)
decode_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const int stages = p.stages;
    const uint32_t bar0 = base + stages * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
    uint8_t* tail = smem_raw + (base - raw) + stages * STAGE_BYTES + 16 * stages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail);
    volatile int* ops_done = reinterpret_cast<volatile int*>(tail + 4);     // operations complete on every CTA
    float* scratch = reinterpret_cast<float*>(tail + 16);                   // 33 floats of the row norm's tree

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x;

    if (warp == CONSUMER_WARPS) {
        if (lane == 0) {
            for (int s = 0; s < stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), CONSUMER_WARPS); }
            *abort_flag = 0;
            *ops_done = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    __syncthreads();

    if (warp >= CONSUMER_WARPS) {
        // ------------------------------------------------------------ two producer lanes walk this CTA's units of all
        // products in order.  Warp 4 asks for the weights: as far ahead as stages are free, across the products'
        // boundaries.  Warp 5 follows with each unit's small activation tile, once every operation before the unit's
        // product is complete on all CTAs.  Both kinds of load report to the stage's one barrier.
        if (lane == 0) {
            const bool weights = warp == CONSUMER_WARPS;
            if (weights) pdl_launch_dependents();
            else pdl_wait();                                   // the first product's input is an earlier kernel's output
            int s = 0; uint32_t use = 0;                       // the next unit's stage; how often it has been used before
            bool ok = true;
            for (int k = 0; k < p.n_ops && ok; ++k) {
                const ChainOp& op = p.ops[k];
                if (op.type != OP_GEMV) continue;
                const int KB = (op.K + TILE_K - 1) / TILE_K;
                const int U = ((op.N + TILE_N - 1) / TILE_N) * KB;
                const int u0 = first_unit(blockIdx.x, U, G), u1 = first_unit(blockIdx.x + 1, U, G);
                if (u0 == u1) continue;
                const CUtensorMap* map = weights ? &maps.w[op.map] : &maps.a[op.map];
                if (!weights) {
                    // operations 0 .. k - 1 are complete everywhere once the consumers have passed the barrier behind k - 1
                    const unsigned long long t0 = global_ns();
                    for (unsigned int i = 1; *ops_done < k; ++i) {
                        if ((i & 63u) == 0u) {
                            if (*abort_flag) { ok = false; break; }
                            if (global_ns() - t0 > RS_WAIT_LIMIT_NS) {
                                *abort_flag = 1; atomicOr(p.status, RS_STATUS_WAIT_EXPIRED); ok = false; break;
                            }
                        }
                    }
                    if (!ok) break;
                    // written by other CTAs through the generic proxy, read from here on by the async proxy
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                int tile = u0 / KB, kb = u0 % KB;
                for (int u = u0; u < u1; ++u) {
                    if (use != 0 && !mbar_wait(empty_bar(s), (use - 1) & 1u, abort_flag, p.status)) { ok = false; break; }
                    const uint32_t dst = base + s * STAGE_BYTES;
                    if (weights) {
                        mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
                        for (int b = 0; b < BOXES; ++b)
                            tma_load_2d(dst + b * W_BOX_BYTES, map, kb * TILE_K + b * BOX_K, tile * TILE_N, full_bar(s));
                    } else {
#pragma unroll
                        for (int b = 0; b < BOXES; ++b)
                            tma_load_2d(dst + W_BYTES + b * X_BOX_BYTES, map, kb * TILE_K + b * BOX_K, 0, full_bar(s));
                    }
                    if (++s == stages) { s = 0; ++use; }
                    if (++kb == KB) { kb = 0; ++tile; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ consumers: the operations in order
        const int g = lane >> 2, t = lane & 3;
        pdl_wait();                                            // outputs and the workspace belong to earlier kernels until now
        bool ok = true;
        int cs = 0; uint32_t cphase = 0;                       // stage and phase of the next unit to consume (all products)
        for (int k = 0; k < p.n_ops; ++k) {
            const ChainOp& op = p.ops[k];
            if (op.type == OP_GEMV) {
                const int KB = (op.K + TILE_K - 1) / TILE_K;
                const int U = ((op.N + TILE_N - 1) / TILE_N) * KB;
                const int u0 = first_unit(blockIdx.x, U, G), u1 = first_unit(blockIdx.x + 1, U, G);
                SkinnyParams sp;
                sp.C = op.C; sp.ldc = op.ldc; sp.M = op.M; sp.N = op.N; sp.K = op.K; sp.stages = stages;
                sp.workspace = p.workspace; sp.status = p.status;
                float acc[NT][4], acc2[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
                    acc2[j][0] = acc2[j][1] = acc2[j][2] = acc2[j][3] = 0.f;
                }
                int seg_start = u0;
                int tile = u0 / KB, kb = u0 % KB;
                for (int u = u0; u < u1; ++u) {
                    const int s = cs;
                    if (ok) ok = mbar_wait(full_bar(s), cphase, abort_flag, p.status);
                    if (++cs == stages) { cs = 0; cphase ^= 1u; }
                    const uint32_t wst = base + s * STAGE_BYTES, xst = wst + W_BYTES;
                    if (ok) {
                        consume_unit<NT>(wst, xst, warp, g, t, acc, acc2);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_bar(s));
                    }
                    if (kb == KB - 1 || u == u1 - 1) {
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) { acc[j][i] += acc2[j][i]; acc2[j][i] = 0.f; }
                        const int tile_first = tile * KB;
                        const bool whole = seg_start == tile_first && kb == KB - 1;
                        const int slot = (u0 >= tile_first) ? 0 : 1;
                        if (ok) {                                  // a CTA that gave up writes nothing
                            if (op.epi == EPI_STORE_BF16) gemv_segment_end<EPI_STORE_BF16>(sp, acc, whole, ok, slot, tile, warp, g, t);
                            else if (op.epi == EPI_STORE_F32) gemv_segment_end<EPI_STORE_F32>(sp, acc, whole, ok, slot, tile, warp, g, t);
                            else if (op.epi == EPI_ADD_F32) gemv_segment_end<EPI_ADD_F32>(sp, acc, whole, ok, slot, tile, warp, g, t);
                            else gemv_segment_end<EPI_SWIGLU_BF16>(sp, acc, whole, ok, slot, tile, warp, g, t);
                        }
#pragma unroll
                        for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
                        seg_start = u + 1;
                    }
                    if (++kb == KB) { kb = 0; ++tile; }
                }
            } else if (op.type == OP_REDUCE) {
                if (ok && (int)blockIdx.x < G - 1) {
                    const SharedTile st = shared_tile_of_boundary(blockIdx.x + 1, op.N, op.K, G);
                    if (st.acts) {
                        SkinnyParams sp;
                        sp.C = op.C; sp.ldc = op.ldc; sp.M = op.M; sp.N = op.N; sp.K = op.K; sp.stages = stages;
                        sp.workspace = p.workspace; sp.status = p.status;
                        if (op.epi == EPI_STORE_BF16) finish_shared_tile<NT, EPI_STORE_BF16>(sp, st, G, warp, g, t);
                        else if (op.epi == EPI_STORE_F32) finish_shared_tile<NT, EPI_STORE_F32>(sp, st, G, warp, g, t);
                        else if (op.epi == EPI_ADD_F32) finish_shared_tile<NT, EPI_ADD_F32>(sp, st, G, warp, g, t);
                        else finish_shared_tile<NT, EPI_SWIGLU_BF16>(sp, st, G, warp, g, t);
                    }
                }
            } else {
                if (ok) {
                    for (int m = blockIdx.x; m < op.M; m += G) {
                        if (op.N <= NORM_VIRTUAL * 4) rownorm<1>(op, p.workspace, G, m, scratch);
                        else if (op.N <= NORM_VIRTUAL * 8) rownorm<2>(op, p.workspace, G, m, scratch);
                        else rownorm<4>(op, p.workspace, G, m, scratch);
                    }
                }
            }
            if (k + 1 < p.n_ops) {
                if (!grid_barrier(p.barrier, (unsigned int)G, abort_flag, p.status)) ok = false;
                if (threadIdx.x == 0) *ops_done = k + 1;
            }
        }
    }
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);          // let loads already issued land
    }
    __syncthreads();
}
}  // namespace

// One operation of a chain as the host states it (see decode_chain_kernel).  For a GEMV, A/lda/a_rows/W/ldw describe
// the operands as in rs_skinny_gemm_bf16.
struct RsChainOp {
    int type, M, N, K, epi, owed, w_dt, reserved;
    long lda, a_rows, ldw, ldc, out_stride;
    const void* A; const void* W; void* C; const void* w; void* out;
    float eps; int reserved2;
};

RS_EXPORT int rs_decode_chain_max_ops() { return MAX_OPS; }
RS_EXPORT int rs_decode_chain_max_products() { return MAX_GEMV; }
RS_EXPORT int rs_decode_chain_max_rows() { return 8 * NT; }
RS_EXPORT int rs_decode_chain_max_norm_width() { return NORM_VIRTUAL * 4 * NORM_MAX_VPT; }

// Runs the operations in order as one kernel.  workspace: rs_skinny_gemm_workspace_floats() float32 values; barrier: two
// 32-bit words that were zero before the first launch ever and are touched by nothing else; launches that share them or
// the workspace must not overlap on the GPU.  Returns cudaErrorInvalidValue for a list the kernel does not take.
RS_EXPORT int rs_decode_chain(const RsChainOp* ops, int n_ops, float* workspace, unsigned int* barrier, int* status, void* stream) {
    if (n_ops <= 0) return 0;
    if (n_ops > MAX_OPS || workspace == nullptr || barrier == nullptr || status == nullptr) return (int)cudaErrorInvalidValue;
    ChainParams p;
    ChainMaps maps;
    memset(&maps, 0, sizeof(maps));
    p.n_ops = n_ops; p.workspace = workspace; p.barrier = barrier; p.status = status;
    int n_gemv = 0;
    for (int k = 0; k < n_ops; ++k) {
        const RsChainOp& h = ops[k];
        ChainOp& o = p.ops[k];
        memset(&o, 0, sizeof(o));
        o.type = h.type; o.M = h.M; o.N = h.N; o.K = h.K; o.epi = h.epi; o.owed = h.owed; o.w_dt = h.w_dt;
        o.C = h.C; o.ldc = h.ldc; o.w = h.w; o.out = h.out; o.out_stride = h.out_stride; o.eps = h.eps;
        if (h.M <= 0 || h.M > 8 * NT || h.N <= 0 || h.K <= 0 || h.C == nullptr) return (int)cudaErrorInvalidValue;
        if (h.type == OP_GEMV) {
            if (n_gemv == MAX_GEMV || h.K % 8 || h.lda % 8 || h.ldw % 8 || ((long)h.A & 15) || ((long)h.W & 15) || h.a_rows < h.M ||
                h.epi < EPI_STORE_BF16 || h.epi > EPI_SWIGLU_BF16 || (h.epi == EPI_SWIGLU_BF16 && (h.N & 1)))
                return (int)cudaErrorInvalidValue;
            int rc = rs_tma::get_map(h.W, h.N, h.K, h.ldw, TILE_N, &maps.w[n_gemv]);
            if (rc) return rc;
            rc = rs_tma::get_map(h.A, h.a_rows, h.K, h.lda, 8 * NT, &maps.a[n_gemv]);
            if (rc) return rc;
            o.map = n_gemv++;
        } else if (h.type == OP_REDUCE) {
            if (k == 0 || ops[k - 1].type != OP_GEMV || ops[k - 1].C != h.C || ops[k - 1].N != h.N || ops[k - 1].K != h.K ||
                ops[k - 1].epi != h.epi || ops[k - 1].M != h.M)
                return (int)cudaErrorInvalidValue;
        } else if (h.type == OP_ROWNORM) {
            if (h.N % 4 || h.N > NORM_VIRTUAL * 4 * NORM_MAX_VPT || h.ldc % 4 || h.out_stride % 4 || ((long)h.C & 15) || ((long)h.out & 7) ||
                ((long)h.w & 15) || h.w == nullptr || h.out == nullptr || (h.w_dt != RS_F32 && h.w_dt != RS_BF16))
                return (int)cudaErrorInvalidValue;
            if (h.owed && (k == 0 || ops[k - 1].type != OP_GEMV || ops[k - 1].epi != EPI_ADD_F32 || ops[k - 1].C != h.C ||
                           ops[k - 1].N != h.N || ops[k - 1].K != h.K || ops[k - 1].M != h.M || ops[k - 1].ldc != h.ldc))
                return (int)cudaErrorInvalidValue;
        } else {
            return (int)cudaErrorInvalidValue;
        }
    }
    if (n_gemv == 0) return (int)cudaErrorInvalidValue;
    int stages = SMEM_BUDGET / STAGE_BYTES;
    if (stages > 24) stages = 24;
    p.stages = stages;
    const int smem = stages * STAGE_BYTES + 1024 + 16 * stages + 16 + 33 * 4 + 64;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    return rs_launch_pdl(decode_chain_kernel, dim3((unsigned)rs_tma::sm_count()), dim3(CHAIN_THREADS), (size_t)smem, (cudaStream_t)stream, maps, p);
}
