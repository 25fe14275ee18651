// Attention of prompt portions in the bfloat16 engine: a tile of queries over the paged keys 0..position
// (or the window), flash-attention style on the warp-level tensor cores.
//
// A CTA of 4 warps owns 64 rows; a row is (query token, query head) with P heads of one kv group packed side
// by side (P = the largest power of two dividing the group, at most 16), so K and V tiles brought into
// shared memory serve P heads.  Keys are walked in blocks of 64 at absolute positions (block b = keys
// [64 b, 64 b + 64)), double-buffered with cp.async through the block table; per block each warp computes
// S = Q K^T for its 16 rows (mma.sync m16n8k16), masks (causal, window, length), runs the online softmax
// in float32 with exp2, and accumulates O += P V.  Since blocks sit at absolute positions, the order in
// which a query's keys are reduced does not depend on how the prompt was cut into portions.
//
// Reference counterpart: attn_prefill_* (src/cuda/kernels.cu:2813-3156): 64 queries x 32 keys, f16 inputs,
// one head per block, reads the cache so earlier portions are visible.
#include "mma_helpers.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int ROWS = 64;               // rows per CTA (16 per warp)
constexpr int BKV = 64;                // keys per block

struct PrefillParams {
    const __nv_bfloat16* q; long q_stride;
    __nv_bfloat16* out; long out_stride;
    const __nv_bfloat16* cache; long page_stride;
    int num_pages, page_size;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len; const int* work;    // work: [n][2] = (sequence, first query of the tile)
    int n_q, n_kv, group, pack, tokens_per_cta;
    int window;
    float scale_log2;
    int* status;
};

__host__ __device__ inline int pack_of(int group) {
    int p = 1;
    while (p < 16 && group % (2 * p) == 0) p *= 2;
    return p;
}

template <int HD>
__global__ void __launch_bounds__(WARPS * 32) prefill_attention_kernel(const PrefillParams p) {
    constexpr int LD = HD + 8, KS = HD / 16, DT = HD / 8, CHUNKS = HD / 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [2][BKV][LD]
    __nv_bfloat16* Vs = Ks + 2 * BKV * LD;                               // [2][BKV][LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int seq = p.work[2 * blockIdx.x], q_off = p.work[2 * blockIdx.x + 1];
    const int chunks_per_group = p.group / p.pack;
    const int kvh = blockIdx.y / chunks_per_group;
    const int head0 = kvh * p.group + (blockIdx.y % chunks_per_group) * p.pack;
    const int row0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - row0;
    const int kv_len = p.kv_len[seq];
    const int n_tok = min(p.tokens_per_cta, q_len - q_off);
    const int n_rows = n_tok * p.pack;
    const int qpos0 = kv_len - q_len + q_off;
    const int key_lo = p.window > 0 ? max(0, qpos0 - p.window + 1) : 0;
    const int key_hi = min(kv_len, qpos0 + n_tok);
    const int blk_lo = key_lo / BKV, blk_hi = (key_hi + BKV - 1) / BKV;
    const int* table = p.block_table + (size_t)seq * p.table_stride;

    // 128 threads, 64 key rows per block: two threads share a row (one page lookup each), each copies half of its chunks
    auto load_block = [&](int blk, int stage) {
        const int j = tid >> 1;
        __nv_bfloat16* kd = Ks + stage * BKV * LD + j * LD;
        __nv_bfloat16* vd = Vs + stage * BKV * LD + j * LD;
        const int kpos = blk * BKV + j;
        const __nv_bfloat16* src = nullptr;
        if (kpos >= key_lo && kpos < key_hi) {
            const int page = table[kpos / p.page_size];
            if (page >= 0 && page < p.num_pages)
                src = p.cache + (size_t)page * p.page_stride + ((size_t)kvh * p.page_size + (kpos % p.page_size)) * HD;
            else if ((tid & 1) == 0)
                atomicOr(p.status, RS_STATUS_BAD_PAGE);
        }
        const int c0 = (tid & 1) * (CHUNKS / 2);
        if (src != nullptr) {
            const __nv_bfloat16* vsrc = src + (size_t)p.n_kv * p.page_size * HD;
#pragma unroll
            for (int c = 0; c < CHUNKS / 2; ++c) {
                cp_async16(smem_addr(kd + (c0 + c) * 8), src + (c0 + c) * 8);
                cp_async16(smem_addr(vd + (c0 + c) * 8), vsrc + (c0 + c) * 8);
            }
        } else {
#pragma unroll
            for (int c = 0; c < CHUNKS / 2; ++c) {
                *reinterpret_cast<uint4*>(kd + (c0 + c) * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + (c0 + c) * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };

    load_block(blk_lo, 0);

    // this lane's two rows: r_a = 16 warp + g, r_b = r_a + 8; row r = (token r / pack, head r % pack)
    const int ra = 16 * warp + g, rb = ra + 8;
    const bool va = ra < n_rows, vb = rb < n_rows;
    const int qpos_a = qpos0 + ra / p.pack, qpos_b = qpos0 + rb / p.pack;
    const __nv_bfloat16* qa = p.q + (size_t)(row0 + q_off + ra / p.pack) * p.q_stride + (size_t)(head0 + ra % p.pack) * HD;
    const __nv_bfloat16* qb = p.q + (size_t)(row0 + q_off + rb / p.pack) * p.q_stride + (size_t)(head0 + rb % p.pack) * HD;
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int d0 = 16 * ks + 2 * t;
        qf[ks][0] = va ? *reinterpret_cast<const uint32_t*>(qa + d0) : 0u;
        qf[ks][1] = vb ? *reinterpret_cast<const uint32_t*>(qb + d0) : 0u;
        qf[ks][2] = va ? *reinterpret_cast<const uint32_t*>(qa + d0 + 8) : 0u;
        qf[ks][3] = vb ? *reinterpret_cast<const uint32_t*>(qb + d0 + 8) : 0u;
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    // rows of this warp span query positions [wq_lo, wq_hi]
    const int wq_lo = qpos0 + (16 * warp) / p.pack;
    const int wq_hi = qpos0 + min(n_rows - 1, 16 * warp + 15) / p.pack;
    const bool warp_live = 16 * warp < n_rows;

    for (int blk = blk_lo; blk < blk_hi; ++blk) {
        const int stage = (blk - blk_lo) & 1;
        if (blk + 1 < blk_hi) load_block(blk + 1, stage ^ 1);
        if (blk + 1 < blk_hi) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        const __nv_bfloat16* kb = Ks + stage * BKV * LD;
        const __nv_bfloat16* vbk = Vs + stage * BKV * LD;
        const int k0 = blk * BKV;
        // a warp skips blocks none of its rows can see (all keys after its last query, or before the window of its first)
        const bool block_visible = warp_live && k0 <= wq_hi && (p.window <= 0 || k0 + BKV - 1 > wq_lo - p.window);
        if (block_visible) {
            float s[BKV / 8][4];
#pragma unroll
            for (int nt = 0; nt < BKV / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int np = 0; np < BKV / 16; ++np) {
                    uint32_t b00, b01, b10, b11;
                    const int row = 16 * np + (lane >> 4) * 8 + (lane & 7);
                    const int col = 16 * ks + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(smem_addr(kb + row * LD + col), b00, b01, b10, b11);
                    mma16816(s[2 * np], qf[ks], b00, b01);
                    mma16816(s[2 * np + 1], qf[ks], b10, b11);
                }
            }
            const bool need_mask = (k0 + BKV - 1 > wq_lo) || (k0 + BKV > key_hi) || (p.window > 0 && k0 <= wq_hi - p.window) ||
                                   k0 < key_lo;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < BKV / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = s[nt][i] * p.scale_log2;
                    if (need_mask) {
                        const int kpos = k0 + 8 * nt + 2 * t + (i & 1);
                        const int qp = (i >> 1) ? qpos_b : qpos_a;
                        const bool ok = kpos <= qp && kpos < key_hi && kpos >= key_lo && (p.window <= 0 || kpos > qp - p.window);
                        v = ok ? v : -INFINITY;
                    }
                    s[nt][i] = v;
                    mx[i >> 1] = fmaxf(mx[i >> 1], v);
                }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                corr[r] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[r] - m_new);
                m_run[r] = m_new;
            }
            float rs[2] = {0.f, 0.f};
            uint32_t pf[BKV / 16][4];
#pragma unroll
            for (int nt = 0; nt < BKV / 8; ++nt) {
                float e[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float mm = m_run[i >> 1];
                    e[i] = (mm == -INFINITY) ? 0.f : fast_exp2(s[nt][i] - mm);
                    rs[i >> 1] += e[i];
                }
                pf[nt >> 1][(nt & 1) * 2] = pack_bf16(e[0], e[1]);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e[2], e[3]);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
                rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
                l_run[r] = l_run[r] * corr[r] + rs[r];
            }
#pragma unroll
            for (int d = 0; d < DT; ++d) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
                for (int d = 0; d < DT; d += 2) {
                    uint32_t v00, v01, v10, v11;
                    const int row = 16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int col = 8 * (d + (lane >> 4));
                    ldmatrix_x4_trans(smem_addr(vbk + row * LD + col), v00, v01, v10, v11);
                    mma16816(o[d], pf[kk], v00, v01);
                    mma16816(o[d + 1], pf[kk], v10, v11);
                }
            }
        }
        __syncthreads();                                   // the stage may be overwritten by the next load
    }

    // ---- normalise and store: d0,d1 → row a, dims 8 d + 2 t, +1; d2,d3 → row b
    const float inv_a = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    __nv_bfloat16* oa = p.out + (size_t)(row0 + q_off + ra / p.pack) * p.out_stride + (size_t)(head0 + ra % p.pack) * HD;
    __nv_bfloat16* ob = p.out + (size_t)(row0 + q_off + rb / p.pack) * p.out_stride + (size_t)(head0 + rb % p.pack) * HD;
#pragma unroll
    for (int d = 0; d < DT; ++d) {
        if (va) *reinterpret_cast<uint32_t*>(oa + 8 * d + 2 * t) = pack_bf16(o[d][0] * inv_a, o[d][1] * inv_a);
        if (vb) *reinterpret_cast<uint32_t*>(ob + 8 * d + 2 * t) = pack_bf16(o[d][2] * inv_b, o[d][3] * inv_b);
    }
}

template <int HD>
int launch(const PrefillParams& p, int n_work, cudaStream_t s) {
    constexpr size_t smem = (size_t)4 * BKV * (HD + 8) * 2;
    auto kern = prefill_attention_kernel<HD>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    kern<<<dim3(n_work, p.n_kv * (p.group / p.pack)), WARPS * 32, smem, s>>>(p);
    return rs_launch_result();
}
}  // namespace

RS_EXPORT int rs_attention_prefill_bf16_supported(int n_q, int n_kv, int hd) {
    if (n_kv <= 0 || n_q % n_kv) return 0;
    return hd == 32 || hd == 64 || hd == 96 || hd == 128;
}

// Query tokens per CTA: the host cuts each sequence's queries into tiles of this many.
RS_EXPORT int rs_attention_prefill_bf16_q_per_cta(int n_q, int n_kv) { return ROWS / pack_of(n_q / n_kv); }

RS_EXPORT int rs_attention_prefill_bf16(const void* q, long q_stride, void* out, long out_stride, const void* cache,
                                        long page_stride, int num_pages, int page_size, const int* block_table,
                                        int table_stride, const int* q_start, const int* kv_len, const int* work,
                                        int n_work, int n_q, int n_kv, int hd, int window, float scale, int* status,
                                        void* stream) {
    if (n_work <= 0) return 0;
    if (!rs_attention_prefill_bf16_supported(n_q, n_kv, hd) || (q_stride % 2) || (out_stride % 2) || ((long)q & 3) ||
        ((long)out & 3) || ((long)cache & 15) || (page_stride % 8))
        return (int)cudaErrorInvalidValue;
    PrefillParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.cache = (const __nv_bfloat16*)cache; p.page_stride = page_stride; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work;
    p.n_q = n_q; p.n_kv = n_kv; p.group = n_q / n_kv; p.pack = pack_of(p.group); p.tokens_per_cta = ROWS / p.pack;
    p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    switch (hd) {
        case 32: return launch<32>(p, n_work, s);
        case 64: return launch<64>(p, n_work, s);
        case 96: return launch<96>(p, n_work, s);
        case 128: return launch<128>(p, n_work, s);
    }
    return (int)cudaErrorInvalidValue;
}
