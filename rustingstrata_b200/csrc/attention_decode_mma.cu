// Decode attention of the bfloat16 engine: one query token per sequence over its paged keys and values.
//
// grid = (sequences, kv heads, splits); a CTA takes one split of SPLIT keys (fixed, at absolute positions)
// of one kv head and serves all query heads of that group at once, so K and V are read from HBM exactly
// once per group.  The CTA brings its whole split into shared memory with 16-byte cp.async copies through
// the block table (all loads in flight together), then each of its 4 warps takes a quarter of the keys:
// scores S = Q K^T and the weighted sum O += P V run as mma.sync m16n8k16 (the group's heads are the 16-row
// operand, padded with zero rows), softmax is float32 with exp2 on pre-scaled scores.  The warps' (max, sum,
// O) are combined through shared memory and written as one un-normalised partial per (sequence, split,
// head); the merge kernel adds the splits in ascending order.  Keys of a split are visited in the same
// order whatever the batch holds, so a row's result does not depend on its neighbours.
//
// Reference counterparts: attn_decode_gqa_* + attn_merge (src/cuda/kernels.cu:2571-2625): K/V of a group
// read once with cp.async double buffering, CUDA-core dot products, 32 splits.
#include "mma_helpers.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 8;
constexpr int SPLIT = 128;             // keys per CTA; must equal the split size the host plans with
constexpr int KEYS_PER_WARP = SPLIT / WARPS;   // 16: warps 0-3 work on the first half of the split, 4-7 on the second

struct DecodeParams {
    const __nv_bfloat16* q; long q_stride;
    __nv_bfloat16* out; long out_stride;
    const __nv_bfloat16* cache; long page_stride;
    int num_pages, page_size;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len; const int* work;
    int n_q, n_kv, group;
    int window;
    float scale_log2;                  // scale * log2(e)
    const int* split_start;
    float* partial;                    // [slot][n_q][hd + 2]: acc, max (log2 units), sum
    int* status;
};

template <int HD>
__global__ void __launch_bounds__(WARPS * 32) decode_attention_kernel(const DecodeParams p) {
    constexpr int LD = HD + 8;                       // padded row: ldmatrix rows fall into distinct banks
    constexpr int KS = HD / 16;                      // k-steps of Q K^T
    constexpr int DT = HD / 8;                       // 8-wide output tiles of P V
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [SPLIT][LD]
    __nv_bfloat16* Vs = Ks + SPLIT * LD;                                   // [SPLIT][LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int w = blockIdx.x, kvh = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();                                      // the new key and value of this step come from the previous kernel
    const int seq = p.work[w];
    const int kv_len = p.kv_len[seq];
    int key_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
    const int first_split = key_lo / SPLIT;
    const int split = first_split + blockIdx.z;
    key_lo = max(key_lo, split * SPLIT);
    const int key_hi = min(kv_len, (split + 1) * SPLIT);
    if (key_lo >= key_hi) return;
    const int k_base = split * SPLIT;

    // ---- bring the split's keys and values in: one 16-byte chunk per cp.async
    const int* table = p.block_table + (size_t)seq * p.table_stride;
    constexpr int CHUNKS = HD / 8;                   // 16-byte chunks per row
    const int n_keys = key_hi - k_base;              // rows [0, n_keys) of the tile are real keys (some may be below key_lo)
    // two halves of SPLIT/2 keys, each its own cp.async group: the first half is computed on while the second lands
    constexpr int HALF = SPLIT / 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        // 256 threads, 64 key rows per half: 4 threads share a row, each taking a quarter of its chunks
        const int j = half * HALF + (tid >> 2);
        const int kpos = k_base + j;
        const __nv_bfloat16* src = nullptr;
        if (j < n_keys && kpos >= key_lo) {
            const int page = table[kpos / p.page_size];
            if (page >= 0 && page < p.num_pages)
                src = p.cache + (size_t)page * p.page_stride + ((size_t)kvh * p.page_size + (kpos % p.page_size)) * HD;
            else if ((tid & 3) == 0)
                atomicOr(p.status, RS_STATUS_BAD_PAGE);
        }
        for (int c = (tid & 3); c < CHUNKS; c += 4) {
            if (src != nullptr) {
                cp_async16(smem_addr(Ks + j * LD + c * 8), src + c * 8);
                cp_async16(smem_addr(Vs + j * LD + c * 8), src + (size_t)p.n_kv * p.page_size * HD + c * 8);
            } else {                                  // masked keys still take part in the MMAs: keep them finite
                *reinterpret_cast<uint4*>(Ks + j * LD + c * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(Vs + j * LD + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    }

    // ---- query fragments (rows = heads of the group, zero beyond the group), loaded while the copies fly
    const int head0 = kvh * p.group;
    const __nv_bfloat16* qrow = p.q + (size_t)p.q_start[seq] * p.q_stride + (size_t)head0 * HD;
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int d0 = 16 * ks + 2 * t;
        qf[ks][0] = g < p.group ? ld_dep(reinterpret_cast<const uint32_t*>(qrow + (size_t)g * HD + d0)) : 0u;
        qf[ks][1] = g + 8 < p.group ? ld_dep(reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * HD + d0)) : 0u;
        qf[ks][2] = g < p.group ? ld_dep(reinterpret_cast<const uint32_t*>(qrow + (size_t)g * HD + d0 + 8)) : 0u;
        qf[ks][3] = g + 8 < p.group ? ld_dep(reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * HD + d0 + 8)) : 0u;
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

    cp_async_wait<0>();
    __syncthreads();                                            // the whole split has landed
    {
        const int j0 = warp * 16;                               // first key row of this warp's 16-key block
        const bool warp_has_keys = k_base + j0 < key_hi;
        if (warp_has_keys) {
        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t b00, b01, b10, b11;
            const int row = j0 + (lane >> 4) * 8 + (lane & 7);
            const int col = 16 * ks + ((lane >> 3) & 1) * 8;
            ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Ks + row * LD + col), b00, b01, b10, b11);
            mma16816(s[0], qf[ks], b00, b01);
            mma16816(s[1], qf[ks], b10, b11);
        }
        // mask and scale (log2 units); key of s[nt][i]: j0 + 8 nt + 2 t + (i & 1)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kpos = k_base + j0 + 8 * nt + 2 * t + (i & 1);
                const bool ok = kpos >= key_lo && kpos < key_hi;
                s[nt][i] = ok ? s[nt][i] * p.scale_log2 : -INFINITY;
                mx[i >> 1] = fmaxf(mx[i >> 1], s[nt][i]);
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
        uint32_t pf[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float e[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mm = m_run[i >> 1];
                e[i] = (mm == -INFINITY) ? 0.f : fast_exp2(s[nt][i] - mm);
                rs[i >> 1] += e[i];
            }
            pf[2 * nt] = pack_bf16(e[0], e[1]);         // a0 / a2: row g
            pf[2 * nt + 1] = pack_bf16(e[2], e[3]);     // a1 / a3: row g + 8
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * corr[r] + rs[r];
        }
#pragma unroll
        for (int d = 0; d < DT; ++d) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
        // O += P V: V^T fragments through ldmatrix.trans, two 8-wide output tiles per instruction
#pragma unroll
        for (int d = 0; d < DT; d += 2) {
            uint32_t v00, v01, v10, v11;
            const int row = j0 + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int col = 8 * (d + (lane >> 4));
            ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(Vs + row * LD + col), v00, v01, v10, v11);
            mma16816(o[d], pf, v00, v01);
            mma16816(o[d + 1], pf, v10, v11);
        }
        }
    }
    cp_async_wait<0>();

    // ---- combine the warps: (max, sum, O) of each warp → shared memory, then one partial per head
    __syncthreads();                                            // everyone is done reading K and V
    float* Os = reinterpret_cast<float*>(smem_raw);            // [WARPS][16][HD + 2]
    constexpr int OLD = HD + 8;                                 // row stride = 8 mod 32 floats: 8-byte stores of a half-warp hit distinct banks
    if (g < p.group) {
        float* r0 = Os + ((size_t)warp * 16 + g) * OLD;
#pragma unroll
        for (int d = 0; d < DT; ++d) *reinterpret_cast<float2*>(r0 + 8 * d + 2 * t) = make_float2(o[d][0], o[d][1]);
        if (t == 0) { r0[HD] = m_run[0]; r0[HD + 1] = l_run[0]; }
    }
    if (g + 8 < p.group) {
        float* r1 = Os + ((size_t)warp * 16 + g + 8) * OLD;
#pragma unroll
        for (int d = 0; d < DT; ++d) *reinterpret_cast<float2*>(r1 + 8 * d + 2 * t) = make_float2(o[d][2], o[d][3]);
        if (t == 0) { r1[HD] = m_run[1]; r1[HD + 1] = l_run[1]; }
    }
    __syncthreads();
    const size_t slot = (size_t)p.split_start[w] + blockIdx.z;
    for (int i = tid; i < p.group * (HD + 2); i += WARPS * 32) {
        const int r = i / (HD + 2), d = i % (HD + 2);
        float M = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < WARPS; ++ww) M = fmaxf(M, Os[((size_t)ww * 16 + r) * OLD + HD]);
        float val;
        if (d == HD) {
            val = M;
        } else {
            val = 0.f;
#pragma unroll
            for (int ww = 0; ww < WARPS; ++ww) {
                const float mw = Os[((size_t)ww * 16 + r) * OLD + HD];
                const float e = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
                val += Os[((size_t)ww * 16 + r) * OLD + (d < HD ? d : HD + 1)] * e;
            }
        }
        p.partial[(slot * p.n_q + head0 + r) * (HD + 2) + d] = val;
    }
}

// out[token of seq, head, :] = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in ascending order
template <int HD>
__global__ void decode_merge_kernel(const DecodeParams p) {
    const int w = blockIdx.x, h = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();
    const int seq = p.work[w];
    const int kv_len = p.kv_len[seq];
    const int key_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
    const int n_splits = (kv_len + SPLIT - 1) / SPLIT - key_lo / SPLIT;
    const float* base = p.partial + ((size_t)p.split_start[w] * p.n_q + h) * (HD + 2);
    const size_t stride = (size_t)p.n_q * (HD + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ld_dep(base + s * stride + HD));
    __nv_bfloat16* dst = p.out + (size_t)p.q_start[seq] * p.out_stride + (size_t)h * HD;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float num = 0.f, den = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float* ps = base + s * stride;
            const float e = fast_exp2(ld_dep(ps + HD) - M);
            num = fmaf(ld_dep(ps + d), e, num);
            den = fmaf(ld_dep(ps + HD + 1), e, den);
        }
        dst[d] = __float2bfloat16_rn(num / den);
    }
}

template <int HD>
int launch(const DecodeParams& p, int n_work, int max_splits, cudaStream_t s) {
    constexpr int LD = HD + 8;
    constexpr size_t kv_bytes = (size_t)2 * SPLIT * LD * 2;
    constexpr size_t o_bytes = (size_t)WARPS * 16 * (HD + 8) * 4;
    constexpr size_t smem = kv_bytes > o_bytes ? kv_bytes : o_bytes;
    auto kern = decode_attention_kernel<HD>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    int rc = rs_launch_pdl(kern, dim3(n_work, p.n_kv, max_splits), dim3(WARPS * 32), smem, s, p);
    if (rc != 0) return rc;
    return rs_launch_pdl(decode_merge_kernel<HD>, dim3(n_work, p.n_q), dim3(HD >= 128 ? 128 : 64), 0, s, p);
}
}  // namespace

// Head sizes this kernel is built for; other sizes (and groups above 16 heads) go to the CUDA-core kernel.
RS_EXPORT int rs_attention_decode_bf16_supported(int n_q, int n_kv, int hd) {
    if (n_kv <= 0 || n_q % n_kv || n_q / n_kv > 16) return 0;
    return hd == 32 || hd == 64 || hd == 96 || hd == 128;
}

RS_EXPORT int rs_attention_decode_bf16_split_keys() { return SPLIT; }

// Same arguments and partial-workspace layout as the decode form of rs_attention_simt; bfloat16 only.
RS_EXPORT int rs_attention_decode_bf16(const void* q, long q_stride, void* out, long out_stride, const void* cache,
                                       long page_stride, int num_pages, int page_size, const int* block_table,
                                       int table_stride, const int* q_start, const int* kv_len, const int* work,
                                       int n_work, int n_q, int n_kv, int hd, int window, float scale, int split_keys,
                                       int max_splits, const int* split_start, float* partial, int* status,
                                       void* stream) {
    if (n_work <= 0) return 0;
    if (!rs_attention_decode_bf16_supported(n_q, n_kv, hd) || split_keys != SPLIT || max_splits <= 0 ||
        partial == nullptr || split_start == nullptr || (q_stride % 2) || ((long)q & 3) || ((long)cache & 15) ||
        (page_stride % 8))
        return (int)cudaErrorInvalidValue;
    DecodeParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.cache = (const __nv_bfloat16*)cache; p.page_stride = page_stride; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work;
    p.n_q = n_q; p.n_kv = n_kv; p.group = n_q / n_kv; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.split_start = split_start; p.partial = partial; p.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    switch (hd) {
        case 32: return launch<32>(p, n_work, max_splits, s);
        case 64: return launch<64>(p, n_work, max_splits, s);
        case 96: return launch<96>(p, n_work, max_splits, s);
        case 128: return launch<128>(p, n_work, max_splits, s);
    }
    return (int)cudaErrorInvalidValue;
}
