// Paged causal attention on CUDA cores, for any head size that is a multiple of 16 up
// to 256, any number of heads and groups, float32 or bfloat16 cache: the attention of
// the 32-bit engine and the general fallback of the bfloat16 engine.
//
// Two launch forms share one kernel body:
//  * portions ("prefill"): a host-built list of (sequence, first query of the tile);
//    a CTA takes a tile of queries of one group of heads that share a KV head and
//    walks the keys 0..position (or the window) through the block table;
//  * decode: one query token per sequence, the keys cut into fixed splits of
//    SPLIT_KEYS at absolute positions, each split a CTA that writes an un-normalised
//    partial (acc, max, sum); a merge kernel combines the splits in ascending order.
// Key tiles start at multiples of 32 from key 0, so the order in which a query's
// scores are reduced depends only on its position, not on how the prompt was cut or
// what else is in the batch.  Scores, softmax and the weighted sum are float32.
//
// Reference counterparts (src/cuda/kernels.cu): attn_prefill_* :2813-3156,
// attn_decode_gqa_* :2571-2580, attn_merge :2594-2625; formulas src/model.rs:778-791.
#include "common.cuh"
#include <math.h>
#include <atomic>

namespace {
constexpr int RS_MAX_DEVICES = 64;   // devices per process the per-device tables below have room for
constexpr int KT = 32;        // keys per tile = lanes of a warp
constexpr int WARPS = 4;
constexpr int RPW = 4;        // query rows per warp
constexpr int ROWS = WARPS * RPW;

struct AttnParams {
    const void* q; long q_stride;          // [tokens, q_stride], head h at h*hd
    void* out; long out_stride;            // [tokens, out_stride]
    const void* cache; long page_stride;   // [pages][2][n_kv][page_size][hd]
    int num_pages, page_size;
    const int* block_table; int table_stride;
    const int* q_start;                    // [n_seqs + 1] first token row of each sequence in this step
    const int* kv_len;                     // [n_seqs] keys of each sequence after this step
    const int* work;                       // portions: [n_work][2] (seq, query offset); decode: [n_work] seq
    int n_q, n_kv, hd, group, heads_per_cta, chunks_per_group, q_per_cta;
    int window;                            // 0 = all keys
    float scale;
    const float* slopes;                   // [n_q] or null: slopes[h] * (key position - query position) is added to a score
    int decode, split_keys, max_splits;
    const int* split_start;                // decode: [n_work] first partial slot of each sequence
    float* partial;                        // decode: [slot][n_q][hd + 2], slot = split_start[w] + split
    int partial_slots;                     // decode: slots `partial` holds; a slot beyond it is flagged, not written
    int* status;
};

template <typename T, int HDL, bool PRECISE>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kernel(const AttnParams p) {
    extern __shared__ float smem[];
    const int hd = p.hd, ldk = hd + 1;
    float* Ks = smem;                       // [KT][ldk]
    float* Vs = Ks + KT * ldk;              // [KT][ldk]
    float* Qs = Vs + KT * ldk;              // [ROWS][hd]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* q = (const T*)p.q;
    const T* cache = (const T*)p.cache;

    const int kvh = blockIdx.y / p.chunks_per_group;
    const int head0 = kvh * p.group + (blockIdx.y % p.chunks_per_group) * p.heads_per_cta;
    const int n_heads = min(p.heads_per_cta, (kvh + 1) * p.group - head0);

    int seq, q_off, n_q_tok;
    if (p.decode) { seq = p.work[blockIdx.x]; q_off = 0; n_q_tok = 1; }
    else { seq = p.work[2 * blockIdx.x]; q_off = p.work[2 * blockIdx.x + 1]; }
    const int row0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - row0;
    const int kv_len = p.kv_len[seq];
    if (!p.decode) n_q_tok = min(p.q_per_cta, q_len - q_off);
    const int n_rows = n_q_tok * n_heads;
    const int qpos0 = kv_len - q_len + q_off;                 // position of the tile's first query

    int key_lo = p.window > 0 ? max(0, qpos0 - p.window + 1) : 0;
    int key_hi = min(kv_len, qpos0 + n_q_tok);
    int split_local = 0;
    if (p.decode) {
        const int first_split = key_lo / p.split_keys;
        split_local = blockIdx.z;
        const int s = first_split + split_local;
        key_lo = max(key_lo, s * p.split_keys);
        key_hi = min(key_hi, (s + 1) * p.split_keys);
        if (key_lo >= key_hi) return;
    }

    // queries of this CTA as float32: row r = token (r / n_heads), head (r % n_heads)
    for (int i = tid; i < n_rows * hd; i += WARPS * 32) {
        const int r = i / hd, d = i % hd;
        const int tok = row0 + q_off + r / n_heads, h = head0 + r % n_heads;
        Qs[r * hd + d] = to_f32<T>(q[(size_t)tok * p.q_stride + (size_t)h * hd + d]);
    }

    float m[RPW], l[RPW], acc[RPW][HDL];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < HDL; ++i) acc[r][i] = 0.f;
    }

    const int* table = p.block_table + (size_t)seq * p.table_stride;
    for (int k0 = (key_lo / KT) * KT; k0 < key_hi; k0 += KT) {
        __syncthreads();
        for (int i = tid; i < KT * hd; i += WARPS * 32) {
            const int j = i / hd, d = i % hd;
            const int kpos = k0 + j;
            float kv = 0.f, vv = 0.f;
            if (kpos >= key_lo && kpos < key_hi) {
                const int page = table[kpos / p.page_size];
                if (page >= 0 && page < p.num_pages) {
                    const T* base = cache + (size_t)page * p.page_stride +
                                    ((size_t)kvh * p.page_size + (kpos % p.page_size)) * hd + d;
                    kv = to_f32<T>(base[0]);
                    vv = to_f32<T>(base[(size_t)p.n_kv * p.page_size * hd]);
                } else if (d == 0) {
                    atomicOr(p.status, RS_STATUS_BAD_PAGE);
                }
            }
            Ks[j * ldk + d] = kv;
            Vs[j * ldk + d] = vv;
        }
        __syncthreads();
        const int kpos = k0 + lane;
#pragma unroll
        for (int rr = 0; rr < RPW; ++rr) {
            const int r = warp + rr * WARPS;
            if (r >= n_rows) continue;                       // uniform per warp
            const int qpos = qpos0 + r / n_heads;
            const float* qr = Qs + r * hd;
            const float* kr = Ks + lane * ldk;
            float s = 0.f;
            for (int d = 0; d < hd; ++d) s = fmaf(qr[d], kr[d], s);
            s *= p.scale;
            if (p.slopes != nullptr) s = fmaf(p.slopes[head0 + r % n_heads], (float)(kpos - qpos), s);   // a bias linear in the distance
            const bool ok = kpos >= key_lo && kpos < key_hi && kpos <= qpos &&
                            (p.window <= 0 || kpos > qpos - p.window);
            s = ok ? s : -INFINITY;
            const float m_new = fmaxf(m[rr], warp_max(s));
            if (m_new == -INFINITY) continue;                 // nothing visible yet for this row
            const float corr = PRECISE ? expf(m[rr] - m_new) : __expf(m[rr] - m_new);
            const float pr = ok ? (PRECISE ? expf(s - m_new) : __expf(s - m_new)) : 0.f;
            l[rr] = l[rr] * corr + warp_sum(pr);
            m[rr] = m_new;
#pragma unroll
            for (int i = 0; i < HDL; ++i) acc[rr][i] *= corr;
            for (int j = 0; j < KT; ++j) {
                const float pj = __shfl_sync(0xffffffffu, pr, j);
#pragma unroll
                for (int i = 0; i < HDL; ++i) {
                    const int d = lane + 32 * i;
                    if (d < hd) acc[rr][i] = fmaf(pj, Vs[j * ldk + d], acc[rr][i]);
                }
            }
        }
    }

#pragma unroll
    for (int rr = 0; rr < RPW; ++rr) {
        const int r = warp + rr * WARPS;
        if (r >= n_rows) continue;
        const int tok = row0 + q_off + r / n_heads, h = head0 + r % n_heads;
        if (p.decode) {
            const size_t slot = (size_t)p.split_start[blockIdx.x] + split_local;
            if (slot >= (size_t)p.partial_slots) {
                if (lane == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
                continue;
            }
            float* dst = p.partial + (slot * p.n_q + h) * (hd + 2);
#pragma unroll
            for (int i = 0; i < HDL; ++i) { const int d = lane + 32 * i; if (d < hd) dst[d] = acc[rr][i]; }
            if (lane == 0) { dst[hd] = m[rr]; dst[hd + 1] = l[rr]; }
        } else {
            T* dst = (T*)p.out + (size_t)tok * p.out_stride + (size_t)h * hd;
            const float inv = 1.0f / l[rr];
#pragma unroll
            for (int i = 0; i < HDL; ++i) { const int d = lane + 32 * i; if (d < hd) dst[d] = from_f32<T>(acc[rr][i] * inv); }
        }
    }
}

// out[token of seq, head, :] = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M), splits in ascending order
template <typename T, bool PRECISE>
__global__ void attention_merge_kernel(const AttnParams p) {
    const int w = blockIdx.x, h = blockIdx.y;
    const int seq = p.work[w];
    const int kv_len = p.kv_len[seq];
    const int key_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
    const int n_splits = (kv_len + p.split_keys - 1) / p.split_keys - key_lo / p.split_keys;
    const int hd = p.hd;
    if ((size_t)p.split_start[w] + n_splits > (size_t)p.partial_slots) {       // flagged by the split kernel too
        if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
        return;
    }
    const float* base = p.partial + ((size_t)p.split_start[w] * p.n_q + h) * (hd + 2);
    const size_t split_stride = (size_t)p.n_q * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[s * split_stride + hd]);
    T* dst = (T*)p.out + (size_t)p.q_start[seq] * p.out_stride + (size_t)h * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float num = 0.f, den = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float* ps = base + s * split_stride;
            const float e = PRECISE ? expf(ps[hd] - M) : __expf(ps[hd] - M);
            num = fmaf(ps[d], e, num);
            den = fmaf(ps[hd + 1], e, den);
        }
        dst[d] = from_f32<T>(num / den);
    }
}

template <typename T, int HDL, bool PRECISE>
int launch_attention(const AttnParams& p, int n_work, cudaStream_t s) {
    const size_t smem = ((size_t)2 * KT * (p.hd + 1) + (size_t)ROWS * p.hd) * sizeof(float);
    auto kern = paged_attention_kernel<T, HDL, PRECISE>;
    // The opt-in to more than 48 KB of shared memory is a property of (kernel, device): raised once per size on each
    // device, and not while a stream is capturing (the engine runs every shape once eagerly before it captures).
    static std::atomic<size_t> smem_allowed[RS_MAX_DEVICES];
    cudaError_t e;
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= RS_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (smem > smem_allowed[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        size_t seen = smem_allowed[dev].load(std::memory_order_relaxed);
        while (seen < smem && !smem_allowed[dev].compare_exchange_weak(seen, smem, std::memory_order_release)) {}
    }
    dim3 grid(n_work, p.n_kv * p.chunks_per_group, p.decode ? p.max_splits : 1);
    kern<<<grid, WARPS * 32, smem, s>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess || !p.decode) return (int)e;
    attention_merge_kernel<T, PRECISE><<<dim3(n_work, p.n_q), 128, 0, s>>>(p);
    return rs_launch_result();
}

template <typename T, bool PRECISE>
int dispatch_hd(const AttnParams& p, int n_work, cudaStream_t s) {
    if (p.hd <= 32) return launch_attention<T, 1, PRECISE>(p, n_work, s);
    if (p.hd <= 64) return launch_attention<T, 2, PRECISE>(p, n_work, s);
    if (p.hd <= 128) return launch_attention<T, 4, PRECISE>(p, n_work, s);
    return launch_attention<T, 8, PRECISE>(p, n_work, s);
}
}  // namespace

// Queries per CTA of the portion form: the host cuts each sequence's queries into tiles of this many.
RS_EXPORT int rs_attention_simt_q_per_cta(int n_q, int n_kv) {
    const int group = n_q / n_kv;
    const int hpc = group < ROWS ? group : ROWS;
    return ROWS / hpc;
}

// Floats of partial workspace the decode form needs for `total_splits` (sequence, split) pairs.
RS_EXPORT long rs_attention_simt_partial_floats(int total_splits, int n_q, int hd) {
    return (long)total_splits * n_q * (hd + 2);
}

RS_EXPORT int rs_attention_simt(const void* q, long q_stride, void* out, long out_stride, int dt, const void* cache,
                                long page_stride, int num_pages, int page_size, const int* block_table,
                                int table_stride, const int* q_start, const int* kv_len, const int* work, int n_work,
                                int n_q, int n_kv, int hd, int window, float scale, int decode, int split_keys,
                                int max_splits, const int* split_start, float* partial, int partial_slots,
                                const float* slopes, int* status, void* stream) {
    if (n_work <= 0) return 0;
    if (hd % 16 || hd > 256 || hd <= 0 || n_q % n_kv) return (int)cudaErrorInvalidValue;
    if (decode && (split_keys % KT || split_keys <= 0 || max_splits <= 0 || partial == nullptr || partial_slots <= 0 ||
                   split_start == nullptr))
        return (int)cudaErrorInvalidValue;
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
    p.cache = cache; p.page_stride = page_stride; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work;
    p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.group = n_q / n_kv;
    p.heads_per_cta = p.group < ROWS ? p.group : ROWS;
    p.chunks_per_group = (p.group + p.heads_per_cta - 1) / p.heads_per_cta;
    p.q_per_cta = decode ? 1 : ROWS / p.heads_per_cta;
    p.window = window; p.scale = scale; p.decode = decode; p.split_keys = split_keys; p.max_splits = max_splits;
    p.split_start = split_start; p.partial = partial; p.partial_slots = partial_slots; p.status = status;
    p.slopes = slopes;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == RS_F32) return dispatch_hd<float, true>(p, n_work, s);
    if (dt == RS_BF16) return dispatch_hd<__nv_bfloat16, false>(p, n_work, s);
    return (int)cudaErrorInvalidValue;
}

// =============================================================================================
// Decode attention without a caller-supplied workspace (see attention_decode_noalloc.h).
// The array below is the workspace.  In host code its name is only a handle for the runtime,
// not a device address: the address each device maps it to is asked for once per device with
// cudaGetSymbolAddress and passed to the kernels like any other pointer.
// =============================================================================================
#include "attention_decode_noalloc.h"
#include <mutex>
#include <stdio.h>

static __device__ __align__(256) float rs_noalloc_partial[RS_NOALLOC_MAX_FLOATS];

namespace {
constexpr int RS_NOALLOC_MAX_DEVICES = RS_MAX_DEVICES;
float* g_noalloc_address[RS_NOALLOC_MAX_DEVICES] = {nullptr};
std::mutex g_noalloc_mutex;
thread_local char g_noalloc_error[256] = "";

int noalloc_fail(int code, const char* fmt, long a = 0, long b = 0) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), fmt, a, b);
    return code;
}

// Device address of the array on the current device; looked up at the first call per device.
int noalloc_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return noalloc_fail((int)e, "cudaGetDevice failed with CUDA error %ld", (long)e);
    if (dev < 0 || dev >= RS_NOALLOC_MAX_DEVICES)
        return noalloc_fail(RS_NOALLOC_BAD_ARGUMENT, "device index %ld is beyond the %ld devices this entry point tracks",
                            dev, RS_NOALLOC_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_address[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, rs_noalloc_partial);
        if (e != cudaSuccess || p == nullptr)
            return noalloc_fail(e != cudaSuccess ? (int)e : RS_NOALLOC_BAD_ARGUMENT,
                                "cudaGetSymbolAddress for the built-in workspace failed with CUDA error %ld", (long)e);
        g_noalloc_address[dev] = p;
    }
    *out = g_noalloc_address[dev];
    return 0;
}
}  // namespace

RS_EXPORT long rs_attention_decode_noalloc_capacity(void) { return RS_NOALLOC_MAX_FLOATS; }

RS_EXPORT const char* rs_attention_decode_noalloc_error(void) { return g_noalloc_error; }

RS_EXPORT int rs_attention_decode_noalloc(const void* q, long q_stride, void* out, long out_stride, int dt,
                                          const void* cache, long page_stride, int num_pages, int page_size,
                                          const int* block_table, int table_stride, const int* q_start,
                                          const int* kv_len, const int* work, int n_work, int n_q, int n_kv, int hd,
                                          int window, float scale, int split_keys, int max_splits,
                                          const int* split_start, int total_splits, int* status, void* stream) {
    g_noalloc_error[0] = 0;
    if (n_work <= 0) return 0;
    if (hd <= 0 || hd % 16 || hd > 256 || n_kv <= 0 || n_q <= 0 || n_q % n_kv)
        return noalloc_fail(RS_NOALLOC_BAD_ARGUMENT, "head size %ld must be a multiple of 16 up to 256 and the %ld query "
                            "heads a multiple of the key/value heads", hd, n_q);
    if (split_keys <= 0 || split_keys % KT || max_splits <= 0 || total_splits <= 0 || split_start == nullptr)
        return noalloc_fail(RS_NOALLOC_BAD_ARGUMENT, "split_keys %ld must be a positive multiple of 32 and the split "
                            "counts positive (total_splits %ld)", split_keys, total_splits);
    const long need = (long)total_splits * n_q * (hd + 2);
    if (need > (long)RS_NOALLOC_MAX_FLOATS)
        return noalloc_fail(RS_NOALLOC_TOO_LARGE, "this call needs %ld float32 values of partial results, the built-in "
                            "workspace holds %ld; use rs_attention_simt with your own buffer", need,
                            (long)RS_NOALLOC_MAX_FLOATS);
    float* partial = nullptr;
    const int rc = noalloc_address(&partial);
    if (rc != 0) return rc;
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
    p.cache = cache; p.page_stride = page_stride; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work;
    p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.group = n_q / n_kv;
    p.heads_per_cta = p.group < ROWS ? p.group : ROWS;
    p.chunks_per_group = (p.group + p.heads_per_cta - 1) / p.heads_per_cta;
    p.q_per_cta = 1;
    p.window = window; p.scale = scale; p.decode = 1; p.split_keys = split_keys; p.max_splits = max_splits;
    p.split_start = split_start; p.partial = partial; p.status = status; p.slopes = nullptr;
    // what the array really holds for this shape, not what the caller said it would use: a split list that
    // disagrees with total_splits is flagged by the kernels (RS_STATUS_BAD_PLAN) instead of written past the array
    p.partial_slots = (int)((long)RS_NOALLOC_MAX_FLOATS / ((long)n_q * (hd + 2)));
    cudaStream_t s = (cudaStream_t)stream;
    int e;
    if (dt == RS_F32) e = dispatch_hd<float, true>(p, n_work, s);
    else if (dt == RS_BF16) e = dispatch_hd<__nv_bfloat16, false>(p, n_work, s);
    else return noalloc_fail(RS_NOALLOC_BAD_ARGUMENT, "element type code %ld is neither float32 (0) nor bfloat16 (1)", dt);
    if (e != 0) return noalloc_fail(e, "a kernel launch failed with CUDA error %ld", (long)e);
    return 0;
}
