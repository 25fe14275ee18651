// Memory-bound kernels of the step: token embedding, RMSNorm (optionally gathering
// rows), per-head QK-norm + rotary encoding + write of K and V into cache pages,
// SiLU(gate)*up.  Each is templated on the activation element type so the 32-bit and
// the bfloat16 engine run the same code; reductions and the rotation are float32.
//
// Reference counterparts (RustingStrata, src/cuda/kernels.cu): rms_norm :1504-1552,
// rms_norm_rope :2196-2228, swiglu :1622-1625; host formulas src/ops.rs:3-7,14,36-45.
#include "common.cuh"

// --------------------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32 (the residual stream is float32 in both engines).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int H, int V, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ld_dep(ids + t);
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(status, RS_STATUS_BAD_TOKEN);
        id = 0;
    }
    const T* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

RS_EXPORT int rs_embed(const void* table, int table_dt, const int* ids, float* out, int T_, int H, int V,
                       int* status, void* stream) {
    if (T_ <= 0) return 0;
    RS_DISPATCH_DTYPE(table_dt, T,
        return rs_launch_pdl(embed_kernel<T>, dim3(T_), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids, out, H, V,
                             status));
    return 0;
}

// --------------------------------------------------------------------------- RMSNorm
// out[r, i] = x[src(r), i] * rsqrt(mean(x[src(r), :]^2) + eps) * w[i], src(r) = rows ? rows[r] : r.
// x is the float32 residual stream; w is float32 or bfloat16; out is the activation type.
// The sum of squares is float32 with a fixed order per row (thread-strided partials,
// then a tree), so a row's result does not depend on what else is in the batch.
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, long x_stride, const int* __restrict__ rows,
                               const void* __restrict__ w, int w_dt, float eps, TO* __restrict__ out, long out_stride,
                               int n) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * x_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { float v = ld_dep(xr + i); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(ss / (float)n + eps);
    TO* o = out + (size_t)r * out_stride;
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f32<TO>(ld_dep(xr + i) * s * load_any(w, w_dt, i));
}

// The same for a bfloat16 output when the row fits the block's registers (n <= 512 * 4 * VPT, n % 4 == 0, 16-byte
// aligned rows): one read of x with float4 loads, the row kept in registers between the sum and the scaling.
template <int VPT>
__global__ void __launch_bounds__(512) rmsnorm_bf16_vec_kernel(const float* x, long x_stride, const int* __restrict__ rows,
                                                               const void* __restrict__ w, int w_dt, float eps,
                                                               __nv_bfloat16* __restrict__ out, long out_stride, int n) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int n4 = n >> 2;
    // the weights are the model's, not the previous kernel's: they are fetched while that kernel is still at work
    float wv[VPT][4];
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = threadIdx.x + u * 512;
        wv[u][0] = wv[u][1] = wv[u][2] = wv[u][3] = 0.f;
        if (i < n4) {
            if (w_dt == RS_F32) {
                const float4 f = reinterpret_cast<const float4*>(w)[i];
                wv[u][0] = f.x; wv[u][1] = f.y; wv[u][2] = f.z; wv[u][3] = f.w;
            } else {
                const uint2 h = reinterpret_cast<const uint2*>(w)[i];
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&h.x), b = *reinterpret_cast<const __nv_bfloat162*>(&h.y);
                wv[u][0] = __low2float(a); wv[u][1] = __high2float(a); wv[u][2] = __low2float(b); wv[u][3] = __high2float(b);
            }
        }
    }
    pdl_wait();
    const int r = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * x_stride);
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = threadIdx.x + u * 512;
        v[u] = i < n4 ? ld_dep(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss); ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(ss / (float)n + eps);
    __nv_bfloat16* o = out + (size_t)r * out_stride;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = threadIdx.x + u * 512;
        if (i < n4) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x * s * wv[u][0], v[u].y * s * wv[u][1]);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(v[u].z * s * wv[u][2], v[u].w * s * wv[u][3]);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo); pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            reinterpret_cast<uint2*>(o)[i] = pk;
        }
    }
}

RS_EXPORT int rs_rmsnorm(const float* x, long x_stride, const int* rows, const void* w, int w_dt, float eps,
                         void* out, int out_dt, long out_stride, int n_rows, int n, void* stream) {
    if (n_rows <= 0) return 0;
    if (out_dt == RS_BF16 && n % 4 == 0 && n <= 512 * 4 * 4 && x_stride % 4 == 0 && out_stride % 4 == 0 && ((long)x & 15) == 0 &&
        ((long)out & 7) == 0 && ((long)w & 15) == 0) {
        auto* o = (__nv_bfloat16*)out;
        cudaStream_t s = (cudaStream_t)stream;
        if (n <= 512 * 4) return rs_launch_pdl(rmsnorm_bf16_vec_kernel<1>, dim3(n_rows), dim3(512), 0, s, x, x_stride, rows, w, w_dt, eps, o, out_stride, n);
        if (n <= 512 * 8) return rs_launch_pdl(rmsnorm_bf16_vec_kernel<2>, dim3(n_rows), dim3(512), 0, s, x, x_stride, rows, w, w_dt, eps, o, out_stride, n);
        return rs_launch_pdl(rmsnorm_bf16_vec_kernel<4>, dim3(n_rows), dim3(512), 0, s, x, x_stride, rows, w, w_dt, eps, o, out_stride, n);
    }
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    RS_DISPATCH_DTYPE(out_dt, TO,
        return rs_launch_pdl(rmsnorm_kernel<TO>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, x, x_stride, rows, w,
                             w_dt, eps, (TO*)out, out_stride, n));
    return 0;
}

// --------------------------------------------------------------------------- QK-norm + RoPE + KV write
// One warp per (token, head).  The fused projection row of a token is
// [q heads | k heads | v heads], each head `hd` wide.  q heads and k heads get an
// RMSNorm over hd with a weight shared by all heads (optional), then the NEOX rotation
// of pairs (i, i + n_rot/2) with cos/sin taken from a table indexed by position
// (optional).  A token carries pos_stride position values ("streams"): stream 0 is its
// place in the cache, and the rotation follows stream rot_stream (0 for plain text).  q is written back in place; k and v go to the token's cache page:
//   cache[page][0 = K, 1 = V][kv head][slot in page][hd],  page = table[seq][pos / page_size].
// With write_kv == 0 the call reads another call's cache and only q is processed.
template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, long row_stride, int n_q, int n_kv, int hd,
                                       const void* __restrict__ q_w, const void* __restrict__ k_w, int w_dt, float eps,
                                       const float* __restrict__ cos_sin, int n_rot, int table_rows,
                                       const int* __restrict__ positions, int pos_stride, int rot_stream,
                                       const int* __restrict__ seq_of_token,
                                       const int* __restrict__ block_table, int table_stride, int page_size,
                                       T* __restrict__ cache, long page_stride, int num_pages, int write_kv,
                                       int n_tokens, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int heads_per_token = n_q + (write_kv ? 2 * n_kv : 0);
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_tokens * heads_per_token) return;
    const int t = warp / heads_per_token;
    const int h = warp % heads_per_token;
    const int pos = positions[(size_t)t * pos_stride];                  // stream 0: where the token lies in the cache
    const int rpos = positions[(size_t)t * pos_stride + rot_stream];    // the stream this layer's rotation follows
    if (cos_sin != nullptr && (rpos < 0 || rpos >= table_rows)) {
        if (lane == 0) atomicOr(status, RS_STATUS_BAD_PLAN);
        return;
    }
    T* src = qkv + (size_t)t * row_stride + (size_t)h * hd;   // q heads, then k heads, then v heads are contiguous

    T* dst = src;                                              // q: in place
    if (h >= n_q) {
        const int kvh = (h - n_q) % n_kv;
        const int is_v = (h - n_q) / n_kv;
        const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(status, RS_STATUS_BAD_PAGE);
            return;
        }
        dst = cache + (size_t)page * page_stride + ((size_t)(is_v * n_kv + kvh) * page_size + (pos % page_size)) * hd;
        if (is_v) {
            for (int i = lane; i < hd; i += 32) dst[i] = src[i];
            return;
        }
    }
    const void* w = h < n_q ? q_w : k_w;
    float scale = 1.f;
    if (w != nullptr) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) { float v = to_f32<T>(src[i]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    const int half = n_rot / 2;
    const float* cs = cos_sin ? cos_sin + (size_t)rpos * n_rot : nullptr;  // [position][cos(half) | sin(half)]
    for (int i = lane; i < half; i += 32) {
        float a = to_f32<T>(src[i]) * scale, b = to_f32<T>(src[i + half]) * scale;
        if (w != nullptr) { a *= load_any(w, w_dt, i); b *= load_any(w, w_dt, i + half); }
        if (cs) {
            const float c = cs[i], s = cs[half + i];
            const float ra = a * c - b * s, rb = a * s + b * c;
            a = ra; b = rb;
        }
        dst[i] = from_f32<T>(a);
        dst[i + half] = from_f32<T>(b);
    }
    for (int i = n_rot + lane; i < hd; i += 32) {               // dims beyond the rotated ones
        float a = to_f32<T>(src[i]) * scale;
        if (w != nullptr) a *= load_any(w, w_dt, i);
        dst[i] = from_f32<T>(a);
    }
}

// bfloat16 fast path: whole head rotated (n_rot == hd), bfloat16 norm weights (or none), aligned rows.
// A lane owns E consecutive elements of the lower half of a head and the E it pairs with in the upper half (E = 8:
// 16-byte accesses, when half a head is a multiple of 8; else E = 4), so a head takes L = hd / (2 E) lanes; when L is
// a power of two a warp serves 32 / L heads side by side.
template <int E>
__global__ void qk_norm_rope_kv_bf16_kernel(__nv_bfloat16* qkv, long row_stride, int n_q, int n_kv, int hd,
                                            const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w,
                                            float eps, const float* __restrict__ cos_sin, int table_rows,
                                            const int* __restrict__ positions, int pos_stride, int rot_stream,
                                            const int* __restrict__ seq_of_token,
                                            const int* __restrict__ block_table, int table_stride, int page_size,
                                            __nv_bfloat16* __restrict__ cache, long page_stride, int num_pages, int write_kv,
                                            int n_tokens, int lanes_shift, int page_shift, int* status) {
    struct alignas(2 * E) Vec { uint32_t w[E / 2]; };           // E bfloat16 values
    const int lanes_per_head = 1 << lanes_shift;
    pdl_launch_dependents();
    // Positions, block tables, norm weights and the rotation table are in place before the step's first kernel, so they
    // are fetched here, while the projection before this kernel is still at work; only qkv has to wait for it.
    const int heads_per_token = n_q + (write_kv ? 2 * n_kv : 0);
    // The kernel is bound by instructions (over 400 per warp for 16 elements a lane), so token and head come without a
    // division: blockIdx.x is the token, blockIdx.y and the thread number give the head; lanes per head and, where it
    // is one, the page size are powers of two.
    const int lane = threadIdx.x & 31;
    const int sub = lane & (lanes_per_head - 1);
    const int t = blockIdx.x;
    const int head = (int)((blockIdx.y * blockDim.x + threadIdx.x) >> lanes_shift);
    const bool live = head < heads_per_token;
    const int h = live ? head : 0;
    const int pos = positions[(size_t)t * pos_stride];                  // stream 0: where the token lies in the cache
    const int rpos = positions[(size_t)t * pos_stride + rot_stream];    // the stream this layer's rotation follows
    __nv_bfloat16* src = qkv + (size_t)t * row_stride + (size_t)h * hd;
    __nv_bfloat16* dst = src;
    bool is_v = false, ok = live, bad_page = false;
    const bool bad_pos = rpos < 0 || rpos >= table_rows;
    if (bad_pos) ok = false;
    if (h >= n_q) {
        const int plane = h - n_q;                                       // (K|V) * n_kv + kv head: the page's planes in that order
        is_v = plane >= n_kv;
        const int block = page_shift >= 0 ? pos >> page_shift : pos / page_size;
        const int in_page = pos - block * page_size;
        const int page = block_table[(size_t)seq_of_token[t] * table_stride + block];
        if (page < 0 || page >= num_pages) {
            bad_page = sub == 0 && live;
            ok = false;
        } else {
            dst = cache + (size_t)page * page_stride + ((size_t)plane * page_size + in_page) * hd;
        }
    }
    const __nv_bfloat16* w = h < n_q ? q_w : k_w;
    const int half = hd >> 1;
    auto unpack = [](const Vec& u, float* f) {
#pragma unroll
        for (int k = 0; k < E / 2; ++k) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.w[k]);
            f[2 * k] = __low2float(a); f[2 * k + 1] = __high2float(a);
        }
    };
    auto pack = [](const float* f) {
        Vec u;
#pragma unroll
        for (int k = 0; k < E / 2; ++k) {
            const __nv_bfloat162 a = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
            u.w[k] = *reinterpret_cast<const uint32_t*>(&a);
        }
        return u;
    };
    const int i = sub * E;
    const bool mine = ok && i < half;
    float wa[E], wb[E], cc[E], sv[E];
#pragma unroll
    for (int u = 0; u < E; ++u) { wa[u] = wb[u] = 1.f; cc[u] = sv[u] = 0.f; }
    if (mine && !is_v) {
        if (w != nullptr) { unpack(*reinterpret_cast<const Vec*>(w + i), wa); unpack(*reinterpret_cast<const Vec*>(w + half + i), wb); }
#pragma unroll
        for (int u = 0; u < E; u += 4) {
            const float4 c = *reinterpret_cast<const float4*>(cos_sin + (size_t)rpos * hd + i + u);
            const float4 sn = *reinterpret_cast<const float4*>(cos_sin + (size_t)rpos * hd + half + i + u);
            cc[u] = c.x; cc[u + 1] = c.y; cc[u + 2] = c.z; cc[u + 3] = c.w;
            sv[u] = sn.x; sv[u + 1] = sn.y; sv[u + 2] = sn.z; sv[u + 3] = sn.w;
        }
    }
    pdl_wait();
    if (bad_page) atomicOr(status, RS_STATUS_BAD_PAGE);         // nothing is written before the wait
    if (bad_pos && live && sub == 0) atomicOr(status, RS_STATUS_BAD_PLAN);
    Vec ua, ub;
#pragma unroll
    for (int k = 0; k < E / 2; ++k) ua.w[k] = ub.w[k] = 0u;
    if (mine) { ua = *reinterpret_cast<const Vec*>(src + i); ub = *reinterpret_cast<const Vec*>(src + half + i); }
    if (is_v) {                                    // values are copied as they are
        if (mine) { *reinterpret_cast<Vec*>(dst + i) = ua; *reinterpret_cast<Vec*>(dst + half + i) = ub; }
#pragma unroll
        for (int k = 0; k < E / 2; ++k) ua.w[k] = ub.w[k] = 0u;
    }
    float a[E], b[E];
    unpack(ua, a); unpack(ub, b);
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < E; ++u) { ss = fmaf(a[u], a[u], ss); ss = fmaf(b[u], b[u], ss); }
    for (int o = lanes_per_head >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // within the head's lanes
    if (!mine || is_v) return;
    const float scale = w != nullptr ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.f;       // as the row norms compute it
    float ra[E], rb[E];
#pragma unroll
    for (int u = 0; u < E; ++u) {
        float x = a[u] * scale, y = b[u] * scale;
        if (w != nullptr) { x *= wa[u]; y *= wb[u]; }
        ra[u] = x * cc[u] - y * sv[u];
        rb[u] = x * sv[u] + y * cc[u];
    }
    *reinterpret_cast<Vec*>(dst + i) = pack(ra);
    *reinterpret_cast<Vec*>(dst + half + i) = pack(rb);
}

RS_EXPORT int rs_qk_norm_rope_kv(void* qkv, int dt, long row_stride, int n_q, int n_kv, int hd, const void* q_w,
                                 const void* k_w, int w_dt, float eps, const float* cos_sin, int n_rot, int table_rows,
                                 const int* positions, int pos_stride, int rot_stream, const int* seq_of_token,
                                 const int* block_table,
                                 int table_stride, int page_size, void* cache, long page_stride, int num_pages,
                                 int write_kv, int n_tokens, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_rot % 2 || n_rot > hd || pos_stride <= 0 || rot_stream < 0 || rot_stream >= pos_stride ||
        (cos_sin != nullptr && table_rows <= 0))
        return (int)cudaErrorInvalidValue;
    if (cos_sin == nullptr) { rot_stream = 0; table_rows = 1 << 30; }
    const long warps = (long)n_tokens * (n_q + (write_kv ? 2 * n_kv : 0));
    const int threads = 256;
    const long blocks = (warps * 32 + threads - 1) / threads;
    const bool weights_ok = (q_w == nullptr && k_w == nullptr) || (w_dt == RS_BF16 && (q_w == nullptr) == (k_w == nullptr || !write_kv) &&
                                                                  ((long)q_w & 7) == 0 && ((long)k_w & 7) == 0);
    if (dt == RS_BF16 && warps < (1L << 26) && cos_sin != nullptr && n_rot == hd && hd % 8 == 0 && hd <= 256 && row_stride % 4 == 0 && page_stride % 4 == 0 &&
        ((long)qkv & 7) == 0 && ((long)cache & 7) == 0 && ((long)cos_sin & 15) == 0 && weights_ok && (q_w != nullptr || k_w == nullptr)) {
        // 16-byte accesses when half a head is a multiple of 8 elements and everything is 16-byte aligned
        const bool wide = hd % 16 == 0 && row_stride % 8 == 0 && page_stride % 8 == 0 && ((long)qkv & 15) == 0 && ((long)cache & 15) == 0 &&
                          ((long)q_w & 15) == 0 && ((long)k_w & 15) == 0;
        int lanes = hd / (wide ? 16 : 8);                     // lanes a head needs; a power of two packs several heads per warp
        if (lanes & (lanes - 1)) lanes = 32;
        int lanes_shift = 0;
        while ((1 << lanes_shift) < lanes) ++lanes_shift;
        int page_shift = -1;
        if ((page_size & (page_size - 1)) == 0) { page_shift = 0; while ((1 << page_shift) < page_size) ++page_shift; }
        const int token_threads = (n_q + (write_kv ? 2 * n_kv : 0)) << lanes_shift;       // threads a token's heads need
        const int rope_threads = 128;
        const dim3 rope_grid((unsigned)n_tokens, (unsigned)((token_threads + rope_threads - 1) / rope_threads));
        auto kern = wide ? qk_norm_rope_kv_bf16_kernel<8> : qk_norm_rope_kv_bf16_kernel<4>;
        return rs_launch_pdl(kern, rope_grid, dim3(rope_threads), 0, (cudaStream_t)stream,
                             (__nv_bfloat16*)qkv, row_stride, n_q, n_kv, hd, (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, eps,
                             cos_sin, table_rows, positions, pos_stride, rot_stream, seq_of_token, block_table, table_stride,
                             page_size, (__nv_bfloat16*)cache, page_stride, num_pages, write_kv, n_tokens, lanes_shift, page_shift, status);
    }
    RS_DISPATCH_DTYPE(dt, T,
        return rs_launch_pdl(qk_norm_rope_kv_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream,
                             (T*)qkv, row_stride, n_q, n_kv, hd, q_w, k_w, w_dt, eps, cos_sin, n_rot, table_rows, positions,
                             pos_stride, rot_stream, seq_of_token, block_table, table_stride, page_size, (T*)cache,
                             page_stride, num_pages, write_kv, n_tokens, status));
    return 0;
}

// --------------------------------------------------------------------------- SiLU(gate) * up
// in: [rows, 2*I] with gate in columns [0, I) and up in [I, 2I); out: [rows, I].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, long in_stride, T* __restrict__ out, long out_stride,
                                int rows, int I) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)rows * I) return;
    const int r = (int)(idx / I), c = (int)(idx % I);
    const float g = to_f32<T>(in[(size_t)r * in_stride + c]);
    const float u = to_f32<T>(in[(size_t)r * in_stride + I + c]);
    out[(size_t)r * out_stride + c] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

RS_EXPORT int rs_silu_mul(const void* in, long in_stride, void* out, long out_stride, int dt, int rows, int I,
                          void* stream) {
    if (rows <= 0) return 0;
    const long n = (long)rows * I;
    RS_DISPATCH_DTYPE(dt, T,
        silu_mul_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const T*)in, in_stride,
                                                                                       (T*)out, out_stride, rows, I));
    return rs_launch_result();
}

// --------------------------------------------------------------------------- residual add of a delta
// x[r, :] += delta[r, :] in float32 (for parts that cannot add inside their last kernel).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ d, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_f32<T>(d[i]);
}

RS_EXPORT int rs_residual_add(float* x, const void* delta, int dt, long n, void* stream) {
    if (n <= 0) return 0;
    RS_DISPATCH_DTYPE(dt, T,
        residual_add_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, (const T*)delta, n));
    return rs_launch_result();
}

// dst[i] = src[idx[i]]: the ids a step chose, brought into the order of the next step's rows on the device
__global__ void gather_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ idx, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = ld_dep(src + __ldg(idx + i));
}

RS_EXPORT int rs_gather_i32(int* dst, const int* src, const int* idx, int n, void* stream) {
    if (n <= 0) return 0;
    return rs_launch_pdl(gather_i32_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, dst, src, idx, n);
}

// ---- random weights ------------------------------------------------------------------------------------
// Element i of a tensor's stream: z = mix64(key + (first + i + 1) * GOLDEN); floating tensors take
// shift + scale * table[z >> 48] (table: 65,536 normal quantiles as float32, made on the host), integer
// tables the low bit of z.  Integer arithmetic, one look-up, one float32 multiply and one float32 add, none of
// them contracted: the host's numpy generator (weights/random_init.py) produces the same bits.
namespace {
__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_random_kernel(T* out, long n, unsigned long long key, long first, const float* table, float scale,
                                   float shift) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const unsigned long long z = mix64(key + (unsigned long long)(first + i + 1) * 0x9E3779B97F4A7C15ull);
        out[i] = from_f32<T>(__fadd_rn(__fmul_rn(scale, __ldg(table + (z >> 48))), shift));
    }
}

__global__ void fill_random_bits_kernel(int* out, long n, unsigned long long key, long first) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        out[i] = (int)(mix64(key + (unsigned long long)(first + i + 1) * 0x9E3779B97F4A7C15ull) & 1ull);
}
}  // namespace

// dt: RS_F32, RS_BF16, or 2 for an int32 table of random bits (table, scale and shift unused).
RS_EXPORT int rs_fill_random(void* out, int dt, long n, unsigned long long key, long first, const float* table,
                             float scale, float shift, void* stream) {
    if (n <= 0) return 0;
    if (dt != 2 && table == nullptr) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == 2) { fill_random_bits_kernel<<<blocks, threads, 0, s>>>((int*)out, n, key, first); return rs_launch_result(); }
    RS_DISPATCH_DTYPE(dt, T, fill_random_kernel<T><<<blocks, threads, 0, s>>>((T*)out, n, key, first, table, scale, shift));
    return rs_launch_result();
}

// Turns programmatic dependent launch on or off for every kernel of this library (default on).
RS_EXPORT void rs_core_set_pdl(int on) { rs_pdl_switch() = on ? 1 : 0; }
