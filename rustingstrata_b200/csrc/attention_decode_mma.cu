// Decode attention of the bfloat16 engine: one query token per sequence over its paged keys and values.
//
// Work items are (sequence, kv head, split of SPLIT keys at absolute positions); an item serves all query
// heads of its group at once, so K and V are read from HBM exactly once per group.  Persistent CTAs (one per
// SM) walk the items round-robin; inside a CTA the live items go to G consumer groups in turn, and every
// group owns `depth` stages of shared memory (K tile, V tile, the group's query rows):
//   warp 4G (producer)   - lane i looks page i of the item up in the block table and issues ONE 5-d TMA load for
//                          it: (64 dims, tokens of the page, 64-wide halves of the head, K|V, block), 128-byte
//                          swizzle.  The TMA unit spends a fixed time on every load, so few large loads stream
//                          faster than many small ones.  (If the driver refuses the 5-d map, one 2-d load per
//                          K/V and half goes to the same places.)  All lanes copy the query rows.  Table entry
//                          and query of the next item are fetched before the wait for a free stage, so their
//                          latency hides behind the loads in flight.
//   warp 4G + 1          - prefetcher: asks the pages of the next few items into L2 (TMA prefetch), because the
//                          shared-memory ring alone holds too few bytes in flight to cover the latency of loaded DRAM.
//   warps 4g .. 4g+3     - consumer group g.  Each warp takes 32 keys of the item in one pass: scores
//                          S = Q K^T (mma.sync m16n8k16, the group's query heads are the 16-row operand, padded
//                          with zero rows), float32 softmax with exp2 on pre-scaled scores, then O = P V.  Its
//                          (O, max, sum) go over its own rows of the K and V tiles, which nobody reads any more;
//                          the four warps' results meet there and leave as one un-normalised partial per
//                          (sequence, split, head).  Then the stage goes back to the producer.
// With few warps per SM every dependent instruction's latency shows, so the consumers do as little as they
// can (one pass, no running maximum) and three groups overlap one another's chains.
// The merge kernel adds the splits of a head in an order that the sequence's length alone fixes (see there).  Keys of
// a split are visited in the same order whatever the batch holds, so a row's result does not depend on its neighbours.  Pages an item does
// not own (beyond the sequence, given back by a window) are replaced by page 0: their keys are masked and
// their values only have to be finite.  Waits on mbarriers are bounded (tma_helpers.cuh).
//
// Reference counterparts: attn_decode_gqa_* + attn_merge (src/cuda/kernels.cu:2571-2625): K/V of a group
// read once with cp.async double buffering, CUDA-core dot products, 32 splits.
#include "tma_helpers.cuh"
#include "mma_helpers.cuh"
#include <math.h>

namespace {
constexpr int GROUP_WARPS = 4;
constexpr int MAX_GROUPS = 3;
constexpr int MAX_THREADS = (MAX_GROUPS * GROUP_WARPS + 2) * 32;
constexpr int PREFETCH_AHEAD = 4;      // items whose pages are asked into L2 before their stage is free
constexpr int SPLIT = 128;             // keys per item; must equal the split size the host plans with
constexpr int KEYS_PER_WARP = SPLIT / GROUP_WARPS;
constexpr int Q_ROWS = 16;             // rows of the query operand
static_assert(KEYS_PER_WARP == 32, "a warp's pass covers two 16-key blocks");

struct DecodeParams {
    const __nv_bfloat16* q; long q_stride;
    __nv_bfloat16* out; long out_stride;
    int num_pages, page_size;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len; const int* work;
    int n_q, n_kv, group;
    int window;
    float scale_log2;                  // scale * log2(e)
    const int* split_start;
    const int* items;                  // [split_start[n_work] * n_kv] live items, packed by pack_item
    float* partial;                    // [slot][n_q][hd + 2]: acc, max (log2 units), sum
    int partial_slots;                 // slots `partial` holds; a slot beyond it is flagged and not written
    int* status;
    int n_work, max_splits, total;     // total: items = (partial slot, kv head) pairs; the kernel reads it from split_start[n_work]
    int groups, depth;                 // consumer groups and stages per group
    int one_load_per_page;             // the 5-d map is in use
};

struct Item { int w, kvh, split_local, seq, key_lo, key_hi, k_base, kv_len; };

// The metadata arrays are uploaded before the step's first kernel, and the list of items is written by a kernel that
// has ended before this one starts, so the read-only path is safe for them.
// The items are the live (sequence, kv head, split) triples only, whatever the launch shape was rounded up to, so the
// CTAs, which take ids round robin, get the same number of items to within one.  Sequence w owns the ids from
// split_start[w] * n_kv (split_start[w] is its first partial slot); inside a sequence the split runs fastest, then the
// kv head: CTAs that work side by side then read pages that lie far apart, which streams faster than neighbours
// reading the adjacent 4 KiB pieces of one page (126.8 against 112.4 us at 64 x 2,048 keys).  Finding an id's triple
// takes a bisection and a division; every role of every CTA needs it for every item, in all layers of a step, and that
// arithmetic showed in the kernel's time (+18 % at batch 64).  So a small kernel writes the list of triples once per
// step (decode_items_kernel), and the attention kernels of all layers look an id up with one load.
__host__ __device__ __forceinline__ int pack_item(int w, int kvh, int split_local) { return (w << 20) | (kvh << 12) | split_local; }
constexpr int ITEM_MAX_SEQS = 1 << 11, ITEM_MAX_KV = 1 << 8, ITEM_MAX_SPLITS = 1 << 12;

__device__ __forceinline__ Item decode_item(const DecodeParams& p, int id) {
    Item it;
    const int packed = __ldg(p.items + id);
    it.w = packed >> 20;
    it.kvh = (packed >> 12) & (ITEM_MAX_KV - 1);
    it.split_local = packed & (ITEM_MAX_SPLITS - 1);
    it.seq = __ldg(p.work + it.w);
    const int kv_len = __ldg(p.kv_len + it.seq);
    it.kv_len = kv_len;
    const int lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
    const int split = lo / SPLIT + it.split_local;
    it.key_lo = max(lo, split * SPLIT);
    it.key_hi = min(kv_len, (split + 1) * SPLIT);
    it.k_base = split * SPLIT;
    return it;
}

// The item with this id, if there is one; every role steps through the ids the same way and skips none.  (An item
// without visible keys cannot come from a well-formed list; it would load page 0 and leave an empty partial.)
__device__ __forceinline__ int item_at(const DecodeParams& p, int id, Item& it) {
    if (id >= p.total) return p.total;
    it = decode_item(p, id);
    return id;
}

template <int HD>
__global__ void __launch_bounds__(MAX_THREADS, 1) decode_attention_kernel(const __grid_constant__ CUtensorMap map_kv, const DecodeParams p_launch) {
    // the step's metadata is in place before its first kernel: the number of live items is read, not launched with
    DecodeParams p = p_launch;
    p.total = __ldg(p.split_start + p.n_work) * p.n_kv;
    // A stage holds the item's pages one after the other; a page's block is [K | V][half of the head][token][64 dims],
    // every (K|V, half) piece a multiple of 1 KiB, so a token's swizzle phase is its index mod 8.
    constexpr int HALVES = HD / 64;                  // 64-wide (128-byte) column blocks of a head
    constexpr int STAGE_BYTES = 2 * HALVES * SPLIT * 128;
    constexpr int WARP_BYTES = 2 * HALVES * KEYS_PER_WARP * 128;
    constexpr int Q_BYTES = Q_ROWS * HD * 2;
    constexpr int KS = HD / 16, DT = HD / 8, VEC = HD / 8;
    constexpr int OLD = HD + 8;                      // float row stride = 8 mod 32: 8-byte stores of a half-warp hit distinct banks
    constexpr int CHUNK_BYTES = KEYS_PER_WARP * 128; // a warp's tokens of one (K|V, half) piece
    constexpr int ROWS_PER_CHUNK = CHUNK_BYTES / (OLD * 4);
    static_assert(ROWS_PER_CHUNK * 2 * HALVES >= Q_ROWS && Q_ROWS * OLD * 4 <= WARP_BYTES, "a warp's K and V rows hold its results");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw);
    const int stages = p.groups * p.depth;
    const uint32_t q0 = base + stages * STAGE_BYTES;
    const uint32_t bar0 = q0 + stages * Q_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + (size_t)stages * (STAGE_BYTES + Q_BYTES + 16));
    volatile int* produced = abort_flag + 1;         // live items whose loads have been issued

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int piece = p.page_size * 128;             // bytes of one (K|V, half) piece of a page
    const int page_block = 2 * HALVES * piece;
    const int page_shift = __ffs(p.page_size) - 1;
    const int producer_warp = p.groups * GROUP_WARPS;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), GROUP_WARPS); }
        *abort_flag = 0;
        *produced = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // query rows past the group stay zero for the whole kernel
    for (int i = threadIdx.x; i < stages * Q_BYTES / 16; i += blockDim.x)
        *reinterpret_cast<uint4*>(aligned + (size_t)stages * STAGE_BYTES + (size_t)i * 16) = make_uint4(0, 0, 0, 0);
    __syncthreads();
    pdl_launch_dependents();
    // The query and the new token's key and value come from the previous kernel: every role waits for it before it
    // touches them; the producer first starts the loads that cannot hold the new token.

    if (warp == producer_warp) {
        // ------------------------------------------------------------ producer
        const int pages_per_item = SPLIT / p.page_size;
        const int nvec = p.group * VEC;              // 16-byte pieces of an item's query rows
        constexpr int QV = Q_ROWS * VEC / 32;
        auto fetch = [&](const Item& it, int& page, uint4 (&qv)[QV]) {
            const int kpos = it.k_base + lane * p.page_size;
            page = 0;
            if (lane < pages_per_item && kpos < it.key_hi && kpos + p.page_size > it.key_lo)
                page = __ldg(p.block_table + (size_t)it.seq * p.table_stride + kpos / p.page_size);
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)__ldg(p.q_start + it.seq) * p.q_stride +
                                                              (size_t)it.kvh * p.group * HD);
#pragma unroll
            for (int i = 0; i < QV; ++i)
                if (lane + 32 * i < nvec) qv[i] = ld_dep(src + lane + 32 * i);
        };
        auto load_pages = [&](const Item& it, int page, int s) {
            if (lane < pages_per_item) {
                const uint32_t dst = base + s * STAGE_BYTES + lane * page_block;
                if (p.one_load_per_page) {
                    tma_load_5d(dst, &map_kv, 0, 0, 0, 0, page * 2 * p.n_kv + it.kvh, full_bar(s));
                } else {
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {
                        const int row = ((page * 2 + kv) * p.n_kv + it.kvh) * p.page_size;
#pragma unroll
                        for (int h = 0; h < HALVES; ++h)
                            tma_load_2d(dst + (kv * HALVES + h) * piece, &map_kv, h * 64, row, full_bar(s));
                    }
                }
            }
        };
        auto stage_of = [&](int n) { return (n % p.groups) * p.depth + (n / p.groups) % p.depth; };
        // Before waiting for the previous kernel: keys and values of this CTA's first items, as far as their splits
        // end before the position that kernel is writing (the sequence's last).  Their stages are fresh.
        int early = 0;
        {
            Item it;
            int id_e = item_at(p, blockIdx.x, it);
            while (id_e < p.total && early < stages && it.k_base + SPLIT < it.kv_len) {
                const int kpos = it.k_base + lane * p.page_size;
                int pg = 0;
                if (lane < pages_per_item && kpos < it.key_hi && kpos + p.page_size > it.key_lo)
                    pg = __ldg(p.block_table + (size_t)it.seq * p.table_stride + kpos / p.page_size);
                if (pg < 0 || pg >= p.num_pages) { atomicOr(p.status, RS_STATUS_BAD_PAGE); pg = 0; }
                const int s = stage_of(early);
                if (lane == 0)
                    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(STAGE_BYTES) : "memory");
                __syncwarp();                        // the byte count is expected before any lane's load can land
                load_pages(it, pg, s);
                ++early;
                id_e = item_at(p, id_e + gridDim.x, it);
            }
        }
        pdl_wait();
        Item cur, nxt;
        int page, page_n = 0;
        uint4 qv[QV], qn[QV];
        int id = item_at(p, blockIdx.x, cur);
        if (id < p.total) fetch(cur, page, qv);
        for (int n = 0; id < p.total; ++n) {
            const int id_n = item_at(p, id + gridDim.x, nxt);
            if (id_n < p.total) fetch(nxt, page_n, qn);
            const int k = n / p.groups;
            const int s = stage_of(n);
            const uint32_t parity = (uint32_t)(k / p.depth) & 1u;
            if (page < 0 || page >= p.num_pages) { atomicOr(p.status, RS_STATUS_BAD_PAGE); page = 0; }
            const bool loaded = n < early;           // its keys and values are already on their way
            int ok = 1;
            if (lane == 0 && !loaded) ok = mbar_wait(empty_bar(s), parity ^ 1u, abort_flag, p.status) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const uint32_t qdst = q0 + s * Q_BYTES;
#pragma unroll
            for (int i = 0; i < QV; ++i) {
                const int v = lane + 32 * i;
                if (v < nvec) {
                    const int r = v / VEC, c = v % VEC;
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(qdst + r * (HD * 2) + ((c ^ (r & 7)) << 4)),
                                 "r"(qv[i].x), "r"(qv[i].y), "r"(qv[i].z), "r"(qv[i].w) : "memory");
                }
            }
            __syncwarp();                            // every lane's query rows are written before lane 0 arrives
            if (lane == 0) {
                if (loaded) mbar_arrive(full_bar(s));
                else mbar_expect_tx(full_bar(s), STAGE_BYTES);
            }
            __syncwarp();                            // ... and the byte count is expected before any lane's load can land
            if (!loaded) load_pages(cur, page, s);
            if (lane == 0) *produced = n + 1;
            id = id_n; cur = nxt; page = page_n;
#pragma unroll
            for (int i = 0; i < QV; ++i) qv[i] = qn[i];
        }
    } else if (warp == producer_warp + 1) {
        // ------------------------------------------------------------ prefetcher: the smem ring holds too little to cover
        // the latency of loaded DRAM, so the pages of the next few items are asked into L2 ahead of the producer
        pdl_wait();
        if (p.one_load_per_page) {
            const int pages_per_item = SPLIT / p.page_size;
            Item it;
            int n = 0;
            bool go = true;
            for (int id = item_at(p, blockIdx.x, it); id < p.total && go; id = item_at(p, id + gridDim.x, it), ++n) {
                const int kpos = it.k_base + lane * p.page_size;
                int page = -1;
                if (lane < pages_per_item && kpos < it.key_hi && kpos + p.page_size > it.key_lo)
                    page = __ldg(p.block_table + (size_t)it.seq * p.table_stride + kpos / p.page_size);
                unsigned long long t0 = 0;                // the clock is slow to read: every 64 naps only
                for (uint32_t i = 1; n >= *produced + PREFETCH_AHEAD; ++i) {
                    __nanosleep(200);
                    if (*abort_flag) { go = false; break; }
                    if ((i & 63u) == 0u) {
                        const unsigned long long now = global_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > RS_WAIT_LIMIT_NS) { go = false; break; }
                    }
                }
                if (go && page >= 0 && page < p.num_pages) tma_prefetch_5d(&map_kv, 0, 0, 0, 0, page * 2 * p.n_kv + it.kvh);
            }
        }
    } else if (warp < producer_warp) {
        // ------------------------------------------------------------ consumers: group g takes the items g, g + G, ... of the CTA
        const int grp = warp / GROUP_WARPS, gw = warp % GROUP_WARPS;
        const int g = lane >> 2, t = lane & 3;
        auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(GROUP_WARPS * 32) : "memory"); };
        // A warp whose wait ran out keeps walking its items without touching them, so that the group's named
        // barrier below always finds all four warps.
        pdl_wait();                                  // the workspace of partials belongs to earlier kernels until now
        bool ok = true;
        Item it;
        // the CTA's n-th item has id blockIdx.x + n * gridDim.x: a group looks at its own only
        for (int n = grp, id = blockIdx.x + grp * gridDim.x; id < p.total; n += p.groups, id += p.groups * gridDim.x) {
            it = decode_item(p, id);
            const int k = n / p.groups;
            const int s = grp * p.depth + k % p.depth;
            const uint32_t parity = (uint32_t)(k / p.depth) & 1u;
            const uint32_t st_smem = base + s * STAGE_BYTES, q_smem = q0 + s * Q_BYTES;
            // where warp ww leaves row r of its result: over its own tokens' keys and values
            auto result_row = [&](int ww, int r) {
                if (p.page_size <= KEYS_PER_WARP) return st_smem + ww * WARP_BYTES + r * (OLD * 4);   // whole pages, contiguous
                const int c = r / ROWS_PER_CHUNK, row = ww * KEYS_PER_WARP;
                return st_smem + (row >> page_shift) * page_block + c * piece + (row & (p.page_size - 1)) * 128 +
                       (r % ROWS_PER_CHUNK) * (OLD * 4);
            };
            if (ok) ok = mbar_wait(full_bar(s), parity, abort_flag, p.status);
            if (ok) {
                // address of the 16-byte chunk holding dims [col, col + 8) of token `row`'s key (kv = 0) or value (kv = 1)
                auto chunk_addr = [&](int kv, int row, int col) {
                    return st_smem + (row >> page_shift) * page_block + (kv * HALVES + (col >> 6)) * piece +
                           (row & (p.page_size - 1)) * 128 + (((((col & 63) >> 3) ^ row) & 7) << 4);
                };
                const int j0 = gw * KEYS_PER_WARP;
                float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
                float o[DT][4];
#pragma unroll
                for (int d = 0; d < DT; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
                if (it.k_base + j0 < it.key_hi && it.k_base + j0 + KEYS_PER_WARP > it.key_lo) {      // uniform per warp
                    float sc[4][4];
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        uint32_t qa[4], b0[4], b1[4];
                        {
                            const int mi = lane >> 3, row = (lane & 7) + (mi & 1) * 8, c = 2 * ks + (mi >> 1);
                            ldmatrix_x4(q_smem + row * (HD * 2) + ((c ^ (row & 7)) << 4), qa[0], qa[1], qa[2], qa[3]);
                        }
                        const int row = j0 + (lane >> 4) * 8 + (lane & 7);
                        const int col = 16 * ks + ((lane >> 3) & 1) * 8;
                        ldmatrix_x4(chunk_addr(0, row, col), b0[0], b0[1], b0[2], b0[3]);
                        ldmatrix_x4(chunk_addr(0, row + 16, col), b1[0], b1[1], b1[2], b1[3]);
                        mma16816(sc[0], qa, b0[0], b0[1]);
                        mma16816(sc[1], qa, b0[2], b0[3]);
                        mma16816(sc[2], qa, b1[0], b1[1]);
                        mma16816(sc[3], qa, b1[2], b1[3]);
                    }
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int kpos = it.k_base + j0 + 8 * nt + 2 * t + (i & 1);
                            const bool vis = kpos >= it.key_lo && kpos < it.key_hi;
                            sc[nt][i] = vis ? sc[nt][i] * p.scale_log2 : -INFINITY;
                            m_row[i >> 1] = fmaxf(m_row[i >> 1], sc[nt][i]);
                        }
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        m_row[r] = fmaxf(m_row[r], __shfl_xor_sync(0xffffffffu, m_row[r], 1));
                        m_row[r] = fmaxf(m_row[r], __shfl_xor_sync(0xffffffffu, m_row[r], 2));
                    }
                    // the warp's range holds a visible key, so both maxima are finite
                    uint32_t pf[2][4];
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        float e[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            e[i] = fast_exp2(sc[nt][i] - m_row[i >> 1]);
                            l_row[i >> 1] += e[i];
                        }
                        pf[nt >> 1][2 * (nt & 1)] = pack_bf16(e[0], e[1]);
                        pf[nt >> 1][2 * (nt & 1) + 1] = pack_bf16(e[2], e[3]);
                    }
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
                        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
                    }
#pragma unroll
                    for (int d = 0; d < DT; d += 2) {
                        uint32_t v0[4], v1[4];
                        const int row = j0 + ((lane >> 3) & 1) * 8 + (lane & 7);
                        const int col = 8 * (d + (lane >> 4));
                        ldmatrix_x4_trans(chunk_addr(1, row, col), v0[0], v0[1], v0[2], v0[3]);
                        ldmatrix_x4_trans(chunk_addr(1, row + 16, col), v1[0], v1[1], v1[2], v1[3]);
                        mma16816(o[d], pf[0], v0[0], v0[1]);
                        mma16816(o[d + 1], pf[0], v0[2], v0[3]);
                        mma16816(o[d], pf[1], v1[0], v1[1]);
                        mma16816(o[d + 1], pf[1], v1[2], v1[3]);
                    }
                }
                __syncwarp();                        // all lanes are done reading the warp's key and value rows
                if (g < p.group) {
                    const uint32_t r0 = result_row(gw, g);
#pragma unroll
                    for (int d = 0; d < DT; ++d)
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(r0 + (8 * d + 2 * t) * 4), "f"(o[d][0]), "f"(o[d][1]) : "memory");
                    if (t == 0)
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(r0 + HD * 4), "f"(m_row[0]), "f"(l_row[0]) : "memory");
                }
                if (g + 8 < p.group) {
                    const uint32_t r1 = result_row(gw, g + 8);
#pragma unroll
                    for (int d = 0; d < DT; ++d)
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(r1 + (8 * d + 2 * t) * 4), "f"(o[d][2]), "f"(o[d][3]) : "memory");
                    if (t == 0)
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(r1 + HD * 4), "f"(m_row[1]), "f"(l_row[1]) : "memory");
                }
            }
            group_sync();
            if (ok) {
                // one partial per head: the four warps' sums on a common maximum
                const size_t slot = (size_t)__ldg(p.split_start + it.w) + it.split_local;
                float* dst = p.partial + (slot * p.n_q + (size_t)it.kvh * p.group) * (HD + 2);
                auto lds = [&](uint32_t a) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a)); return v; };
                const bool in_workspace = slot < (size_t)p.partial_slots;
                if (!in_workspace && gw == 0 && lane == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
                // a warp takes the heads gw, gw + 4, ...: the four warps' maxima and weights of a head once, then a
                // lane per column of the partial (head dims, then maximum and sum)
                for (int r = gw; in_workspace && r < p.group; r += GROUP_WARPS) {
                    float mw[GROUP_WARPS], e[GROUP_WARPS], M = -INFINITY;
#pragma unroll
                    for (int ww = 0; ww < GROUP_WARPS; ++ww) { mw[ww] = lds(result_row(ww, r) + HD * 4); M = fmaxf(M, mw[ww]); }
#pragma unroll
                    for (int ww = 0; ww < GROUP_WARPS; ++ww) e[ww] = (mw[ww] == -INFINITY) ? 0.f : fast_exp2(mw[ww] - M);
                    for (int d = lane; d < HD + 2; d += 32) {
                        float val = M;
                        if (d != HD) {
                            val = 0.f;
#pragma unroll
                            for (int ww = 0; ww < GROUP_WARPS; ++ww)
                                val = fmaf(lds(result_row(ww, r) + (d < HD ? d : HD + 1) * 4), e[ww], val);
                        }
                        dst[r * (HD + 2) + d] = val;
                    }
                }
                // the next writes to these rows come from TMA
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(s));
            }
        }
    }
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);      // let loads already issued land
    }
    __syncthreads();
}

// out[token of seq, head, :] = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// The splits are added in four interleaved chains (split s goes to chain s mod 4, each chain in ascending order)
// that meet as (c0 + c1) + (c2 + c3): the order depends on the number of splits alone, that is on the sequence's
// length, never on the batch.  One CTA per (sequence, head).  TG = 4: four threads per head dim, one per chain (small
// batches: many loads in flight); TG = 1: one thread per head dim runs all four chains (large batches: small CTAs).
// Both give the same bits.
constexpr int MERGE_CHAINS = 4;
constexpr int MERGE_MAX_SPLITS = 512;      // weights kept in shared memory; longer sequences go in rounds of this many
template <int HD, int TG>
__global__ void __launch_bounds__(TG * HD) decode_merge_kernel(const DecodeParams p) {
    constexpr int NT = TG * HD;
    __shared__ float wgt[MERGE_MAX_SPLITS], wl[MERGE_MAX_SPLITS];
    __shared__ float red[NT / 32];
    __shared__ float part[2][MERGE_CHAINS][HD];
    const int w = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int d = tid % HD, g = tid / HD;
    pdl_launch_dependents();
    // the step's metadata is in place before its first kernel: it is read while the attention kernel is still at work
    const int seq = __ldg(p.work + w);
    const int kv_len = __ldg(p.kv_len + seq);
    const int key_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
    const int n_splits = (kv_len + SPLIT - 1) / SPLIT - key_lo / SPLIT;
    const float* base = p.partial + ((size_t)__ldg(p.split_start + w) * p.n_q + h) * (HD + 2);
    const size_t stride = (size_t)p.n_q * (HD + 2);
    __nv_bfloat16* const out_row = p.out + (size_t)__ldg(p.q_start + seq) * p.out_stride + (size_t)h * HD;
    pdl_wait();
    if ((size_t)__ldg(p.split_start + w) + n_splits > (size_t)p.partial_slots) {      // flagged by the split kernel too
        if (tid == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
        return;
    }
    // Everything the first round needs is asked for at once, before anything is waited for: the splits' maxima and
    // sums (kept in registers when there is at most one split per thread) and the first accumulators of this
    // thread's chain(s).  The arithmetic and its order are the same as if they were loaded where they are used.
    constexpr int ROUND = TG == MERGE_CHAINS ? 8 : 16;            // accumulator loads in flight per thread
    const int n_first = min(MERGE_MAX_SPLITS, n_splits);
    const bool mine_only = n_splits <= NT;                         // uniform
    float my_m = -INFINITY, my_l = 0.f;
    if (mine_only && tid < n_splits) {
        my_m = ld_dep(base + tid * stride + HD);
        my_l = ld_dep(base + tid * stride + HD + 1);
    }
    float a0[ROUND];
#pragma unroll
    for (int j = 0; j < ROUND; ++j) {
        const int s = TG == MERGE_CHAINS ? g + MERGE_CHAINS * j : j;
        a0[j] = s < n_first ? ld_dep(base + s * stride + d) : 0.f;
    }
    // the row's maximum over all splits
    float M = my_m;
    if (!mine_only)
        for (int s = tid; s < n_splits; s += NT) M = fmaxf(M, ld_dep(base + s * stride + HD));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if ((tid & 31) == 0) red[tid >> 5] = M;
    __syncthreads();
    M = red[0];
#pragma unroll
    for (int i = 1; i < NT / 32; ++i) M = fmaxf(M, red[i]);
    float num[MERGE_CHAINS / TG], den[MERGE_CHAINS / TG];
#pragma unroll
    for (int c = 0; c < MERGE_CHAINS / TG; ++c) num[c] = den[c] = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += MERGE_MAX_SPLITS) {
        const int n = min(MERGE_MAX_SPLITS, n_splits - s0);
        const float* ps = base + (size_t)s0 * stride;
        __syncthreads();
        if (mine_only) {
            if (tid < n) {
                const float e = fast_exp2(my_m - M);
                wgt[tid] = e;
                wl[tid] = e * my_l;
            }
        } else {
            for (int s = tid; s < n; s += NT) {
                const float e = fast_exp2(ld_dep(ps + s * stride + HD) - M);
                wgt[s] = e;
                wl[s] = e * ld_dep(ps + s * stride + HD + 1);
            }
        }
        __syncthreads();
        if (TG == MERGE_CHAINS) {
            for (int i = g; i < n; i += MERGE_CHAINS * ROUND) {          // my chain: splits g, g + 4, ...; eight loads in flight
                float a[ROUND];
                const bool first = s0 == 0 && i == g;
#pragma unroll
                for (int j = 0; j < ROUND; ++j) {
                    const int s = i + MERGE_CHAINS * j;
                    a[j] = first ? a0[j] : (s < n ? ld_dep(ps + s * stride + d) : 0.f);
                }
#pragma unroll
                for (int j = 0; j < ROUND; ++j) {
                    const int s = i + MERGE_CHAINS * j;
                    if (s < n) { num[0] = fmaf(a[j], wgt[s], num[0]); den[0] += wl[s]; }
                }
            }
        } else {
            for (int i = 0; i < n; i += ROUND) {                           // all chains: sixteen loads in flight
                float a[ROUND];
                const bool first = s0 == 0 && i == 0;
#pragma unroll
                for (int j = 0; j < ROUND; ++j) a[j] = first ? a0[j] : (i + j < n ? ld_dep(ps + (i + j) * stride + d) : 0.f);
#pragma unroll
                for (int j = 0; j < ROUND; ++j)
                    if (i + j < n) { num[j % MERGE_CHAINS] = fmaf(a[j], wgt[i + j], num[j % MERGE_CHAINS]); den[j % MERGE_CHAINS] += wl[i + j]; }
            }
        }
    }
    float nn, dd;
    if (TG == MERGE_CHAINS) {
        part[0][g][d] = num[0]; part[1][g][d] = den[0];
        __syncthreads();
        nn = (part[0][0][d] + part[0][1][d]) + (part[0][2][d] + part[0][3][d]);
        dd = (part[1][0][d] + part[1][1][d]) + (part[1][2][d] + part[1][3][d]);
    } else {
        nn = (num[0] + num[MERGE_CHAINS / TG > 1 ? 1 : 0]) + (num[MERGE_CHAINS / TG > 2 ? 2 : 0] + num[MERGE_CHAINS / TG > 3 ? 3 : 0]);
        dd = (den[0] + den[MERGE_CHAINS / TG > 1 ? 1 : 0]) + (den[MERGE_CHAINS / TG > 2 ? 2 : 0] + den[MERGE_CHAINS / TG > 3 ? 3 : 0]);
    }
    if (g == 0) out_row[d] = __float2bfloat16_rn(nn / dd);
}

// 5-d map of the cache: (64 dims, token of the page, half of the head, K|V, block = page * 2 * n_kv + kv head); one
// box is everything an item needs of a page.  Returns non-zero if the driver does not take it.
int page_map(const void* cache, int num_pages, int n_kv, int page_size, int hd, CUtensorMap* out) {
    using namespace rs_tma;
    EncodeTiledFn enc = get_encoder();
    if (!enc) return 1;
    const cuuint64_t row = (cuuint64_t)hd * 2;
    cuuint64_t dims[5] = {64, (cuuint64_t)page_size, (cuuint64_t)(hd / 64), 2, (cuuint64_t)num_pages * 2 * n_kv - n_kv};
    cuuint64_t strides[4] = {row, 128, (cuuint64_t)n_kv * page_size * row, (cuuint64_t)page_size * row};
    cuuint32_t box[5] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64), 2, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1;
}

struct PageMapKey { const void* cache; int num_pages, n_kv, page_size, hd; };
struct PageMapEntry { PageMapKey key; int refused; CUtensorMap map; };
std::vector<PageMapEntry> g_page_maps;
std::mutex g_page_maps_mutex;
int g_last_loads_per_page = 0;

int cached_page_map(const void* cache, int num_pages, int n_kv, int page_size, int hd, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_page_maps_mutex);
    for (auto& e : g_page_maps)
        if (e.key.cache == cache && e.key.num_pages == num_pages && e.key.n_kv == n_kv && e.key.page_size == page_size &&
            e.key.hd == hd) { *out = e.map; return e.refused; }
    PageMapEntry e{PageMapKey{cache, num_pages, n_kv, page_size, hd}, 0, {}};
    e.refused = page_map(cache, num_pages, n_kv, page_size, hd, &e.map);
    if (g_page_maps.size() > 64) g_page_maps.clear();
    g_page_maps.push_back(e);
    *out = e.map;
    return e.refused;
}

// One thread per (sequence, kv head, split of the launch shape): a live one writes its triple to its id.
// The attention kernel reads the list before it waits for the kernel in front of it (its first loads start early), so
// this kernel is an ordinary launch that lets nothing start before it has ended: whatever follows it in the stream,
// launched early or not, finds the list complete.
__global__ void decode_items_kernel(const int* __restrict__ split_start, int n_work, int n_kv, int max_splits, int* __restrict__ items) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_work * n_kv * max_splits) return;
    const int s = i % max_splits, r = i / max_splits;
    const int kvh = r % n_kv, w = r / n_kv;
    const int first = split_start[w], n_splits = split_start[w + 1] - first;
    if (s < n_splits) items[first * n_kv + kvh * n_splits + s] = pack_item(w, kvh, s);
}

template <int HD>
int launch(const CUtensorMap& mkv, DecodeParams p, cudaStream_t s) {
    constexpr size_t stage_bytes = (size_t)2 * (HD / 64) * SPLIT * 128 + Q_ROWS * HD * 2 + 16;
    constexpr size_t budget = 225 * 1024 - 1024 - 16;
    const int stages = (int)(budget / stage_bytes);
    p.groups = stages < MAX_GROUPS ? stages : MAX_GROUPS;
    p.depth = stages / p.groups < 2 ? stages / p.groups : 2;
    const size_t smem = (size_t)p.groups * p.depth * stage_bytes + 1024 + 16;
    auto kern = decode_attention_kernel<HD>;
    static size_t smem_allowed = 0;
    if (smem > smem_allowed) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        smem_allowed = smem;
    }
    const int sms = rs_tma::sm_count();
    const int grid = p.total < sms ? p.total : sms;
    int rc = rs_launch_pdl(kern, dim3(grid), dim3((p.groups * GROUP_WARPS + 2) * 32), smem, s, mkv, p);
    if (rc != 0) return rc;
    // a small batch: four threads per head dim; else small CTAs (the same bits either way)
    if ((long)p.n_work * p.n_q <= 1024)
        return rs_launch_pdl(decode_merge_kernel<HD, MERGE_CHAINS>, dim3(p.n_work, p.n_q), dim3(MERGE_CHAINS * HD), 0, s, p);
    return rs_launch_pdl(decode_merge_kernel<HD, 1>, dim3(p.n_work, p.n_q), dim3(HD), 0, s, p);
}
}  // namespace

// Shapes this kernel is built for; other head sizes, groups above 16 heads and page sizes that are not a power of
// two from 8 to 128 go to the CUDA-core kernel.
RS_EXPORT int rs_attention_decode_bf16_supported(int n_q, int n_kv, int hd, int page_size) {
    if (n_kv <= 0 || n_q % n_kv || n_q / n_kv > Q_ROWS) return 0;
    if (hd != 64 && hd != 128) return 0;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

RS_EXPORT int rs_attention_decode_bf16_split_keys() { return SPLIT; }

// The list of live items of a step (see decode_item): items[split_start[n_work] * n_kv], to be built once per step
// and handed to every rs_attention_decode_bf16 call of the step with the same work list, split_start, n_kv.  max_splits:
// at least the largest number of splits of a sequence (the launch shape).
RS_EXPORT int rs_attention_decode_build_items(const int* split_start, int n_work, int n_kv, int max_splits, int* items, void* stream) {
    if (n_work <= 0) return 0;
    if (split_start == nullptr || items == nullptr || n_kv <= 0 || n_kv > ITEM_MAX_KV || n_work > ITEM_MAX_SEQS || max_splits <= 0 ||
        max_splits > ITEM_MAX_SPLITS || (long)n_work * n_kv * max_splits > 0x7fff0000L)
        return (int)cudaErrorInvalidValue;
    const int n = n_work * n_kv * max_splits;
    decode_items_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(split_start, n_work, n_kv, max_splits, items);
    return (int)cudaGetLastError();
}

// TMA loads per page of an item in the most recent launch: 1 with the 5-d map, else 2 * head size / 64.
RS_EXPORT int rs_attention_decode_bf16_loads_per_page() { return g_last_loads_per_page; }

// Same arguments and partial-workspace layout as the decode form of rs_attention_simt; bfloat16 only.
RS_EXPORT int rs_attention_decode_bf16(const void* q, long q_stride, void* out, long out_stride, const void* cache,
                                       long page_stride, int num_pages, int page_size, const int* block_table,
                                       int table_stride, const int* q_start, const int* kv_len, const int* work,
                                       int n_work, int n_q, int n_kv, int hd, int window, float scale, int split_keys,
                                       int max_splits, const int* split_start, const int* items, float* partial,
                                       int partial_slots, int* status, void* stream) {
    if (n_work <= 0) return 0;
    if (!rs_attention_decode_bf16_supported(n_q, n_kv, hd, page_size) || split_keys != SPLIT || max_splits <= 0 ||
        partial == nullptr || partial_slots <= 0 || split_start == nullptr || items == nullptr || n_kv > ITEM_MAX_KV ||
        n_work > ITEM_MAX_SEQS || max_splits > ITEM_MAX_SPLITS || (q_stride % 8) || ((long)q & 15) || ((long)cache & 15) ||
        page_stride != (long)2 * n_kv * page_size * hd || (long)n_work * n_kv * max_splits > 0x7fff0000L)
        return (int)cudaErrorInvalidValue;
    DecodeParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work;
    p.n_q = n_q; p.n_kv = n_kv; p.group = n_q / n_kv; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.split_start = split_start; p.items = items; p.partial = partial; p.partial_slots = partial_slots; p.status = status;
    p.n_work = n_work; p.max_splits = max_splits;
    p.total = n_work * n_kv * max_splits;          // an upper bound, for the size of the grid
    p.groups = p.depth = 0;
    CUtensorMap mkv;
    p.one_load_per_page = cached_page_map(cache, num_pages, n_kv, page_size, hd, &mkv) == 0;
    if (!p.one_load_per_page) {
        int rc = rs_tma::get_map(cache, (long)num_pages * 2 * n_kv * page_size, hd, hd, page_size, &mkv);
        if (rc) return rc;
    }
    g_last_loads_per_page = p.one_load_per_page ? 1 : 2 * (hd / 64);
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch<64>(mkv, p, s);
    return launch<128>(mkv, p, s);
}
