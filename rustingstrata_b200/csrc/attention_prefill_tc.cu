// Attention of prompt portions on the 5th-generation tensor cores (sm_100a), head sizes 64 and 128.
//
// A CTA owns 128 rows; a row is (query token, query head) with P heads of one kv group packed side by side,
// so a key/value tile in shared memory serves P heads.  Keys are walked in blocks of 128 at absolute
// positions.  Per block
//   S = Q K^T      tcgen05.mma, Q (128 x hd) and the K block (128 keys x hd) both K-major in shared memory
//                  (TMA, 128-byte swizzle), S in tensor memory.  A K or V block lies in shared memory as
//                  [group of 8 keys][64-wide half of the head][8 keys][64 dims]: every (group, half) piece is one
//                  1 KiB swizzle atom, the groups are evenly spaced whatever the page size is, and a cache page
//                  arrives with ONE 5-d TMA load (the TMA unit spends a fixed time per load, so fewer and larger
//                  loads feed the tensor cores faster);
//   softmax        eight warps, two threads per row (each half of the block's keys): tcgen05.ld the scores, mask
//                  (causal, window, length), running max and sum in float32 with exp2, P rounded to bfloat16 and
//                  written back over S with tcgen05.st (two values per 32-bit column);
//   O += P V       tcgen05.mma with P as the tensor-memory operand and the V block (keys x hd, hd contiguous =
//                  MN-major) in shared memory, accumulated in tensor memory over all blocks.  The reference maximum
//                  of a row only moves when a block exceeds it by more than 2^8; only then are the row's sum and
//                  its O (loaded, scaled, stored back) corrected, which after the first blocks is rare.
// Warp 8 issues the MMAs (one elected lane) and owns the tensor-memory allocation; warp 9 streams the keys and warp
// 10 the values (lane i looks page i of a block up, three blocks ahead, and loads it).  The scores have three buffers
// in tensor memory, so Q K^T runs two blocks ahead of P V and the softmax warps never wait for scores.  The CTAs are
// persistent: one per SM, each walks several tiles (longest first, dealt in a snake), loads the next tile's queries
// and first keys under this tile's last blocks, and stores a result through a staging tile in shared memory (whole
// tiles by TMA store).  Every mbarrier wait is bounded (tma_helpers.cuh).  Cache pages a block does not own (beyond
// the sequence, given back by a window) are replaced by page 0: their keys are masked, and their values only have to
// be finite.
//
// Reference counterpart: attn_prefill_* (src/cuda/kernels.cu:2813-3156), an mma.sync kernel with f16 inputs.
#include "tma_helpers.cuh"
#include <math.h>

namespace {
constexpr int ROWS = 128;              // rows per CTA = TMEM lanes
constexpr int BKV = 128;               // keys per block
constexpr int PARTS = 2;                // softmax threads per row: each takes 128 / PARTS keys of a block and hd / PARTS dims of O
                                        // (four threads per row, 16 softmax warps, were 4 % slower: the softmax is not short of warps)
constexpr int SOFTMAX_WARPS = 4 * PARTS;
constexpr int MMA_WARP = SOFTMAX_WARPS, TMA_WARP = SOFTMAX_WARPS + 1;
constexpr int THREADS = (SOFTMAX_WARPS + 3) * 32;        // the warp after TMA_WARP loads the values, TMA_WARP the keys
constexpr int KV_STAGES = 2;
constexpr int LOCAL_ITEMS = 64;        // items of a CTA whose description is kept in shared memory (later ones are worked out when met)

struct TcParams {
    __nv_bfloat16* out; long out_stride;
    int page_size, num_pages;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len; const int* work; int n_work;
    int n_q, n_kv, group, pack, pack_shift, tokens_per_cta;      // pack = 1 << pack_shift heads side by side in a tile
    int window;
    float scale_log2;
    int* status;
    int one_load_per_page;             // the 5-d map of the cache is in use (else 2-d loads of 8 keys x 64 dims)
    int out_by_tma;                    // the result has a tensor map: whole tiles are stored by the TMA unit
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// shared memory -> global, tiled; completion is tracked by the issuing thread's bulk groups
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc) : "memory");
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr, uint32_t sbo = 1024) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand tile (the contiguous direction is N), 128-byte swizzle: 64 elements of N contiguous per row of
// 128 bytes, groups of 8 rows of K `sbo` bytes apart, blocks of 64 N-elements `lbo` bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// What a CTA needs to know of one work item: a tile of query rows (sequence, first query, kv group and heads).
struct TcItem { int seq, q_off, kvh, head0, row0, n_tok, n_rows, qpos0, key_lo, key_hi, blk_lo, n_blocks; };

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const __grid_constant__ CUtensorMap map_out, const TcParams p) {
    constexpr int HALVES = HD / 64;                      // 64-wide (128-byte) column blocks of a head
    constexpr int HALF_BYTES = 128 * 128;                // 128 rows x 128 bytes
    constexpr int TILE_BYTES = HALVES * HALF_BYTES;      // one Q, K or V tile
    constexpr int GROUP_BYTES = HALVES * 1024;           // 8 keys of a K or V tile: one swizzle atom per half of the head
    constexpr int TMEM_COLS = 512;                       // S0 | S1 | S2 | O  (3 x 128 + HD columns)
    constexpr int S_BUFS = 3, O_COL = S_BUFS * 128;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t q_smem = base, k_smem = base + TILE_BYTES, v_smem = k_smem + KV_STAGES * TILE_BYTES;
    const uint32_t bar0 = v_smem + KV_STAGES * TILE_BYTES;
    // barriers: q_full, q_empty, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[3], p_ready[3], o_full[3], o_empty.
    // A wait by parity cannot tell "this phase is over" from "the phase before the one before it is not over yet".  Every
    // barrier but o_full is waited for phase by phase, so its waiter is never that far ahead.  The softmax warps look at
    // o_full only when they rescale O and at an item's end, and with three score buffers they can be two P V ahead of
    // the tensor core (values that arrive late hold P V up, scores do not need them): block b's P V completes barrier
    // b % 3, and scores of block b exist only after P V (b - 3) is over, so a waiter is at most one phase ahead.
    enum { Q_FULL = 0, Q_EMPTY = 1, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, P_READY = 13, O_FULL = 16,
           O_EMPTY = 19, NBAR = 20 };
    auto bar = [&](int i) { return bar0 + 8u * i; };
    uint8_t* aligned = smem_raw + (base - raw);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aligned + (bar0 - base) + 8 * NBAR);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xchg = reinterpret_cast<float*>(tmem_slot + 4);     // [2 blocks parity][PARTS][ROWS] maxima, then [PARTS][ROWS] sums
    TcItem* item_table = reinterpret_cast<TcItem*>(xchg + 3 * PARTS * ROWS);                       // [LOCAL_ITEMS]
    // results on their way out: [SOFTMAX_WARPS][32 rows][HD / PARTS] bf16, which for 64 dims per part is the layout of
    // the query tile ([half of the head][row][128 bytes], chunks swizzled by the row), 1 KiB aligned for the TMA unit
    uint8_t* stage_out = aligned + ((reinterpret_cast<uint8_t*>(item_table + LOCAL_ITEMS) - aligned + 1023) & ~(size_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // The CTAs stay: one per SM, each walks several items.  An item's start (barriers, tensor memory, the first loads'
    // latency, the first scores) and its end (the last P V, O read back, normalised and stored) keep the tensor cores
    // and the softmax warps idle for about as long as four blocks of keys take, which at 2,048 tokens was a third of
    // a CTA's life.  Here the barriers and the tensor memory are set up once, the next item's queries and first keys
    // are loaded while this item's last blocks are at work, and its first Q K^T is issued while the softmax warps
    // store this item's result.  All barrier phases count on across the items (g: blocks before this item, nq: items
    // before it).  The host sorts the items by the keys they walk, longest first; round r gives CTA b item r G + b or,
    // in odd rounds, r G + (G - 1 - b), so that every CTA gets long and short ones and the sums come out even.
    const int chunks_per_group = p.group / p.pack;
    const int ny = p.n_kv * chunks_per_group;
    const int total = p.n_work * ny;
    const int G = (int)gridDim.x;
    auto item_of_round = [&](int round) {
        return round * G + ((round & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
    };
    auto compute_item = [&](int id) {
        TcItem I;
        const int x = id / ny, y = id - x * ny;
        I.seq = __ldg(p.work + 2 * x);
        I.q_off = __ldg(p.work + 2 * x + 1);
        I.kvh = y / chunks_per_group;
        I.head0 = I.kvh * p.group + (y % chunks_per_group) * p.pack;
        I.row0 = __ldg(p.q_start + I.seq);
        const int q_len = __ldg(p.q_start + I.seq + 1) - I.row0;
        const int kv_len = __ldg(p.kv_len + I.seq);
        I.n_tok = min(p.tokens_per_cta, q_len - I.q_off);
        I.n_rows = I.n_tok * p.pack;
        I.qpos0 = kv_len - q_len + I.q_off;
        I.key_lo = p.window > 0 ? max(0, I.qpos0 - p.window + 1) : 0;
        I.key_hi = min(kv_len, I.qpos0 + I.n_tok);
        I.blk_lo = I.key_lo / BKV;
        I.n_blocks = (I.key_hi + BKV - 1) / BKV - I.blk_lo;
        return I;
    };
    // What the items of this CTA's first rounds are is worked out once, side by side (three dependent loads each), and
    // kept in shared memory: every role looks an item up when it gets there, and none waits for global memory then.
    if (threadIdx.x < LOCAL_ITEMS) {
        const int id = item_of_round(threadIdx.x);
        if (threadIdx.x * G < total && id < total) item_table[threadIdx.x] = compute_item(id);
    }
    auto get_item = [&](int round, int id) { return round < LOCAL_ITEMS ? item_table[round] : compute_item(id); };

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        mbar_init(bar(Q_EMPTY), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(K_FULL + s), 1); mbar_init(bar(K_EMPTY + s), 1);
            mbar_init(bar(V_FULL + s), 1); mbar_init(bar(V_EMPTY + s), 1);
        }
        for (int s = 0; s < S_BUFS; ++s) {
            mbar_init(bar(S_FULL + s), 1); mbar_init(bar(P_READY + s), SOFTMAX_WARPS); mbar_init(bar(O_FULL + s), 1);
        }
        mbar_init(bar(O_EMPTY), SOFTMAX_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    if (warp >= TMA_WARP) {
        // ------------------------------------------------------------ TMA producers: one warp streams the keys, the
        // next one the values; lane i loads page i of a block.  A warp needs of the order of 80 cycles per load it
        // issues and 800 for a block-table entry from L2.  One warp doing both for keys and values, and looking a
        // block's pages up while the block before it was on its way, took as long per block of 128 keys as the block
        // takes everything else (2,400 cycles at pages of 16: per-block timestamps of a throw-away build) and was what
        // the kernel waited for.  So the two streams have a warp each, and the pages are looked up three blocks ahead.
        const int kv = warp - TMA_WARP;
        const int pages_per_block = BKV / p.page_size;
        const uint32_t tiles = kv ? v_smem : k_smem;
        pdl_wait();                                           // q and the portion's keys and values come from the kernel before
        int g = 0, nq = 0;
        bool alive = true;
        for (int round = 0; round * G < total && alive; ++round) {
            const int id = item_of_round(round);
            if (id >= total) continue;
            const TcItem I = get_item(round, id);
            if (I.n_blocks <= 0) continue;
            if (kv == 0 && lane == 0) {
                // the queries' tile is free once the last Q K^T of the item before has read it
                if (nq == 0 || mbar_wait(bar(Q_EMPTY), (nq - 1) & 1, abort_flag, p.status)) {
                    mbar_expect_tx(bar(Q_FULL), TILE_BYTES);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_3d(q_smem + h * HALF_BYTES, &map_q, h * 64, I.head0, I.row0 + I.q_off, bar(Q_FULL));
                }
            }
            const int* table = p.block_table + (size_t)I.seq * p.table_stride;
            auto lookup = [&](int j) {                            // the value is not looked at before it is used
                const int kpos = (I.blk_lo + j) * BKV + lane * p.page_size;
                int page = 0;
                if (j < I.n_blocks && lane < pages_per_block && kpos < I.key_hi && kpos + p.page_size > I.key_lo)
                    page = __ldg(table + kpos / p.page_size);
                return page;
            };
            constexpr int AHEAD = 3;
            int pages[AHEAD];
#pragma unroll
            for (int a = 0; a < AHEAD; ++a) pages[a] = lookup(a);
            for (int j = 0; j < I.n_blocks; ++j) {
                const int jj = g + j;
                const int s = jj & 1;
                const uint32_t par = ((jj >> 1) & 1) ^ 1u;
                const int page_later = lookup(j + AHEAD);
                const uint32_t full = bar((kv ? V_FULL : K_FULL) + s);
                int ok = 1;
                if (lane == 0) {
                    ok = mbar_wait(bar((kv ? V_EMPTY : K_EMPTY) + s), par, abort_flag, p.status) ? 1 : 0;
                    if (ok) mbar_expect_tx(full, TILE_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);              // also orders the expect_tx before every lane's loads
                if (!ok) { alive = false; break; }
                int page = pages[0];
                if (page < 0 || page >= p.num_pages) { atomicOr(p.status, RS_STATUS_BAD_PAGE); page = 0; }
                if (lane < pages_per_block) {
                    const uint32_t dst = tiles + s * TILE_BYTES + lane * (p.page_size / 8) * GROUP_BYTES;
                    const int block = (page * 2 + kv) * p.n_kv + I.kvh;
                    if (p.one_load_per_page) {
                        tma_load_5d(dst, &map_kv, 0, 0, 0, 0, block, full);
                    } else {
                        for (int g8 = 0; g8 < p.page_size / 8; ++g8)
#pragma unroll
                            for (int h = 0; h < HALVES; ++h)
                                tma_load_2d(dst + g8 * GROUP_BYTES + h * 1024, &map_kv, h * 64, block * p.page_size + g8 * 8, full);
                    }
                }
#pragma unroll
                for (int a = 0; a + 1 < AHEAD; ++a) pages[a] = pages[a + 1];
                pages[AHEAD - 1] = page_later;
            }
            g += I.n_blocks;
            ++nq;
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = idesc_bf16(ROWS, BKV, 0), idesc_pv = idesc_bf16(ROWS, HD, 1);
            int g = 0, nq = 0;
            bool ok = true;
            for (int round = 0; round * G < total && ok; ++round) {
                const int id = item_of_round(round);
                if (id >= total) continue;
                const TcItem I = get_item(round, id);
                const int n_blocks = I.n_blocks;
                if (n_blocks <= 0) continue;
                ok = mbar_wait(bar(Q_FULL), nq & 1, abort_flag, p.status);
                // Scores have three buffers: Q K^T of block j + 2 is issued before P V of block j, so the scores of a
                // block are ready a whole block before the softmax warps ask for them, and those never wait for this
                // thread (with two buffers Q K^T (j + 2) could only follow P V (j), which follows the softmax of block
                // j: the two roles then ran in turn for part of every block).  Buffer (j + 2) % 3 held P of block
                // j - 1, which P V (j - 1) has read: it was issued earlier by this thread, and the tensor core runs
                // them in order.
                auto issue_qk = [&](int j) {
                    const int jj = g + j;
                    const int s = jj & 1, sb = jj % S_BUFS;
                    if (!mbar_wait(bar(K_FULL + s), (jj >> 1) & 1, abort_flag, p.status)) return false;
                    tc_fence_after();
                    const uint32_t d = tmem_base + sb * 128;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        umma_ss(d, desc_kmajor(q_smem + (ks >> 2) * HALF_BYTES + (ks & 3) * 32),
                                desc_kmajor(k_smem + s * TILE_BYTES + (ks >> 2) * 1024 + (ks & 3) * 32, GROUP_BYTES), idesc_qk, ks ? 1u : 0u);
                    }
                    umma_commit(bar(K_EMPTY + s));           // the K stage is free once these have read it
                    umma_commit(bar(S_FULL + sb));
                    if (j == n_blocks - 1) umma_commit(bar(Q_EMPTY));      // ... and so are the queries after the item's last block
                    return true;
                };
                if (ok) ok = issue_qk(0);
                if (ok && n_blocks > 1) ok = issue_qk(1);
                for (int j = 0; j < n_blocks && ok; ++j) {
                    const int jj = g + j;
                    const int s = jj & 1, sb = jj % S_BUFS;
                    if (j + 2 < n_blocks) ok = issue_qk(j + 2);
                    if (!ok) break;
                    if (!mbar_wait(bar(P_READY + sb), (jj / S_BUFS) & 1, abort_flag, p.status)) { ok = false; break; }
                    // the first P V of an item overwrites O: the softmax warps must have read the item before out of it
                    if (j == 0 && nq > 0 && !mbar_wait(bar(O_EMPTY), (nq - 1) & 1, abort_flag, p.status)) { ok = false; break; }
                    if (!mbar_wait(bar(V_FULL + s), (jj >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < BKV / 16; ++kk)
                        umma_ts(tmem_base + O_COL, tmem_base + sb * 128 + kk * 8,
                                desc_mnmajor(v_smem + s * TILE_BYTES + kk * 2 * GROUP_BYTES, 1024, GROUP_BYTES), idesc_pv, (j | kk) ? 1u : 0u);
                    umma_commit(bar(V_EMPTY + s));
                    umma_commit(bar(O_FULL + sb));            // O holds the item's blocks 0..j
                }
                g += n_blocks;
                ++nq;
            }
        }
    } else {
        // ------------------------------------------------------------ softmax warps: PARTS threads per row
        // The warps w, w + 4, w + 8, ... own the same 32 rows (tensor-memory lanes 32 (w & 3) ..): warp number `part`
        // of them takes the keys [part * HK, +HK) of a block and the head dims [part * HO, +HO) of O.  They exchange
        // their row maxima through shared memory once per block; their partial sums meet at the end.  A warp whose
        // wait ran out keeps walking the items and blocks without touching them, so that the named barriers stay in step.
        constexpr int HK = BKV / PARTS, HO = HD / PARTS;
        static_assert(HK % 32 == 0 && (HO % 32 == 0 || HO == 16), "scores in loads of 32 columns; O in loads of 32 or 16 columns");
        constexpr int OC = HO >= 32 ? 32 : 16;       // columns of O per load
        constexpr float RESCALE_ABOVE = 8.f;         // log2 units: keep the old maximum while the new one is within 2^8 of it
        const int quarter = warp & 3, part = warp >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t o_addr = lane_base + O_COL + part * HO;
        bool ok = true;
        auto row_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + quarter), "n"(PARTS * 32) : "memory"); };
        int g = 0;
        for (int round = 0; round * G < total; ++round) {
            const int id = item_of_round(round);
            if (id >= total) continue;
            const TcItem I = get_item(round, id);
            const int n_blocks = I.n_blocks;
            if (n_blocks <= 0) continue;
            const int qpos0 = I.qpos0, key_lo = I.key_lo, key_hi = I.key_hi, n_tok = I.n_tok;
            const int qpos = qpos0 + (r >> p.pack_shift);
            float m_used = -INFINITY, l_run = 0.f;
            for (int j = 0; j < n_blocks; ++j) {
                const int jj = g + j;
                const int s = jj % S_BUFS;
                const int kb0 = (I.blk_lo + j) * BKV;
                const int k0 = kb0 + part * HK;                            // first key of this thread's part of the block
                if (ok) ok = mbar_wait(bar(S_FULL + s), (jj / S_BUFS) & 1, abort_flag, p.status);
                ok = __all_sync(0xffffffffu, ok);                          // tensor-memory loads and stores are warp-wide
                float x[HK];
                float mx = -INFINITY;
                if (ok) {
                    tc_fence_after();
                    const bool need_mask = (kb0 + BKV - 1 > qpos0) || (kb0 + BKV > key_hi) || kb0 < key_lo ||
                                           (p.window > 0 && kb0 <= qpos0 + n_tok - 1 - p.window);
                    // the row's scores of this part of the block, once, into registers (masked)
                    {
                        uint32_t v[HK];
#pragma unroll
                        for (int c = 0; c < HK; c += 32) tmem_ld32(lane_base + s * 128 + part * HK + c, v + c);
                        tmem_ld_wait();                                   // one wait for all of the row's loads
#pragma unroll
                        for (int i = 0; i < HK; ++i) x[i] = __uint_as_float(v[i]);          // raw scores: the scale goes into the exponent's FMA
                    }
                    if (need_mask) {
                        // the keys a row sees are an interval: one subtraction and one unsigned comparison per score
                        const int first = max(key_lo, p.window > 0 ? qpos - p.window + 1 : 0) - k0;
                        const unsigned n_vis = (unsigned)max(0, min(qpos + 1, key_hi) - k0 - first);
#pragma unroll
                        for (int i = 0; i < HK; ++i) x[i] = (unsigned)(i - first) < n_vis ? x[i] : -INFINITY;
                    }
                    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < HK; i += 4) {
                        mx0 = fmaxf(mx0, x[i]); mx1 = fmaxf(mx1, x[i + 1]); mx2 = fmaxf(mx2, x[i + 2]); mx3 = fmaxf(mx3, x[i + 3]);
                    }
                    mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;         // the scale is positive: it commutes with the maximum
                }
                xchg[((j & 1) * PARTS + part) * ROWS + r] = mx;
                row_sync();
                float m_blk = mx;
#pragma unroll
                for (int q = 0; q < PARTS; ++q) m_blk = fmaxf(m_blk, xchg[((j & 1) * PARTS + q) * ROWS + r]);
                if (!ok) continue;
                // The reference maximum only moves when the block's maximum exceeds it by more than 2^8 (or it was
                // still -inf): then everything accumulated so far, O in tensor memory included, is rescaled.  All
                // threads of a row see the same numbers and take the same decision.
                const bool move = m_blk > m_used + RESCALE_ABOVE || (m_used == -INFINITY && m_blk > -INFINITY);
                if (__any_sync(0xffffffffu, move)) {
                    const float corr = move ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_blk)) : 1.f;
                    if (j > 0) {                                          // O holds the products of the item's blocks 0..j-1
                        ok = __all_sync(0xffffffffu, mbar_wait(bar(O_FULL + (jj - 1) % S_BUFS), ((jj - 1) / S_BUFS) & 1, abort_flag, p.status));
                        if (ok) {
                            tc_fence_after();
#pragma unroll
                            for (int c = 0; c < HO; c += OC) {
                                uint32_t v[32];
                                if (OC == 32) tmem_ld32(o_addr + c, v); else tmem_ld16(o_addr + c, v);
                                tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < OC; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                                tmem_st16(o_addr + c, v);
                                if (OC == 32) tmem_st16(o_addr + c + 16, v + 16);
                            }
                            tmem_st_wait();
                        }
                    }
                    l_run *= corr;
                    if (move) m_used = m_blk;
                }
                if (!ok) continue;
                // P = 2^(x - m), its sum, and P as bfloat16 pairs written over S
                const float sub = (m_used == -INFINITY) ? 0.f : m_used;     // nothing visible yet: every x is -inf, P = 0
                float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
                for (int c = 0; c < HK; c += 32) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float e0 = fast_exp2(fmaf(x[c + i], p.scale_log2, -sub)), e1 = fast_exp2(fmaf(x[c + i + 1], p.scale_log2, -sub));
                        rs0 += e0; rs1 += e1;
                        __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
                        pk[i >> 1] = *reinterpret_cast<uint32_t*>(&b);
                    }
                    tmem_st16(lane_base + s * 128 + ((part * HK + c) >> 1), pk);
                }
                tmem_st_wait();
                l_run += rs0 + rs1;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(P_READY + s));
            }
            // the row's sum: all parts used the same reference maxima, so their partial sums simply add (in a fixed order)
            xchg[(2 * PARTS + part) * ROWS + r] = l_run;
            row_sync();
            l_run = 0.f;
#pragma unroll
            for (int q = 0; q < PARTS; ++q) l_run += xchg[(2 * PARTS + q) * ROWS + r];
            if (ok) ok = mbar_wait(bar(O_FULL + (g + n_blocks - 1) % S_BUFS), ((g + n_blocks - 1) / S_BUFS) & 1, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            // Normalised and rounded, the thread's part of its row goes to the warp's staging rows in shared memory
            // (16-byte chunks, swizzled by the row).  Whole tiles of 64 dims per part then leave through the TMA unit:
            // the staging rows are laid out as the query tile is, one thread issues two stores, and nothing queues up
            // in front of the other warps' memory instructions.  (Stored straight from the registers, every lane of
            // an instruction hit a line of its own, 256 lines per warp, and for as long as that took the MMA thread
            // could not issue the next item's first Q K^T: they share the queue to the memory pipes.)  A sequence's
            // last, partial tile is read back with consecutive lanes on consecutive chunks of a row and stored row by
            // row, because the rows after it in the buffer belong to the next sequence.  The barriers among the
            // softmax warps are taken by all of them, also by a warp whose wait ran out.
            constexpr int CH = HO / 8;                                 // 16-byte chunks per row part
            constexpr int PITCH = HO * 2, ROWS_PER_LINE = 128 / PITCH > 0 ? 128 / PITCH : 1;
            const bool tma_out = HO == 64 && p.out_by_tma;
            const bool tile_by_tma = tma_out && I.n_tok == p.tokens_per_cta;
            uint8_t* mine = stage_out + (size_t)warp * 32 * PITCH;
            if (tma_out) {
                if (warp == 0 && lane == 0) tma_store_wait_read();       // the store of the item before has read the staging rows
                asm volatile("bar.sync 5, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
            }
            if (ok) {
                tc_fence_after();
                // the whole of this thread's part of the row leaves tensor memory first, so that the next item's P V
                // may start while the result is normalised and stored
                uint32_t v[HO];
#pragma unroll
                for (int c = 0; c < HO; c += OC) {                         // warp-collective: rows beyond the tile load too
                    if (OC == 32) tmem_ld32(o_addr + c, v + c); else tmem_ld16(o_addr + c, v + c);
                }
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(O_EMPTY));
                const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    uint32_t w[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2 * u]) * inv, __uint_as_float(v[8 * c + 2 * u + 1]) * inv);
                        w[u] = *reinterpret_cast<uint32_t*>(&b);
                    }
                    *reinterpret_cast<uint4*>(mine + lane * PITCH + ((c ^ ((lane / ROWS_PER_LINE) & (CH - 1))) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            if (tile_by_tma) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 6, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
                if (ok && warp == 0 && lane == 0) {
#pragma unroll
                    for (int h = 0; h < PARTS; ++h)
                        tma_store_3d(&map_out, smem_u32(stage_out) + h * 4 * 32 * PITCH, h * 64, I.head0, I.row0 + I.q_off);
                    tma_store_commit();
                }
            } else if (ok) {
                __syncwarp();
#pragma unroll
                for (int k = 0; k < CH; ++k) {
                    const int lr = k * (32 / CH) + lane / CH, c = lane % CH;   // row of the warp's 32, chunk of the row part
                    const int rr = quarter * 32 + lr;
                    const uint4 val = *reinterpret_cast<const uint4*>(mine + lr * PITCH + ((c ^ ((lr / ROWS_PER_LINE) & (CH - 1))) << 4));
                    if (rr < I.n_rows)
                        *reinterpret_cast<uint4*>(p.out + (size_t)(I.row0 + I.q_off + (rr >> p.pack_shift)) * p.out_stride +
                                                  (I.head0 + (rr & (p.pack - 1))) * HD + part * HO + c * 8) = val;
                }
                __syncwarp();                                              // the rows are read before the next item writes them
            }
            g += n_blocks;
        }
    }
    if (threadIdx.x == 0) tma_store_wait_all();                 // thread 0 (softmax warp 0, lane 0) issued the result stores
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

__host__ __device__ inline int pack_of(int group) {
    int p = 1;
    while (p < 16 && group % (2 * p) == 0) p *= 2;
    return p;
}

// 3-D map of the query part of the projection buffer: (head dim, head, token), box 64 x pack x (128 / pack).
int q_map(const void* q, long q_stride, long tokens, int n_q, int hd, int pack, CUtensorMap* out) {
    using namespace rs_tma;
    EncodeTiledFn enc = get_encoder();
    if (!enc) return (int)cudaErrorNotSupported;
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)n_q, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)pack, (cuuint32_t)(ROWS / pack)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

struct QMapKey { const void* q; long stride, tokens; int n_q, hd, pack; };
std::vector<std::pair<QMapKey, CUtensorMap>> g_qmaps;
std::mutex g_qmaps_mutex;

int cached_q_map(const void* q, long q_stride, long tokens, int n_q, int hd, int pack, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_qmaps_mutex);
    for (auto& e : g_qmaps)
        if (e.first.q == q && e.first.stride == q_stride && e.first.tokens == tokens && e.first.n_q == n_q && e.first.hd == hd &&
            e.first.pack == pack) { *out = e.second; return 0; }
    CUtensorMap m;
    int rc = q_map(q, q_stride, tokens, n_q, hd, pack, &m);
    if (rc) return rc;
    if (g_qmaps.size() > 64) g_qmaps.clear();
    g_qmaps.push_back({QMapKey{q, q_stride, tokens, n_q, hd, pack}, m});
    *out = m;
    return 0;
}

// 5-d map of the cache: (64 dims, key within a group of 8, half of the head, group of the page, block = (page * 2 + K|V) *
// n_kv + kv head); one box is a page's keys (or values) of one kv head.  Returns non-zero if the driver does not take it.
int page_map(const void* cache, int num_pages, int n_kv, int page_size, int hd, CUtensorMap* out) {
    using namespace rs_tma;
    EncodeTiledFn enc = get_encoder();
    if (!enc) return 1;
    const cuuint64_t row = (cuuint64_t)hd * 2;
    cuuint64_t dims[5] = {64, 8, (cuuint64_t)(hd / 64), (cuuint64_t)(page_size / 8), (cuuint64_t)num_pages * 2 * n_kv};
    cuuint64_t strides[4] = {row, 128, 8 * row, (cuuint64_t)page_size * row};
    cuuint32_t box[5] = {64, 8, (cuuint32_t)(hd / 64), (cuuint32_t)(page_size / 8), 1};
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

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const CUtensorMap& mo, const TcParams& p, int n_work, cudaStream_t s) {
    constexpr int smem = (1 + 2 * KV_STAGES) * (HD / 64) * 128 * 128 + 1024 + 8 * 20 + 256 + 3 * PARTS * ROWS * 4 +
                         LOCAL_ITEMS * (int)sizeof(TcItem) + 1024 + ROWS * HD * 2;
    auto kern = prefill_attention_tc_kernel<HD>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const long total = (long)n_work * p.n_kv * (p.group / p.pack);
    const int grid = (int)(total < rs_tma::sm_count() ? total : rs_tma::sm_count());      // one CTA per SM; each walks its items
    return rs_launch_pdl(kern, dim3(grid), dim3(THREADS), (size_t)smem, s, mq, mkv, mo, p);
}
}  // namespace

RS_EXPORT int rs_attention_prefill_tc_supported(int n_q, int n_kv, int hd, int page_size) {
    if (n_kv <= 0 || n_q % n_kv) return 0;
    if (hd != 64 && hd != 128) return 0;
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// TMA loads per cache page (keys and values together) in the most recent launch: 2 with the 5-d map.
RS_EXPORT int rs_attention_prefill_tc_loads_per_page() { return g_last_loads_per_page; }

// Query tokens per CTA: the host cuts each sequence's queries into tiles of this many.
RS_EXPORT int rs_attention_prefill_tc_q_per_cta(int n_q, int n_kv) { return ROWS / pack_of(n_q / n_kv); }

// q: the projection buffer [q_rows, q_stride] whose first n_q * hd columns of every row are the queries.
RS_EXPORT int rs_attention_prefill_tc(const void* q, long q_stride, long q_rows, void* out, long out_stride, const void* cache,
                                      long page_stride, int num_pages, int page_size, const int* block_table,
                                      int table_stride, const int* q_start, const int* kv_len, const int* work, int n_work,
                                      int n_q, int n_kv, int hd, int window, float scale, int* status, void* stream) {
    if (n_work <= 0) return 0;
    if (!rs_attention_prefill_tc_supported(n_q, n_kv, hd, page_size) || (q_stride % 8) || (out_stride % 8) || ((long)q & 15) ||
        ((long)out & 15) || ((long)cache & 15) || page_stride != (long)2 * n_kv * page_size * hd)
        return (int)cudaErrorInvalidValue;
    TcParams p;
    p.out = (__nv_bfloat16*)out; p.out_stride = out_stride; p.page_size = page_size; p.num_pages = num_pages;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work; p.n_work = n_work;
    p.n_q = n_q; p.n_kv = n_kv; p.group = n_q / n_kv; p.pack = pack_of(p.group); p.tokens_per_cta = ROWS / p.pack;
    p.pack_shift = 0;
    while ((1 << p.pack_shift) < p.pack) ++p.pack_shift;
    p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    CUtensorMap mq, mkv, mo;
    int rc = cached_q_map(q, q_stride, q_rows, n_q, hd, p.pack, &mq);
    if (rc) return rc;
    // the result as (head dim, head, token), the queries' layout; its rows are the queries' rows
    p.out_by_tma = hd == 128 && cached_q_map(out, out_stride, q_rows, n_q, hd, p.pack, &mo) == 0;
    if (!p.out_by_tma) mo = mq;
    p.one_load_per_page = cached_page_map(cache, num_pages, n_kv, page_size, hd, &mkv) == 0;
    if (!p.one_load_per_page) {
        rc = rs_tma::get_map(cache, (long)num_pages * 2 * n_kv * page_size, hd, hd, 8, &mkv);
        if (rc) return rc;
    }
    g_last_loads_per_page = p.one_load_per_page ? 2 : 2 * (hd / 64) * (page_size / 8);
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch<64>(mq, mkv, mo, p, n_work, s);
    return launch<128>(mq, mkv, mo, p, n_work, s);
}
