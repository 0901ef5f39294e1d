// Causal grouped-query flash attention for prompts on the tcgen05 tensor cores (bfloat16).
//
// One CTA owns 128 query rows of one head of one sequence and walks the sequence's cache in
// tiles of 64 keys (one cache block) up to the causal limit.  Per tile:
//   S = Q·K^T        tcgen05.mma, M = 128, N = 64, K = d, accumulator in TMEM;
//   softmax          four warps, one thread per query row: tcgen05.ld of the row's 64 scores,
//                    scale, mask, running maximum and sum in float32 (exp2 of log2e-scaled
//                    scores); P is written as bfloat16 into shared memory in the swizzled
//                    K-major layout that the tensor core reads;
//   O += P·V         tcgen05.mma, M = 128, N = d, K = 64 keys, accumulating in TMEM; V is used as
//                    it lies in the cache ([key][d], i.e. MN-major for the B operand).
// The running maximum of a row is only raised when the new maximum exceeds it by more than 2^8;
// then the row's O in TMEM is rescaled (tcgen05.ld, multiply, tcgen05.st).  Until then P is
// taken relative to the older maximum, which gives the same quotient O / l.
// Q, K and V tiles arrive by TMA (128-byte swizzle).  S is double-buffered in tensor memory: the scores of
// tile i + 1 are computed while the softmax warps work on tile i, and P·V of tile i runs while they work on
// tile i + 1.  So K(i + 1) is needed at the same time as V(i), and the two travel together under one barrier;
// K(0) comes with Q.  V has two slots and K three: P(i) is written over K(i), which therefore stays until
// P·V of tile i is through, while K(i + 1) is in use and K(i + 2) is landing.  With K and V of a tile in one
// slot of two, the copy of tile i + 2 could only start after P·V of tile i, and its latency lay on every
// tile's path.  mbarriers order producer, MMA issuer and softmax warps; every wait is bounded.
// Formulas: src/HyMT2Sharp/Ops.cs:359-455 (scores, kv head = head / group), :198-325 (softmax
// over the visible keys), :535-595 (combine).  A query at position p sees keys
// [max(0, p - window + 1), p].
// Takes head sizes 64 and 128 and cache blocks of 64 tokens; other shapes stay with the general kernel.
#include "tc_common.cuh"

namespace {

constexpr int Q_ROWS = 128, KEY_TILE = 64, NUM_THREADS = 256, KV_STAGES = 2, K_SLOTS = 3;
// The numbers of the barrier protocol (why these: see the kernel).  hymt2_attention_prefill_tc_protocol hands them to the
// test that explores every interleaving of the roles, so that the protocol explored is the one compiled here.
constexpr int P_BARS = K_SLOTS;      // "P of tile i is written": one barrier per K slot, tile mod P_BARS
constexpr int O_BARS = 3;            // "P·V of tile i is through": tile mod O_BARS
constexpr int S_BUFFERS = 2;         // score buffers in tensor memory, each with a barrier
constexpr int STAGE_HOLDERS = 2;     // who must let go of a K/V stage before it is filled again: P·V and the score issuer
constexpr int NUM_BARS = 2 * KV_STAGES + 1 + O_BARS + S_BUFFERS + P_BARS;

struct PrefillParams {
    __nv_bfloat16* out;        // [T, nh * d]
    const int* block_table;
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    int table_stride, nh, nkv, window;
    int batch, qtiles, sm_count;
    float scale_log2;          // scale * log2(e)
    int* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}


template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillParams p) {
    constexpr int D_BOXES = D / 64;                         // TMA boxes of 64 elements along d
    constexpr int Q_BYTES = Q_ROWS * D * 2, KV_TILE_BYTES = KEY_TILE * D * 2, P_BYTES = Q_ROWS * KEY_TILE * 2;
    // P of a tile (16 KB) takes the place of the tile's K (free once S is computed): a K slot holds the larger of the two
    constexpr int K_SLOT_BYTES = KV_TILE_BYTES >= P_BYTES ? KV_TILE_BYTES : P_BYTES;
    constexpr int BARS_OFFSET = Q_BYTES + K_SLOTS * K_SLOT_BYTES + KV_STAGES * KV_TILE_BYTES;
    constexpr int TMEM_COLS = 256;                          // S of even tiles: columns [0, 64), of odd tiles [64, 128); O: [128, 128 + D)
    constexpr uint32_t S_COL = 0, O_COL = 128;
    // D float32, A and B bfloat16; S: both K-major, N = 64; O: B is MN-major, N = D
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KEY_TILE >> 3) << 17) | ((uint32_t)(Q_ROWS >> 4) << 24);
    constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(Q_ROWS >> 4) << 24);

    // No static shared memory: the dynamic part then starts on a 1 KB boundary, which the swizzled tiles need,
    // and two CTAs of 112 KB fit an SM.  Barriers and the two words lie behind the tiles.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + BARS_OFFSET);
    uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(smem_raw + BARS_OFFSET + NUM_BARS * 8);
    int& abort_s = *reinterpret_cast<int*>(smem_raw + BARS_OFFSET + NUM_BARS * 8 + 4);

    // The last query tiles of a prompt walk the most keys: CTAs are numbered by falling query tile, so the long
    // ones start first and the short ones fill the gaps.  When all CTAs fit on the SMs at once (two each), the
    // ones beyond the first per SM are numbered by RISING length instead: the SM that got the longest tile also
    // gets the shortest.
    int n = blockIdx.x;
    const int total = gridDim.x, per_qtile = p.nh * p.batch;
    if (total <= 2 * p.sm_count && n >= p.sm_count) n = p.sm_count + (total - 1 - n);
    const int qtile = p.qtiles - 1 - n / per_qtile, head = (n % per_qtile) % p.nh, b = (n % per_qtile) / p.nh;
    const int slot = p.slot_ids[b];
    const int tok0 = p.cu_seqlens[b], T_b = p.cu_seqlens[b + 1] - tok0;
    if (slot < 0 || qtile * Q_ROWS >= T_b) return;
    const int kv_len = p.kv_lens[b], start = kv_len - T_b;
    const int kvh = head / (p.nh / p.nkv);
    const int rows_here = min(Q_ROWS, T_b - qtile * Q_ROWS);
    const int first_pos = start + qtile * Q_ROWS, last_pos = first_pos + rows_here - 1;
    const int tile_begin = p.window > 0 ? max(0, first_pos - p.window + 1) / KEY_TILE : 0;
    const int tile_end = last_pos / KEY_TILE + 1;
    const int num_tiles = tile_end - tile_begin;

    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {   // never seen; a swizzled tile off its boundary would give wrong numbers, not a fault
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 119);
        return;
    }
    const uint32_t q_smem = base, k_smem = q_smem + Q_BYTES, v_smem = k_smem + K_SLOTS * K_SLOT_BYTES;
    auto k_of = [&](int tile) { return k_smem + (tile % K_SLOTS) * K_SLOT_BYTES; };   // K of a tile, then its P
    auto v_of = [&](int tile) { return v_smem + (tile % KV_STAGES) * KV_TILE_BYTES; };
    const uint32_t kv_full = smem_u32(&bars[0]), kv_empty = smem_u32(&bars[KV_STAGES]);
    const uint32_t q_full = smem_u32(&bars[2 * KV_STAGES]), o_full = q_full + 8;
    const uint32_t s_full = o_full + 8 * O_BARS, p_full = s_full + 8 * S_BUFFERS;   // s_full: one for even, one for odd tiles
    // Why these counts.  A parity cannot tell a barrier's phase from the one two later, so no reader may fall two
    // phases behind a barrier, however long its thread is kept from running.  S(j) is only issued once P·V of tile
    // j - 3 is through: with P's barrier of tile j the one of tile j - 3, P(j) cannot be announced before the
    // P·V issuer has taken P(j - 3); with two barriers it could, while that thread still waited for P(j - 2)'s
    // predecessor: one CTA in tens of thousands then waited for ever (status 114, met with 32 heads and 16,384
    // tokens in a step).  O's barrier has three for the score issuer's sake, who reads P·V(j - 3) after issuing S(j - 1),
    // and the copies' stages are held by both their readers (kv_empty below).
    volatile int* abort_flag = &abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < KV_STAGES; s++) {
            mbar_init(kv_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, STAGE_HOLDERS);   // P·V of the tile is through, and the score issuer has seen the copy land
        }
        mbar_init(q_full, 1);
        for (int t = 0; t < S_BUFFERS; t++) mbar_init(s_full + 8 * t, 1);
        for (int t = 0; t < O_BARS; t++) mbar_init(o_full + 8 * t, 1);
        for (int t = 0; t < P_BARS; t++) mbar_init(p_full + 8 * t, 128);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---- producer: Q with K(0), then K(i + 1) with V(i) ---------------------------------------
        const int* table = p.block_table + (size_t)slot * p.table_stride;
        auto cache_row = [&](int tile) { return (table[tile_begin + tile] * p.nkv + kvh) * KEY_TILE; };
        mbar_expect_tx(q_full, Q_BYTES + KV_TILE_BYTES);
        for (int x = 0; x < D_BOXES; x++) {
            tma_load_2d(q_smem + x * (Q_ROWS * 128), &map_q, q_full, head * D + x * 64, tok0 + qtile * Q_ROWS);
            tma_load_2d(k_of(0) + x * (KEY_TILE * 128), &map_k, q_full, x * 64, cache_row(0));
        }
        int issued = 0;
        for (int i = 0; i < num_tiles; i++) {
            const int s = i % KV_STAGES;
            // P·V of tile i - 2 is through: V's slot is free, and so is the slot of K(i - 2), which takes K(i + 1)
            if (!mbar_wait(kv_empty + 8 * s, ((i / KV_STAGES) & 1) ^ 1, abort_flag, p.status, 111)) break;
            const bool more = i + 1 < num_tiles;
            mbar_expect_tx(kv_full + 8 * s, (more ? 2 : 1) * KV_TILE_BYTES);
            const int v_row = cache_row(i), k_row = more ? cache_row(i + 1) : 0;
            const uint32_t k_dst = k_of(i + 1), v_dst = v_of(i);
            for (int x = 0; x < D_BOXES; x++) {
                if (more) tma_load_2d(k_dst + x * (KEY_TILE * 128), &map_k, kv_full + 8 * s, x * 64, k_row);
                tma_load_2d(v_dst + x * (KEY_TILE * 128), &map_v, kv_full + 8 * s, x * 64, v_row);
            }
            issued = i + 1;
        }
        if (*abort_flag) {   // nothing may still be landing when the CTA leaves
            for (uint32_t t = 0; t < (1u << 16) && !mbar_try_wait(q_full, 0); t++) {}
            for (int i = max(0, issued - KV_STAGES); i < issued; i++)
                for (uint32_t t = 0; t < (1u << 16) && !mbar_try_wait(kv_full + 8 * (i % KV_STAGES), (i / KV_STAGES) & 1); t++) {}
        }
    } else if (warp == 1 && lane == 0) {
        // ---- first MMA issuer: the scores, one tile ahead of the softmax warps ---------------------------
        // Two threads issue, each with a wait or two and a dozen instructions a tile: one thread doing both was
        // the slowest link of the chain.
        // The descriptors of slot 0 once; per instruction only constants are added (the address sits in the
        // low bits in units of 16 bytes, and shared memory is too small to carry out of them).
        const uint64_t q_desc = desc_k_major(q_smem), k_desc0 = desc_k_major(k_smem);
        constexpr uint64_t K_STEP = K_SLOT_BYTES >> 4;
        // S(i) = Q K(i)^T over d in steps of 16, into the S buffer of i's parity.  K(i) has landed; the buffer's
        // last scores, those of tile i - 2, have been read: the softmax warps read a tile's scores before they
        // announce its P, and P(i - 2) is waited for first.
        auto issue_scores = [&](int i) {
            const uint64_t kd = k_desc0 + (i % K_SLOTS) * K_STEP;
#pragma unroll
            for (int k = 0; k < D / 16; k++) {
                const uint64_t q_off = ((k / 4) * (Q_ROWS * 128) + (k % 4) * 32) >> 4, k_off = ((k / 4) * (KEY_TILE * 128) + (k % 4) * 32) >> 4;
                umma_bf16(tmem_base + S_COL + 64 * (i & 1), q_desc + q_off, kd + k_off, IDESC_S, k > 0 ? 1u : 0u);
            }
            umma_commit(s_full + 8 * (i & 1));
        };
        bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 112);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_scores(0);
        }
        for (int i = 0; ok && i + 1 < num_tiles; i++) {
            // K(i + 1) has landed (with V(i))
            if (!mbar_wait(kv_full + 8 * (i % KV_STAGES), (i / KV_STAGES) & 1, abort_flag, p.status, 113)) break;
            mbar_arrive(kv_empty + 8 * (i % KV_STAGES));   // seen: the stage may be filled again once P·V of tile i is through too
            // P·V of tile i - 2 is through.  The softmax warps, who wait for P·V of the tile before theirs only when a
            // maximum rose, then never meet a barrier more than one phase behind (a parity cannot tell two apart).
            if (i >= 2 && !mbar_wait(o_full + 8 * ((i - 2) % O_BARS), ((i - 2) / O_BARS) & 1, abort_flag, p.status, 108)) break;
            // the scores of tile i - 1 have been read: their buffer takes those of tile i + 1
            if (i >= 1 && !mbar_wait(p_full + 8 * ((i - 1) % P_BARS), ((i - 1) / P_BARS) & 1, abort_flag, p.status, 118)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_scores(i + 1);
        }
    } else if (warp == 2 && lane == 0) {
        // ---- second MMA issuer: O += P V once the softmax warps have written P (and rescaled O where a maximum rose)
        const uint64_t p_desc0 = desc_k_major(k_smem), v_desc0 = desc_mn_major(v_smem, KEY_TILE * 128);
        constexpr uint64_t K_STEP = K_SLOT_BYTES >> 4, V_STEP = KV_TILE_BYTES >> 4;
        for (int i = 0; i < num_tiles; i++) {
            const int s = i % KV_STAGES;
            if (!mbar_wait(p_full + 8 * (i % P_BARS), (i / P_BARS) & 1, abort_flag, p.status, 114)) break;
            if (!mbar_wait(kv_full + 8 * s, (i / KV_STAGES) & 1, abort_flag, p.status, 109)) break;   // V(i) has landed
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t pd = p_desc0 + (i % K_SLOTS) * K_STEP, vd = v_desc0 + s * V_STEP;
#pragma unroll
            for (int k = 0; k < KEY_TILE / 16; k++)
                umma_bf16(tmem_base + O_COL, pd + ((k * 32) >> 4), vd + ((k * (16 * 128)) >> 4), IDESC_O, (i > 0 || k > 0) ? 1u : 0u);
            umma_commit(kv_empty + 8 * s);
            umma_commit(o_full + 8 * (i % O_BARS));
        }
    } else if (warp >= 4) {
        // ---- softmax: one thread per query row; O stays in TMEM ------------------------------------
        const int quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int pos = first_pos + r;                                  // position of this row's query
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const bool row_ok = r < rows_here;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < num_tiles; i++) {
            if (!(ok = mbar_wait(s_full + 8 * (i & 1), (i >> 1) & 1, abort_flag, p.status, 115))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int key0 = (tile_begin + i) * KEY_TILE;
            float s[KEY_TILE];
            tmem_load32(lane_addr + S_COL + 64 * (i & 1), s);
            tmem_load32(lane_addr + S_COL + 64 * (i & 1) + 32, s + 32);
            // s stays unscaled: the scale (> 0) goes into the exponent's multiply-add; most tiles lie wholly
            // inside the row's visible range and need no mask
            // four running maxima (and four sums below): one chain of 64 dependent operations would leave
            // the thread waiting on each result, and only two such warps share a scheduler
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (row_ok && key0 >= lo && key0 + KEY_TILE - 1 <= pos) {
#pragma unroll
                for (int c = 0; c < KEY_TILE; c++) mx[c & 3] = fmaxf(mx[c & 3], s[c]);
            } else {
#pragma unroll
                for (int c = 0; c < KEY_TILE; c++) {
                    const int key = key0 + c;
                    s[c] = (row_ok && key >= lo && key <= pos) ? s[c] : -INFINITY;
                    mx[c & 3] = fmaxf(mx[c & 3], s[c]);
                }
            }
            float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
            // raise the row's maximum only when it grows by more than 2^8 (or at its first visible key)
            const bool raise = tile_max > m + 8.0f || (m == -INFINITY && tile_max > -INFINITY);
            const float corr = raise ? exp2f(m - tile_max) : 1.f;   // m = -inf: 0
            if (raise) m = tile_max;
            if (i > 0 && __any_sync(0xffffffffu, raise)) {
                // the O of the tiles so far is complete, then every row of the warp scales its own O
                if (!(ok = mbar_wait(o_full + 8 * ((i - 1) % O_BARS), ((i - 1) / O_BARS) & 1, abort_flag, p.status, 116))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c = 0; c < D; c += 16) {   // 16 columns at a time: the row's 64 scores are live in registers
                    float o[16];
                    tmem_load16(lane_addr + O_COL + c, o);
#pragma unroll
                    for (int j = 0; j < 16; j++) o[j] *= corr;
                    tmem_store16(lane_addr + O_COL + c, o);
                }
            }
            l *= corr;
            float psum[4] = {0.f, 0.f, 0.f, 0.f};
            // a row that has seen no key yet (m = -inf) has only masked scores: -inf * scale + 0 = -inf, exp2 gives 0
            const float neg_m = m == -INFINITY ? 0.f : -m;
            // P as bfloat16 into the swizzled K-major tile: row r, 16-byte chunk c8 at chunk (c8 ^ (r & 7))
            const uint32_t p_dst = k_of(i);
#pragma unroll
            for (int c8 = 0; c8 < KEY_TILE / 8; c8++) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    // the special-function unit is this kernel's scarcest resource: one instruction an element
                    // (exp2f brings a range fix-up of several more; -inf gives 0 either way, and P has 8 bits)
                    const float p0 = ex2_approx(fmaf(s[c8 * 8 + 2 * j], p.scale_log2, neg_m));
                    const float p1 = ex2_approx(fmaf(s[c8 * 8 + 2 * j + 1], p.scale_log2, neg_m));
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    psum[j] += p0 + p1;
                    packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                const uint32_t dst = p_dst + r * 128 + ((c8 ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]),
                             "r"(packed[2]), "r"(packed[3]) : "memory");
            }
            l += (psum[0] + psum[1]) + (psum[2] + psum[3]);
            // rows of V at and past the sequence's length were never written by this sequence: their
            // weight is 0, but 0 x (whatever bits lie there) must stay 0.  Only a sequence's last tile has
            // such rows; V of the tile must have landed before they are overwritten.
            if (key0 + KEY_TILE > kv_len &&
                !(ok = mbar_wait(kv_full + 8 * (i % KV_STAGES), (i / KV_STAGES) & 1, abort_flag, p.status, 110))) break;
            if (r < KEY_TILE && key0 + r >= kv_len) {
#pragma unroll
                for (int x = 0; x < D_BOXES; x++) {
                    const uint32_t rowp = v_of(i) + x * (KEY_TILE * 128) + r * 128;
#pragma unroll
                    for (int c = 0; c < 8; c++)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(rowp + c * 16), "r"(0) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(p_full + 8 * (i % P_BARS));
        }
        if (ok) ok = mbar_wait(o_full + 8 * ((num_tiles - 1) % O_BARS), ((num_tiles - 1) / O_BARS) & 1, abort_flag, p.status, 117);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = p.out + ((size_t)(tok0 + qtile * Q_ROWS + r) * p.nh + head) * D;
#pragma unroll
            for (int c = 0; c < D; c += 32) {
                float o[32];
                tmem_load32(lane_addr + O_COL + c, o);   // all lanes of the warp take part in the load
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        __nv_bfloat162 h[4];
#pragma unroll
                        for (int q = 0; q < 4; q++) h[q] = __floats2bfloat162_rn(o[j + 2 * q] * inv, o[j + 2 * q + 1] * inv);
                        *reinterpret_cast<uint4*>(dst + c + j) = *reinterpret_cast<uint4*>(h);
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, dim3 grid,
           cudaStream_t stream) {
    constexpr size_t kv_tile = KEY_TILE * D * 2, p_tile = Q_ROWS * KEY_TILE * 2;
    constexpr size_t smem = Q_ROWS * D * 2 + K_SLOTS * (kv_tile >= p_tile ? kv_tile : p_tile) + KV_STAGES * kv_tile +
                            NUM_BARS * 8 + 8;   // tiles, barriers, two words
    auto kernel = attention_prefill_tc_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { hymt2_set_error("attention_prefill_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);   // two CTAs an SM
        configured = true;
    }
    kernel<<<grid, NUM_THREADS, smem, stream>>>(mq, mk, mv, p);
    return hymt2_check_launch("attention_prefill_tc");
}

}  // namespace

// The numbers of the kernel's barrier protocol: out[0] stages of the K/V copies, [1] K slots, [2] barriers for "P written",
// [3] barriers for "P·V through", [4] holders of a stage, [5] score buffers.
HYMT2_API int hymt2_attention_prefill_tc_protocol(int* out) {
    static_assert(S_BUFFERS == 2, "the score buffers are addressed by a tile's parity");
    out[0] = KV_STAGES; out[1] = K_SLOTS; out[2] = P_BARS; out[3] = O_BARS; out[4] = STAGE_HOLDERS; out[5] = S_BUFFERS;
    return HYMT2_OK;
}

// out, q: [tokens, nh * d] bfloat16; k_cache, v_cache: one layer's planes [blocks][nkv][64][d] bfloat16.
HYMT2_API int hymt2_attention_prefill_tc(void* out, const void* q, const void* k_cache, const void* v_cache,
                                         long cache_blocks, const int* block_table, int table_stride, int block_tokens,
                                         const int* cu_seqlens, const int* slot_ids, const int* kv_lens, int batch,
                                         int tokens, int max_new_tokens, int nh, int nkv, int d, float scale, int window,
                                         int* status, cudaStream_t stream) {
    if (tokens == 0 || batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(d == 64 || d == 128, "attention_prefill_tc: head_dim %d is not taken (64 and 128 are)", d);
    HYMT2_REQUIRE(block_tokens == KEY_TILE, "attention_prefill_tc: cache blocks must hold %d tokens", KEY_TILE);
    HYMT2_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0 && batch <= 65535 && nh <= 65535, "attention_prefill_tc: bad sizes");
    HYMT2_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) &&
                  ((uintptr_t)out % 16 == 0), "attention_prefill_tc: tensors must be 16-byte aligned");
    HYMT2_REQUIRE(status != nullptr, "attention_prefill_tc: a status word is needed");
    CUtensorMap mq, mk, mv;
    const long cache_rows = cache_blocks * nkv * KEY_TILE;
    const bool ok = make_map(&mq, q, tokens, (long)nh * d, (long)nh * d, Q_ROWS) &&
                    make_map(&mk, k_cache, cache_rows, d, d, KEY_TILE) && make_map(&mv, v_cache, cache_rows, d, d, KEY_TILE);
    HYMT2_REQUIRE(ok, "attention_prefill_tc: cuTensorMapEncodeTiled refused the operands");
    const int qtiles = (max_new_tokens + Q_ROWS - 1) / Q_ROWS;
    HYMT2_REQUIRE((long)qtiles * nh * batch <= 2147483647L, "attention_prefill_tc: too many tiles");
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    PrefillParams p{(__nv_bfloat16*)out, block_table, cu_seqlens, slot_ids, kv_lens, table_stride, nh, nkv, window,
                    batch, qtiles, sms, scale * 1.4426950408889634f, status};
    dim3 grid((unsigned)(qtiles * nh * batch), 1, 1);
    return d == 128 ? launch<128>(mq, mk, mv, p, grid, stream) : launch<64>(mq, mk, mv, p, grid, stream);
}
