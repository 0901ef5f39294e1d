// Decode attention on the tcgen05 tensor cores (bfloat16, head_dim 128): one new token per
// sequence attends over its paged cache, with the KEYS on the 128-row side of the tensor core.
//
// A CTA owns (a chunk of 128 keys = two cache blocks, one kv head, one sequence):
//   S^T[key, head]   = K[128 keys, d] · Q^T[d, 16]      tcgen05.mma, M = 128, N = 16, K = d;
//   softmax          one thread per key: the key's scores for the g heads of the group come
//                    out of tensor memory, are scaled and masked; maximum and sum per head
//                    are reduced over the 128 threads in float32; P^T is written as
//                    bfloat16 into shared memory as the next product's B operand;
//   O^T[d, head]     = V^T[d, 128 keys] · P^T[keys, 16]  tcgen05.mma, M = d = 128, N = 16; V is
//                    used as it lies in the cache (MN-major A operand);
//   one thread per d writes the unnormalised partial (O^T, max, sum) of the chunk.
// The K and V blocks of the chunk arrive by TMA, all in flight at once, so a step's cache
// traffic is streamed at full tile size whatever the batch is; the tensor core sees the
// cache once per kv head (all heads of the group share it).  The warps that computed a
// row's last chunk fold all chunks of the row in chunk order, each for its quarter of d.
// Formulas: src/HyMT2Sharp/Ops.cs:462-532 (the reference's fused decode attention).
#include "tc_common.cuh"

namespace {

constexpr int CHUNK = 128, BLOCK_KEYS = 64, D = 128, NQ = 16;
constexpr int NUM_THREADS = 352;   // warp 0 TMA, warp 1 MMAs of the scores, warps 2-5 and 6-9: two softmax groups that take turns, warp 10 MMAs of the sums

struct DecodeTcParams {
    __nv_bfloat16* out;        // [rows, nh * d]
    const int* block_table;
    const int* slot_ids;
    const int* kv_lens;
    float* part_acc;           // [rows, nh, max_splits, d]
    float* part_ml;            // [rows, nh, max_splits, 4 quarters of d, 2]  (maximum in log2 units, sum)
    int* counters;             // [rows, nkv, 4 quarters of d]
    int table_stride, nh, nkv, window, max_splits, rows;
    float scale_log2;
    int* status;
};

constexpr int STAGES = 3;        // chunks whose keys and values are in shared memory or on their way
constexpr int MAX_ITEMS = 64;    // chunks that one CTA holds in shared memory at a time (one round)
constexpr int MAX_ROWS = 512;    // sequences in one launch
constexpr int MAX_CHUNKS = 2048; // chunks of one sequence (262,144 positions); an item keeps chunk numbers in 16 bits
static_assert(MAX_CHUNKS <= 32767, "an item keeps chunk numbers in 16 bits");
constexpr int FOLD_BATCH = 20;   // chunks whose partials are loaded together when a row is folded

template <int G>   // query heads per kv head that the softmax loops cover (the group size rounded up)
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, DecodeTcParams p) {
    // Persistent: a CTA takes the work items (sequence, kv head, chunk) w = blockIdx.x, + gridDim.x, ...
    // Per stage of shared memory: K [d half][128 keys x 128 B], V [key block][d half][64 keys x 128 B],
    // Q [d half][16 x 128 B], P^T [key block][16 x 128 B].  Two (S^T, O^T) pairs alternate in tensor memory,
    // so the tensor core computes the next chunk's scores while the softmax warps work on this one.
    constexpr int K_BYTES = CHUNK * D * 2, V_BYTES = CHUNK * D * 2, Q_BYTES = NQ * D * 2, P_BYTES = 2 * NQ * 128;
    constexpr int STAGE_BYTES = K_BYTES + V_BYTES + Q_BYTES + P_BYTES;
    constexpr int HALF_K = CHUNK * 128, BOX = BLOCK_KEYS * 128;
    constexpr uint32_t TMEM_COLS = 64;   // buffer t: S^T at 32 t, O^T at 32 t + 16
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NQ >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    constexpr uint32_t IDESC_O = IDESC_S | (1u << 15);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[3 * STAGES + 8];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ float red_max[2][4][NQ], red_sum[2][4][NQ];
    __shared__ int n_items_s;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    auto k_of = [&](int s) { return base + s * STAGE_BYTES; };
    auto v_of = [&](int s) { return base + s * STAGE_BYTES + K_BYTES; };
    auto q_of = [&](int s) { return base + s * STAGE_BYTES + K_BYTES + V_BYTES; };
    auto p_of = [&](int s) { return base + s * STAGE_BYTES + K_BYTES + V_BYTES + Q_BYTES; };
    const uint32_t kq_full = smem_u32(&bars[0]), v_full = kq_full + 8 * STAGES, stage_free = kq_full + 16 * STAGES;
    const uint32_t s_done = smem_u32(&bars[3 * STAGES]), p_ready = s_done + 16, o_done = s_done + 32, tmem_free = s_done + 48;
    volatile int* abort_flag = &abort_s;
    const int g = p.nh / p.nkv;

    // Three things at the same time: thread 0 sets up the barriers, warp 1 allocates tensor memory, and
    // warps 2 and 3 find the items of this CTA.  The items' facts come from global memory (slots, lengths,
    // block numbers) and are read BEFORE the wait for the kernel in front (see the producer): lengths,
    // tables and every cache block but the one of the newest position were written by kernels that are
    // long complete.
    //
    // Only chunks that hold visible keys are items: warp 2 counts them row by row (a running sum in shared
    // memory), so w = blockIdx.x, + gridDim.x, ... below the total is always a real chunk and every CTA
    // gets the same number of them, give or take one.
    struct Item { int b, kvh, kv_len, pos, lo, chunk_begin, blocks_here, first_block, row0, row1; short split, folder; };
    __shared__ Item items[MAX_ITEMS];
    __shared__ int row_first[MAX_ROWS + 1], row_slot[MAX_ROWS], row_len[MAX_ROWS];
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // A CTA keeps MAX_ITEMS items in shared memory at a time; if it has more (many long sequences), it goes
    // through them in rounds: the barriers are set up again, the next items are found, the pipeline refills.
    for (int round = 0;; round++) {
        if (threadIdx.x == 0) {
            for (int s = 0; s < STAGES; s++) {
                mbar_init(kq_full + 8 * s, 1);
                mbar_init(v_full + 8 * s, 1);
                mbar_init(stage_free + 8 * s, 1);
            }
            for (int t = 0; t < 2; t++) {
                mbar_init(s_done + 8 * t, 1);
                mbar_init(p_ready + 8 * t, 128);
                mbar_init(o_done + 8 * t, 1);
                mbar_init(tmem_free + 8 * t, 128);
            }
            abort_s = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            if (round == 0) {
                asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_k) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_v) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_q) : "memory");
            }
        }
        if (warp == 2 || warp == 3) {
            if (warp == 2 && round == 0) {
                int running = 0;
                for (int r0 = 0; r0 < p.rows; r0 += 32) {
                    const int r = r0 + lane;
                    int mine = 0;
                    if (r < p.rows) {
                        const int slot = p.slot_ids[r], len = p.kv_lens[r];
                        const int pos = len - 1, lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
                        row_slot[r] = slot;
                        row_len[r] = len;
                        if (slot >= 0 && len > 0) mine = (pos / CHUNK + 1 - lo / CHUNK) * p.nkv;
                    }
                    int incl = mine;
    #pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int up = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += up;
                    }
                    if (r < p.rows) row_first[r + 1] = running + incl;
                    running += __shfl_sync(0xffffffffu, incl, 31);
                }
                if (lane == 0) row_first[0] = 0;
            }
            asm volatile("bar.sync 3, 64;" ::: "memory");
            const int total = row_first[p.rows];
            const int w = blockIdx.x + (round * MAX_ITEMS + (int)threadIdx.x - 64) * gridDim.x;
            if (w < total) {
                int b = 0;                                        // the last row whose first item is <= w
                for (int step = MAX_ROWS / 2; step > 0; step >>= 1)
                    if (b + step < p.rows && row_first[b + step] <= w) b += step;
                Item it;
                it.b = b;
                it.kv_len = row_len[b];
                it.pos = it.kv_len - 1;
                it.lo = p.window > 0 ? max(0, it.pos - p.window + 1) : 0;
                const int chunks = it.pos / CHUNK + 1 - it.lo / CHUNK, rem = w - row_first[b];
                it.kvh = rem / chunks;
                it.split = it.lo / CHUNK + rem % chunks;
                // Who folds the row: the holder of its last chunk, unless the rows' chunks fall on the same CTAs again and
                // again (the number of chunks and of CTAs share a divisor: 18 chunks a row on 144 CTAs would leave all the
                // folding to 8 CTAs, measured 57 against 34 us); then the holder of a chunk that differs from row to row.
                // With more items than a CTA holds at once (rounds) it stays the last chunk: its holder never waits
                // for a chunk of a later round.
                {
                    int gcd = (int)gridDim.x, rest = chunks;
                    while (rest) { const int x = gcd % rest; gcd = rest; rest = x; }
                    const bool one_round = total <= MAX_ITEMS * (int)gridDim.x;
                    it.folder = (one_round && gcd > 2) ? it.lo / CHUNK + (b * p.nkv + it.kvh) % chunks : it.pos / CHUNK;
                }
                it.chunk_begin = it.split * CHUNK;
                it.blocks_here = min(2, (it.pos - it.chunk_begin) / BLOCK_KEYS + 1);
                // With a window, the chunk's first block may lie wholly below the oldest visible key; the cache has
                // then handed that block back and its table entry is -1.  Such a block is not loaded at all (its
                // keys are masked and its rows of V are zeroed in shared memory), and its table entry is not read.
                it.first_block = it.lo >= it.chunk_begin + BLOCK_KEYS ? 1 : 0;
                const int* table = p.block_table + (size_t)row_slot[b] * p.table_stride + it.chunk_begin / BLOCK_KEYS;
                it.row0 = it.first_block == 0 ? (table[0] * p.nkv + it.kvh) * BLOCK_KEYS : 0;
                it.row1 = it.blocks_here > 1 ? (table[1] * p.nkv + it.kvh) * BLOCK_KEYS : 0;
                items[threadIdx.x - 64] = it;
            }
            if (threadIdx.x == 64) {
                const int mine = total > (int)blockIdx.x ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;   // of all rounds
                n_items_s = max(0, min(MAX_ITEMS, mine - round * MAX_ITEMS));
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = tmem_base_s;
        const int n_items = n_items_s;
        if (n_items == 0) break;

        if (warp == 0) {
            // ---- producer: lane 0 announces the bytes, then every lane requests one box ---------------------
            // The kernel in front of this one (rotation and cache append) writes q and the cache rows of the
            // newest position, and lets this kernel start only once everything before ITSELF is complete.  So the
            // keys and values of the first chunks, all but a sequence's last, are requested at once; q and the last
            // chunks follow after the wait.
            // box j of an item: 0, 1 q halves; 2 + 4 kb + {0, 1} the K halves of block kb, + {2, 3} its V halves
            auto load_box = [&](const Item& it, int s, int j) {
                if (j < 2) {
                    tma_load_2d(q_of(s) + j * (NQ * 128), &map_q, kq_full + 8 * s, j * 64, it.b * p.nh + it.kvh * g);
                } else {
                    const int kb = (j - 2) >> 2, x = j & 1;
                    if (kb >= it.blocks_here || kb < it.first_block) return;
                    const int row = kb == 0 ? it.row0 : it.row1;
                    if (((j - 2) & 2) == 0) tma_load_2d(k_of(s) + x * HALF_K + kb * BOX, &map_k, kq_full + 8 * s, x * 64, row);
                    else tma_load_2d(v_of(s) + (kb * 2 + x) * BOX, &map_v, v_full + 8 * s, x * 64, row);
                }
            };
            const int ahead = min(STAGES, n_items);
            if (lane < ahead) {
                const Item& it = items[lane];
                mbar_expect_tx(kq_full + 8 * lane, Q_BYTES + (it.blocks_here - it.first_block) * BOX * 2);
                mbar_expect_tx(v_full + 8 * lane, (it.blocks_here - it.first_block) * BOX * 2);
            }
            __syncwarp();
            const int my_n = lane / 10, my_j = lane % 10;     // three items of ten boxes each
            const bool mine = my_n < ahead;
            const bool early = mine && my_j >= 2 && items[my_n].split != items[my_n].pos / CHUNK;
            if (early) load_box(items[my_n], my_n, my_j);
            pdl_wait();
            if (mine && !early) load_box(items[my_n], my_n, my_j);
            for (int n = ahead; n < n_items; n++) {
                const Item& it = items[n];
                const int s = n % STAGES;
                int freed = lane == 0 ? (int)mbar_wait(stage_free + 8 * s, (uint32_t)(((n / STAGES) - 1) & 1), abort_flag, p.status, 120) : 1;
                freed = __shfl_sync(0xffffffffu, freed, 0);
                if (!freed) break;
                if (lane == 0) {
                    mbar_expect_tx(kq_full + 8 * s, Q_BYTES + (it.blocks_here - it.first_block) * BOX * 2);
                    mbar_expect_tx(v_full + 8 * s, (it.blocks_here - it.first_block) * BOX * 2);
                }
                __syncwarp();
                if (lane < 10) load_box(it, s, lane);
            }
        } else if (warp == 1 && lane == 0) {
            // ---- MMAs of the scores: S^T(n) = K(n) Q^T as soon as the keys have landed and the accumulator pair of
            // n's parity is free.  (A thread that issues MMAs is slow at it: an MMA costs it ~56 cycles and a look
            // at a barrier ~190, so the two kinds of product have a thread each.  The descriptors of stage 0 are
            // built once; per instruction only constants are added: the address sits in the low bits in units of
            // 16 bytes, and shared memory is too small to carry out of them.)
            const uint64_t k_desc0 = desc_k_major(k_of(0)), q_desc0 = desc_k_major(q_of(0));
            constexpr uint64_t STAGE_STEP = STAGE_BYTES >> 4;
            for (int n = 0; n < n_items; n++) {
                const int s = n % STAGES, t = n & 1;
                if (!mbar_wait(kq_full + 8 * s, (uint32_t)((n / STAGES) & 1), abort_flag, p.status, 121)) break;
                if (n >= 2 && !mbar_wait(tmem_free + 8 * t, (uint32_t)(((n >> 1) - 1) & 1), abort_flag, p.status, 123)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t kd = k_desc0 + s * STAGE_STEP, qd = q_desc0 + s * STAGE_STEP;
    #pragma unroll
                for (int k = 0; k < D / 16; k++) {
                    constexpr int HALF_Q = NQ * 128;
                    const uint64_t k_off = ((k / 4) * HALF_K + (k % 4) * 32) >> 4, q_off = ((k / 4) * HALF_Q + (k % 4) * 32) >> 4;
                    umma_bf16(tmem_base + 32 * t, kd + k_off, qd + q_off, IDESC_S, k > 0 ? 1u : 0u);
                }
                umma_commit(s_done + 8 * t);
            }
        } else if (warp == 10 && lane == 0) {
            // ---- MMAs of the weighted sums: O^T(n) = V(n)^T P^T(n) once P^T is written and the values have landed
            const uint64_t p_desc0 = desc_k_major(p_of(0)), v_desc0 = desc_mn_major(v_of(0), BOX);
            constexpr uint64_t STAGE_STEP = STAGE_BYTES >> 4;
            int n = 0;
            for (; n < n_items; n++) {
                const int s = n % STAGES, t = n & 1;
                if (!mbar_wait(p_ready + 8 * t, (uint32_t)((n >> 1) & 1), abort_flag, p.status, 127)) break;
                if (!mbar_wait(v_full + 8 * s, (uint32_t)((n / STAGES) & 1), abort_flag, p.status, 129)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t vd = v_desc0 + s * STAGE_STEP, pd = p_desc0 + s * STAGE_STEP;
                const int blocks_here = items[n].blocks_here;
    #pragma unroll
                for (int kb = 0; kb < 2; kb++) {
                    if (kb < blocks_here) {
    #pragma unroll
                        for (int k = 0; k < BLOCK_KEYS / 16; k++)
                            umma_bf16(tmem_base + 32 * t + 16, vd + ((kb * 2 * BOX + k * (16 * 128)) >> 4),
                                      pd + ((kb * (NQ * 128) + k * 32) >> 4), IDESC_O, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(o_done + 8 * t);
                umma_commit(stage_free + 8 * s);
            }
            // the last commits have arrived before the barriers are set up again for another round
            for (int m = max(0, n - STAGES); m < n && !*abort_flag; m++)
                mbar_wait(stage_free + 8 * (m % STAGES), (uint32_t)((m / STAGES) & 1), abort_flag, p.status, 122);
        } else if (warp >= 2 && warp < 10) {
            // ---- softmax (thread = key), then partial output (thread = d).  Two groups of four warps take turns:
            // group 0 the even items of this CTA with accumulator pair 0, group 1 the odd ones with pair 1.
            const int grp = (warp - 2) >> 2, quarter = warp & 3, t = quarter * 32 + lane;
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + 32 * grp;
            auto group_sync = [&]() {
                if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                else asm volatile("bar.sync 2, 128;" ::: "memory");
            };
            bool ok = true;
            // The rows of P^T beyond the group are zero for good: their columns of O^T are never read, but must be
            // finite.  Nothing else writes there, so they are cleared once, before the first P^T of this CTA.
            if (round == 0) {
                for (int i = threadIdx.x - 64; i < STAGES * P_BYTES / 16; i += 256)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(p_of(i / (P_BYTES / 16)) + (i % (P_BYTES / 16)) * 16), "r"(0) : "memory");
                asm volatile("bar.sync 4, 256;" ::: "memory");
            }
            pdl_wait();   // the partials, the counters and the output may still be in use by the kernels before
            for (int n = grp; ok && n < n_items; n += 2) {
                const Item& it = items[n];
                const int s = n % STAGES, use = n >> 1;   // `use`: how often this group's accumulators were used before
                const int key = it.chunk_begin + t;
                const bool visible = key >= it.lo && key <= it.pos;
                const int head0 = it.kvh * g;
                float sc[NQ];
                if (!(ok = mbar_wait(s_done + 8 * grp, (uint32_t)(use & 1), abort_flag, p.status, 124))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                tmem_load16(lane_base, sc);
    #pragma unroll
                for (int h = 0; h < G; h++) sc[h] = (visible && h < g) ? sc[h] * p.scale_log2 : -INFINITY;
                float mx[G];
    #pragma unroll
                for (int h = 0; h < G; h++) {
                    mx[h] = sc[h];
    #pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
                }
                group_sync();   // red_max and red_sum of this group's item before are read
                if (lane < G) {
                    float mine = mx[0];
    #pragma unroll
                    for (int h = 1; h < G; h++) mine = lane == h ? mx[h] : mine;
                    red_max[grp][quarter][lane] = mine;
                }
                group_sync();
                float psum[G];
                const int kb = t / BLOCK_KEYS, kin = t % BLOCK_KEYS;
                const uint32_t p_dst = p_of(s);
    #pragma unroll
                for (int h = 0; h < G; h++) {
                    const float M = fmaxf(fmaxf(red_max[grp][0][h], red_max[grp][1][h]), fmaxf(red_max[grp][2][h], red_max[grp][3][h]));
                    const float pj = (M == -INFINITY || sc[h] == -INFINITY) ? 0.f : exp2f(sc[h] - M);
                    const __nv_bfloat16 pb = __float2bfloat16_rn(pj);
                    psum[h] = __bfloat162float(pb);   // the sum uses what the tensor core multiplies with
                    mx[h] = M;
                    // P^T[h][key]: row h of the block's 16 x 128 B tile, 16-byte chunk (kin / 8) ^ (h & 7)
                    const uint32_t dst = p_dst + kb * (NQ * 128) + h * 128 + ((((uint32_t)kin >> 3) ^ (h & 7)) << 4) + (kin & 7) * 2;
                    asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst), "h"(*reinterpret_cast<const unsigned short*>(&pb)) : "memory");
                }
                // rows of V at and past the sequence's length have never been written by this sequence, and the rows of
                // a block that was not loaded hold what an earlier chunk left: their weight is 0, but
                // 0 x (whatever bits lie there) must stay 0
                if ((key >= it.kv_len || kb < it.first_block) && kb < it.blocks_here) {
                    for (int x = 0; x < 2; x++) {
                        const uint32_t rowp = v_of(s) + (kb * 2 + x) * BOX + kin * 128;
                        if (x == 0 && !mbar_wait(v_full + 8 * s, (uint32_t)((n / STAGES) & 1), abort_flag, p.status, 125)) break;
    #pragma unroll
                        for (int c = 0; c < 8; c++)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(rowp + c * 16), "r"(0) : "memory");
                    }
                }
    #pragma unroll
                for (int h = 0; h < G; h++)
    #pragma unroll
                    for (int o = 16; o > 0; o >>= 1) psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], o);
                if (lane < G) {
                    float mine = psum[0];
    #pragma unroll
                    for (int h = 1; h < G; h++) mine = lane == h ? psum[h] : mine;
                    red_sum[grp][quarter][lane] = mine;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(p_ready + 8 * grp);
                // partial output: thread = d
                if (!(ok = mbar_wait(o_done + 8 * grp, (uint32_t)(use & 1), abort_flag, p.status, 126))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float o[NQ];
                tmem_load16(lane_base + 16, o);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(tmem_free + 8 * grp);   // this pair of accumulators may be filled again
                group_sync();                       // red_sum of all four warps is written
    #pragma unroll
                for (int h = 0; h < G; h++) {
                    if (h < g) {
                        const size_t row = ((size_t)it.b * p.nh + head0 + h) * p.max_splits + it.split;
                        p.part_acc[row * D + t] = o[h];
                    }
                }
                if (lane < g) {   // every warp keeps its own copy of (maximum, sum): a warp folds what warps of its quarter wrote
                    float mine = mx[0];
    #pragma unroll
                    for (int h = 1; h < G; h++) mine = lane == h ? mx[h] : mine;
                    const size_t row = ((size_t)it.b * p.nh + head0 + lane) * p.max_splits + it.split;
                    *reinterpret_cast<float2*>(p.part_ml + (row * 4 + quarter) * 2) =
                        make_float2(mine, red_sum[grp][0][lane] + red_sum[grp][1][lane] + red_sum[grp][2][lane] + red_sum[grp][3][lane]);
                }
            }
            // All partials of this warp are written.  One counter per (sequence, kv head, quarter of d) counts the
            // chunks whose partials are in memory; a warp raises the counters of all its items at once (lane l the
            // l-th item of the group).  A row is folded, in chunk order, by the warps that computed ONE of the row's
            // chunks (which one: below), each for its quarter of d, so that the folding is spread over the CTAs: the
            // warp waits, with a limit, until its counter shows that all chunks are in.
            __threadfence();
            __syncwarp();
            if (ok && grp + 2 * lane < n_items) {
                const Item& it = items[grp + 2 * lane];
                atomicAdd(p.counters + ((size_t)it.b * p.nkv + it.kvh) * 4 + quarter, 1);
            }
            for (int i = grp; ok && i < n_items; i += 2) {
                const Item& it = items[i];
                const int s_begin = it.lo / CHUNK, n_chunks = it.pos / CHUNK + 1 - s_begin;
                if (it.split != it.folder) continue;          // another CTA folds this row
                int* counter = p.counters + ((size_t)it.b * p.nkv + it.kvh) * 4 + quarter;
                int seen = 0;
                if (lane == 0) {
                    uint32_t spins = 0;
                    while ((seen = *reinterpret_cast<volatile int*>(counter)) < n_chunks && ++spins < (1u << 22)) __nanosleep(20);
                    if (seen >= n_chunks) *counter = 0;          // ready for the next launch
                    else atomicExch(p.status, 128);              // a chunk never arrived: flag it, leave the row
                }
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (seen < n_chunks) continue;
                __threadfence();
                // a lane takes four neighbouring d of one head: 8 lanes per head, 4 heads per round
                const int head0 = it.kvh * g;
                for (int unit = lane; unit < g * 8; unit += 32) {
                    const int h = unit >> 3, dd = quarter * 32 + (unit & 7) * 4;
                    const size_t row = ((size_t)it.b * p.nh + head0 + h) * p.max_splits + s_begin;
                    float M = -INFINITY, L = 0.f;
                    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int cb = 0; cb < n_chunks; cb += FOLD_BATCH) {
                        float2 ml[FOLD_BATCH];
                        float4 v[FOLD_BATCH];
    #pragma unroll
                        for (int j = 0; j < FOLD_BATCH; j++) {   // all loads of the batch are in flight together
                            const bool in = cb + j < n_chunks;
                            ml[j] = in ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((row + cb + j) * 4 + quarter) * 2))
                                       : make_float2(-INFINITY, 0.f);
                            v[j] = in ? __ldcg(reinterpret_cast<const float4*>(p.part_acc + (row + cb + j) * D + dd))
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        float Mb = M;
    #pragma unroll
                        for (int j = 0; j < FOLD_BATCH; j++) Mb = fmaxf(Mb, ml[j].x);
                        const float keep = M == -INFINITY ? 0.f : exp2f(M - Mb);
                        L *= keep; a.x *= keep; a.y *= keep; a.z *= keep; a.w *= keep;
    #pragma unroll
                        for (int j = 0; j < FOLD_BATCH; j++) {
                            const float wc = ml[j].x == -INFINITY ? 0.f : exp2f(ml[j].x - Mb);
                            L = fmaf(ml[j].y, wc, L);
                            a.x = fmaf(v[j].x, wc, a.x); a.y = fmaf(v[j].y, wc, a.y);
                            a.z = fmaf(v[j].z, wc, a.z); a.w = fmaf(v[j].w, wc, a.w);
                        }
                        M = Mb;
                    }
                    const float inv = L > 0.f ? 1.0f / L : 0.f;
                    __nv_bfloat162 o2[2] = {__floats2bfloat162_rn(a.x * inv, a.y * inv), __floats2bfloat162_rn(a.z * inv, a.w * inv)};
                    *reinterpret_cast<uint2*>(p.out + ((size_t)it.b * p.nh + head0 + h) * D + dd) = *reinterpret_cast<uint2*>(o2);
                }
            }
        }

        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();   // every role is through with this round
        if (n_items < MAX_ITEMS) break;
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

// The numbers of the kernel's barrier protocol: out[0] stages of K/V in shared memory, [1] pairs of accumulators in
// tensor memory (one per group of softmax warps).
HYMT2_API int hymt2_attention_decode_tc_protocol(int* out) {
    out[0] = STAGES; out[1] = 2;
    return HYMT2_OK;
}

// out, q: [rows, nh * 128] bfloat16, one new token per row; k_cache, v_cache: one layer's planes
// [blocks][nkv][64][128].  max_splits >= ceil(longest kv_len / 128); part_acc holds
// rows*nh*max_splits*128 floats, part_ml rows*nh*max_splits*8, counters rows*nkv*4 zeroed ints.
HYMT2_API int hymt2_attention_decode_tc(void* out, const void* q, const void* k_cache, const void* v_cache,
                                        long cache_blocks, const int* block_table, int table_stride, int block_tokens,
                                        const int* slot_ids, const int* kv_lens, int rows, int nh, int nkv, int d,
                                        float scale, int window, int max_splits, float* part_acc, float* part_ml,
                                        int* counters, int* status, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(d == D, "attention_decode_tc: head_dim %d is not taken (128 is)", d);
    HYMT2_REQUIRE(block_tokens == BLOCK_KEYS, "attention_decode_tc: cache blocks must hold %d tokens", BLOCK_KEYS);
    HYMT2_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= NQ, "attention_decode_tc: at most %d heads per kv head", NQ);
    HYMT2_REQUIRE(max_splits > 0 && max_splits <= MAX_CHUNKS, "attention_decode_tc: at most %d chunks of 128 keys are taken, got %d", MAX_CHUNKS, max_splits);
    HYMT2_REQUIRE(part_acc && part_ml && counters && status, "attention_decode_tc: scratch is needed");
    HYMT2_REQUIRE(rows <= MAX_ROWS, "attention_decode_tc: at most %d sequences in one launch, got %d", MAX_ROWS, rows);
    CUtensorMap mq, mk, mv;
    const long cache_rows = cache_blocks * nkv * BLOCK_KEYS;
    const bool ok = make_map(&mq, q, (long)rows * nh, d, d, NQ) && make_map(&mk, k_cache, cache_rows, d, d, BLOCK_KEYS) &&
                    make_map(&mv, v_cache, cache_rows, d, d, BLOCK_KEYS);
    HYMT2_REQUIRE(ok, "attention_decode_tc: cuTensorMapEncodeTiled refused the operands");
    DecodeTcParams p{(__nv_bfloat16*)out, block_table, slot_ids, kv_lens, part_acc, part_ml, counters, table_stride, nh, nkv,
                     window, max_splits, rows, scale * 1.4426950408889634f, status};
    constexpr size_t smem = (size_t)STAGES * (2 * CHUNK * D * 2 + NQ * D * 2 + 2 * NQ * 128) + 1024;
    const int g = nh / nkv;
    auto kernel = g <= 1 ? attention_decode_tc_kernel<1> : g <= 2 ? attention_decode_tc_kernel<2>
                : g <= 4 ? attention_decode_tc_kernel<4> : g <= 8 ? attention_decode_tc_kernel<8>
                : attention_decode_tc_kernel<16>;
    static bool configured[5] = {};
    const int which = g <= 1 ? 0 : g <= 2 ? 1 : g <= 4 ? 2 : g <= 8 ? 3 : 4;
    if (!configured[which]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { hymt2_set_error("attention_decode_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        configured[which] = true;
    }
    // one CTA per SM walks the (sequence, kv head, chunk) items, MAX_ITEMS at a time.  All CTAs must run at the
    // same time (a row is folded by a CTA that waits for the others' chunks): never more CTAs than SMs.
    const long total = (long)rows * nkv * max_splits;
    int sms = 148;
    {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // Not quite every SM: behind the q/k/v projection (clusters of CTAs, placed whole inside GPCs) the CTAs numbered past
    // the last multiple of 8 were placed 5 to 8 us after the others, on SMs that had been idle all along (B200, 148 SMs,
    // stamps of the device clock at each CTA's entry), and the rows they held chunks of were folded that much later.
    if (sms >= 16) sms -= sms % 8;
    const long ctas = total < sms ? total : sms;
    cudaError_t e = launch_pdl(kernel, dim3((unsigned)ctas), dim3(NUM_THREADS), smem, stream, mq, mk, mv, p);
    if (e != cudaSuccess) { hymt2_set_error("attention_decode_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
    return hymt2_check_launch("attention_decode_tc");
}
