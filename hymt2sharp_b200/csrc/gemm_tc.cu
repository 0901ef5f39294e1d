// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   C = epilogue(X[T,K] · W[N,K]^T), float32 accumulation in tensor memory (TMEM).
//
// A CTA computes 128 x BN tiles with `tcgen05.mma` (cta_group::1, M = 128, K = 16 per
// instruction).  Operand tiles of 64 K-elements (128 bytes a row, 128-byte swizzle) are brought
// into shared memory by TMA (`cp.async.bulk.tensor.2d`) through a ring of stages guarded by
// mbarriers; one thread issues the TMA loads, one thread issues the MMAs, four warps read the
// accumulator back with `tcgen05.ld` and run the epilogue.
//
// Two orientations:
//   normal   the 128-row side holds tokens, the BN side holds output features (more than 128 tokens): a
//            persistent kernel with one CTA per SM that walks tiles of a width chosen to fill whole waves
//            (see gemm_tc_persistent_kernel and make_plan);
//   swapped  the 128-row side holds output features (weight rows), the BN side holds tokens
//            (BN = 16..128): a decode step streams every weight tile once at full tile height
//            whatever the batch is.  With `splits` > 1 the K range is cut over gridDim.z.  The
//            split CTAs of a tile form a thread-block cluster: each leaves its partial tile in
//            its own shared memory, and after the cluster's barrier every CTA adds the partials
//            of all ranks for its share of the token columns through distributed shared memory,
//            in rank order (so the sum is the same every time), and runs the epilogue for them.
//            (Where a ring for two CTAs on an SM would be too shallow, each split CTA has an SM to
//            itself and a deep ring; partial tiles then go through a global workspace, folded by the
//            CTA that arrives last at the tile's counter, also in split order.)
// Epilogues: store, accumulate into float32 C, SwiGLU (silu(gate) * up; W holds N gate rows,
// then N up rows; src/HyMT2Sharp/Ops.cs:1053), and for the fused q/k/v projection with heads of 128 the rotation, the
// per-head norm and the append to the paged cache (RopeEpilogue).  Rows and K beyond the matrices are zero-filled
// by TMA and masked in the epilogue, so any T and N are taken; K, lda and ldw must be multiples
// of 8 elements (TMA's 16-byte rule).
//
// Every wait on an mbarrier is bounded: when it gives up it sets the status word and the abort
// flag, all roles leave their loops, TMEM is freed and the kernel returns.
#include "tc_common.cuh"

namespace {

constexpr int BLOCK_K = 64, UMMA_K = 16, TILE_M = 128, MAX_STAGES = 8;
constexpr int EPILOGUE_GROUPS = 2;        // persistent kernel: groups of four epilogue warps, one per accumulator
constexpr int NUM_THREADS = 64 + 128 * EPILOGUE_GROUPS;   // warp 0 TMA, warp 1 MMAs, then the epilogue groups
// one-tile kernel: with few accumulator columns a second warp issues MMAs too (warp 6), see ISSUERS in the kernel
__host__ __device__ constexpr int tile_issuers(int bn, int epi) {
    return bn * (epi == 2 ? 2 : 1) <= 32 ? 2 : 1;   // measured: no gain with 64 columns and more
}
__host__ __device__ constexpr int tile_threads(int bn, int epi) { return tile_issuers(bn, epi) > 1 ? 224 : 192; }
constexpr int A_TILE_BYTES = TILE_M * BLOCK_K * 2;
constexpr int PERSISTENT_BN = 256;   // tile width of the persistent kernel for many tokens

enum { EPI_STORE = 0, EPI_ACCUMULATE = 1, EPI_SWIGLU = 2, EPI_ROPE_KV = 3 };

// What the EPI_ROPE_KV epilogue needs: the product is the fused q/k/v projection of a few tokens with heads of 128 (one
// tile of 128 output features = one head), and the epilogue does what the rotation kernel would do next
// (src/HyMT2Sharp/Ops.cs:98-195, src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:53-61): rotate-half rotation of q and k heads,
// per-head RMSNorm after it, q to its own tensor, k and v to their rows of the paged cache.
struct RopeEpilogue {
    __nv_bfloat16* q_out;      // [T, nh * 128]
    __nv_bfloat16* k_cache;    // one layer's plane [blocks][nkv][block_tokens][128]
    __nv_bfloat16* v_cache;
    const int* block_table;
    const int* token_seq;      // [T] batch row of each token
    const int* token_pos;      // [T] position of each token
    const int* slot_ids;       // [B] cache slot of each batch row, -1: padding
    const float* inv_freq;     // [rope_dim / 2], null when rope_dim == 0
    const float* angles;       // [T][rope_dim / 2] (cos, sin) of position * inv_freq: where tokens are the accumulator's rows
    const void* q_gain;        // [128] or null
    const void* k_gain;
    int table_stride, block_tokens, nh, nkv, rope_dim, write_kv, gain_bf16;
    float eps;
};

// An RMSNorm (src/HyMT2Sharp/Ops.cs:29-89) folded into the products around it.  The row scale r = 1/sqrt(mean(x^2) + eps) of the
// norm commutes with the product that follows it: (r * (x * gain)) W^T = r * ((x * gain) W^T).  So a product that ADDS into the
// residual (the only place where a residual row changes) can leave bf16(x * gain) and the row's sum of squares behind,
// and the product after it multiplies its sums by r: no kernel of its own reads the row again.  The sums of squares are
// partial, several per token; the consumer adds them in the order of the features.  The kernel for few tokens leaves one per
// tile of 128 features.  The persistent kernel, whose tile width depends on the number of tokens of the step, leaves one per
// 16 features, each summed in the order of the features: a prompt's rows then get the same sums bit for bit whatever else is
// in the step (with one sum per tile the last bit depended on the tile width, and within two layers the roundings to
// bfloat16 behind it had spread that bit to every logit: measured, 24 elements of one product differed, then all).
struct NormSide {
    // producer (EPI_ACCUMULATE): null, or where bf16(C_new * gain) goes ([T, N] contiguous), with the gain and the partial sums
    __nv_bfloat16* out;
    const void* gain;
    int gain_bf16;
    float* ss_out;           // [T][ss_out_tiles]
    int ss_out_tiles;
    // consumer: null, or the partial sums of the activations' rows ([T][ss_in_tiles]), the width of a row and the norm's eps
    const float* ss_in;
    int ss_in_tiles, ss_width;
    float ss_eps;
};

__device__ __forceinline__ float norm_row_scale(const NormSide& ns, int t) {
    // always in the same order: the same partial sums give the same scale bit for bit
    const float* row = ns.ss_in + (size_t)t * ns.ss_in_tiles;
    float ss = 0.f;
    int m = 0;
    if ((ns.ss_in_tiles & 3) == 0 && (((uintptr_t)ns.ss_in) & 15) == 0) {
        // four running sums, one per place in a group of four, then (0 + 1) + (2 + 3): a fixed order with a quarter of the chain
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
        for (; m < ns.ss_in_tiles; m += 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + m);     // (written by the kernel in front: a plain load)
            s4[0] += v.x; s4[1] += v.y; s4[2] += v.z; s4[3] += v.w;
        }
        ss = (s4[0] + s4[1]) + (s4[2] + s4[3]);
    }
    for (; m < ns.ss_in_tiles; m++) ss += row[m];
    return 1.0f / sqrtf(ss / (float)ns.ss_width + ns.ss_eps);
}
__device__ __forceinline__ float norm_gain_at(const NormSide& ns, int n) {
    return ns.gain_bf16 ? __bfloat162float(((const __nv_bfloat16*)ns.gain)[n]) : ((const float*)ns.gain)[n];
}

struct GemmTcParams {
    void* C;
    long ldc;
    int T, N, K;             // tokens, output features, reduction length
    int stages;
    int bn;                  // persistent kernel: the tile's width in weight rows (<= its template width, a multiple of 16; SwiGLU: of 32)
    int splits, k_blocks_per_split;
    int cluster;             // splits > 1: the split CTAs of a tile form a cluster and reduce through shared memory
    float* workspace;        // [tile][split][acc][BN][128] partial tiles (splits > 1)
    int* counters;           // [tile] arrivals, zero between launches
    int* status;
    RopeEpilogue rope;       // EPI_ROPE_KV only
    uint32_t wait_limit;     // tries of a bounded wait in the one-tile kernel (WAIT_LIMIT, less in the debug entry)
    int withhold_block;      // -1; the debug entry names a k block whose copies the producer does NOT issue
    NormSide norm;
    int together = 0;        // splits through the workspace: every CTA of a tile folds a share of its columns (all of them are resident)
};

// The copies of one stage (activations, weights, and for a split weight tile its second half) with, in front of them, a
// look (mbarrier.test_wait, which never suspends the thread) at the barrier of the stage that comes next: the answer
// takes a few hundred cycles under load, which pass
// while the copies are issued instead of in front of the next ones.  Returns what the look saw.
__device__ __forceinline__ bool tma_stage_looking_ahead(uint32_t bar, uint32_t bytes, uint32_t a_dst, const CUtensorMap* map_a, int ax,
                                                        int ay, uint32_t b_dst, const CUtensorMap* map_b, int bx, int by,
                                                        uint32_t b2_dst, int b2y, uint32_t has_b2, uint32_t next_bar,
                                                        uint32_t next_parity) {
    uint32_t seen;
    asm volatile(
        "{\n\t.reg .pred look, second;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 look, [%13], %14;\n\t"
        "setp.ne.b32 second, %12, 0;\n\t"
        "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%1], %2;\n\t"
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%7], [%8, {%9, %10}], [%1];\n\t"
        "@second cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%11], [%8, {%9, %15}], [%1];\n\t"
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%3], [%4, {%5, %6}], [%1];\n\t"
        "selp.u32 %0, 1, 0, look;\n\t}"
        : "=r"(seen)
        : "r"(bar), "r"(bytes), "r"(a_dst), "l"((uint64_t)map_a), "r"(ax), "r"(ay), "r"(b_dst), "l"((uint64_t)map_b), "r"(bx), "r"(by),
          "r"(b2_dst), "r"(has_b2), "r"(next_bar), "r"(next_parity), "r"(b2y)
        : "memory");
    return seen != 0;
}

// the same with "add to what the accumulator holds" fixed, so that no predicate has to be computed
__device__ __forceinline__ void umma_bf16_add(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.eq.u32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
// The four MMAs of a k block (BLOCK_K / UMMA_K) and the release of its stage with, in front of them, a look at the
// barrier of the stage that comes next (see tma_stage_looking_ahead).  Returns what the look saw.
__device__ __forceinline__ bool umma_block_looking_ahead(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                         uint32_t accumulate, uint32_t empty_bar, uint32_t next_bar,
                                                         uint32_t next_parity) {
    static_assert(BLOCK_K / UMMA_K == 4 && ((UMMA_K * 2) >> 4) == 2, "four MMAs a k block, descriptors 2 units apart");
    uint32_t seen;
    asm volatile(
        "{\n\t.reg .pred look, first, yes;\n\t.reg .b64 a, b;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 look, [%7], %8;\n\t"
        "setp.ne.b32 first, %5, 0;\n\t"
        "setp.eq.u32 yes, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, first;\n\t"
        "add.u64 a, %2, 2;\n\tadd.u64 b, %3, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n\t"
        "add.u64 a, %2, 4;\n\tadd.u64 b, %3, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n\t"
        "add.u64 a, %2, 6;\n\tadd.u64 b, %3, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n\t"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
        "selp.u32 %0, 1, 0, look;\n\t}"
        : "=r"(seen)
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(empty_bar), "r"(next_bar), "r"(next_parity)
        : "memory");
    return seen != 0;
}
template <int N>
__device__ __forceinline__ void tmem_load(uint32_t taddr, float* v);
template <>
__device__ __forceinline__ void tmem_load<16>(uint32_t taddr, float* v) { tmem_load16(taddr, v); }
template <>
__device__ __forceinline__ void tmem_load<32>(uint32_t taddr, float* v) {
    tmem_load16(taddr, v);
    tmem_load16(taddr + 16, v + 16);
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ void store_bf16x16(__nv_bfloat16* dst, const float* v) {   // dst is 32-byte aligned
    __nv_bfloat162 h[8];
#pragma unroll
    for (int q = 0; q < 8; q++) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(h)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(h)[1];
}

// The EPI_ROPE_KV epilogue where tokens are the accumulator's rows (many tokens): this thread owns token t and finds one
// head's 128 projected values in its lane of tensor memory from `head_at` on.  It does what the rotation kernel does
// (src/HyMT2Sharp/Ops.cs:98-195): the values as the projection would have stored them (bfloat16), rotate-half rotation
// over all 128 (rope_dim 128) or none (0), RMSNorm over the head where the model has it, then q to its tensor, k and v
// to the token's row of the paged cache.  Every thread of the warp comes along (the tensor-memory accesses are
// warp-wide); `active` says whether the token exists.
__device__ __forceinline__ void rope_head_from_tmem(uint32_t head_at, int t, int head, bool active, const RopeEpilogue& rp, float row_scale) {
    const bool is_q = head < rp.nh, is_k = !is_q && head < rp.nh + rp.nkv;
    int pos = 0, slot = -1;
    if (active) {
        pos = rp.token_pos[t];
        slot = rp.slot_ids[rp.token_seq[t]];
    }
    __nv_bfloat16* dst = nullptr;                      // where this head's 128 values go; null: nowhere
    if (is_q) {
        if (active) dst = rp.q_out + ((size_t)t * rp.nh + head) * TILE_M;
    } else if (rp.write_kv && slot >= 0) {
        const int block = rp.block_table[(size_t)slot * rp.table_stride + pos / rp.block_tokens];
        const int kvh = is_k ? head - rp.nh : head - rp.nh - rp.nkv;
        dst = (is_k ? rp.k_cache : rp.v_cache) + (((size_t)block * rp.nkv + kvh) * rp.block_tokens + (pos % rp.block_tokens)) * TILE_M;
    }
    const void* gain = is_q ? rp.q_gain : is_k ? rp.k_gain : nullptr;
    const bool rotate = (is_q || is_k) && rp.rope_dim == TILE_M;
    constexpr int HALF = TILE_M / 2;
    // the head's 128 values stay in registers between the rotation and the norm (the persistent kernel has one CTA
    // per SM and registers to spare; through tensor memory, tcgen05.st and back, it took four times as long);
    // every index below is known when the loops are unrolled
    float v[TILE_M];
#pragma unroll
    for (int c = 0; c < TILE_M; c += 16) tmem_load<16>(head_at + c, v + c);
#pragma unroll
    for (int i = 0; i < TILE_M; i++) v[i] = bf16_round(v[i] * row_scale);      // what the projection would have stored
    if (rotate) {
        const float4* angles = reinterpret_cast<const float4*>(rp.angles) + (size_t)(active ? t : 0) * (HALF / 2);
#pragma unroll
        for (int c = 0; c < HALF; c += 8) {
            float4 a[4];                                   // (cos, sin) of 8 angles
#pragma unroll
            for (int j = 0; j < 4; j++) a[j] = __ldg(angles + c / 2 + j);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float x = v[c + j], y = v[HALF + c + j];
                const float cs = j & 1 ? a[j / 2].z : a[j / 2].x, sn = j & 1 ? a[j / 2].w : a[j / 2].y;
                v[c + j] = x * cs - y * sn;
                v[HALF + c + j] = x * sn + y * cs;
            }
        }
    }
    if (gain) {
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < TILE_M; i++) ss[i & 3] += v[i] * v[i];
        const float scale = 1.0f / sqrtf(((ss[0] + ss[1]) + (ss[2] + ss[3])) / (float)TILE_M + rp.eps);
#pragma unroll
        for (int i = 0; i < TILE_M; i++) {
            const float gv = rp.gain_bf16 ? __bfloat162float(((const __nv_bfloat16*)gain)[i]) : ((const float*)gain)[i];
            v[i] = v[i] * scale * gv;
        }
    }
    if (dst) {
#pragma unroll
        for (int c = 0; c < TILE_M; c += 16) store_bf16x16(dst + c, v + c);
    }
}

// sincosf, not inlined: its slow path for large arguments is long, and an epilogue that rotates several columns would
// carry a copy for each
__device__ __noinline__ void sincos_once(float angle, float* sn, float* cs) { sincosf(angle, sn, cs); }

// --------------------------------------------------------------------------------------------
// The kernel for up to 128 tokens (swapped orientation): one CTA computes the tile of 128 output features x BN token
// columns over its cut of K, and the cuts of a tile fold as a cluster or through the workspace (see the top of the file).
// --------------------------------------------------------------------------------------------
template <int BN, int EPI, typename TC>
__global__ void __launch_bounds__(tile_threads(BN, EPI), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmTcParams p) {
    constexpr int NUM_ACC = EPI == EPI_SWIGLU ? 2 : 1;   // accumulators = A tiles per stage (gate rows, up rows)
    constexpr int B_TILE_BYTES = BN * BLOCK_K * 2;
    constexpr int STAGE_BYTES = NUM_ACC * A_TILE_BYTES + B_TILE_BYTES;
    constexpr int ACC_COLS = NUM_ACC * BN;
    // With few columns the thread that issues the MMAs is the bottleneck, not the tensor core (an MMA costs that
    // thread ~56 cycles, a look at an mbarrier ~190, whatever N is).  So two threads of different warps issue:
    // issuer j takes the k blocks that land in the stages j, j + 2, ... of the ring (so each stage's barrier has one
    // reader, who sees every phase of it) and adds them up in an accumulator of its own; the epilogue adds the
    // accumulators, always in the same order.
    constexpr int ISSUERS = tile_issuers(BN, EPI);
    static_assert(ISSUERS == 1 || ACC_COLS <= 32, "two issuers are for narrow accumulators");
    constexpr int PHYS_COLS = ACC_COLS * ISSUERS;   // accumulator a of issuer j: columns (a * ISSUERS + j) * BN ..
    constexpr int TMEM_COLS = PHYS_COLS <= 32 ? 32 : PHYS_COLS <= 64 ? 64 : PHYS_COLS <= 128 ? 128 : PHYS_COLS <= 256 ? 256 : 512;
    constexpr int CH = BN >= 32 ? 32 : 16;                            // accumulator columns per epilogue chunk
    constexpr int OUT_COLS = BN;                                      // token columns that the tile covers
    // instruction descriptor: D float32, A and B bfloat16, both K-major, N = BN, M = 128
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES + 1];
    // (the kernel that follows the q/k/v epilogue, attention, reads lengths, tables and old cache blocks before its
    // own wait: it may only start once everything in front of THIS kernel is complete, see the epilogue warps)
    if (EPI != EPI_ROPE_KV) pdl_launch_dependents();
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s, last_s;
    __shared__ float scale_s[BN];
    __shared__ int rope_pos_s[EPI == EPI_ROPE_KV ? BN : 1];
    __shared__ long long rope_at_s[EPI == EPI_ROPE_KV ? BN : 1];
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;     // 1024-byte aligned stage ring
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = p.stages;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[MAX_STAGES]), done_bar = smem_u32(&bars[2 * MAX_STAGES]);
    volatile int* abort_flag = &abort_s;

    const int num_k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int kb_begin = blockIdx.z * p.k_blocks_per_split;
    const int kb_end = min(num_k_blocks, kb_begin + p.k_blocks_per_split);
    const int my_blocks = max(0, kb_end - kb_begin);
    const int a_row0 = blockIdx.x * TILE_M;
    const int b_row0 = blockIdx.y * OUT_COLS;   // first token of the tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done_bar, ISSUERS);
        abort_s = 0;
        last_s = 0;
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
        // ---- TMA producer -------------------------------------------------------------------
        // Weights do not depend on the kernel before this one: the first ring of weight tiles is
        // requested at once, then the producer waits for that kernel and requests the activations.
        auto load_weights = [&](int i) {
            const int s = i % stages;
            const uint32_t bar = full0 + 8 * s, a_dst = tiles + s * STAGE_BYTES;
            const int k = (kb_begin + i) * BLOCK_K;
            tma_load_2d(a_dst, &map_a, bar, k, a_row0);
            if (NUM_ACC == 2) tma_load_2d(a_dst + A_TILE_BYTES, &map_a, bar, k, p.N + a_row0);
        };
        auto load_activations = [&](int i) {
            const int s = i % stages;
            const uint32_t bar = full0 + 8 * s, b_dst = tiles + s * STAGE_BYTES + NUM_ACC * A_TILE_BYTES;
            tma_load_2d(b_dst, &map_b, bar, (kb_begin + i) * BLOCK_K, b_row0);
        };
        // (p.withhold_block, -1 in every ordinary launch: the debug entry makes the producer announce that block's
        // bytes and never copy them, so that the wait for them runs out; see hymt2_gemm_tc_debug)
        const int ahead = min(stages, my_blocks);
        for (int i = 0; i < ahead; i++) {   // fresh stages: nothing to wait for
            mbar_expect_tx(full0 + 8 * (i % stages), STAGE_BYTES);
            if (kb_begin + i != p.withhold_block) load_weights(i);
        }
        pdl_wait();
        for (int i = 0; i < ahead; i++)
            if (kb_begin + i != p.withhold_block) load_activations(i);
        int issued = ahead;
        for (int i = ahead; i < my_blocks; i++) {
            const int s = i % stages;
            if (!mbar_wait(empty0 + 8 * s, ((i / stages) & 1) ^ 1, abort_flag, p.status, 101, p.wait_limit)) break;
            mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
            if (kb_begin + i != p.withhold_block) {
                load_weights(i);
                load_activations(i);
            }
            issued = i + 1;
        }
        if (*abort_flag) {
            // copies that are in flight must land before the CTA's shared memory goes away
            const uint32_t tries = p.withhold_block >= 0 ? p.wait_limit : (1u << 16);   // a withheld block never lands
            for (int i = max(0, issued - stages); i < issued; i++)
                for (uint32_t t = 0; t < tries && !mbar_try_wait(full0 + 8 * (i % stages), (i / stages) & 1); t++) {}
        }
    } else if ((warp == 1 || (warp >= 6 && warp - 5 < ISSUERS)) && lane == 0) {
        // ---- MMA issuers: warp 1 is issuer 0, warp 6 is issuer 1 ------------------------------------
        // The loop carries the stage's descriptor along (the address sits in the low bits, in units of 16 bytes,
        // and the ring is far too small to carry out of them) and adds constants: a chain of address arithmetic
        // per MMA would cost the issuing thread more than the MMA.
        constexpr uint64_t K_STEP = (UMMA_K * 2) >> 4, A2_STEP = A_TILE_BYTES >> 4, B_STEP = (NUM_ACC * A_TILE_BYTES) >> 4;
        const int me = warp == 1 ? 0 : warp - 5;
        const uint32_t acc0 = tmem_base + me * BN, acc1 = tmem_base + (ISSUERS + me) * BN;
        const uint64_t desc0 = desc_k_major(tiles);
        uint32_t s = 0, phase = 0, any = 0;
        for (int i = 0; i < my_blocks; i++) {
            if ((int)(s % ISSUERS) == me) {
                if (!mbar_wait(full0 + 8 * s, phase, abort_flag, p.status, 102, p.wait_limit)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = desc0 + (uint64_t)s * (uint64_t)(STAGE_BYTES >> 4), bdesc = adesc + B_STEP;
                umma_bf16(acc0, adesc, bdesc, IDESC, any);
                if (NUM_ACC == 2) umma_bf16(acc1, adesc + A2_STEP, bdesc, IDESC, any);
                any = 1;
#pragma unroll
                for (int k = 1; k < BLOCK_K / UMMA_K; k++) {
                    umma_bf16_add(acc0, adesc + k * K_STEP, bdesc + k * K_STEP, IDESC);
                    if (NUM_ACC == 2) umma_bf16_add(acc1, adesc + A2_STEP + k * K_STEP, bdesc + k * K_STEP, IDESC);
                }
                umma_commit(empty0 + 8 * s);   // the stage is free once these MMAs have read it
            }
            if (++s == (uint32_t)stages) { s = 0; phase ^= 1; }
        }
        umma_commit(done_bar);             // this issuer's accumulator is complete once its MMAs are done
    } else if (warp >= 2 && warp < 6) {
        // ---- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 31 --------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                   // row of the tile that this thread owns
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        pdl_wait();   // C, the workspace and the counters may still be in use by the kernel before
        if (EPI == EPI_ROPE_KV && threadIdx.x == 64) pdl_launch_dependents();   // wait first, release after
        if (EPI != EPI_ACCUMULATE && p.norm.ss_in) {
            // the row scale of the norm in front of this product, for the tile's tokens (see NormSide)
            const int tl = threadIdx.x - 64;
            if (tl < BN) scale_s[tl] = b_row0 + tl < p.T ? norm_row_scale(p.norm, b_row0 + tl) : 0.f;
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const bool scaled = EPI != EPI_ACCUMULATE && p.norm.ss_in != nullptr;
        TC* C = (TC*)p.C;
        // The cluster's fold: this CTA's share of the token columns that exist in the tile.  Where the fold adds into C,
        // the old values of the first batch of columns are asked for now, under the MMAs.
        constexpr int MAX_RANKS = 8;                           // a portable cluster
        // In the fold a warp owns a column (a token) and a lane four neighbouring rows (features): 16-byte loads from the
        // ranks' shared memory, a column's 128 features inside one warp (sums of squares and rotation partners need
        // no barrier), the four warps on four columns at a time, FOLD_COLS of each warp's columns in flight.
        constexpr int FOLD_COLS = (EPI == EPI_SWIGLU || BN < 64) ? 1 : 2;   // (narrow tiles: a warp rarely has a second column, and the registers are worth more)
        const int n4 = a_row0 + 4 * lane;                      // this lane's first feature in the fold
        int c_begin = 0, c_end = 0;
        float4 old_first[FOLD_COLS];
#pragma unroll
        for (int q = 0; q < FOLD_COLS; q++) old_first[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        const bool c_vec = (p.ldc & 3) == 0 && (((uintptr_t)C) & (4 * sizeof(TC) - 1)) == 0 && (a_row0 & 3) == 0 && n4 + 4 <= p.N;
        if (p.cluster && p.splits > 1) {
            const int cols = min(BN, p.T - b_row0);
            const int share = (cols + p.splits - 1) / p.splits;
            c_begin = (int)blockIdx.z * share;
            c_end = min(cols, c_begin + share);
            if constexpr (EPI == EPI_ACCUMULATE && sizeof(TC) == 4) {
#pragma unroll
                for (int q = 0; q < FOLD_COLS; q++) {
                    const int c = c_begin + quarter + 4 * q;
                    if (c < c_end && c_vec) old_first[q] = *reinterpret_cast<const float4*>(C + (size_t)(b_row0 + c) * p.ldc + n4);
                }
            }
        }
        // (the gains of the norm that this product's output feeds, for this lane's features: asked for now as well)
        float gain_ahead[4] = {0.f, 0.f, 0.f, 0.f};
        if (EPI == EPI_ACCUMULATE && p.norm.out) {
#pragma unroll
            for (int i = 0; i < 4; i++) if (n4 + i < p.N) gain_ahead[i] = norm_gain_at(p.norm, n4 + i);
        }
        // The rotation epilogue: where each of this CTA's tokens stands and where its k or v row lies in the cache is
        // a chain of three loads (position, slot, block).  It is walked now, under the MMAs, one thread a token.
        float rope_inv_freq[4] = {0.f, 0.f, 0.f, 0.f}, rope_gain[4] = {1.f, 1.f, 1.f, 1.f};
        if constexpr (EPI == EPI_ROPE_KV) {
            const RopeEpilogue& rp = p.rope;
            const int head = blockIdx.x, tl = threadIdx.x - 64;
            const bool is_q = head < rp.nh, is_k = !is_q && head < rp.nh + rp.nkv;
            if (tl < c_end - c_begin && tl < BN) {
                const int t = b_row0 + c_begin + tl;
                const int pos = rp.token_pos[t], slot = rp.slot_ids[rp.token_seq[t]];
                long long at = -1;
                if (!is_q && rp.write_kv && slot >= 0) {
                    const int block = rp.block_table[(size_t)slot * rp.table_stride + pos / rp.block_tokens];
                    const int kvh = is_k ? head - rp.nh : head - rp.nh - rp.nkv;
                    at = (((long long)block * rp.nkv + kvh) * rp.block_tokens + (pos % rp.block_tokens)) * TILE_M;
                }
                rope_pos_s[tl] = pos;
                rope_at_s[tl] = at;
            }
            const int half = rp.rope_dim / 2;
            const void* gain = is_q ? rp.q_gain : is_k ? rp.k_gain : nullptr;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int d = 4 * lane + i;
                if (d < rp.rope_dim && (is_q || is_k)) rope_inv_freq[i] = rp.inv_freq[d < half ? d : d - half];
                if (gain) rope_gain[i] = rp.gain_bf16 ? __bfloat162float(((const __nv_bfloat16*)gain)[d]) : ((const float*)gain)[d];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }

        bool ok = my_blocks > 0 ? mbar_wait(done_bar, 0, abort_flag, p.status, 103, p.wait_limit) : true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // CH columns of the accumulators from column c on (c counts gate columns, then up columns): the sum over the
        // issuers that had a k block, in issuer order (issuer 1 has one as soon as there are two blocks and two stages)
        const int used = min(ISSUERS, min(my_blocks, stages));
        auto acc_load = [&](int c, float* g) {
            const uint32_t at = lane_addr + (uint32_t)((c / BN) * ISSUERS * BN + c % BN);
            tmem_load<CH>(at, g);
#pragma unroll
            for (int j = 1; j < ISSUERS; j++) {
                if (j < used) {
                    float more[CH];
                    tmem_load<CH>(at + j * BN, more);
#pragma unroll
                    for (int q = 0; q < CH; q++) g[q] += more[q];
                }
            }
        };

        // one chunk of CH accumulator columns: g (and u for SwiGLU) -> C
        auto emit = [&](int c, const float* g, const float* u) {
            const int n = a_row0 + row;                    // output feature
            if (n >= p.N) return;
            float old[CH];
            if (EPI == EPI_ACCUMULATE) {                   // all loads first: they do not wait for each other
#pragma unroll
                for (int j = 0; j < CH; j++) {
                    const int t = b_row0 + c + j;
                    old[j] = t < p.T ? to_float(C[(size_t)t * p.ldc + n]) : 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < CH; j++) {
                const int t = b_row0 + c + j;              // token
                if (t >= p.T) break;
                TC* dst = C + (size_t)t * p.ldc + n;
                const float r = scaled ? scale_s[c + j] : 1.0f;
                if (EPI == EPI_STORE) *dst = from_float<TC>(g[j] * r);
                else if (EPI == EPI_ACCUMULATE) *dst = from_float<TC>(old[j] + g[j]);
                else *dst = from_float<TC>(silu_mul(g[j] * r, u[j] * r));
            }
        };

        if (p.splits == 1) {
            if (ok) {
                for (int c = 0; c < OUT_COLS; c += CH) {
                    float g[CH], u[CH];
                    acc_load(c, g);
                    if (EPI == EPI_SWIGLU) acc_load(BN + c, u);
                    emit(c, g, u);
                }
            }
        } else if (p.cluster) {
            // partial tile -> this CTA's shared memory (the stage ring is free now), [column][row].  After the
            // cluster's barrier every CTA of the cluster takes a share of the token columns that exist, adds the
            // partials of all ranks for them through distributed shared memory (in rank order: the sum is the
            // same every time) and writes them out: the adding is spread over the cluster, and no one reads
            // columns beyond the last token.
            for (int c = 0; c < ACC_COLS; c += CH) {
                float g[CH];
                if (ok && my_blocks > 0) acc_load(c, g);
                else {
#pragma unroll
                    for (int j = 0; j < CH; j++) g[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < CH; j++)
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(tiles + ((c + j) * TILE_M + row) * 4), "f"(g[j]) : "memory");
            }
            __syncwarp();
            cluster_sync_all();
            for (int c0 = c_begin + quarter; c0 < c_end; c0 += 4 * FOLD_COLS) {
                // all loads first (they do not wait for each other): the residual's old values, then every rank's partials
                float4 old[FOLD_COLS];
                if constexpr (EPI == EPI_ACCUMULATE && sizeof(TC) == 4) {
#pragma unroll
                    for (int q = 0; q < FOLD_COLS; q++) {
                        const int c = c0 + 4 * q;
                        if (c0 == c_begin + quarter) old[q] = old_first[q];
                        else old[q] = (c < c_end && c_vec) ? *reinterpret_cast<const float4*>(C + (size_t)(b_row0 + c) * p.ldc + n4)
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                float4 g[FOLD_COLS], u[FOLD_COLS];
                {
                    float4 pg[FOLD_COLS][MAX_RANKS], pu[FOLD_COLS][MAX_RANKS];
#pragma unroll
                    for (int q = 0; q < FOLD_COLS; q++)
#pragma unroll
                        for (int r = 0; r < MAX_RANKS; r++) {
                            const int c = c0 + 4 * q;
                            const bool in = r < p.splits && c < c_end;
                            pg[q][r] = in ? ld_cluster_f32x4(tiles + (c * TILE_M + 4 * lane) * 4, r) : make_float4(0.f, 0.f, 0.f, 0.f);
                            pu[q][r] = (in && EPI == EPI_SWIGLU) ? ld_cluster_f32x4(tiles + ((BN + c) * TILE_M + 4 * lane) * 4, r)
                                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                    for (int q = 0; q < FOLD_COLS; q++) {
                        g[q] = make_float4(0.f, 0.f, 0.f, 0.f); u[q] = g[q];
#pragma unroll
                        for (int r = 0; r < MAX_RANKS; r++) {   // rank order
                            g[q].x += pg[q][r].x; g[q].y += pg[q][r].y; g[q].z += pg[q][r].z; g[q].w += pg[q][r].w;
                            u[q].x += pu[q][r].x; u[q].y += pu[q][r].y; u[q].z += pu[q][r].z; u[q].w += pu[q][r].w;
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < FOLD_COLS; q++) {
                    const int c = c0 + 4 * q;                      // warp-uniform
                    if (c >= c_end) continue;
                    const int t = b_row0 + c;                      // the token
                    const float r = scaled ? scale_s[c] : 1.0f;
                    float gv[4] = {g[q].x * r, g[q].y * r, g[q].z * r, g[q].w * r};
                    if constexpr (EPI == EPI_ROPE_KV) {
                        // this tile is head blockIdx.x of token t; this lane holds its values d = 4 lane .. 4 lane + 3
                        const RopeEpilogue& rp = p.rope;
                        const int head = blockIdx.x;
                        const bool is_q = head < rp.nh, is_k = !is_q && head < rp.nh + rp.nkv;
                        const int pos = rope_pos_s[c - c_begin];
                        const long long at = rope_at_s[c - c_begin];
                        float x[4], y[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) x[i] = __bfloat162float(__float2bfloat16_rn(gv[i]));   // what the projection would have stored
                        if (!is_q && !is_k) {   // a value head: as it is
                            if (at >= 0) {
                                __nv_bfloat162 h[2] = {__floats2bfloat162_rn(x[0], x[1]), __floats2bfloat162_rn(x[2], x[3])};
                                *reinterpret_cast<uint2*>(rp.v_cache + at + 4 * lane) = *reinterpret_cast<const uint2*>(h);
                            }
                            continue;
                        }
                        // rotation partners d and d +- rope_dim / 2 trade through this warp's 128 words behind the partials
                        const uint32_t ex = tiles + ACC_COLS * TILE_M * 4 + quarter * (TILE_M * 4);
                        const int half = rp.rope_dim / 2;
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ex + lane * 16), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]) : "memory");
                        __syncwarp();
                        float ss = 0.f;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int d = 4 * lane + i;
                            y[i] = x[i];
                            if (d < rp.rope_dim) {
                                const bool low = d < half;
                                float other, sn, cs;
                                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(other) : "r"(ex + (low ? d + half : d - half) * 4) : "memory");
                                sincos_once((float)pos * rope_inv_freq[i], &sn, &cs);
                                y[i] = low ? x[i] * cs - other * sn : other * sn + x[i] * cs;
                            }
                            ss = fmaf(y[i], y[i], ss);
                        }
                        __syncwarp();                              // the warp's next column trades through the same words
                        if ((is_q ? rp.q_gain : rp.k_gain) != nullptr) {
                            const float scale = 1.0f / sqrtf(warp_sum(ss) / (float)TILE_M + rp.eps);
#pragma unroll
                            for (int i = 0; i < 4; i++) y[i] = y[i] * scale * rope_gain[i];
                        }
                        __nv_bfloat162 h[2] = {__floats2bfloat162_rn(y[0], y[1]), __floats2bfloat162_rn(y[2], y[3])};
                        if (is_q) *reinterpret_cast<uint2*>(rp.q_out + ((size_t)t * rp.nh + head) * TILE_M + 4 * lane) = *reinterpret_cast<const uint2*>(h);
                        else if (at >= 0) *reinterpret_cast<uint2*>(rp.k_cache + at + 4 * lane) = *reinterpret_cast<const uint2*>(h);
                    } else {
                        const float uv[4] = {u[q].x * r, u[q].y * r, u[q].z * r, u[q].w * r};
                        TC* dst = C + (size_t)t * p.ldc + n4;
                        float o[4];
                        if constexpr (EPI == EPI_ACCUMULATE) {
                            if (c_vec) { o[0] = old[q].x + gv[0]; o[1] = old[q].y + gv[1]; o[2] = old[q].z + gv[2]; o[3] = old[q].w + gv[3]; }
                            else {
#pragma unroll
                                for (int i = 0; i < 4; i++) o[i] = n4 + i < p.N ? to_float(dst[i]) + gv[i] : 0.f;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; i++) o[i] = EPI == EPI_STORE ? gv[i] : silu_mul(gv[i], uv[i]);
                        }
                        if (c_vec) {
                            if constexpr (sizeof(TC) == 4) *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                            else {
                                __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
                                *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; i++) if (n4 + i < p.N) dst[i] = from_float<TC>(o[i]);
                        }
                        if (EPI == EPI_ACCUMULATE && p.norm.out) {
                            // for the norm that follows: bf16(value * gain), and the token's sum of squares over the tile's
                            // 128 features, which all lie in this warp
                            float sq = 0.f;
                            __nv_bfloat16 nb[4];
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const float v = n4 + i < p.N ? o[i] : 0.f;
                                sq = fmaf(v, v, sq);
                                nb[i] = __float2bfloat16_rn(v * gain_ahead[i]);
                            }
                            __nv_bfloat16* nd = p.norm.out + (size_t)t * p.N + n4;
                            if (n4 + 4 <= p.N && (p.N & 3) == 0) *reinterpret_cast<uint2*>(nd) = *reinterpret_cast<const uint2*>(nb);
                            else {
#pragma unroll
                                for (int i = 0; i < 4; i++) if (n4 + i < p.N) nd[i] = nb[i];
                            }
                            sq = warp_sum(sq);
                            if (lane == 0) p.norm.ss_out[(size_t)t * p.norm.ss_out_tiles + blockIdx.x] = sq;
                        }
                    }
                }
            }
            __syncwarp();
            cluster_sync_all();   // every CTA keeps its shared memory until its peers have read it
        } else {
            // partial tile -> workspace [tile][split][acc][column][row]; the last arrival reduces
            const int tile = blockIdx.y * gridDim.x + blockIdx.x;
            float* ws_tile = p.workspace + (size_t)tile * p.splits * (ACC_COLS * TILE_M);
            float* mine = ws_tile + (size_t)blockIdx.z * (ACC_COLS * TILE_M);
            for (int c = 0; c < ACC_COLS; c += CH) {
                float g[CH];
                if (ok && my_blocks > 0) acc_load(c, g);
                else {
#pragma unroll
                    for (int j = 0; j < CH; j++) g[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < CH; j++) mine[(size_t)(c + j) * TILE_M + row] = g[j];
            }
            // The fold of the columns [col_begin, col_end) from the partial tiles in memory: a thread takes four neighbouring
            // rows (features) of every fourth column with 16-byte loads, two columns and up to four splits in flight (a
            // batch of 4-byte loads, a row a thread, took 1.2 us where the same bytes by 16-byte loads take 0.45: the
            // requests, not the bytes, bound it).  Sums in split order from zero, as ever: the same bits every time.
            auto fold_from_memory = [&](int col_begin, int col_end) {
                constexpr int FCB = 2, SG = 4;
                const int tid = threadIdx.x - 64, rg = tid & 31, cg = tid >> 5;
                const int n0 = a_row0 + 4 * rg;
                if (n0 >= p.N) return;
                const bool whole = n0 + 4 <= p.N;
                for (int c0 = col_begin + cg; c0 < col_end; c0 += 4 * FCB) {
                    float4 g[FCB], u[FCB];
#pragma unroll
                    for (int q = 0; q < FCB; q++) { g[q] = make_float4(0.f, 0.f, 0.f, 0.f); u[q] = g[q]; }
                    for (int s0 = 0; s0 < p.splits; s0 += SG) {
                        float4 pg[SG][FCB], pu[SG][FCB];
#pragma unroll
                        for (int k = 0; k < SG; k++) {
                            const bool in_s = s0 + k < p.splits;
                            const float* part = ws_tile + (size_t)(in_s ? s0 + k : 0) * (ACC_COLS * TILE_M) + 4 * rg;
#pragma unroll
                            for (int q = 0; q < FCB; q++) {
                                const int c = c0 + 4 * q;
                                const bool in = in_s && c < col_end;
                                pg[k][q] = in ? __ldcg(reinterpret_cast<const float4*>(part + (size_t)c * TILE_M)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                pu[k][q] = (in && EPI == EPI_SWIGLU) ? __ldcg(reinterpret_cast<const float4*>(part + (size_t)(BN + c) * TILE_M))
                                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
#pragma unroll
                        for (int k = 0; k < SG; k++)
#pragma unroll
                            for (int q = 0; q < FCB; q++) {
                                g[q].x += pg[k][q].x; g[q].y += pg[k][q].y; g[q].z += pg[k][q].z; g[q].w += pg[k][q].w;
                                u[q].x += pu[k][q].x; u[q].y += pu[k][q].y; u[q].z += pu[k][q].z; u[q].w += pu[k][q].w;
                            }
                    }
#pragma unroll
                    for (int q = 0; q < FCB; q++) {
                        const int c = c0 + 4 * q;
                        if (c >= col_end) continue;
                        const float r = scaled ? scale_s[c] : 1.0f;
                        const float gv[4] = {g[q].x, g[q].y, g[q].z, g[q].w}, uv[4] = {u[q].x, u[q].y, u[q].z, u[q].w};
                        TC* dst = C + (size_t)(b_row0 + c) * p.ldc + n0;
                        float o[4];
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            o[i] = EPI == EPI_STORE ? gv[i] * r : EPI == EPI_ACCUMULATE ? gv[i] : silu_mul(gv[i] * r, uv[i] * r);
                        if (whole && (((uintptr_t)dst) & (4 * sizeof(TC) - 1)) == 0) {
                            if constexpr (sizeof(TC) == 4) {
                                float4 v = make_float4(o[0], o[1], o[2], o[3]);
                                if (EPI == EPI_ACCUMULATE) {
                                    const float4 old = *reinterpret_cast<const float4*>(dst);
                                    v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                                }
                                *reinterpret_cast<float4*>(dst) = v;
                            } else {
                                __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
                                *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                if (n0 + i < p.N) dst[i] = from_float<TC>(EPI == EPI_ACCUMULATE ? to_float(dst[i]) + o[i] : o[i]);
                        }
                    }
                }
            };
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            bool together = false;
            if constexpr (BN >= 64) together = p.together != 0;   // (compiled for wide tiles only: the narrow ones keep their registers, and with them their place beside other kernels' CTAs)
            if (together) {
              if constexpr (BN >= 64) {
                // Every CTA of the tile is on an SM at this time (the launch has no more CTAs than there are SMs).  Each
                // waits, with a limit, until all the partials are in memory, then adds them up for its share of the token
                // columns, in split order, and writes those: a third of the work each instead of all of it for the CTA
                // that happened to come last, whose fold stood between this kernel and the next (20 us at 64 tokens).
                if (warp == 2 && lane == 0) {
                    atomicAdd(&p.counters[tile], 1);
                    int seen = 0;
                    for (uint32_t tries = 0; tries < p.wait_limit; tries++) {
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile) : "memory");
                        if (seen >= p.splits || *abort_flag) break;
                        __nanosleep(32);
                    }
                    if (seen < p.splits) { *abort_flag = 1; atomicExch(p.status, 106); }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!*abort_flag) {
                    __threadfence();
                    const int cols = min(BN, p.T - b_row0);
                    const int share = (cols + p.splits - 1) / p.splits;
                    const int mine_begin = (int)blockIdx.z * share;
                    fold_from_memory(mine_begin, min(cols, mine_begin + share));
                }
                // the CTA that leaves last puts the counter back to zero for the next launch
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0 && !*abort_flag) {
                    const int left = atomicAdd(&p.counters[tile], 1);
                    if (left == 2 * p.splits - 1) p.counters[tile] = 0;
                }
              }
            } else {
            if (warp == 2 && lane == 0) {
                const int arrived = atomicAdd(&p.counters[tile], 1);
                last_s = arrived == p.splits - 1;
                if (last_s) p.counters[tile] = 0;              // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (last_s) {
                __threadfence();
                fold_from_memory(0, min(BN, p.T - b_row0));
            }
            }
        }
    }

    if (p.cluster && p.splits > 1 && (warp < 2 || warp >= 6)) {   // the warps without an epilogue take part in both barriers
        __syncwarp();
        cluster_sync_all();
        cluster_sync_all();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// --------------------------------------------------------------------------------------------
// Persistent kernel for many tokens (normal orientation): one CTA per SM walks the output tiles
// (token tiles fastest, so that neighbours in time share a weight tile in L2).  The stage ring
// runs on across tiles, and two accumulators in tensor memory alternate: while the epilogue
// warps drain one, the MMA thread already fills the other with the next tile.
// --------------------------------------------------------------------------------------------
template <int BN, int EPI, typename TC>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmTcParams p) {
    // BN is the widest tile (the accumulators lie BN columns apart); the width in use comes with the launch, chosen so
    // that the tiles fill whole waves of SMs
    constexpr bool SPLIT_B = EPI == EPI_SWIGLU;
    const int bn = p.bn;
    const int B_TILE_BYTES = bn * BLOCK_K * 2;
    const int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    constexpr int TMEM_COLS = 2 * BN;                       // 256 or 512
    const int OUT_COLS = SPLIT_B ? bn / 2 : bn;
    const uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    if (EPI != EPI_ROPE_KV) pdl_launch_dependents();
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = p.stages;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[MAX_STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * MAX_STAGES]), acc_empty0 = acc_full0 + 16;
    volatile int* abort_flag = &abort_s;
    const int num_k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int tiles_m = (p.T + TILE_M - 1) / TILE_M, tiles_n = (p.N + OUT_COLS - 1) / OUT_COLS;
    const int num_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 128);
        }
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
        // ---- producer: the first stage's weights (B) before the wait, then everything in order ----
        // Stage and phase are counted along; whether the next stage is free was looked up while this one's copies
        // were issued (the stages of the first round are free anyway).
        uint32_t s = 0, round = 0;
        bool first = true, looked = true;
        for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
            const int a_row0 = (tile % tiles_m) * TILE_M, b_row0 = (tile / tiles_m) * OUT_COLS;
            for (int kb = 0; kb < num_k_blocks; kb++) {
                if (round > 0 && !looked && !mbar_wait(empty0 + 8 * s, (round & 1) ^ 1, abort_flag, p.status, 101)) break;
                const uint32_t bar = full0 + 8 * s, a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + A_TILE_BYTES;
                const int k = kb * BLOCK_K;
                const uint32_t s_next = s + 1 == (uint32_t)stages ? 0 : s + 1, round_next = s_next ? round : round + 1;
                if (first) {
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(b_dst, &map_b, bar, k, b_row0);
                    if (SPLIT_B) tma_load_2d(b_dst + B_TILE_BYTES / 2, &map_b, bar, k, p.N + b_row0);
                    pdl_wait();   // the activations come from the kernel before
                    tma_load_2d(a_dst, &map_a, bar, k, a_row0);
                    first = false;
                    looked = round_next == 0;
                } else {
                    const bool seen = tma_stage_looking_ahead(bar, STAGE_BYTES, a_dst, &map_a, k, a_row0, b_dst, &map_b, k, b_row0,
                                                              b_dst + B_TILE_BYTES / 2, p.N + b_row0, SPLIT_B ? 1u : 0u,
                                                              empty0 + 8 * s_next, (round_next & 1) ^ 1);
                    looked = round_next == 0 || seen;
                }
                s = s_next;
                round = round_next;
            }
        }
        if (first) pdl_wait();
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: the stage's descriptor is carried along, see gemm_tc_kernel --------------
        const uint64_t desc0 = desc_k_major(tiles);
        uint64_t adesc = desc0;
        uint32_t s = 0, phase = 0;
        bool looked = false;   // whether the stage's barrier was already seen complete
        int j = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, j++) {
            const int buf = j & 1;
            if (j >= 2 && !mbar_wait(acc_empty0 + 8 * buf, (uint32_t)((((j >> 1) - 1) & 1)), abort_flag, p.status, 104)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            bool ok = true;
            const uint32_t acc_at = tmem_base + buf * BN;
            for (int kb = 0; kb < num_k_blocks; kb++) {
                if (!looked && !(ok = mbar_wait(full0 + 8 * s, phase, abort_flag, p.status, 102))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t s_next = s + 1 == (uint32_t)stages ? 0 : s + 1, phase_next = s_next ? phase : phase ^ 1;
                // a look at a stage that will never be filled (behind the last one) is thrown away by the loops' ends
                looked = umma_block_looking_ahead(acc_at, adesc, adesc + (A_TILE_BYTES >> 4), IDESC, kb > 0 ? 1u : 0u, empty0 + 8 * s,
                                                  full0 + 8 * s_next, phase_next);
                s = s_next;
                phase = phase_next;
                adesc = s ? adesc + (uint64_t)(STAGE_BYTES >> 4) : desc0;
            }
            if (!ok) break;
            umma_commit(acc_full0 + 8 * buf);
        }
    } else if (warp >= 2) {
        // ---- epilogue ---------------------------------------------------------------------------------
        // Two groups of four warps, one per accumulator: group 0 takes this CTA's tiles 0, 2, 4, ..., group 1 the tiles
        // 1, 3, 5, ...  An epilogue that reads and writes memory (the add into the residual, the rotation) lasts longer
        // than a short tile's MMAs; with a group per accumulator two epilogues run at the same time.
        const int quarter = warp & 3, row = quarter * 32 + lane, group = (warp - 2) >> 2;
        pdl_wait();   // C may still be in use by the kernel before
        // the kernel after this one may read the cache before its own wait; it must not start while the kernel
        // before this one still runs: wait first, release after
        if (EPI == EPI_ROPE_KV && threadIdx.x == 64) pdl_launch_dependents();
        TC* C = (TC*)p.C;
        static_assert(EPILOGUE_GROUPS == 2, "a group serves the accumulator of its number");
        // The CTA's LAST tile has nothing behind it that would hide its epilogue, so both groups take it: its owner the
        // lower half of its columns, the other group, once through with its own tiles, the upper half.
        // (The helper reads a barrier it has not followed.  When it gets there it has drained tile last - 1, whose
        // MMAs were issued after those of tile last - 2 were complete, so the barrier of the last tile's accumulator is in
        // the last tile's own phase or past it, never one behind: the parity cannot be taken for an older one.)
        const int my_tiles = (int)blockIdx.x < num_tiles ? (num_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const int last = my_tiles - 1;
        const int split_at = EPI == EPI_ROPE_KV ? (bn / TILE_M / 2) * TILE_M : ((OUT_COLS / 16 + 1) / 2) * 16;   // whole heads, whole chunks
        const bool can_share = split_at > 0 && split_at < OUT_COLS;
        for (int item = 0;; item++) {
            // this group's own tiles first, then (where the last tile is the other group's) the upper half of that one
            int j, c_begin = 0, c_end = OUT_COLS;
            bool own = true;
            if (group + EPILOGUE_GROUPS * item < my_tiles) {
                j = group + EPILOGUE_GROUPS * item;
                if (j == last && can_share) c_end = split_at;
            } else if (my_tiles > 0 && can_share && (last & 1) != group && group + EPILOGUE_GROUPS * (item - 1) < my_tiles && !*abort_flag) {
                j = last; own = false; c_begin = split_at;
            } else break;
            const int tile = blockIdx.x + j * gridDim.x;
            const int buf = j & 1;
            const int a_row0 = (tile % tiles_m) * TILE_M, b_row0 = (tile / tiles_m) * OUT_COLS;
            // (the threads of a warp leave the wait at different times; what follows reads tensor memory warp-wide, so the
            // warp comes together first, and gives up together)
            const int m = a_row0 + row;
            // a norm folded into this product (see NormSide): the row scale of this thread's token, added up from the row's
            // partial sums while the tile's MMAs still run
            const float row_scale = (EPI != EPI_ACCUMULATE && p.norm.ss_in && m < p.T) ? norm_row_scale(p.norm, m) : 1.0f;
            const bool landed = mbar_wait(acc_full0 + 8 * buf, (uint32_t)((j >> 1) & 1), abort_flag, p.status, 103);
            if (!__all_sync(0xffffffffu, landed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
            if constexpr (EPI == EPI_ROPE_KV) {
                // the tile holds BN / 128 heads of 128 tokens: this thread's token, head after head
                const int heads = p.rope.nh + 2 * p.rope.nkv;
#pragma unroll 1
                for (int h = c_begin / TILE_M; h < c_end / TILE_M; h++) {
                    const int head = b_row0 / TILE_M + h;
                    if (head < heads) rope_head_from_tmem(lane_addr + h * TILE_M, m, head, m < p.T, p.rope, row_scale);
                }
            } else
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 16) {
                float g[16], u[16];
                tmem_load<16>(lane_addr + c, g);
                if (EPI == EPI_SWIGLU) tmem_load<16>(lane_addr + bn / 2 + c, u);
                if (m >= p.T) continue;
                const int n0 = b_row0 + c;
                if (n0 >= p.N) continue;
                float ss_acc = 0.f;     // of these 16 features: a tile starts at a multiple of 16, so the groups are the same for every tile width
                TC* dst = C + (size_t)m * p.ldc + n0;
                const bool vec = n0 + 16 <= p.N && (((uintptr_t)dst) & 15) == 0;
#pragma unroll
                for (int j8 = 0; j8 < 16; j8 += 8) {
                    float o[8];
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        o[q] = EPI == EPI_SWIGLU ? silu_mul(g[j8 + q] * row_scale, u[j8 + q] * row_scale)
                             : EPI == EPI_STORE ? g[j8 + q] * row_scale : g[j8 + q];
                    if (vec) {
                        if constexpr (sizeof(TC) == 4) {
                            float4* d4 = reinterpret_cast<float4*>(dst + j8);
#pragma unroll
                            for (int q = 0; q < 2; q++) {
                                float4 v = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                                if (EPI == EPI_ACCUMULATE) {
                                    const float4 old = d4[q];
                                    v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                                    o[4 * q] = v.x; o[4 * q + 1] = v.y; o[4 * q + 2] = v.z; o[4 * q + 3] = v.w;
                                }
                                d4[q] = v;
                            }
                            if (EPI == EPI_ACCUMULATE && p.norm.out) {
                                __nv_bfloat162 h[4];
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    const float a = o[2 * q], b = o[2 * q + 1];
                                    ss_acc = fmaf(a, a, ss_acc); ss_acc = fmaf(b, b, ss_acc);
                                    h[q] = __floats2bfloat162_rn(a * norm_gain_at(p.norm, n0 + j8 + 2 * q), b * norm_gain_at(p.norm, n0 + j8 + 2 * q + 1));
                                }
                                *reinterpret_cast<uint4*>(p.norm.out + (size_t)m * p.N + n0 + j8) = *reinterpret_cast<uint4*>(h);
                            }
                        } else {
                            __nv_bfloat162 h[4];
#pragma unroll
                            for (int q = 0; q < 4; q++) h[q] = __floats2bfloat162_rn(o[2 * q], o[2 * q + 1]);
                            *reinterpret_cast<uint4*>(dst + j8) = *reinterpret_cast<uint4*>(h);
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            if (n0 + j8 + q >= p.N) break;
                            const float v = EPI == EPI_ACCUMULATE ? to_float(dst[j8 + q]) + o[q] : o[q];
                            dst[j8 + q] = from_float<TC>(v);
                            if (EPI == EPI_ACCUMULATE && p.norm.out) {
                                ss_acc = fmaf(v, v, ss_acc);
                                p.norm.out[(size_t)m * p.N + n0 + j8 + q] = __float2bfloat16_rn(v * norm_gain_at(p.norm, n0 + j8 + q));
                            }
                        }
                    }
                }
                if (EPI == EPI_ACCUMULATE && p.norm.out) p.norm.ss_out[(size_t)m * p.norm.ss_out_tiles + (n0 >> 4)] = ss_acc;
            }
            if (!own) break;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty0 + 8 * buf);   // this thread has taken its row out of the accumulator
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// --------------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------------
template <int BN, int EPI, typename TC>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmTcParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kernel = gemm_tc_kernel<BN, EPI, TC>;
    static bool configured = false;   // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) { hymt2_set_error("gemm_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        configured = true;
    }
    cudaError_t e;
    if (p.cluster && p.splits > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(tile_threads(BN, EPI));
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = hymt2_pdl_enabled() ? 1 : 0;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = (unsigned)p.splits;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        e = cudaLaunchKernelEx(&cfg, kernel, ma, mb, p);
    } else {
        e = launch_pdl(kernel, grid, dim3(tile_threads(BN, EPI)), smem, stream, ma, mb, p);
    }
    if (e != cudaSuccess) { hymt2_set_error("gemm_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
    return hymt2_check_launch("gemm_tc");
}

template <int BN>
int dispatch_epilogue(const CUtensorMap& ma, const CUtensorMap& mb, const GemmTcParams& p, dim3 grid, size_t smem,
                      int epilogue, int c_dtype, cudaStream_t stream) {
    if (epilogue == EPI_STORE && c_dtype == HYMT2_BF16) return launch<BN, EPI_STORE, __nv_bfloat16>(ma, mb, p, grid, smem, stream);
    if (epilogue == EPI_STORE && c_dtype == HYMT2_F32) return launch<BN, EPI_STORE, float>(ma, mb, p, grid, smem, stream);
    if (epilogue == EPI_ACCUMULATE && c_dtype == HYMT2_F32) return launch<BN, EPI_ACCUMULATE, float>(ma, mb, p, grid, smem, stream);
    if (epilogue == EPI_SWIGLU && c_dtype == HYMT2_BF16) return launch<BN, EPI_SWIGLU, __nv_bfloat16>(ma, mb, p, grid, smem, stream);
    hymt2_set_error("gemm_tc: epilogue %d with output type %d is not built", epilogue, c_dtype);
    return HYMT2_ERR_ARGUMENT;
}

struct Plan {
    bool swapped;
    int bn, splits, k_blocks_per_split, stages;
    bool cluster, persistent;
    int sm_count;
    dim3 grid;
    size_t smem, workspace_floats;
    int tiles;
};

bool make_plan(int T, int N, int K, int epilogue, int sm_count, Plan* plan) {
    const int num_k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    Plan& pl = *plan;
    pl.sm_count = sm_count;
    pl.persistent = false;
    pl.swapped = T <= 128;
    pl.splits = 1;
    int num_acc = 1;
    if (pl.swapped) {
        pl.bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
        num_acc = epilogue == EPI_SWIGLU ? 2 : 1;
        const int tiles = (N + TILE_M - 1) / TILE_M;
        pl.grid = dim3(tiles, 1, 1);
        // too few tiles to pull the whole memory bandwidth: cut K so that about one wave of CTAs runs;
        // the cut depends on N and K only, never on the number of tokens
        if (tiles < sm_count / 2) {
            int want = sm_count / tiles;
            want = want > 8 ? 8 : want;   // a portable cluster holds at most 8 CTAs
            while (want > 1 && num_k_blocks / want < 2) want--;
            pl.splits = want;
        }
        // 128 token columns of split partials no longer fold inside a cluster (the ring of two CTAs on an SM gets too
        // shallow) and fold slowly through memory; two tiles of 64 columns do fold as clusters, and the second reading of
        // a weight tile, by the CTA beside the first, comes from L2
        if (T > 64 && pl.splits > 1 && num_acc == 1) {
            pl.bn = 64;
            pl.grid.y = (T + 63) / 64;
        }
        pl.tiles = tiles * (int)pl.grid.y;
    } else {
        // More than 128 tokens: the persistent kernel (one CTA per SM, wide tiles, a tile's epilogue hidden behind the
        // next tile's MMAs, the last one shared by both epilogue groups).  Tiles of 128 x 128 with two CTAs per SM were
        // measured against it for the products that add into the residual: slower at every size once the last tile's
        // epilogue was shared (down projection at 2,048 tokens 56 -> 49 us, at 1,536 tokens 54 -> 45 us).
        const int row_tiles = (T + TILE_M - 1) / TILE_M;
        pl.persistent = true;
        pl.bn = 128;
        {
            // The tile's width: the one whose tiles fill whole waves of SMs best.  A k block of a tile bn wide
            // costs about 350 + 1.84 bn cycles (measured at 192 to 256), and a wave lasts as long as one tile; behind
            // the last wave one epilogue stands alone, which costs about 60 cycles a column where it rotates and
            // norms heads (measured: tiles of one head win up to a few thousand tokens, of two heads beyond), 30
            // where it adds into float32, 15 else.
            const int step = epilogue == EPI_SWIGLU ? 32 : epilogue == EPI_ROPE_KV ? TILE_M : 16;   // SwiGLU: gate and up halves in chunks of 16; rotation: whole heads
            double best = 0;
            for (int bn = PERSISTENT_BN; bn >= 128; bn -= step) {
                const int out = epilogue == EPI_SWIGLU ? bn / 2 : bn;
                const long tiles = (long)row_tiles * ((N + out - 1) / out);
                const double epilogue_cycles = (epilogue == EPI_ROPE_KV ? 60.0 : epilogue == EPI_ACCUMULATE ? 30.0 : 15.0) * bn;
                const double cost = (double)((tiles + sm_count - 1) / sm_count) * num_k_blocks * (350.0 + 1.84 * bn) + epilogue_cycles;
                if (bn == PERSISTENT_BN || cost < best) { best = cost; pl.bn = bn; }
            }
        }
        const int out_cols = epilogue == EPI_SWIGLU ? pl.bn / 2 : pl.bn;
        pl.grid = dim3((T + TILE_M - 1) / TILE_M, (N + out_cols - 1) / out_cols, 1);
        pl.tiles = pl.grid.x * pl.grid.y;
    }
    pl.k_blocks_per_split = (num_k_blocks + pl.splits - 1) / pl.splits;
    pl.splits = (num_k_blocks + pl.k_blocks_per_split - 1) / pl.k_blocks_per_split;
    pl.grid.z = pl.splits;
    const int stage_bytes = num_acc * A_TILE_BYTES + pl.bn * BLOCK_K * 2;
    const long ctas = (long)pl.grid.x * pl.grid.y * pl.splits;
    // Splits go the cluster way when a ring for two CTAs on an SM still holds four stages (clusters must be placed
    // whole inside a GPC; with one CTA per SM they would not all fit at once): the fold through distributed shared
    // memory is quick.  Wide stages (two accumulators) stream best with one CTA per SM and a deep ring, and fold
    // through the global workspace.
    constexpr int CLUSTER_RING_BYTES = 110 * 1024;
    pl.cluster = pl.splits > 1 && pl.splits <= 8 && CLUSTER_RING_BYTES / stage_bytes >= 4 &&
                 (size_t)num_acc * pl.bn * TILE_M * 4 <= 96 * 1024;
    // one wave of CTAs: each takes what an SM has; more: two CTAs share an SM, one's epilogue hides behind the other's loads
    // (the persistent kernel: one CTA per SM, all it has)
    const int ring_bytes = pl.cluster ? CLUSTER_RING_BYTES : pl.persistent ? 224 * 1024 : ctas <= sm_count ? 200 * 1024 : 100 * 1024;
    int stages = ring_bytes / stage_bytes;
    stages = stages > MAX_STAGES ? MAX_STAGES : stages < 2 ? 2 : stages;
    if (pl.swapped && stages > pl.k_blocks_per_split) stages = pl.k_blocks_per_split < 2 ? 2 : pl.k_blocks_per_split;
    pl.stages = stages;
    pl.smem = (size_t)stages * stage_bytes + 1024;
    if ((size_t)num_acc * pl.bn * TILE_M * 4 > (size_t)stages * stage_bytes) pl.cluster = false;   // the partial must fit the ring
    pl.workspace_floats = (pl.splits > 1 && !pl.cluster) ? (size_t)pl.tiles * pl.splits * num_acc * pl.bn * TILE_M : 0;
    return true;
}

template <int BN, int EPI, typename TC>
int launch_persistent_one(const CUtensorMap& ma, const CUtensorMap& mb, const GemmTcParams& p, int ctas, size_t smem,
                          cudaStream_t stream) {
    auto kernel = gemm_tc_persistent_kernel<BN, EPI, TC>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) { hymt2_set_error("gemm_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        configured = true;
    }
    cudaError_t e = launch_pdl(kernel, dim3(ctas), dim3(NUM_THREADS), smem, stream, ma, mb, p);
    if (e != cudaSuccess) { hymt2_set_error("gemm_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
    return hymt2_check_launch("gemm_tc (persistent)");
}

int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmTcParams& p, const Plan& pl, int epilogue,
                      int c_dtype, cudaStream_t stream) {
    const int ctas = pl.tiles < pl.sm_count ? pl.tiles : pl.sm_count;
    if (epilogue == EPI_STORE && c_dtype == HYMT2_BF16) return launch_persistent_one<PERSISTENT_BN, EPI_STORE, __nv_bfloat16>(ma, mb, p, ctas, pl.smem, stream);
    if (epilogue == EPI_STORE && c_dtype == HYMT2_F32) return launch_persistent_one<PERSISTENT_BN, EPI_STORE, float>(ma, mb, p, ctas, pl.smem, stream);
    if (epilogue == EPI_ACCUMULATE && c_dtype == HYMT2_F32) return launch_persistent_one<PERSISTENT_BN, EPI_ACCUMULATE, float>(ma, mb, p, ctas, pl.smem, stream);
    if (epilogue == EPI_SWIGLU && c_dtype == HYMT2_BF16) return launch_persistent_one<PERSISTENT_BN, EPI_SWIGLU, __nv_bfloat16>(ma, mb, p, ctas, pl.smem, stream);
    hymt2_set_error("gemm_tc: epilogue %d with output type %d is not built", epilogue, c_dtype);
    return HYMT2_ERR_ARGUMENT;
}

int sm_count_of_current_device() {
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

}  // namespace

// The numbers of the kernels' barrier protocols: out[0] the most stages of a ring, [1] accumulators of the persistent
// kernel that alternate, [2] the most MMA issuers of the one-tile kernel, [3] 1: issuer j owns the stages j, j + issuers, ...,
// [4] epilogue groups of the persistent kernel (group g drains the tiles g, g + groups, ... of its CTA)
HYMT2_API int hymt2_gemm_tc_protocol(int* out) {
    out[0] = MAX_STAGES; out[1] = 2; out[2] = tile_issuers(16, EPI_STORE); out[3] = 1; out[4] = EPILOGUE_GROUPS;
    return HYMT2_OK;
}

// Whether the tensor-core kernel takes this problem, and what scratch it wants:
// workspace_floats of float32 and counters ints (zeroed once; the kernel leaves them zero).
HYMT2_API int hymt2_gemm_tc_plan(int T, int N, int K, int epilogue, long* workspace_floats, int* counters) {
    Plan pl;
    make_plan(T, N, K, epilogue, sm_count_of_current_device(), &pl);
    *workspace_floats = (long)pl.workspace_floats;
    *counters = (pl.splits > 1 && !pl.cluster) ? pl.tiles : 0;
    return HYMT2_OK;
}

// How a product of T tokens onto N features over K would be run (epilogue 0 store, 1 add, 2 SwiGLU, 3 the q/k/v epilogue),
// on a device of sm_count SMs (0: the current one): out[0] weight rows on the 128-row side (few tokens), [1] the
// persistent kernel, [2] the tile's width, [3] stages of the ring, [4] splits of K, [5] whether the splits fold as a cluster,
// [6] tiles, [7] CTAs.  For tests and for reading a profile; nothing is launched.
HYMT2_API int hymt2_gemm_tc_describe(int T, int N, int K, int epilogue, int sm_count, int* out) {
    HYMT2_REQUIRE(T > 0 && N > 0 && K > 0 && epilogue >= 0 && epilogue <= 3 && out, "gemm_tc_describe: bad arguments");
    Plan pl;
    make_plan(T, N, K, epilogue, sm_count > 0 ? sm_count : sm_count_of_current_device(), &pl);
    out[0] = pl.swapped ? 1 : 0;
    out[1] = pl.persistent ? 1 : 0;
    out[2] = pl.bn;
    out[3] = pl.stages;
    out[4] = pl.splits;
    out[5] = pl.cluster ? 1 : 0;
    out[6] = pl.tiles;
    out[7] = pl.persistent ? (pl.tiles < pl.sm_count ? pl.tiles : pl.sm_count) : (int)(pl.grid.x * pl.grid.y * pl.grid.z);
    return HYMT2_OK;
}

namespace {
// How many partial sums of squares per token a product that adds into the residual leaves behind for the norm after it:
// one per tile of 128 output features in steps of few tokens, one per 16 features from the persistent kernel (0: this plan
// cannot, and the norm runs as a kernel of its own).
int norm_out_tiles(const Plan& pl, int epilogue, int N) {
    if (epilogue != EPI_ACCUMULATE) return 0;
    if (pl.swapped) return (pl.splits > 1 && pl.cluster) ? (int)pl.grid.x : 0;   // the cluster's fold holds (token, tile) whole
    return (N + 15) / 16;   // the persistent kernel: one partial sum per 16 features, the same for every tile width
}

int run_gemm_tc(void* C, int c_dtype, const void* X, const void* W, int T, int N, int K, long lda, long ldw, long ldc,
                int epilogue, float* workspace, long workspace_floats, int* counters, int num_counters, int* status,
                cudaStream_t stream, uint32_t wait_limit, int withhold_block, NormSide norm = NormSide{}) {
    if (T == 0 || N == 0) return HYMT2_OK;
    HYMT2_REQUIRE(T > 0 && N > 0 && K > 0, "gemm_tc: bad sizes T=%d N=%d K=%d", T, N, K);
    HYMT2_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_tc: K, lda and ldw must be multiples of 8 (K=%d lda=%ld ldw=%ld)", K, lda, ldw);
    HYMT2_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    HYMT2_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tc: unknown epilogue %d", epilogue);
    HYMT2_REQUIRE(status != nullptr, "gemm_tc: a status word is needed");
    Plan pl;
    make_plan(T, N, K, epilogue, sm_count_of_current_device(), &pl);
    HYMT2_REQUIRE(pl.grid.y <= 65535 && pl.grid.x <= 2147483647u, "gemm_tc: grid too large");
    if (pl.splits > 1 && !pl.cluster)
        HYMT2_REQUIRE(workspace && counters && workspace_floats >= (long)pl.workspace_floats && num_counters >= pl.tiles,
                      "gemm_tc: the split needs %zu floats of workspace and %d counters", pl.workspace_floats, pl.tiles);
    const long w_rows = epilogue == EPI_SWIGLU ? 2L * N : N;
    CUtensorMap ma, mb;
    bool ok;
    if (pl.swapped) {
        ok = make_map(&ma, W, w_rows, K, ldw, TILE_M) && make_map(&mb, X, T, K, lda, pl.bn);
    } else {
        ok = make_map(&ma, X, T, K, lda, TILE_M) && make_map(&mb, W, w_rows, K, ldw, epilogue == EPI_SWIGLU ? pl.bn / 2 : pl.bn);
    }
    HYMT2_REQUIRE(ok, "gemm_tc: cuTensorMapEncodeTiled refused the operands");
    if (norm.out) {
        HYMT2_REQUIRE(c_dtype == HYMT2_F32 && norm_out_tiles(pl, epilogue, N) > 0 && norm.gain && norm.ss_out && N % 8 == 0 &&
                      (uintptr_t)norm.out % 16 == 0, "gemm_tc: this product (T=%d N=%d K=%d epilogue %d) cannot leave a norm's input behind", T, N, K, epilogue);
        norm.ss_out_tiles = norm_out_tiles(pl, epilogue, N);
    }
    if (norm.ss_in) HYMT2_REQUIRE(epilogue != EPI_ACCUMULATE && norm.ss_in_tiles > 0 && norm.ss_width > 0, "gemm_tc: bad row-scale arguments");
    GemmTcParams p{C, ldc, T, N, K, pl.stages, pl.bn, pl.splits, pl.k_blocks_per_split, pl.cluster ? 1 : 0, workspace, counters, status,
                   RopeEpilogue{}, wait_limit, withhold_block, norm};
    // (from 64 token columns on: below that the fold is short, and two thirds of the CTAs leaving early, so that the next
    // kernel's CTAs find room, is worth more; batch 8: 1.63 against 1.82 ms a step, batch 64: 4.05 against 3.95)
    p.together = (pl.swapped && pl.splits > 1 && !pl.cluster && pl.bn >= 64 && (long)pl.grid.x * pl.grid.y * pl.splits <= pl.sm_count) ? 1 : 0;
    if (withhold_block >= 0)
        HYMT2_REQUIRE(pl.swapped && pl.splits == 1, "gemm_tc_debug: only the one-tile kernel without a cut of K can withhold a block "
                      "(T=%d N=%d K=%d gives swapped=%d splits=%d)", T, N, K, (int)pl.swapped, pl.splits);
    if (pl.swapped) {
        switch (pl.bn) {
            case 16: return dispatch_epilogue<16>(ma, mb, p, pl.grid, pl.smem, epilogue, c_dtype, stream);
            case 32: return dispatch_epilogue<32>(ma, mb, p, pl.grid, pl.smem, epilogue, c_dtype, stream);
            case 64: return dispatch_epilogue<64>(ma, mb, p, pl.grid, pl.smem, epilogue, c_dtype, stream);
            default: return dispatch_epilogue<128>(ma, mb, p, pl.grid, pl.smem, epilogue, c_dtype, stream);
        }
    }
    return launch_persistent(ma, mb, p, pl, epilogue, c_dtype, stream);
}
}  // namespace

// C[T,N] (ldc) = epilogue(X[T,K] (lda) · W[N,K]^T (ldw)), X and W bfloat16; for SwiGLU W has 2N rows.
HYMT2_API int hymt2_gemm_tc(void* C, int c_dtype, const void* X, const void* W, int T, int N, int K, long lda, long ldw,
                            long ldc, int epilogue, float* workspace, long workspace_floats, int* counters,
                            int num_counters, int* status, cudaStream_t stream) {
    return run_gemm_tc(C, c_dtype, X, W, T, N, K, lda, ldw, ldc, epilogue, workspace, workspace_floats, counters, num_counters,
                       status, stream, WAIT_LIMIT, -1);
}

// hymt2_gemm_tc with an RMSNorm folded in (see NormSide).  As a consumer (ss_in): the activations X are bf16(x * gain) and the sums
// are multiplied by 1/sqrt(sum_tiles ss_in[t] / ss_width + ss_eps) (store and SwiGLU epilogues).  As a producer (norm_out, accumulate
// epilogue into float32): bf16(C_new * gain) goes to norm_out [T, N] and the partial sums of squares to ss_out [T][tiles], tiles as
// hymt2_gemm_tc_norm_tiles says (0: not offered for this shape).
HYMT2_API int hymt2_gemm_tc_norm_tiles(int T, int N, int K, int epilogue) {
    if (T <= 0 || N <= 0 || K <= 0 || N % 8) return 0;
    Plan pl;
    make_plan(T, N, K, epilogue, sm_count_of_current_device(), &pl);
    return norm_out_tiles(pl, epilogue, N);
}

HYMT2_API int hymt2_gemm_tc_norm(void* C, int c_dtype, const void* X, const void* W, int T, int N, int K, long lda, long ldw,
                                 long ldc, int epilogue, float* workspace, long workspace_floats, int* counters,
                                 int num_counters, int* status, cudaStream_t stream, const float* ss_in, int ss_in_tiles,
                                 int ss_width, float ss_eps, void* norm_out, const void* norm_gain, int norm_gain_dtype,
                                 float* ss_out) {
    HYMT2_REQUIRE(!norm_out || norm_gain_dtype == HYMT2_BF16 || norm_gain_dtype == HYMT2_F32, "gemm_tc_norm: the gain must be bfloat16 or float32");
    NormSide ns{(__nv_bfloat16*)norm_out, norm_gain, norm_gain_dtype == HYMT2_BF16 ? 1 : 0, ss_out, 0, ss_in, ss_in_tiles, ss_width, ss_eps};
    return run_gemm_tc(C, c_dtype, X, W, T, N, K, lda, ldw, ldc, epilogue, workspace, workspace_floats, counters, num_counters,
                       status, stream, WAIT_LIMIT, -1, ns);
}

// The same product with one fault put in on purpose, for the test of the bounded waits: the producer announces
// the bytes of k block `withhold_block` and never copies them, and every wait gives up after `wait_limit` tries
// (a few thousand: milliseconds).  The MMA issuer's wait for that block then runs out: it writes 102 into the
// status word and raises the CTA's abort flag, every role leaves its loop, the producer waits (bounded) for the
// copies that are in flight, tensor memory is freed, the kernel returns, and the context stays usable.  What the
// launch wrote into C is not a product.  Only a product of few tokens whose K is not cut is taken (the smallest
// launch there is): no cluster, no workspace, no counters that a half-finished run could leave set.
HYMT2_API int hymt2_gemm_tc_debug(void* C, int c_dtype, const void* X, const void* W, int T, int N, int K, long lda, long ldw,
                                  long ldc, int epilogue, int* status, cudaStream_t stream, int wait_limit,
                                  int withhold_block) {
    HYMT2_REQUIRE(wait_limit > 0 && wait_limit <= (1 << 16), "gemm_tc_debug: wait_limit %d must be in [1, 65536]", wait_limit);
    HYMT2_REQUIRE(withhold_block >= 0 && withhold_block < (K + BLOCK_K - 1) / BLOCK_K, "gemm_tc_debug: K has no block %d", withhold_block);
    return run_gemm_tc(C, c_dtype, X, W, T, N, K, lda, ldw, ldc, epilogue, nullptr, 0, nullptr, 0, status, stream,
                       (uint32_t)wait_limit, withhold_block);
}

// Whether hymt2_gemm_tc_rope_kv takes a projection of T tokens onto N = (nh + 2 nkv) * 128 features over K.  A few tokens
// need the split-K cluster plan, whose CTAs each hold whole heads of a few tokens, and take any even rope_dim; more than
// 128 tokens are an accumulator's rows, whose threads rotate all of a head or nothing.
HYMT2_API int hymt2_gemm_tc_rope_kv_supported(int T, int N, int K, int rope_dim) {
    if (T <= 0 || N <= 0 || N % TILE_M || K <= 0 || K % 8) return 0;
    Plan pl;
    make_plan(T, N, K, EPI_ROPE_KV, sm_count_of_current_device(), &pl);
    if (pl.swapped) return (pl.cluster && pl.bn <= 64) ? 1 : 0;
    return (rope_dim == 0 || rope_dim == TILE_M) ? 1 : 0;   // tokens as rows: a thread rotates its token's whole head
}

// Whether hymt2_gemm_tc_rope_kv wants `angles`, the table that hymt2_rope_angles makes of the step's positions: where
// tokens are the accumulator's rows and are rotated.
HYMT2_API int hymt2_gemm_tc_rope_kv_wants_angles(int T, int rope_dim) { return (T > TILE_M && rope_dim > 0) ? 1 : 0; }

// The fused q/k/v projection of a few tokens with everything that follows it up to the cache: q_out[T, nh*128] gets the
// rotated (and normed) queries, the cache planes get the rotated (and normed) keys and the values of every token whose
// batch row has a slot.  X[T, K] (lda), W[(nh + 2 nkv) * 128, K] (ldw), both bfloat16; head_dim is 128.
HYMT2_API int hymt2_gemm_tc_rope_kv(const void* X, const void* W, int T, int K, long lda, long ldw, void* q_out, void* k_cache,
                                    void* v_cache, const int* block_table, int table_stride, int block_tokens,
                                    const int* token_seq, const int* token_pos, const int* slot_ids, const float* inv_freq,
                                    const float* angles, int rope_dim, const void* q_gain, const void* k_gain, int gain_dtype,
                                    float eps, int nh, int nkv, int write_kv, int* status, cudaStream_t stream,
                                    const float* ss_in, int ss_in_tiles, int ss_width, float ss_eps) {
    if (T == 0) return HYMT2_OK;
    const int N = (nh + 2 * nkv) * TILE_M;
    HYMT2_REQUIRE(!ss_in || (ss_in_tiles > 0 && ss_width > 0), "gemm_tc_rope_kv: bad row-scale arguments");
    HYMT2_REQUIRE(T > 0 && nh > 0 && nkv > 0 && K > 0, "gemm_tc_rope_kv: bad sizes T=%d nh=%d nkv=%d K=%d", T, nh, nkv, K);
    HYMT2_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_tc_rope_kv: K, lda and ldw must be multiples of 8");
    HYMT2_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc_rope_kv: operands must be 16-byte aligned");
    HYMT2_REQUIRE(rope_dim >= 0 && rope_dim <= TILE_M && rope_dim % 2 == 0, "gemm_tc_rope_kv: rope_dim %d must be even and at most 128", rope_dim);
    HYMT2_REQUIRE(rope_dim == 0 || inv_freq, "gemm_tc_rope_kv: rope_dim %d needs a frequency table", rope_dim);
    HYMT2_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "gemm_tc_rope_kv: q and k gains come together");
    HYMT2_REQUIRE(!q_gain || gain_dtype == HYMT2_BF16 || gain_dtype == HYMT2_F32, "gemm_tc_rope_kv: gains must be bfloat16 or float32");
    HYMT2_REQUIRE(block_tokens > 0 && q_out && status, "gemm_tc_rope_kv: missing arguments");
    HYMT2_REQUIRE(!write_kv || (k_cache && v_cache), "gemm_tc_rope_kv: the cache planes are needed to write keys and values");
    HYMT2_REQUIRE(hymt2_gemm_tc_rope_kv_supported(T, N, K, rope_dim), "gemm_tc_rope_kv: T=%d N=%d K=%d rope_dim=%d is not taken", T, N, K, rope_dim);
    Plan pl;
    make_plan(T, N, K, EPI_ROPE_KV, sm_count_of_current_device(), &pl);
    CUtensorMap ma, mb;
    const bool maps = pl.swapped ? make_map(&ma, W, N, K, ldw, TILE_M) && make_map(&mb, X, T, K, lda, pl.bn)
                                 : make_map(&ma, X, T, K, lda, TILE_M) && make_map(&mb, W, N, K, ldw, pl.bn);
    HYMT2_REQUIRE(maps, "gemm_tc_rope_kv: cuTensorMapEncodeTiled refused the operands");
    HYMT2_REQUIRE(!hymt2_gemm_tc_rope_kv_wants_angles(T, rope_dim) || (angles && (uintptr_t)angles % 16 == 0),
                  "gemm_tc_rope_kv: %d tokens are the accumulator's rows and need the table of their angles (hymt2_rope_angles)", T);
    RopeEpilogue rope{(__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, block_table, token_seq, token_pos,
                      slot_ids, inv_freq, angles, q_gain, k_gain, table_stride, block_tokens, nh, nkv, rope_dim, write_kv,
                      gain_dtype == HYMT2_BF16 ? 1 : 0, eps};
    GemmTcParams p{nullptr, 0, T, N, K, pl.stages, pl.bn, pl.splits, pl.k_blocks_per_split, pl.cluster ? 1 : 0, nullptr, nullptr, status, rope,
                   WAIT_LIMIT, -1, NormSide{nullptr, nullptr, 0, nullptr, 0, ss_in, ss_in_tiles, ss_width, ss_eps}};
    if (pl.persistent) {
        const int ctas = pl.tiles < pl.sm_count ? pl.tiles : pl.sm_count;
        return launch_persistent_one<PERSISTENT_BN, EPI_ROPE_KV, __nv_bfloat16>(ma, mb, p, ctas, pl.smem, stream);
    }
    switch (pl.bn) {
        case 16: return launch<16, EPI_ROPE_KV, __nv_bfloat16>(ma, mb, p, pl.grid, pl.smem, stream);
        case 32: return launch<32, EPI_ROPE_KV, __nv_bfloat16>(ma, mb, p, pl.grid, pl.smem, stream);
        default: return launch<64, EPI_ROPE_KV, __nv_bfloat16>(ma, mb, p, pl.grid, pl.smem, stream);
    }
}
