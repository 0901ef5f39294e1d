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
// cache once per kv head (all heads of the group share it).  The chunk that arrives last
// at a row's counter folds all chunks of its heads in chunk order.
// Formulas: src/HyMT2Sharp/Ops.cs:462-532 (the reference's fused decode attention).
#include "common.cuh"

#include <cuda.h>

namespace {

constexpr int CHUNK = 128, BLOCK_KEYS = 64, D = 128, NQ = 16, NUM_THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 21;

struct DecodeTcParams {
    __nv_bfloat16* out;        // [rows, nh * d]
    const int* block_table;
    const int* slot_ids;
    const int* kv_lens;
    float* part_acc;           // [rows, nh, max_splits, d]
    float* part_ml;            // [rows, nh, max_splits, 2]  (maximum in log2 units, sum)
    int* counters;             // [rows, nkv]
    int table_stride, nh, nkv, window, max_splits;
    float scale_log2;
    int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(status, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t mn_group_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(mn_group_bytes >> 4) << 16) | (64ull << 32) | (1ull << 46) |
           (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int G>   // query heads per kv head that the softmax loops cover (the group size rounded up)
__global__ void __launch_bounds__(NUM_THREADS)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, DecodeTcParams p) {
    // shared memory: K [d half][128 keys x 128 B], V [key block][d half][64 keys x 128 B],
    // Q [d half][16 x 128 B], P^T [key block][16 x 128 B]
    constexpr int K_BYTES = CHUNK * D * 2, V_BYTES = CHUNK * D * 2, Q_BYTES = NQ * D * 2;
    constexpr int HALF_K = CHUNK * 128, BOX = BLOCK_KEYS * 128;
    constexpr uint32_t S_COL = 0, O_COL = 16, TMEM_COLS = 32;
    // D float32, A and B bfloat16, N = 16, M = 128; S^T: both K-major; O^T: A (V^T) is MN-major
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NQ >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    constexpr uint32_t IDESC_O = IDESC_S | (1u << 15);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s, last_s;
    __shared__ float red_max[4][NQ], red_sum[4][NQ];

    pdl_launch_dependents();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t k_smem = base, v_smem = k_smem + K_BYTES, q_smem = v_smem + V_BYTES, p_smem = q_smem + Q_BYTES;
    const uint32_t kq_full = smem_u32(&bars[0]), v_full = kq_full + 8, s_done = kq_full + 16, p_ready = kq_full + 24;
    volatile int* abort_flag = &abort_s;
    pdl_wait();   // q, the cache and the lengths come from the kernels before

    const int slot = p.slot_ids[b];
    if (slot < 0) return;
    const int kv_len = p.kv_lens[b], pos = kv_len - 1;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int chunk_begin = split * CHUNK;
    if (chunk_begin > pos || chunk_begin + CHUNK <= lo) return;   // no visible key here: the merge skips it
    const int g = p.nh / p.nkv, head0 = kvh * g;
    const int blocks_here = min(2, (pos - chunk_begin) / BLOCK_KEYS + 1);   // cache blocks of the chunk that hold keys

    if (threadIdx.x == 0) {
        mbar_init(kq_full, 1);
        mbar_init(v_full, 1);
        mbar_init(s_done, 1);
        mbar_init(p_ready, 128);
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
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ---- producer: everything at once ------------------------------------------------------
        const int* table = p.block_table + (size_t)slot * p.table_stride;
        mbar_expect_tx(kq_full, Q_BYTES + blocks_here * BOX * 2);
        mbar_expect_tx(v_full, blocks_here * BOX * 2);
        for (int x = 0; x < 2; x++) tma_load_2d(q_smem + x * (NQ * 128), &map_q, kq_full, x * 64, b * p.nh + head0);
        for (int kb = 0; kb < blocks_here; kb++) {
            const int block = table[chunk_begin / BLOCK_KEYS + kb];
            const int row = (block * p.nkv + kvh) * BLOCK_KEYS;
            for (int x = 0; x < 2; x++) tma_load_2d(k_smem + x * HALF_K + kb * BOX, &map_k, kq_full, x * 64, row);
            for (int x = 0; x < 2; x++) tma_load_2d(v_smem + (kb * 2 + x) * BOX, &map_v, v_full, x * 64, row);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------------
        if (mbar_wait(kq_full, 0, abort_flag, p.status, 121)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k = 0; k < D / 16; k++) {
                const uint32_t half = k / 4, in_box = (k % 4) * 32;
                umma_bf16(tmem_base + S_COL, desc_k_major(k_smem + half * HALF_K + in_box),
                          desc_k_major(q_smem + half * (NQ * 128) + in_box), IDESC_S, k > 0 ? 1u : 0u);
            }
            umma_commit(s_done);
            if (mbar_wait(p_ready, 0, abort_flag, p.status, 122) && mbar_wait(v_full, 0, abort_flag, p.status, 123)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < blocks_here; kb++)
#pragma unroll
                    for (int k = 0; k < BLOCK_KEYS / 16; k++)
                        umma_bf16(tmem_base + O_COL, desc_mn_major(v_smem + kb * 2 * BOX + k * (16 * 128), BOX),
                                  desc_k_major(p_smem + kb * (NQ * 128) + k * 32), IDESC_O, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(kq_full);   // second phase of this barrier: O^T is complete
        }
    } else if (warp >= 2) {
        // ---- softmax: thread = key -------------------------------------------------------------------
        const int quarter = warp & 3, t = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int key = chunk_begin + t;
        const bool visible = key >= lo && key <= pos;
        float s[NQ];
        ok = mbar_wait(s_done, 0, abort_flag, p.status, 124);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_load16(lane_addr + S_COL, s);
#pragma unroll
        for (int h = 0; h < G; h++) s[h] = (visible && h < g) ? s[h] * p.scale_log2 : -INFINITY;
        // maximum per head over the 128 keys
        float mx[G];
#pragma unroll
        for (int h = 0; h < G; h++) {
            mx[h] = s[h];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
        }
        if (lane < G) {
            float mine = mx[0];
#pragma unroll
            for (int h = 1; h < G; h++) mine = lane == h ? mx[h] : mine;
            red_max[quarter][lane] = mine;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        float psum[G];
        const int kb = t / BLOCK_KEYS, kin = t % BLOCK_KEYS;
        // the rows of P^T beyond the group stay zero: their columns of O^T are never read, but must be finite
#pragma unroll
        for (int h = G; h < NQ; h++) {
            const uint32_t dst = p_smem + kb * (NQ * 128) + h * 128 + ((((uint32_t)kin >> 3) ^ (h & 7)) << 4) + (kin & 7) * 2;
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst), "h"((unsigned short)0) : "memory");
        }
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float M = fmaxf(fmaxf(red_max[0][h], red_max[1][h]), fmaxf(red_max[2][h], red_max[3][h]));
            const float pj = (M == -INFINITY || s[h] == -INFINITY) ? 0.f : exp2f(s[h] - M);
            const __nv_bfloat16 pb = __float2bfloat16_rn(pj);
            psum[h] = __bfloat162float(pb);   // the sum uses what the tensor core multiplies with
            mx[h] = M;
            // P^T[h][key]: row h of the block's 16 x 128 B tile, 16-byte chunk (kin / 8) ^ (h & 7)
            const uint32_t dst = p_smem + kb * (NQ * 128) + h * 128 + ((((uint32_t)kin >> 3) ^ (h & 7)) << 4) + (kin & 7) * 2;
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst), "h"(*reinterpret_cast<const unsigned short*>(&pb)) : "memory");
        }
        // rows of V at and past the sequence's length have never been written by this sequence:
        // their weight is 0, but 0 x (whatever bits lie there) must stay 0
        if (key >= kv_len && kb < blocks_here) {
            for (int x = 0; x < 2; x++) {
                const uint32_t rowp = v_smem + (kb * 2 + x) * BOX + kin * 128;
                if (x == 0 && !mbar_wait(v_full, 0, abort_flag, p.status, 125)) break;
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
            red_sum[quarter][lane] = mine;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(p_ready);
        // ---- epilogue: thread = d ----------------------------------------------------------------------
        ok = ok && mbar_wait(kq_full, 1, abort_flag, p.status, 126);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float o[NQ];
        tmem_load16(lane_addr + O_COL, o);
        asm volatile("bar.sync 1, 128;" ::: "memory");   // red_sum of all four warps is written
#pragma unroll
        for (int h = 0; h < G; h++) {
            if (h < g) {
                const size_t row = ((size_t)b * p.nh + head0 + h) * p.max_splits + split;
                p.part_acc[row * D + t] = ok ? o[h] : 0.f;
                if (t == h) {
                    p.part_ml[row * 2] = mx[h];
                    p.part_ml[row * 2 + 1] = red_sum[0][h] + red_sum[1][h] + red_sum[2][h] + red_sum[3][h];
                }
            }
        }
        // the chunk that arrives last folds all chunks of this kv head's heads, in chunk order
        const int s_begin = lo / CHUNK, s_end = pos / CHUNK + 1;
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (t == 0) {
            int* counter = p.counters + (size_t)b * p.nkv + kvh;
            const int arrived = atomicAdd(counter, 1);
            last_s = arrived == s_end - s_begin - 1;
            if (last_s) *counter = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (last_s) {
            __threadfence();
            // weights of the chunks first: (maximum, sum) of every (head, chunk) pair is read by one thread
            // each, all at once; then every thread folds its d over heads and chunks with the loads of
            // 16 chunks in flight at a time
            const int n_chunks = s_end - s_begin;
            float* w_s = reinterpret_cast<float*>(smem_raw);           // [g][n_chunks] weights, then [g] 1/L
            for (int base_i = 0; base_i < g * n_chunks; base_i += 128) {
                const int i = base_i + t;
                if (i < g * n_chunks) {
                    const int h = i / n_chunks, sp = s_begin + i % n_chunks;
                    const size_t row = ((size_t)b * p.nh + head0 + h) * p.max_splits + sp;
                    w_s[i] = __ldcg(p.part_ml + row * 2);                    // maxima for now
                    w_s[g * n_chunks + NQ + i] = __ldcg(p.part_ml + row * 2 + 1);   // sums
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (t < g) {
                float M = -INFINITY;
                for (int c = 0; c < n_chunks; c++) M = fmaxf(M, w_s[t * n_chunks + c]);
                float L = 0.f;
                for (int c = 0; c < n_chunks; c++) {
                    const float m_c = w_s[t * n_chunks + c];
                    const float wgt = m_c == -INFINITY ? 0.f : exp2f(m_c - M);
                    L += w_s[g * n_chunks + NQ + t * n_chunks + c] * wgt;
                    w_s[t * n_chunks + c] = wgt;
                }
                w_s[g * n_chunks + t] = L > 0.f ? 1.0f / L : 0.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int h = 0; h < g; h++) {
                const size_t row = ((size_t)b * p.nh + head0 + h) * p.max_splits + s_begin;
                float a = 0.f;
                for (int c0 = 0; c0 < n_chunks; c0 += 16) {
                    float pa[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) pa[j] = c0 + j < n_chunks ? __ldcg(p.part_acc + (row + c0 + j) * D + t) : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; j++) a = fmaf(pa[j], c0 + j < n_chunks ? w_s[h * n_chunks + c0 + j] : 0.f, a);
                }
                p.out[((size_t)b * p.nh + head0 + h) * D + t] = __float2bfloat16_rn(a * w_s[g * n_chunks + h]);
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

bool make_map(CUtensorMap* map, const void* base, long rows, long cols, long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// out, q: [rows, nh * 128] bfloat16, one new token per row; k_cache, v_cache: one layer's planes
// [blocks][nkv][64][128].  max_splits >= ceil(longest kv_len / 128); part_acc holds
// rows*nh*max_splits*128 floats, part_ml rows*nh*max_splits*2, counters rows*nkv zeroed ints.
HYMT2_API int hymt2_attention_decode_tc(void* out, const void* q, const void* k_cache, const void* v_cache,
                                        long cache_blocks, const int* block_table, int table_stride, int block_tokens,
                                        const int* slot_ids, const int* kv_lens, int rows, int nh, int nkv, int d,
                                        float scale, int window, int max_splits, float* part_acc, float* part_ml,
                                        int* counters, int* status, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(d == D, "attention_decode_tc: head_dim %d is not taken (128 is)", d);
    HYMT2_REQUIRE(block_tokens == BLOCK_KEYS, "attention_decode_tc: cache blocks must hold %d tokens", BLOCK_KEYS);
    HYMT2_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= NQ, "attention_decode_tc: at most %d heads per kv head", NQ);
    HYMT2_REQUIRE(rows <= 65535 && nkv <= 65535 && max_splits > 0, "attention_decode_tc: grid too large");
    HYMT2_REQUIRE(part_acc && part_ml && counters && status, "attention_decode_tc: scratch is needed");
    CUtensorMap mq, mk, mv;
    const long cache_rows = cache_blocks * nkv * BLOCK_KEYS;
    const bool ok = make_map(&mq, q, (long)rows * nh, d, d, NQ) && make_map(&mk, k_cache, cache_rows, d, d, BLOCK_KEYS) &&
                    make_map(&mv, v_cache, cache_rows, d, d, BLOCK_KEYS);
    HYMT2_REQUIRE(ok, "attention_decode_tc: cuTensorMapEncodeTiled refused the operands");
    DecodeTcParams p{(__nv_bfloat16*)out, block_table, slot_ids, kv_lens, part_acc, part_ml, counters, table_stride, nh, nkv,
                     window, max_splits, scale * 1.4426950408889634f, status};
    constexpr size_t smem = 2 * CHUNK * D * 2 + NQ * D * 2 + 2 * NQ * 128 + 1024;
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
    cudaError_t e = launch_pdl(kernel, dim3(max_splits, nkv, rows), dim3(NUM_THREADS), smem, stream, mq, mk, mv, p);
    if (e != cudaSuccess) { hymt2_set_error("attention_decode_tc: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
    return hymt2_check_launch("attention_decode_tc");
}
