// Rotary position encoding, per-head RMSNorm of q and k, and the append of k and v
// to the paged cache, in one pass over the fused QKV projection.
//
// For every token t and head: rotate-half rotation with angle = pos * inv_freq[i]
// as a float32 product (src/HyMT2Sharp/Ops.cs:98-195; pairs (i, i+half) :159-164;
// dims at and beyond rope_dim unchanged), then, if gains are given, RMSNorm over
// the head's d values AFTER the rotation
// (src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:53-58), then q goes to its own
// tensor and k, v go to the cache row of (slot, position)
// (src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:60-61).  All arithmetic is float32.
//
// Cache layout of one plane (one layer's keys or values):
//   [block][kv head][token in block][d]
// `block_table[slot * table_stride + pos / block_tokens]` names the block.
// A token whose batch row has slot < 0 is padding: its q is written, its k and v
// are dropped.
#include "common.cuh"

#include <type_traits>

namespace {

struct RopeKvParams {
    const void* qkv;      // [T, (nh + 2 nkv) * d]
    void* q_out;          // [T, nh * d]
    void* k_cache;        // plane base
    void* v_cache;
    const int* block_table;
    const int* token_seq;   // [T] batch row of each token
    const int* token_pos;   // [T] absolute position of each token
    const int* slot_ids;    // [B]
    const float* inv_freq;  // [rope_dim / 2] or null when rope_dim == 0
    const void* q_gain;     // [d] or null
    const void* k_gain;     // [d] or null
    int table_stride, block_tokens, nh, nkv, d, rope_dim, write_kv;
    float eps;
};

template <typename T, typename TG>
__global__ void __launch_bounds__(128)
rope_kv_kernel(RopeKvParams p, int tokens) {
    extern __shared__ float smem[];  // [4 warps][d]
    // Wait first, release after: the attention kernel that follows reads lengths, tables and old cache
    // blocks before its own wait, which is only safe once everything in front of THIS kernel is complete.
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* row = smem + warp * p.d;
    const int total_heads = p.nh + 2 * p.nkv;
    // one warp per (token, head)
    const long item = (long)blockIdx.x * 4 + warp;
    if (item >= (long)tokens * total_heads) return;
    const int t = (int)(item / total_heads), head = (int)(item % total_heads);
    const int d = p.d, half = p.rope_dim / 2;
    const int pos = p.token_pos[t];
    const int slot = p.slot_ids[p.token_seq[t]];
    const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
    const bool write_kv = p.write_kv && slot >= 0;
    if (!is_q && !write_kv) return;
    const T* src = (const T*)p.qkv + ((size_t)t * total_heads + head) * d;

    size_t cache_row = 0;
    if (!is_q) {
        const int block = p.block_table[(size_t)slot * p.table_stride + pos / p.block_tokens];
        const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
        cache_row = (((size_t)block * p.nkv + kvh) * p.block_tokens + (pos % p.block_tokens)) * d;
    }
    if (!is_q && !is_k) {  // value head: a plain copy into the cache
        T* dst = (T*)p.v_cache + cache_row;
        for (int c = lane; c < d; c += 32) dst[c] = src[c];
        return;
    }
    for (int c = lane; c < d; c += 32) row[c] = to_float(src[c]);
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
        const float angle = (float)pos * p.inv_freq[i];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float x0 = row[i], x1 = row[i + half];
        row[i] = x0 * cs - x1 * sn;
        row[i + half] = x0 * sn + x1 * cs;
    }
    __syncwarp();
    const TG* gain = (const TG*)(is_q ? p.q_gain : p.k_gain);
    float scale = 1.f;
    if (gain) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) ss = fmaf(row[c], row[c], ss);
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)d + p.eps);
    }
    T* dst = is_q ? (T*)p.q_out + ((size_t)t * p.nh + head) * d : (T*)p.k_cache + cache_row;
    for (int c = lane; c < d; c += 32) {
        float v = row[c];
        if (gain) v = v * scale * to_float(gain[c]);
        dst[c] = from_float<T>(v);
    }
}

// bfloat16 with the whole head rotated (rope_dim == d, d = 64, 128 or 256): one warp per (token, head),
// every lane holds E = d / 32 neighbouring values (one 4-, 8- or 16-byte load), the partner of a value
// sits 16 lanes away, the sum of squares is a warp sum, nothing goes through shared memory.
template <int E, typename TG>
__global__ void __launch_bounds__(128)
rope_kv_vec_kernel(RopeKvParams p, int tokens) {
    // Wait first, release after: the attention kernel that follows reads lengths, tables and old cache
    // blocks before its own wait, which is only safe once everything in front of THIS kernel is complete.
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_heads = p.nh + 2 * p.nkv;
    const long item = (long)blockIdx.x * 4 + warp;
    if (item >= (long)tokens * total_heads) return;
    const int t = (int)(item / total_heads), head = (int)(item % total_heads);
    constexpr int D = 32 * E;
    const int pos = p.token_pos[t];
    const int slot = p.slot_ids[p.token_seq[t]];
    const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
    const bool write_kv = p.write_kv && slot >= 0;
    if (!is_q && !write_kv) return;
    using Vec = typename std::conditional<E == 2, uint32_t, typename std::conditional<E == 4, uint2, uint4>::type>::type;
    const __nv_bfloat16* src = (const __nv_bfloat16*)p.qkv + ((size_t)t * total_heads + head) * D + lane * E;
    size_t cache_row = 0;
    if (!is_q) {
        const int block = p.block_table[(size_t)slot * p.table_stride + pos / p.block_tokens];
        const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
        cache_row = (((size_t)block * p.nkv + kvh) * p.block_tokens + (pos % p.block_tokens)) * D + lane * E;
    }
    Vec raw = *reinterpret_cast<const Vec*>(src);
    if (!is_q && !is_k) {
        *reinterpret_cast<Vec*>((__nv_bfloat16*)p.v_cache + cache_row) = raw;
        return;
    }
    float x[E];
    const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < E; i++) x[i] = __bfloat162float(rb[i]);
    const bool low = lane < 16;                      // holds x[i] of the pairs (i, i + d/2); else x[i + d/2]
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < E; i++) {
        const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
        const float angle = (float)pos * p.inv_freq[(lane & 15) * E + i];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float x0 = low ? x[i] : other, x1 = low ? other : x[i];
        x[i] = low ? x0 * cs - x1 * sn : x0 * sn + x1 * cs;
        ss = fmaf(x[i], x[i], ss);
    }
    const TG* gain = (const TG*)(is_q ? p.q_gain : p.k_gain);
    if (gain) {
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)D + p.eps);
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = x[i] * scale * to_float(gain[lane * E + i]);
    }
    Vec outv;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&outv);
#pragma unroll
    for (int i = 0; i < E; i++) ob[i] = __float2bfloat16_rn(x[i]);
    __nv_bfloat16* dst = is_q ? (__nv_bfloat16*)p.q_out + ((size_t)t * p.nh + head) * D + lane * E
                              : (__nv_bfloat16*)p.k_cache + cache_row;
    *reinterpret_cast<Vec*>(dst) = outv;
}

// out[t][i] = (cos, sin) of (float)pos[t] * inv_freq[i]: the angles of a step's tokens, the same float32 product and
// the same functions as in the kernels above, for the epilogue of a projection whose threads own whole tokens and
// would otherwise compute every angle once per head and layer.
__global__ void __launch_bounds__(128)
rope_angles_kernel(float2* out, const int* token_pos, const float* inv_freq, int tokens, int half) {
    pdl_wait();
    pdl_launch_dependents();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)tokens * half) return;
    float sn, cs;
    sincosf((float)token_pos[i / half] * inv_freq[i % half], &sn, &cs);
    out[i] = make_float2(cs, sn);
}

}  // namespace

HYMT2_API int hymt2_rope_angles(float* out, const int* token_pos, const float* inv_freq, int tokens, int half,
                                cudaStream_t stream) {
    if (tokens == 0 || half == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && half > 0 && out && token_pos && inv_freq, "rope_angles: bad arguments");
    HYMT2_REQUIRE((uintptr_t)out % 16 == 0, "rope_angles: the table must be 16-byte aligned");
    const long items = (long)tokens * half;
    launch_pdl(rope_angles_kernel, dim3((unsigned)((items + 127) / 128)), dim3(128), 0, stream, (float2*)out, token_pos,
               inv_freq, tokens, half);
    return hymt2_check_launch("rope_angles");
}

HYMT2_API int hymt2_rope_kv(const void* qkv, void* q_out, void* k_cache, void* v_cache, int dtype,
                            const int* block_table, int table_stride, int block_tokens,
                            const int* token_seq, const int* token_pos, const int* slot_ids,
                            const float* inv_freq, int rope_dim, const void* q_gain, const void* k_gain,
                            int gain_dtype, float eps, int tokens, int nh, int nkv, int d, int write_kv,
                            cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && nh > 0 && nkv > 0 && d > 0, "rope_kv: bad sizes");
    HYMT2_REQUIRE(rope_dim >= 0 && rope_dim <= d && rope_dim % 2 == 0, "rope_kv: rope_dim %d must be even and <= head_dim %d", rope_dim, d);
    HYMT2_REQUIRE(rope_dim == 0 || inv_freq, "rope_kv: rope_dim %d needs a frequency table", rope_dim);
    HYMT2_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "rope_kv: q and k gains come together");
    HYMT2_REQUIRE(block_tokens > 0, "rope_kv: block_tokens must be positive");
    RopeKvParams p{qkv, q_out, k_cache, v_cache, block_table, token_seq, token_pos, slot_ids, inv_freq,
                   q_gain, k_gain, table_stride, block_tokens, nh, nkv, d, rope_dim, write_kv, eps};
    const size_t smem = (size_t)4 * d * sizeof(float);
    HYMT2_REQUIRE(smem <= 48 * 1024, "rope_kv: head_dim %d is too large", d);
    const long items = (long)tokens * (nh + 2 * nkv);
    HYMT2_REQUIRE((items + 3) / 4 <= 2147483647L, "rope_kv: too many (token, head) pairs");
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (dtype == HYMT2_BF16 && rope_dim == d && (d == 64 || d == 128 || d == 256) && (uintptr_t)qkv % 16 == 0 &&
        (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0) {
#define HYMT2_ROPE_VEC(E_)                                                                                          \
        if (gain_dtype == HYMT2_BF16) launch_pdl(rope_kv_vec_kernel<E_, __nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, p, tokens); \
        else launch_pdl(rope_kv_vec_kernel<E_, float>, dim3(blocks), dim3(128), 0, stream, p, tokens)
        if (d == 64) { HYMT2_ROPE_VEC(2); } else if (d == 128) { HYMT2_ROPE_VEC(4); } else { HYMT2_ROPE_VEC(8); }
#undef HYMT2_ROPE_VEC
        return hymt2_check_launch("rope_kv");
    }
    HYMT2_DISPATCH_DTYPE(dtype, T, HYMT2_DISPATCH_DTYPE(gain_dtype, TG,
        (launch_pdl(rope_kv_kernel<T, TG>, dim3(blocks), dim3(128), smem, stream, p, tokens))));
    return hymt2_check_launch("rope_kv");
}
