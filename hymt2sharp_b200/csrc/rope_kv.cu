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
    pdl_launch_dependents();
    pdl_wait();
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

}  // namespace

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
    HYMT2_DISPATCH_DTYPE(dtype, T, HYMT2_DISPATCH_DTYPE(gain_dtype, TG,
        (launch_pdl(rope_kv_kernel<T, TG>, dim3(blocks), dim3(128), smem, stream, p, tokens))));
    return hymt2_check_launch("rope_kv");
}
