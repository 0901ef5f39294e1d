// Decode attention in bfloat16: one new token per sequence attends over its paged cache.
// The step is bound by the bytes of keys and values that it must read, so the kernel is
// built around memory traffic: every key and value element goes from global memory
// straight into the registers of the one thread that uses it (16-byte loads, the next
// pair of keys in flight while the current pair is used), and is applied to all query
// heads of its kv group at once, so the cache is read once per kv head, not once per head.
//
// Work of one CTA: (chunk of 256 keys, kv head x group of G query heads, sequence).  A warp
// owns 64 of the keys; inside a warp 8 lanes share a key and each holds d/8 of its values.
// Scores, softmax and the weighted sum are float32; the running maximum and sum follow the
// same formulas as the general kernel (src/HyMT2Sharp/Ops.cs:462-532 is the reference's fused
// decode attention).  Each CTA writes an unnormalised partial (acc, max, sum) per head to
// scratch; the merge kernel of attention_simt.cu folds the chunks in index order.  The chunk
// size is a constant, so the cut depends on a key's index only.
//
// Takes head sizes 64 and 128 and any number of heads and groups; other shapes stay with the
// general kernel.
#include "common.cuh"

namespace {

constexpr int CHUNK_KEYS = 256, WARPS = 4, LANES_PER_KEY = 8, KEYS_PER_ITER = 4;

struct DecodeParams {
    const __nv_bfloat16* q;        // [rows, nh * d]
    const __nv_bfloat16* k_cache;  // [block][nkv][block_tokens][d]
    const __nv_bfloat16* v_cache;
    const int* block_table;
    const int* slot_ids;
    const int* kv_lens;
    __nv_bfloat16* out;            // [rows, nh * d]
    float* part_acc;               // [rows, nh, max_splits, d]
    float* part_ml;                // [rows, nh, max_splits, 2]
    int* counters;                 // [rows, nkv * groups] arrivals of a row's chunks, zero between launches
    int table_stride, block_shift, nh, nkv, window, max_splits;   // block_tokens = 1 << block_shift
    float scale;
};

template <int E>
__device__ __forceinline__ void load_row(const __nv_bfloat16* p, uint4 (&raw)[E / 8], bool ok) {
#pragma unroll
    for (int i = 0; i < E / 8; i++)
        raw[i] = ok ? __ldg(reinterpret_cast<const uint4*>(p) + i) : make_uint4(0, 0, 0, 0);
}

template <int E>
__device__ __forceinline__ void unpack(const uint4 (&raw)[E / 8], float (&f)[E]) {
#pragma unroll
    for (int i = 0; i < E / 8; i++) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // a bfloat16 is the upper half of a float32
            f[i * 8 + 2 * j] = __uint_as_float(w[j] << 16);
            f[i * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

template <int D, int G>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(DecodeParams p) {
    constexpr int E = D / LANES_PER_KEY;   // elements of a key that one lane holds
    constexpr int KEYS_PER_WARP = CHUNK_KEYS / WARPS;
    constexpr int ITERS = KEYS_PER_WARP / KEYS_PER_ITER;   // 16 keys per lane group
    constexpr int PF = 4;                  // keys in flight per lane group
    __shared__ float sm_p[WARPS][KEYS_PER_WARP][G];        // scores, then softmax numerators
    __shared__ float sm_acc[WARPS][G][D];
    __shared__ float sm_ml[WARPS][G][2];
    pdl_launch_dependents();
    pdl_wait();
    const int split = blockIdx.x, b = blockIdx.z;
    const int slot = p.slot_ids[b];
    if (slot < 0) return;
    const int kv_len = p.kv_lens[b];
    const int pos = kv_len - 1;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int chunk_begin = split * CHUNK_KEYS;
    if (chunk_begin > pos || chunk_begin + CHUNK_KEYS <= lo) return;   // no visible key here: the merge skips it
    const int g = p.nh / p.nkv, groups = g / G;
    const int kvh = blockIdx.y / groups, head0 = kvh * g + (blockIdx.y % groups) * G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LANES_PER_KEY, keygrp = lane / LANES_PER_KEY;
    const int* table = p.block_table + (size_t)slot * p.table_stride;
    const int warp_begin = chunk_begin + warp * KEYS_PER_WARP;

    auto address = [&](int it, bool& ok) -> size_t {   // the row of this lane group's key of iteration `it`
        const int key = warp_begin + it * KEYS_PER_ITER + keygrp;
        ok = key >= lo && key <= pos;
        if (!ok) return 0;
        const int block = table[key >> p.block_shift];
        return ((((size_t)block * p.nkv + kvh) << p.block_shift) + (key & ((1 << p.block_shift) - 1))) * D + sub * E;
    };

    // ---- pass 1: scores of the warp's 64 keys; only q and the keys in flight are live --------
    float m[G];
    {
        float q[G][E];
#pragma unroll
        for (int h = 0; h < G; h++) {
            uint4 raw[E / 8];
            load_row<E>(p.q + ((size_t)b * p.nh + head0 + h) * D + sub * E, raw, true);
            unpack<E>(raw, q[h]);
#pragma unroll
            for (int e = 0; e < E; e++) q[h][e] *= p.scale;
            m[h] = -INFINITY;
        }
        uint4 kraw[PF][E / 8];
        bool okv[PF];
#pragma unroll
        for (int i = 0; i < PF; i++) {
            const size_t a = address(i, okv[i]);
            load_row<E>(p.k_cache + a, kraw[i], okv[i]);
        }
#pragma unroll
        for (int it = 0; it < ITERS; it++) {
            const int st = it % PF;
            float kf[E];
            unpack<E>(kraw[st], kf);
            const bool ok = okv[st];
            if (it + PF < ITERS) {   // the freed registers take the key that is PF iterations ahead
                const size_t a = address(it + PF, okv[st]);
                load_row<E>(p.k_cache + a, kraw[st], okv[st]);
            }
            float s[G];
#pragma unroll
            for (int h = 0; h < G; h++) {
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < E; e++) dot = fmaf(q[h][e], kf[e], dot);
                s[h] = dot;
            }
#pragma unroll
            for (int o = 1; o < LANES_PER_KEY; o <<= 1)
#pragma unroll
                for (int h = 0; h < G; h++) s[h] += __shfl_xor_sync(0xffffffffu, s[h], o);
#pragma unroll
            for (int h = 0; h < G; h++) {
                if (!ok) s[h] = -INFINITY;
                m[h] = fmaxf(m[h], s[h]);
            }
            if (sub < G) sm_p[warp][it * KEYS_PER_ITER + keygrp][sub] = s[sub < G ? sub : 0];
        }
    }
    // the warp's maximum per head, then numerators and their sum
#pragma unroll
    for (int o = LANES_PER_KEY; o < 32; o <<= 1)
#pragma unroll
        for (int h = 0; h < G; h++) m[h] = fmaxf(m[h], __shfl_xor_sync(0xffffffffu, m[h], o));
    __syncwarp();
    float l[G];
#pragma unroll
    for (int h = 0; h < G; h++) l[h] = 0.f;
    for (int i = lane; i < KEYS_PER_WARP * G; i += 32) {
        const int key = i / G, h = i - key * G;
        float mh = m[0];
#pragma unroll
        for (int hh = 1; hh < G; hh++) mh = h == hh ? m[hh] : mh;
        const float s = sm_p[warp][key][h];
        const float pj = mh == -INFINITY ? 0.f : expf(s - mh);   // a masked key has s = -inf: 0
        sm_p[warp][key][h] = pj;
#pragma unroll
        for (int hh = 0; hh < G; hh++) l[hh] += h == hh ? pj : 0.f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int h = 0; h < G; h++) l[h] += __shfl_xor_sync(0xffffffffu, l[h], o);
    __syncwarp();

    // ---- pass 2: weighted sum of the values; only the accumulators and the values in flight ----
    float acc[G][E];
#pragma unroll
    for (int h = 0; h < G; h++)
#pragma unroll
        for (int e = 0; e < E; e++) acc[h][e] = 0.f;
    {
        uint4 vraw[PF][E / 8];
        bool okv[PF];
#pragma unroll
        for (int i = 0; i < PF; i++) {
            const size_t a = address(i, okv[i]);
            load_row<E>(p.v_cache + a, vraw[i], okv[i]);
        }
#pragma unroll
        for (int it = 0; it < ITERS; it++) {
            const int st = it % PF;
            float vf[E];
            unpack<E>(vraw[st], vf);
            if (it + PF < ITERS) {
                const size_t a = address(it + PF, okv[st]);
                load_row<E>(p.v_cache + a, vraw[st], okv[st]);
            }
            const float* pr = sm_p[warp][it * KEYS_PER_ITER + keygrp];   // 0 for keys that are not visible
#pragma unroll
            for (int h = 0; h < G; h++) {
                const float pj = pr[h];
#pragma unroll
                for (int e = 0; e < E; e++) acc[h][e] = fmaf(pj, vf[e], acc[h][e]);
            }
        }
    }
    // fold the 4 key groups of a warp (they share the warp's maximum), then the 4 warps, in a fixed order
#pragma unroll
    for (int o = LANES_PER_KEY; o < 32; o <<= 1)
#pragma unroll
        for (int h = 0; h < G; h++)
#pragma unroll
            for (int e = 0; e < E; e++) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], o);
    if (keygrp == 0) {
#pragma unroll
        for (int h = 0; h < G; h++) {
#pragma unroll
            for (int e = 0; e < E; e++) sm_acc[warp][h][sub * E + e] = acc[h][e];
            if (sub == 0) { sm_ml[warp][h][0] = m[h]; sm_ml[warp][h][1] = l[h]; }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
        const int h = i / D, x = i - h * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; w++) M = fmaxf(M, sm_ml[w][h][0]);
        float L = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) {
            const float c = M == -INFINITY ? 0.f : expf(sm_ml[w][h][0] - M);
            L += sm_ml[w][h][1] * c;
            a += sm_acc[w][h][x] * c;
        }
        const size_t row = ((size_t)b * p.nh + head0 + h) * p.max_splits + split;
        p.part_acc[row * D + x] = a;
        if (x == 0) { p.part_ml[row * 2] = M; p.part_ml[row * 2 + 1] = L; }
    }

    // the chunk that arrives last folds all chunks of its heads, in chunk order
    const int s_begin = lo / CHUNK_KEYS, s_end = pos / CHUNK_KEYS + 1;
    __shared__ int last_s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.counters + (size_t)b * gridDim.y + blockIdx.y;
        const int arrived = atomicAdd(counter, 1);
        last_s = arrived == s_end - s_begin - 1;
        if (last_s) *counter = 0;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
        const int h = i / D, x = i - h * D;
        const size_t row = ((size_t)b * p.nh + head0 + h) * p.max_splits;
        float M = -INFINITY;
        for (int s = s_begin; s < s_end; s++) M = fmaxf(M, __ldcg(p.part_ml + (row + s) * 2));
        float L = 0.f, a = 0.f;
        for (int s = s_begin; s < s_end; s++) {
            const float c = expf(__ldcg(p.part_ml + (row + s) * 2) - M);
            L += __ldcg(p.part_ml + (row + s) * 2 + 1) * c;
            a = fmaf(__ldcg(p.part_acc + (row + s) * D + x), c, a);
        }
        p.out[((size_t)b * p.nh + head0 + h) * D + x] = __float2bfloat16_rn(L > 0.f ? a / L : 0.f);
    }
}

template <int D>
int launch_d(const DecodeParams& p, int rows, int g, int splits, cudaStream_t stream) {
    const int G = g % 4 == 0 ? 4 : g % 2 == 0 ? 2 : 1;
    dim3 grid(splits, p.nkv * (g / G), rows);
    if (G == 4) launch_pdl(attention_decode_kernel<D, 4>, grid, dim3(WARPS * 32), 0, stream, p);
    else if (G == 2) launch_pdl(attention_decode_kernel<D, 2>, grid, dim3(WARPS * 32), 0, stream, p);
    else launch_pdl(attention_decode_kernel<D, 1>, grid, dim3(WARPS * 32), 0, stream, p);
    return hymt2_check_launch("attention_decode");
}

}  // namespace

// out, q: [rows, nh * d] bfloat16; one new token per row.  max_splits >= ceil(longest kv_len / 256);
// part_acc holds rows*nh*max_splits*d floats, part_ml rows*nh*max_splits*2, counters rows*nh ints
// that are zero before the first launch (the kernel leaves them zero).
HYMT2_API int hymt2_attention_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                                     const int* block_table, int table_stride, int block_tokens, const int* cu_seqlens,
                                     const int* slot_ids, const int* kv_lens, int rows, int nh, int nkv, int d, float scale,
                                     int window, int max_splits, float* part_acc, float* part_ml, int* counters,
                                     cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad sizes");
    HYMT2_REQUIRE(d == 64 || d == 128, "attention_decode: head_dim %d is not taken (64 and 128 are)", d);
    HYMT2_REQUIRE(max_splits > 0 && part_acc && part_ml && counters, "attention_decode: scratch for the partials is needed");
    int block_shift = 0;
    while ((1 << block_shift) < block_tokens) block_shift++;
    HYMT2_REQUIRE((1 << block_shift) == block_tokens, "attention_decode: block_tokens %d must be a power of two", block_tokens);
    HYMT2_REQUIRE(rows <= 65535 && nkv * (nh / nkv) <= 65535, "attention_decode: grid too large");
    DecodeParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
                   slot_ids, kv_lens, (__nv_bfloat16*)out, part_acc, part_ml, counters, table_stride, block_shift, nh, nkv, window, max_splits, scale};
    const int g = nh / nkv;
    (void)cu_seqlens;
    return d == 128 ? launch_d<128>(p, rows, g, max_splits, stream) : launch_d<64>(p, rows, g, max_splits, stream);
}
