// Causal grouped-query attention over the paged cache on CUDA cores, any head size
// that is a multiple of 8 up to 256, any number of heads and groups, any lengths.
// It serves the 32-bit path in prefill and decode, and the bfloat16 path where the
// tensor-core kernels refuse a shape.
//
// Query t of batch row b (the i-th of its T_b new tokens) sits at position
// p = kv_len_b - T_b + i and sees the keys j in [max(0, p - window + 1), p]
// (window <= 0: all of [0, p]); the new tokens' own keys are already in the cache.
// scores = (q·k) * scale with kv head = head / (nh / nkv)
// (src/HyMT2Sharp/Ops.cs:359-455, group :374, kvh :381); softmax over the visible
// keys in float32 with the row's true maximum (src/HyMT2Sharp/Ops.cs:198-325);
// out = sum_j p_j v_j (src/HyMT2Sharp/Ops.cs:535-595).
//
// A block owns up to 16 (token, head) rows that share one kv head and walks the
// keys in tiles of 32 with an online softmax.  With split_keys > 0 the keys are
// cut into chunks of split_keys (a constant, so the cut depends on nothing but
// the key's own index); each chunk's block writes an unnormalised partial and
// `attention_merge_kernel` folds the partials in chunk order.
#include "common.cuh"

namespace {

constexpr int ROWS = 16, LANES_PER_ROW = 8, KEY_TILE = 32, MAX_D = 256;

struct AttnParams {
    const void* q;        // [T, nh * d]
    void* out;            // [T, nh * d]
    const void* k_cache;  // plane base, [block][nkv][block_tokens][d]
    const void* v_cache;
    const int* block_table;
    const int* cu_seqlens;  // [B + 1] offsets of the batch rows' new tokens
    const int* slot_ids;    // [B]
    const int* kv_lens;     // [B] cached length including the new tokens
    float* part_acc;        // [T, nh, splits, d] when split
    float* part_ml;         // [T, nh, splits, 2]
    int table_stride, block_tokens, nh, nkv, d, window, tokens_per_tile, heads_per_tile, head_chunks;
    int split_keys, max_splits;
    float scale;
    int* status;            // may be null; [0] = 2 when a row is longer than max_splits * split_keys covers
};

template <typename T>
__global__ void __launch_bounds__(ROWS* LANES_PER_ROW)
attention_simt_kernel(AttnParams p) {
    extern __shared__ float smem[];
    const int d = p.d;
    float* Qs = smem;                          // [ROWS][d]
    float* Ks = Qs + ROWS * d;                 // [KEY_TILE][d + 1]
    float* Vs = Ks + KEY_TILE * (d + 1);       // [KEY_TILE][d]
    float* Ps = Vs + KEY_TILE * d;             // [ROWS][KEY_TILE]

    const int b = blockIdx.z / p.max_splits, split = blockIdx.z % p.max_splits;
    const int slot = p.slot_ids[b];
    if (slot < 0) return;
    const int tok0 = p.cu_seqlens[b], T_b = p.cu_seqlens[b + 1] - tok0;
    const int kv_len = p.kv_lens[b];
    const int tile_tok0 = blockIdx.x * p.tokens_per_tile;
    if (tile_tok0 >= T_b) return;
    const int g = p.nh / p.nkv;
    const int kvh = blockIdx.y / p.head_chunks, chunk = blockIdx.y % p.head_chunks;

    const int tid = threadIdx.x, r = tid / LANES_PER_ROW, c = tid % LANES_PER_ROW;
    const int row_tok = tile_tok0 + r / p.heads_per_tile;         // index among the row's new tokens
    const int head_in_group = chunk * p.heads_per_tile + r % p.heads_per_tile;
    const bool row_ok = r < p.tokens_per_tile * p.heads_per_tile && row_tok < T_b && head_in_group < g;
    const int head = kvh * g + head_in_group;
    const int row_pos = kv_len - T_b + row_tok;                   // absolute position of the query
    const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;

    // key range of the whole tile
    const int last_tok = min(T_b, tile_tok0 + p.tokens_per_tile) - 1;
    const int tile_hi = kv_len - T_b + last_tok;                  // inclusive
    const int first_pos = kv_len - T_b + tile_tok0;
    int key_begin = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    int key_end = tile_hi + 1;
    if (p.split_keys > 0) {
        key_begin = max(key_begin, split * p.split_keys);
        key_end = min(key_end, (split + 1) * p.split_keys);
    }

    // stage the queries
    for (int i = tid; i < ROWS * d; i += blockDim.x) {
        const int rr = i / d, x = i - rr * d;
        const int tk = tile_tok0 + rr / p.heads_per_tile;
        const int hg = chunk * p.heads_per_tile + rr % p.heads_per_tile;
        const bool ok = rr < p.tokens_per_tile * p.heads_per_tile && tk < T_b && hg < g;
        Qs[i] = ok ? to_float(((const T*)p.q)[((size_t)(tok0 + tk) * p.nh + kvh * g + hg) * d + x]) : 0.f;
    }

    float acc[MAX_D / LANES_PER_ROW];
#pragma unroll
    for (int i = 0; i < MAX_D / LANES_PER_ROW; i++) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int* table = p.block_table + (size_t)slot * p.table_stride;
    for (int k0 = (key_begin / KEY_TILE) * KEY_TILE; k0 < key_end; k0 += KEY_TILE) {
        __syncthreads();
        // a tile of 32 keys lies inside one block (block_tokens is a multiple of 32)
        const int block = table[k0 / p.block_tokens];
        const size_t base = (((size_t)block * p.nkv + kvh) * p.block_tokens + (k0 % p.block_tokens)) * d;
        const T* kp = (const T*)p.k_cache + base;
        const T* vp = (const T*)p.v_cache + base;
        const int valid = min(KEY_TILE, kv_len - k0);
        for (int i = tid; i < KEY_TILE * d; i += blockDim.x) {
            const int j = i / d, x = i - j * d;
            const bool ok = j < valid && block >= 0;
            Ks[j * (d + 1) + x] = ok ? to_float(kp[i]) : 0.f;
            Vs[i] = ok ? to_float(vp[i]) : 0.f;
        }
        __syncthreads();

        float s[KEY_TILE / LANES_PER_ROW];
        float tile_max = -INFINITY;
#pragma unroll
        for (int kk = 0; kk < KEY_TILE / LANES_PER_ROW; kk++) {
            const int j = c + kk * LANES_PER_ROW, key = k0 + j;
            float dot = 0.f;
            const float* qr = Qs + r * d;
            const float* kr = Ks + j * (d + 1);
            for (int x = 0; x < d; x++) dot = fmaf(qr[x], kr[x], dot);
            const bool visible = row_ok && key >= row_lo && key <= row_pos && key >= key_begin && key < key_end;
            s[kk] = visible ? dot * p.scale : -INFINITY;
            tile_max = fmaxf(tile_max, s[kk]);
        }
#pragma unroll
        for (int o = 1; o < LANES_PER_ROW; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
        const float m_new = fmaxf(m, tile_max);
        float corr = 1.f, psum = 0.f;
        if (m_new > -INFINITY) {
            corr = expf(m - m_new);  // m = -inf gives 0
#pragma unroll
            for (int kk = 0; kk < KEY_TILE / LANES_PER_ROW; kk++) {
                const float pj = expf(s[kk] - m_new);  // masked: exp(-inf) = 0
                Ps[r * KEY_TILE + c + kk * LANES_PER_ROW] = pj;
                psum += pj;
            }
        } else {
#pragma unroll
            for (int kk = 0; kk < KEY_TILE / LANES_PER_ROW; kk++) Ps[r * KEY_TILE + c + kk * LANES_PER_ROW] = 0.f;
        }
#pragma unroll
        for (int o = 1; o < LANES_PER_ROW; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l = l * corr + psum;
        m = m_new;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < MAX_D / LANES_PER_ROW; i++) {
            const int x = c + i * LANES_PER_ROW;
            if (x < d) {
                float a = acc[i] * corr;
                for (int j = 0; j < KEY_TILE; j++) a = fmaf(Ps[r * KEY_TILE + j], Vs[j * d + x], a);
                acc[i] = a;
            }
        }
    }

    if (!row_ok) return;
    const size_t row_index = (size_t)(tok0 + row_tok) * p.nh + head;
    if (p.split_keys > 0) {
        float* pa = p.part_acc + (row_index * p.max_splits + split) * d;
#pragma unroll
        for (int i = 0; i < MAX_D / LANES_PER_ROW; i++) {
            const int x = c + i * LANES_PER_ROW;
            if (x < d) pa[x] = acc[i];
        }
        if (c == 0) {
            float* ml = p.part_ml + (row_index * p.max_splits + split) * 2;
            ml[0] = m;
            ml[1] = l;
        }
    } else {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = (T*)p.out + row_index * d;
#pragma unroll
        for (int i = 0; i < MAX_D / LANES_PER_ROW; i++) {
            const int x = c + i * LANES_PER_ROW;
            if (x < d) o[x] = from_float<T>(acc[i] * inv);
        }
    }
}

// out[row] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M), chunks in index order.
template <typename T>
__global__ void attention_merge_kernel(AttnParams p, int total_tokens) {
    const int row = blockIdx.x;  // token * nh + head
    const int t = row / p.nh;
    // the batch row of token t: cu_seqlens is short, a linear scan is enough
    int b = 0;
    while (p.cu_seqlens[b + 1] <= t) b++;
    if (p.slot_ids[b] < 0) return;
    const int T_b = p.cu_seqlens[b + 1] - p.cu_seqlens[b];
    const int pos = p.kv_lens[b] - T_b + (t - p.cu_seqlens[b]);
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int s_begin = lo / p.split_keys, s_end = pos / p.split_keys + 1;  // chunks that hold visible keys
    if (s_end > p.max_splits) {
        // The row is longer than the chunks the caller made room for: its last keys were never visited and the
        // partials of chunk max_splits and beyond do not exist.  No truncated softmax is returned: the row's
        // output stays as it was, and the status word says so.
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, 2);
        return;
    }
    const float* ml = p.part_ml + (size_t)row * p.max_splits * 2;
    float M = -INFINITY;
    for (int s = s_begin; s < s_end; s++) M = fmaxf(M, ml[2 * s]);
    float L = 0.f;
    for (int s = s_begin; s < s_end; s++) L += ml[2 * s + 1] * expf(ml[2 * s] - M);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    const float* pa = p.part_acc + (size_t)row * p.max_splits * p.d;
    for (int x = threadIdx.x; x < p.d; x += blockDim.x) {
        float a = 0.f;
        for (int s = s_begin; s < s_end; s++) a = fmaf(pa[(size_t)s * p.d + x], expf(ml[2 * s] - M), a);
        ((T*)p.out)[(size_t)row * p.d + x] = from_float<T>(a * inv);
    }
}

}  // namespace

// The merge alone, for other kernels that write partials in the same layout
// (part_acc [token, head, split, d], part_ml [token, head, split, (max, sum)]).
int hymt2_attention_merge_launch(void* out, int dtype, const int* cu_seqlens, const int* slot_ids, const int* kv_lens,
                                 float* part_acc, float* part_ml, int tokens, int nh, int d, int window, int split_keys,
                                 int max_splits, cudaStream_t stream, int* status) {
    AttnParams p{};
    p.status = status;
    p.out = out; p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.part_acc = part_acc; p.part_ml = part_ml; p.nh = nh; p.d = d; p.window = window;
    p.split_keys = split_keys; p.max_splits = max_splits;
    HYMT2_DISPATCH_DTYPE(dtype, T, (attention_merge_kernel<T><<<tokens * nh, 64, 0, stream>>>(p, tokens)));
    return hymt2_check_launch("attention_merge");
}

// Sizes of the scratch that a split run needs, in floats: acc then ml.
HYMT2_API int hymt2_attention_simt_scratch(int tokens, int nh, int d, int max_splits, long* acc_floats, long* ml_floats) {
    *acc_floats = (long)tokens * nh * max_splits * d;
    *ml_floats = (long)tokens * nh * max_splits * 2;
    return HYMT2_OK;
}

HYMT2_API int hymt2_attention_simt(void* out, const void* q, const void* k_cache, const void* v_cache, int dtype,
                                   const int* block_table, int table_stride, int block_tokens,
                                   const int* cu_seqlens, const int* slot_ids, const int* kv_lens,
                                   int batch, int tokens, int max_new_tokens, int nh, int nkv, int d,
                                   float scale, int window, int split_keys, int max_splits,
                                   float* part_acc, float* part_ml, cudaStream_t stream, int* status) {
    if (tokens == 0 || batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(batch > 0 && tokens > 0 && nh > 0 && nkv > 0, "attention: bad sizes");
    HYMT2_REQUIRE(nh % nkv == 0, "attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    HYMT2_REQUIRE(d > 0 && d % 8 == 0 && d <= MAX_D, "attention: head_dim %d must be a multiple of 8, at most %d", d, MAX_D);
    HYMT2_REQUIRE(block_tokens % KEY_TILE == 0, "attention: block_tokens %d must be a multiple of %d", block_tokens, KEY_TILE);
    HYMT2_REQUIRE(split_keys == 0 || (split_keys % KEY_TILE == 0 && max_splits > 0 && part_acc && part_ml),
                  "attention: split_keys %d must be a multiple of %d and comes with scratch", split_keys, KEY_TILE);
    const int g = nh / nkv;
    AttnParams p;
    p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table;
    p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.part_acc = part_acc; p.part_ml = part_ml;
    p.table_stride = table_stride; p.block_tokens = block_tokens; p.nh = nh; p.nkv = nkv; p.d = d;
    p.window = window;
    p.heads_per_tile = g < ROWS ? g : ROWS;
    p.tokens_per_tile = ROWS / p.heads_per_tile;
    if (p.tokens_per_tile > max_new_tokens) p.tokens_per_tile = max_new_tokens > 0 ? max_new_tokens : 1;
    p.head_chunks = (g + p.heads_per_tile - 1) / p.heads_per_tile;
    p.split_keys = split_keys; p.max_splits = split_keys > 0 ? max_splits : 1;
    p.scale = scale;
    p.status = status;
    const size_t smem = sizeof(float) * ((size_t)ROWS * d + (size_t)KEY_TILE * (d + 1) + (size_t)KEY_TILE * d + ROWS * KEY_TILE);
    dim3 grid((max_new_tokens + p.tokens_per_tile - 1) / p.tokens_per_tile, nkv * p.head_chunks, batch * p.max_splits);
    HYMT2_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "attention: grid too large (batch %d x splits %d)", batch, p.max_splits);
    int rc = HYMT2_OK;
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(attention_simt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) { hymt2_set_error("attention: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        }
        attention_simt_kernel<T><<<grid, ROWS * LANES_PER_ROW, smem, stream>>>(p);
        rc = hymt2_check_launch("attention_simt");
        if (rc == HYMT2_OK && split_keys > 0) {
            attention_merge_kernel<T><<<tokens * nh, 64, 0, stream>>>(p, tokens);
            rc = hymt2_check_launch("attention_merge");
        }
    });
    return rc;
}

// ---------------------------------------------------------------------------
// The entry point that allocates nothing (see hymt2_noalloc.h).
// ---------------------------------------------------------------------------
#include "hymt2_noalloc.h"

#include <mutex>

namespace {

// Room for the partial results of hymt2_attention_decode_noalloc: [acc | max,sum].  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_noalloc_scratch[HYMT2_NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_scratch_ptr[NOALLOC_MAX_DEVICES] = {};

// Once per device, with that device current: the array's address on that device.
int noalloc_setup(int device, float** scratch) {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_scratch_ptr[device]) {
        float* s = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&s, g_noalloc_scratch);
        if (e != cudaSuccess || !s) {
            hymt2_set_error("attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return HYMT2_ERR_LAUNCH;
        }
        g_noalloc_scratch_ptr[device] = s;
    }
    *scratch = g_noalloc_scratch_ptr[device];
    return HYMT2_OK;
}

}  // namespace

HYMT2_API int hymt2_attention_decode_noalloc(void* out, const void* q, const void* k_cache, const void* v_cache,
                                             int dtype, const int* block_table, int table_stride, int block_tokens,
                                             const int* cu_seqlens, const int* slot_ids, const int* kv_lens, int rows,
                                             int nh, int nkv,
                                             int d, float scale, int window, int split_keys, int max_splits,
                                             int* status, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(status != nullptr, "attention_decode_noalloc: a status word (one int on the device) is needed");
    HYMT2_REQUIRE(rows > 0, "attention_decode_noalloc: rows %d must be positive", rows);
    HYMT2_REQUIRE(split_keys > 0 && max_splits > 0, "attention_decode_noalloc: split_keys and max_splits must be positive");
    HYMT2_REQUIRE(nh > 0 && d > 0, "attention_decode_noalloc: bad sizes");
    const long long need = (long long)rows * nh * max_splits * (d + 2);
    HYMT2_REQUIRE(need <= HYMT2_NOALLOC_SCRATCH_FLOATS,
                  "attention_decode_noalloc: rows %d x heads %d x splits %d x (head_dim %d + 2) = %lld floats of "
                  "partial results exceed the built-in scratch of %d floats",
                  rows, nh, max_splits, d, need, (int)HYMT2_NOALLOC_SCRATCH_FLOATS);
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= NOALLOC_MAX_DEVICES) {
        hymt2_set_error("attention_decode_noalloc: no usable current device (%s)", cudaGetErrorString(e));
        return HYMT2_ERR_LAUNCH;
    }
    float* scratch = nullptr;
    const int rc = noalloc_setup(device, &scratch);
    if (rc != HYMT2_OK) return rc;
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)rows * nh * max_splits * d;
    return hymt2_attention_simt(out, q, k_cache, v_cache, dtype, block_table, table_stride, block_tokens, cu_seqlens,
                                slot_ids, kv_lens, rows, rows, 1, nh, nkv, d, scale, window, split_keys, max_splits,
                                part_acc, part_ml, stream, status);
}
