// Token sampling on the GPU, one block per row of logits.
//
//  * argmax: the first index that holds the maximum (src/HyMT2Sharp/Sampling.cs:298-334).
//  * filters: repetition penalty over a window of recent tokens
//    (Sampling.cs:141-156), temperature (Sampling.cs:97-99), top-k with exact count
//    under ties (Sampling.cs:171-225), min-p and top-p on the softmax numerators
//    (Sampling.cs:229-293).  They rewrite the row: dropped entries become -inf.
//  * temperature sampling: p_i = exp(x_i - max) (Sampling.cs:105-113), r = u * sum,
//    the first i with p_i > 0 whose running sum reaches r (Sampling.cs:119-129), else
//    the last i with p_i > 0 (Sampling.cs:131-138).  u comes from a xoshiro256**
//    stream seeded through SplitMix64, u = (next >> 40) * 2^-24 (Sampling.cs:375-409);
//    its four 64-bit words live in device memory, one stream per sequence.
//
// The running sum is built from per-thread partial sums over contiguous pieces of
// the vocabulary, scanned in index order, so a pick never depends on the batch.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__global__ void __launch_bounds__(THREADS)
argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, long row_stride, int vocab,
              const int* __restrict__ row_map) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    const int row = blockIdx.x;
    if (row_map && row_map[row] < 0) return;
    const float* x = logits + (size_t)row * row_stride;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    // NaN logits never win a comparison; a row of NaNs gives index 0 below
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = sval[lane]; best_i = sidx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) out[row] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

// Two-stage argmax for wide vocabularies: pieces of ARGMAX_PIECE logits each give their first
// maximum, then one block per row picks the first maximum among the pieces.
constexpr int ARGMAX_PIECE = 4096;

__global__ void __launch_bounds__(256)
argmax_pieces_kernel(float* __restrict__ piece_val, int* __restrict__ piece_idx, const float* __restrict__ logits,
                     long row_stride, int vocab, const int* __restrict__ row_map) {
    __shared__ float sval[8];
    __shared__ int sidx[8];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, piece = blockIdx.x;
    if (row_map && row_map[row] < 0) return;
    const float* x = logits + (size_t)row * row_stride;
    const int begin = piece * ARGMAX_PIECE, end = min(vocab, begin + ARGMAX_PIECE);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (sval[w] > best || (sval[w] == best && sidx[w] < best_i)) { best = sval[w]; best_i = sidx[w]; }
        piece_val[(size_t)row * gridDim.x + piece] = best;
        piece_idx[(size_t)row * gridDim.x + piece] = best_i;
    }
}

__global__ void argmax_final_kernel(int* __restrict__ out, const float* __restrict__ piece_val,
                                    const int* __restrict__ piece_idx, int pieces, const int* __restrict__ row_map) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    if (row_map && row_map[row] < 0) return;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < pieces; i += 32) {
        const float v = piece_val[(size_t)row * pieces + i];
        const int vi = piece_idx[(size_t)row * pieces + i];
        if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) out[row] = best_i == 0x7fffffff ? 0 : best_i;
}

__device__ __forceinline__ uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

__device__ __forceinline__ uint64_t xoshiro_next(uint64_t* s) {
    const uint64_t r = rotl64(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return r;
}

__global__ void seed_rng_kernel(uint64_t* states, const int* rows, const uint64_t* seeds, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint64_t z = seeds[i];
    uint64_t* s = states + (size_t)rows[i] * 4;
    for (int k = 0; k < 4; k++) {
        z += 0x9E3779B97F4A7C15ull;
        uint64_t x = z;
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        s[k] = x ^ (x >> 31);
    }
}

// Exclusive scan of one value per thread over the block, in thread order.
// `warp_totals` holds 32 values of shared memory, `total` one.
template <typename V>
__device__ __forceinline__ V block_exclusive_scan(V v, V* warp_totals, V* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    V inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const V n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        V w = warp_totals[lane];
        V winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const V n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_totals[lane] = winc - w;  // exclusive
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return warp_totals[warp] + (inc - v);
}

// One row: x_i = logits_i * inv_temperature (entries at -inf have probability 0).
__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long row_stride, int vocab,
              const float* __restrict__ inv_temperature, uint64_t* __restrict__ rng_states,
              const int* __restrict__ row_map) {
    __shared__ float scratch[33];
    __shared__ float warp_totals[32];
    __shared__ float total_s;
    __shared__ int pick_s, owner_s;
    const int row = blockIdx.x;
    const int srow = row_map ? row_map[row] : row;  // the sequence's row in the per-sequence arrays
    if (srow < 0) return;
    const float* x = logits + (size_t)row * row_stride;
    const float inv_t = inv_temperature[srow];
    if (!(inv_t > 0.f)) return;  // a greedy row: argmax has written its token
    const int piece = (vocab + THREADS - 1) / THREADS;
    const int begin = min(vocab, (int)threadIdx.x * piece), end = min(vocab, begin + piece);

    float mx = -INFINITY;
    for (int i = begin; i < end; i++) mx = fmaxf(mx, x[i] * inv_t);
    mx = block_max(mx, scratch);

    float part = 0.f;
    for (int i = begin; i < end; i++) {
        const float v = x[i] * inv_t;
        part += v == -INFINITY ? 0.f : expf(v - mx);
    }
    const float before = block_exclusive_scan<float>(part, warp_totals, &total_s);
    const float total = total_s;

    float u = 0.f;
    if (threadIdx.x == 0) {
        uint64_t* s = rng_states + (size_t)srow * 4;
        u = (float)(xoshiro_next(s) >> 40) * (1.0f / 16777216.0f);
        scratch[0] = u;
        owner_s = 0x7fffffff;
        pick_s = -1;
    }
    __syncthreads();
    u = scratch[0];
    const float r = u * total;
    // the first piece whose inclusive running sum reaches r owns the pick
    if (part > 0.f && before + part >= r) atomicMin(&owner_s, (int)threadIdx.x);
    __syncthreads();
    if ((int)threadIdx.x == owner_s) {
        float acc = before;
        int pick = -1, last = -1;
        for (int i = begin; i < end; i++) {
            const float v = x[i] * inv_t;
            const float pr = v == -INFINITY ? 0.f : expf(v - mx);
            if (pr <= 0.f) continue;
            last = i;
            acc += pr;
            if (acc >= r) { pick = i; break; }
        }
        pick_s = pick >= 0 ? pick : last;  // the walk inside a piece may round past r: its last entry
    }
    __syncthreads();
    if (owner_s == 0x7fffffff) {
        // r lies past the last survivor through rounding: take the last entry with p > 0
        int last = -1;
        for (int i = begin; i < end; i++) {
            const float v = x[i] * inv_t;
            if (v != -INFINITY && expf(v - mx) > 0.f) last = i;
        }
        if (last >= 0) atomicMax(&pick_s, last);
        __syncthreads();
    }
    if (threadIdx.x == 0) out[row] = pick_s >= 0 ? pick_s : 0;
}

// ---------------------------------------------------------------------------
// filters: penalty, top-k, min-p, top-p.  One block per row, in place.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float v) {  // monotone: larger float, larger key
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// The value of the k-th largest key among vocab entries (k >= 1), by 4 radix passes.
__device__ uint32_t kth_largest_key(const float* x, float mul, int vocab, int k, int* hist /*256*/, int* misc) {
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const uint32_t key = float_key(x[i] * mul);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int need = remaining, bin = 255;
            for (; bin > 0; bin--) {
                if (hist[bin] >= need) break;
                need -= hist[bin];
            }
            misc[0] = bin;
            misc[1] = need;
        }
        __syncthreads();
        prefix |= (uint32_t)misc[0] << shift;
        mask |= 255u << shift;
        remaining = misc[1];
        __syncthreads();
    }
    return prefix;
}

struct FilterParams {
    float* logits;
    long row_stride;
    int vocab;
    const float* inv_temperature;  // per sequence; <= 0 marks a greedy row (only the penalty applies)
    const int* top_k;              // per sequence, 0 = off
    const float* top_p;            // per sequence, >= 1 = off
    const float* min_p;            // per sequence, <= 0 = off
    const float* penalty;          // per sequence, 1 = off
    const int* history;            // [sequence, history_stride] recent tokens, -1 = empty
    int history_stride;
    const int* row_map;            // logits row -> sequence row, < 0 = skip
};

__global__ void __launch_bounds__(THREADS)
filter_kernel(FilterParams p) {
    __shared__ int hist[256];
    __shared__ int misc[4];
    __shared__ float scratch[33];
    __shared__ float fmisc[2];
    __shared__ int iscan[32];
    __shared__ int iscan_total;
    const int row = blockIdx.x;
    const int srow = p.row_map ? p.row_map[row] : row;
    if (srow < 0) return;
    float* x = p.logits + (size_t)row * p.row_stride;
    const int vocab = p.vocab;
    const int piece = (vocab + THREADS - 1) / THREADS;
    const int begin = min(vocab, (int)threadIdx.x * piece), end = min(vocab, begin + piece);

    // repetition penalty: every entry of the window applies once, repeats included
    const float pen = p.penalty ? p.penalty[srow] : 1.f;
    if (pen != 1.f && p.history) {
        if (threadIdx.x == 0) {
            const int* h = p.history + (size_t)srow * p.history_stride;
            for (int i = 0; i < p.history_stride; i++) {
                const int t = h[i];
                if (t < 0 || t >= vocab) continue;
                const float l = x[t];
                x[t] = l <= 0.f ? l * pen : l / pen;
            }
        }
        __syncthreads();
    }
    const float inv_t = p.inv_temperature[srow];
    if (!(inv_t > 0.f)) return;  // greedy: temperature 0 bypasses every other field (Sampling.cs:81-84)
    const int k = p.top_k ? p.top_k[srow] : 0;
    const float top_p = p.top_p ? p.top_p[srow] : 1.f, min_p = p.min_p ? p.min_p[srow] : 0.f;

    if (k > 0 && k < vocab) {
        const uint32_t kth = kth_largest_key(x, inv_t, vocab, k, hist, misc);
        // entries above the k-th stay; ties at the k-th stay in index order until k survive
        if (threadIdx.x == 0) misc[2] = 0;
        __syncthreads();
        int above = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) above += float_key(x[i] * inv_t) > kth;
        atomicAdd(&misc[2], above);
        __syncthreads();
        const int free_slots = k - misc[2];
        __syncthreads();
        // ties at the k-th value stay in index order until k entries survive
        int ties = 0;
        for (int i = begin; i < end; i++) ties += float_key(x[i] * inv_t) == kth;
        int rank = block_exclusive_scan<int>(ties, iscan, &iscan_total);
        for (int i = begin; i < end; i++) {
            if (float_key(x[i] * inv_t) == kth) {
                if (rank >= free_slots) x[i] = -INFINITY;
                rank++;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            if (float_key(x[i] * inv_t) < kth) x[i] = -INFINITY;
        __syncthreads();
    }

    if (top_p < 1.f || min_p > 0.f) {
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, x[i] * inv_t);
        mx = block_max(mx, scratch);
        // the mass of everything that is left after top-k: top-p's limit is a share of it,
        // also when min-p drops entries first (Sampling.cs:272-274 uses the sum from before)
        float sum = 0.f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = x[i] * inv_t;
            sum += v == -INFINITY ? 0.f : expf(v - mx);
        }
        sum = block_sum(sum, scratch);
        if (min_p > 0.f) {
            // p >= min_p * p_max with p_max = exp(0) = 1
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const float v = x[i] * inv_t;
                if (v != -INFINITY && expf(v - mx) < min_p) x[i] = -INFINITY;
            }
            __syncthreads();
        }
        if (top_p < 1.f) {
            // the largest probabilities, in descending order, while the mass before an entry is
            // below top_p * sum: find the threshold key by radix passes over the mass per bin
            const float limit = top_p * sum;
            __shared__ float mass[256];
            uint32_t prefix = 0, mask = 0;
            float above_mass = 0.f;  // mass of keys strictly above the current prefix range
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int i = threadIdx.x; i < 256; i += blockDim.x) mass[i] = 0.f;
                __syncthreads();
                for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                    const float v = x[i] * inv_t;
                    if (v == -INFINITY) continue;
                    const uint32_t key = float_key(v);
                    if ((key & mask) == prefix) atomicAdd(&mass[(key >> shift) & 255], expf(v - mx));
                }
                __syncthreads();
                if (threadIdx.x == 0) {
                    float acc = above_mass;
                    int bin = 255;
                    for (; bin > 0; bin--) {
                        if (acc + mass[bin] >= limit) break;
                        acc += mass[bin];
                    }
                    misc[0] = bin;
                    fmisc[0] = acc;
                }
                __syncthreads();
                prefix |= (uint32_t)misc[0] << shift;
                mask |= 255u << shift;
                above_mass = fmisc[0];
                __syncthreads();
            }
            // keys above `prefix` stay; entries equal to it (all of one probability) stay in
            // index order while the mass before them is below the limit
            int ties = 0;
            for (int i = begin; i < end; i++) {
                const float v = x[i] * inv_t;
                ties += v != -INFINITY && float_key(v) == prefix;
            }
            int rank = block_exclusive_scan<int>(ties, iscan, &iscan_total);
            for (int i = begin; i < end; i++) {
                const float v = x[i] * inv_t;
                if (v == -INFINITY || float_key(v) != prefix) continue;
                if (above_mass + (float)rank * expf(v - mx) >= limit) x[i] = -INFINITY;
                rank++;
            }
            __syncthreads();
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const float v = x[i] * inv_t;
                if (v != -INFINITY && float_key(v) < prefix) x[i] = -INFINITY;
            }
        }
    }
}

// history[sequence, count % stride] = token; count += 1 (the ring of Sampling.cs:158-169)
__global__ void record_history_kernel(int* history, int* counts, int stride, const int* tokens, const int* row_map,
                                      int rows) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int srow = row_map ? row_map[row] : row;
    if (srow < 0) return;
    const int c = counts[srow];
    history[(size_t)srow * stride + c % stride] = tokens[row];
    counts[srow] = c + 1;
}

}  // namespace

HYMT2_API int hymt2_record_history(int* history, int* counts, int stride, const int* tokens, const int* row_map,
                                   int rows, cudaStream_t stream) {
    if (rows == 0 || stride == 0) return HYMT2_OK;
    record_history_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(history, counts, stride, tokens, row_map, rows);
    return hymt2_check_launch("record_history");
}

// piece_val / piece_idx: scratch of rows * ceil(vocab / 4096) entries each, or null.  With scratch
// and a vocabulary above 2 * 4096 the scan is spread over many blocks per row.
HYMT2_API int hymt2_argmax(int* out, const float* logits, long row_stride, int rows, int vocab,
                           const int* row_map, float* piece_val, int* piece_idx, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && vocab > 0 && row_stride >= vocab, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
    if (piece_val && piece_idx && vocab > 2 * ARGMAX_PIECE && rows <= 65535) {
        const int pieces = (vocab + ARGMAX_PIECE - 1) / ARGMAX_PIECE;
        launch_pdl(argmax_pieces_kernel, dim3(pieces, rows), dim3(256), 0, stream, piece_val, piece_idx, logits, row_stride, vocab, row_map);
        int rc = hymt2_check_launch("argmax (pieces)");
        if (rc != HYMT2_OK) return rc;
        launch_pdl(argmax_final_kernel, dim3(rows), dim3(32), 0, stream, out, (const float*)piece_val, (const int*)piece_idx, pieces, row_map);
        return hymt2_check_launch("argmax (final)");
    }
    argmax_kernel<<<rows, THREADS, 0, stream>>>(out, logits, row_stride, vocab, row_map);
    return hymt2_check_launch("argmax");
}

HYMT2_API int hymt2_seed_rng(uint64_t* states, const int* rows, const uint64_t* seeds, int n, cudaStream_t stream) {
    if (n == 0) return HYMT2_OK;
    seed_rng_kernel<<<(n + 127) / 128, 128, 0, stream>>>(states, rows, seeds, n);
    return hymt2_check_launch("seed_rng");
}

HYMT2_API int hymt2_sample(int* out, const float* logits, long row_stride, int rows, int vocab,
                           const float* inv_temperature, uint64_t* rng_states, const int* row_map,
                           cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    sample_kernel<<<rows, THREADS, 0, stream>>>(out, logits, row_stride, vocab, inv_temperature, rng_states,
                                                row_map);
    return hymt2_check_launch("sample");
}

HYMT2_API int hymt2_filter_logits(float* logits, long row_stride, int rows, int vocab, const float* inv_temperature,
                                  const int* top_k, const float* top_p, const float* min_p, const float* penalty,
                                  const int* history, int history_stride, const int* row_map,
                                  cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && vocab > 0 && row_stride >= vocab, "filter: bad sizes rows=%d vocab=%d", rows, vocab);
    FilterParams p{logits, row_stride, vocab, inv_temperature, top_k, top_p, min_p, penalty, history,
                   history_stride, row_map};
    filter_kernel<<<rows, THREADS, 0, stream>>>(p);
    return hymt2_check_launch("filter_logits");
}
