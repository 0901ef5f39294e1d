// Token embedding: out[t, :] = float(table[ids[t], :]) * scale.  The residual stream
// that it starts is float32 in both precisions.
// Formula: src/HyMT2Sharp/HunyuanDenseModel.cs:494-537 (row gather; that model has no scale, so its
// scale is 1; architectures that multiply their embeddings by a constant give it here).
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int hidden, int vocab, float scale, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {  // never read outside the table: flag it and give zeros
        if (threadIdx.x == 0) atomicExch(status, 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = scale == 1.0f ? to_float(row[i]) : to_float(row[i]) * scale;
}

HYMT2_API int hymt2_embed(float* out, const void* table, int table_dtype, const int* ids, int tokens,
                          int hidden, int vocab, float scale, int* status, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embed: bad sizes tokens=%d hidden=%d vocab=%d", tokens, hidden, vocab);
    HYMT2_DISPATCH_DTYPE(table_dtype, T,
        launch_pdl(embed_kernel<T>, dim3(tokens), dim3(256), 0, stream, out, (const T*)table, ids, hidden, vocab, scale, status));
    return hymt2_check_launch("embed");
}

// After a decode step: every live row of the batch is one token longer.
__global__ void advance_decode_kernel(int* token_pos, int* kv_lens, const int* slot_ids, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= rows || slot_ids[b] < 0) return;
    token_pos[b] += 1;
    kv_lens[b] += 1;
}

HYMT2_API int hymt2_advance_decode(int* token_pos, int* kv_lens, const int* slot_ids, int rows, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    launch_pdl(advance_decode_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, token_pos, kv_lens, slot_ids, rows);
    return hymt2_check_launch("advance_decode");
}

// Asks for `bytes` from `ptr` on to be brought into L2 (cp.async.bulk.prefetch.L2 in pieces of 16 KB), for a stream
// beside the one that computes: a decode step leaves the memory idle most of the time, and the next large product's
// weights can come in meanwhile.  Nothing is written anywhere.
__global__ void l2_prefetch_kernel(const uint8_t* ptr, long bytes) {
    constexpr long PIECE = 16384;
    const long pieces = (bytes + PIECE - 1) / PIECE;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (long)gridDim.x * blockDim.x) {
        const long off = i * PIECE;
        const uint32_t n = (uint32_t)min(PIECE, bytes - off);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr + off), "r"(n) : "memory");
    }
}

HYMT2_API int hymt2_l2_prefetch(const void* ptr, long bytes, cudaStream_t stream) {
    bytes &= ~15L;
    if (bytes <= 0) return HYMT2_OK;
    HYMT2_REQUIRE(ptr != nullptr && (uintptr_t)ptr % 16 == 0, "l2_prefetch: the address must be 16-byte aligned");
    const long pieces = (bytes + 16383) / 16384;
    const unsigned blocks = (unsigned)(pieces < 128 * 32 ? (pieces + 31) / 32 : 128);
    l2_prefetch_kernel<<<blocks, 32, 0, stream>>>((const uint8_t*)ptr, bytes);
    return hymt2_check_launch("l2_prefetch");
}

// The device's clock (nanoseconds of %globaltimer) into out[0]: launched between the kernels of a captured step while
// kernels are being timed, since a graph can hold this where the host cannot look.  Launched without programmatic
// overlap, so a stamp is taken when everything in front of it on the stream is complete.
__global__ void stamp_kernel(unsigned long long* out) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    *out = t;
}

HYMT2_API int hymt2_stamp(unsigned long long* out, cudaStream_t stream) {
    HYMT2_REQUIRE(out != nullptr, "stamp: no place to write");
    stamp_kernel<<<1, 1, 0, stream>>>(out);
    return hymt2_check_launch("stamp");
}
