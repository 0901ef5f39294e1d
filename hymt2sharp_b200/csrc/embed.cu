// Token embedding: out[t, :] = float(table[ids[t], :]).  The residual stream
// that it starts is float32 in both precisions.
// Formula: src/HyMT2Sharp/HunyuanDenseModel.cs:494-537 (row gather, no scale).
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int hidden, int vocab, int* status) {
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
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = to_float(row[i]);
}

HYMT2_API int hymt2_embed(float* out, const void* table, int table_dtype, const int* ids, int tokens,
                          int hidden, int vocab, int* status, cudaStream_t stream) {
    if (tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embed: bad sizes tokens=%d hidden=%d vocab=%d", tokens, hidden, vocab);
    HYMT2_DISPATCH_DTYPE(table_dtype, T,
        launch_pdl(embed_kernel<T>, dim3(tokens), dim3(256), 0, stream, out, (const T*)table, ids, hidden, vocab, status));
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
