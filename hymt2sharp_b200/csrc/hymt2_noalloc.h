// hymt2_noalloc.h: the one entry point of this library that allocates nothing.
//
// This function has no counterpart in sdcb/HyMT2Sharp; it exists for users of
// this library's C interface.
//
// Who it is for.  Every other kernel that needs working memory beyond its inputs
// and outputs takes that memory from its caller, and the Python engine gets it
// from torch's allocator.  Some callers have no allocator to ask: a host program
// that links the library through its C symbols without torch; a serving loop that
// has handed every free byte of the GPU to the key/value cache at start-up and
// must never see cudaMalloc fail (or stall the device, as cudaMalloc does) in the
// middle of a request; code that runs where the CUDA runtime forbids allocation.
// For them the split-key decode attention, which needs room for its partial
// results, is offered in a form that brings its own room.
//
// What it does.  The same computation as hymt2_attention_simt with split_keys > 0
// for decode steps (one new token per batch row): every chunk of `split_keys` keys
// gives an unnormalised partial, and the partials are merged in chunk order.  The
// partials live in a file-scope device array of HYMT2_NOALLOC_SCRATCH_FLOATS floats
// (4 MiB) that every GPU which loads the library holds until the process exits.
//
// Limits and rules.
//   * rows * nh * max_splits * (d + 2) must not exceed HYMT2_NOALLOC_SCRATCH_FLOATS;
//     a larger request is refused with HYMT2_ERR_ARGUMENT and a message, nothing runs.
//   * max_splits * split_keys must cover the longest row: the lengths live on the device, so
//     the host side of this call cannot check it.  The kernels do: a row with
//     kv_len > max_splits * split_keys is not computed (its row of `out` keeps what it held,
//     no partial beyond the array is touched) and status[0] is set to 2.  Read the status
//     word when in doubt; it is only ever written on that fault.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) with that device current.  Make that first call outside
//     of any stream capture.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
//   * All calls share the one array, which keeps what the last call left in it.  A call
//     writes every partial that it later reads, so nothing needs clearing between calls;
//     but two calls that run on the GPU at the same time (different streams) race on
//     the array.  Keep calls on one stream, or order them with events.
#pragma once

#include <cuda_runtime.h>

#define HYMT2_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// out, q: [rows, nh * d]; k_cache, v_cache: one layer's planes [block][nkv][block_tokens][d];
// dtype: 0 = float32, 1 = bfloat16 (q, out and the cache alike); block_table: int32
// [slot][table_stride]; cu_seqlens: int32 [rows + 1] = 0, 1, ..., rows (row b holds token b);
// slot_ids, kv_lens: int32 [rows] (slot < 0: the row is skipped); kv_lens counts the new token;
// status: one int32 on the device, zeroed by the caller (see the rules above).  Returns 0, or a
// negative code with hymt2_last_error() set.
int hymt2_attention_decode_noalloc(void* out, const void* q, const void* k_cache, const void* v_cache, int dtype,
                                   const int* block_table, int table_stride, int block_tokens,
                                   const int* cu_seqlens, const int* slot_ids, const int* kv_lens, int rows, int nh,
                                   int nkv, int d, float scale, int window, int split_keys, int max_splits,
                                   int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
