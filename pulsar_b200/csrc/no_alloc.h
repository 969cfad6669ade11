// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference.  It exists for hosts that give
// all device memory to one arena at start-up, for latency-critical loops that must not
// take the allocator's lock, and for embedders that may launch but not allocate: it
// computes exactly what pb_paged_attention_decode computes, with the scratch for the
// per-split partial results taken from a fixed array inside the library instead of from
// the caller.  It calls no cudaMalloc, no cudaFree and no allocating library routine.
//
//   * Limit: n_seqs * Hq * n_splits * (D + 2) floats must not exceed
//     PB_DECODE_NOALLOC_MAX_FLOATS (1 Mi floats = 4 MiB, resident on every GPU that
//     loads the library until the process exits).  Larger problems are refused with
//     PB_ERR_SCRATCH_TOO_SMALL and nothing is launched; use fewer splits or the entry
//     point that takes the caller's scratch.
//   * The first call on a device looks up the array's device address (a synchronous
//     runtime query made with that device current); make that call before any stream
//     capture starts.
//   * Every call uses the same array and finds the last call's contents in it; nothing
//     needs to be cleared.  Calls that overlap on the GPU race on it: keep them on one
//     stream or order them with events.
//
// Arguments are those of pb_paged_attention_decode without `partial`:
//   dtype 0 float32 / 1 bfloat16; q, out [n_seqs, Hq, D]; pools [pages, Hkv, page_size, D];
//   block_table int32 [n_seqs, table_stride]; kv_len int32 [n_seqs] (context lengths
//   including the query token; a sequence with kv_len 0 gets zeros); window 0 = all keys.
//   Returns 0, a negative refusal, or a cudaError_t.
#pragma once

#include <cuda_runtime.h>

#define PB_DECODE_NOALLOC_MAX_FLOATS (1 << 20)
#define PB_ERR_SCRATCH_TOO_SMALL (-5)

#ifdef __cplusplus
extern "C" {
#endif

long long pb_decode_noalloc_max_floats(void);

int pb_paged_attention_decode_noalloc(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                      const int* block_table, int table_stride, const int* kv_len, int n_seqs, int Hq,
                                      int Hkv, int D, int page_size, float scale, int window, int n_splits,
                                      cudaStream_t stream);

#ifdef __cplusplus
}
#endif
