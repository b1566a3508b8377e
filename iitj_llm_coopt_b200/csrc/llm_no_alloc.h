// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (mohsinmubarak/iitj-llm-coopt): its
// attention is a library call whose workspace the library manages.  It exists for hosts
// that drive this library from outside PyTorch -- a C or C++ serving shell, another
// language's FFI -- and that either have no device allocator at hand or must not use one
// where they call from: a cudaMalloc in the middle of serving synchronises the whole
// device, and in a process that gave all free memory to its key/value pool at start-up
// it may simply fail.
//
// llm_attention_decode_bf16_static does what llm_attention_decode_bf16 does (split-key
// attention of single decoded tokens over the paged cache, bfloat16, head sizes 64 and
// 128) but keeps the per-split partial results in a fixed array inside the library
// instead of in caller-provided scratch.  The caller still passes every input and the
// output.
//
// Limits and rules:
//   * The array holds LLM_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU on which the
//     library is loaded keeps that much memory until the process ends.  A call needs
//     n_items * heads * max_splits * (head_dim + 2) floats; a call that needs more is
//     refused with a negative return code and a message in llm_last_error().
//   * The first call on a device looks up the array's device address (once per device,
//     with that device current).  Make that first call before any stream capture.
//   * All calls share the one array.  Nothing in it has to start at zero -- each call
//     writes every partial it later reads -- but two calls whose kernels may run at the
//     same time on one GPU (different streams, different threads) race on it.  Keep such
//     calls on one stream, or order them with events.
//   * keys_per_split (a multiple of 64) times max_splits must cover the longest item: its
//     position + 1 keys, or with a window the keys from the 64-aligned start of the window.
//     The kernels cannot see what the caller meant, so an item that would need more splits
//     is cut down to max_splits: its last keys are left out, its result is wrong, nothing
//     outside its own partials is touched, and llm_attention_decode_status() returns a
//     non-zero code (6 << 16 | item) until it is read.  The same holds for
//     llm_attention_decode_bf16.
//   * It calls neither cudaMalloc nor cudaFree nor any allocating library routine.
#pragma once

#include <cuda_runtime.h>

#define LLM_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as llm_attention_decode_bf16 without part_o / part_ml.  Returns 0, or a
// negative code with the reason in llm_last_error().
int llm_attention_decode_bf16_static(const void* q, int q_stride, const void* cache, const int* block_table,
                                     int table_width, const int* items, int n_items, const int* token_request,
                                     const int* positions, void* out, int out_stride, int heads, int kv_heads,
                                     int head_dim, int page_size, int window, float scale, int keys_per_split,
                                     int max_splits, cudaStream_t stream);

// Reads and clears the status word of the decode attention kernels (0 = every call since the last read kept the
// contract above).  It copies one int from the device and so waits for the work in flight.
int llm_attention_decode_status(void);

#ifdef __cplusplus
}
#endif
