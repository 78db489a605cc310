// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in NikolayBlagoev/garlic-inference, which allocates inside its
// forward pass; it exists for hosts of this library that cannot call cudaMalloc at the time they need
// attention: code running inside a CUDA graph capture, a plug-in that was handed a fixed memory
// budget and no allocator, or a real-time loop that may not take the allocator's locks.
//
// gi_attention_decode_bf16_static does what gi_attention_decode_bf16 does (split-KV attention of one
// new token per sequence over the paged cache, then the merge of the slices), but the partial results
// of the slices go through a fixed array that lives in the library's device image instead of
// through buffers the caller allocates.  The caller still passes the inputs and the output.
//
//   * Limit: the partials of one call, n_seqs * n_q * n_splits * (head_dim + 2) floats, must fit in
//     GI_STATIC_SCRATCH_FLOATS (2 Mi floats = 8 MiB).  Larger calls are refused with an error
//     (GI_ERR_ARGUMENT, text from gi_last_error()); nothing is launched.  Every GPU that loads the
//     library holds these 8 MiB until the process exits.
//   * The first call on a device looks up the array's device address (one cudaGetSymbolAddress,
//     checked).  Make that first call outside any stream capture, with the device current.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine.
//   * All calls on a device share the one array, and it keeps what the last call left.  Nothing in it
//     has to start at zero: every slice writes its (max, sum) pair before the merge reads it, and the
//     merge never reads the output of a slice that saw no key.  Two calls that overlap on the GPU
//     (different streams, or a graph replayed while another call runs) race on the array; give such
//     callers the allocating entry point with buffers of their own.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define GI_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

int gi_attention_decode_bf16_static(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                    const int* tok_pos, const int* tok_slot, void* out, int n_seqs, int n_q,
                                    int n_kv, int d, int page_size, int max_pages, int n_pool_pages, int window,
                                    float scale, int n_splits, void* stream);

#ifdef __cplusplus
}
#endif
