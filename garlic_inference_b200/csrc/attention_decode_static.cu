// The no-allocation variant of decode attention: see no_alloc.h for who needs it and its limits.
#include "no_alloc.h"

#include "common.cuh"

#include <mutex>

// Partial results of the slices of one call: first the unnormalised outputs
// [n_seqs, n_q, n_splits, head_dim], then the (max, sum) pairs [n_seqs, n_q, n_splits, 2].
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_scratch[GI_STATIC_SCRATCH_FLOATS];

extern "C" int gi_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                        const int* tok_pos, const int* tok_slot, void* out, float* part_o,
                                        float* part_ml, int n_seqs, int n_q, int n_kv, int d, int page_size,
                                        int max_pages, int n_pool_pages, int window, float scale, int n_splits,
                                        void* stream);

#define GI_MAX_DEVICES 64
static float* g_scratch_on_device[GI_MAX_DEVICES];      // the array's address on each device, once looked up
static std::mutex g_scratch_mutex;

// The device address of the array on the current device; looked up at the first call on that device.
static int static_scratch(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { gi_set_error("gi_attention_decode_bf16_static: cudaGetDevice: %s", cudaGetErrorString(e)); return (int)e; }
    GI_REQUIRE(dev >= 0 && dev < GI_MAX_DEVICES, "gi_attention_decode_bf16_static: device %d is beyond %d", dev, GI_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_on_device[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            gi_set_error("gi_attention_decode_bf16_static: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : GI_ERR_ARGUMENT;
        }
        g_scratch_on_device[dev] = p;
    }
    *ptr = g_scratch_on_device[dev];
    return 0;
}

extern "C" int gi_attention_decode_bf16_static(const void* q, const void* k_pool, const void* v_pool,
                                               const int* block_table, const int* tok_pos, const int* tok_slot,
                                               void* out, int n_seqs, int n_q, int n_kv, int d, int page_size,
                                               int max_pages, int n_pool_pages, int window, float scale,
                                               int n_splits, void* stream) {
    GI_REQUIRE(n_seqs >= 0 && n_q > 0 && d > 0 && n_splits >= 1, "gi_attention_decode_bf16_static: sizes must be positive");
    const long long pairs = (long long)n_seqs * n_q * n_splits;
    const long long need = pairs * (d + 2);
    GI_REQUIRE(need <= (long long)GI_STATIC_SCRATCH_FLOATS,
               "gi_attention_decode_bf16_static: %d sequences x %d heads x %d slices x (head_dim %d + 2) = %lld floats "
               "of partial results; the fixed array holds %d (use fewer slices or sequences, or the entry point "
               "that takes the caller's buffers)", n_seqs, n_q, n_splits, d, need, GI_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    float* part_o = scratch;
    float* part_ml = scratch + pairs * d;                 // pairs * d floats: a multiple of 16 elements, so 64-byte aligned
    return gi_attention_decode_bf16(q, k_pool, v_pool, block_table, tok_pos, tok_slot, out, part_o, part_ml, n_seqs,
                                    n_q, n_kv, d, page_size, max_pages, n_pool_pages, window, scale, n_splits, stream);
}
