// Next-token choice from float32 logits: greedy (temperature <= 0) or a draw
// from softmax(logits / temperature): one pass over the row by many blocks, each
// finding the best entry of its chunk, and a small second pass over the chunks' winners.
//
// The draw uses the Gumbel trick: argmax_i( logit_i / temperature + g_i ) with
// g_i = -log(-log(u_i)) is distributed as the softmax, and needs no
// normalisation pass.  u_i comes from a counter-based generator keyed by
// (seed, the row's stream id, the row's token index, i), so a request's tokens
// do not depend on which other requests share its batch.  Ties go to the
// lowest index.  Upstream picks the greedy token only, without a tie rule
// (src/src-cuda/reductions/argmax.cu:7-70).
#include "common.cuh"
#include <math.h>

// Uniform strictly inside (0, 1) from the 23 high bits of a hash: (k + 0.5) / 2^23 with k < 2^23 is exact in
// float32 (24 significant bits), so the largest value is 1 - 2^-24 and never 1.  (With 24 bits k + 0.5 would
// round to even, reach 2^24 and give u = 1, whose Gumbel term is +infinity.)
__host__ __device__ __forceinline__ float gi_uniform_from_hash(unsigned long long h) {
    return ((float)(h >> 41) + 0.5f) * (1.0f / 8388608.0f);
}

__host__ __device__ __forceinline__ float gi_uniform(unsigned long long seed, unsigned long long stream,
                                                     unsigned long long counter, unsigned long long index) {
    unsigned long long h = gi_mix64(seed);
    h = gi_mix64(h ^ stream);
    h = gi_mix64(h ^ counter);
    h = gi_mix64(h ^ index);
    return gi_uniform_from_hash(h);
}

#define SM_THREADS 256
#define SM_CHUNK 4096        // vocabulary entries per block of the first pass

__device__ __forceinline__ bool sm_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// First pass: block (chunk, row) finds the best entry of its chunk of the row.
__global__ void __launch_bounds__(SM_THREADS)
sample_partial_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                      const float* __restrict__ temperature, const long long* __restrict__ streams,
                      const int* __restrict__ counters, unsigned long long seed, float* __restrict__ part_v,
                      int* __restrict__ part_i) {
    gi_pdl_start();
    __shared__ float best_v[SM_THREADS / 32];
    __shared__ int best_i[SM_THREADS / 32];
    const int r = blockIdx.y, chunk = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const unsigned long long stream = streams ? (unsigned long long)streams[r] : 0ull;
    const unsigned long long counter = counters ? (unsigned long long)counters[r] : 0ull;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    const int end = min(vocab, (chunk + 1) * SM_CHUNK);
    for (int i = chunk * SM_CHUNK + threadIdx.x; i < end; i += SM_THREADS) {
        float v = row[i];
        if (temp > 0.f) {
            const float u = gi_uniform(seed, stream, counter, (unsigned long long)i);
            v = v / temp - logf(-logf(u));
        }
        if (v > bv) { bv = v; bi = i; }      // ascending i within a thread: the first maximum stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (sm_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SM_THREADS / 32; ++w)
            if (sm_better(best_v[w], best_i[w], bv, bi)) { bv = best_v[w]; bi = best_i[w]; }
        part_v[(size_t)r * gridDim.x + chunk] = bv;
        part_i[(size_t)r * gridDim.x + chunk] = bi;
    }
}

// Second pass: one warp per row picks the best of the chunks' winners (ties to the lowest index).
__global__ void sample_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int n_chunks,
                                    int* __restrict__ out) {
    gi_pdl_start();
    const int r = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const float v = part_v[(size_t)r * n_chunks + c];
        const int i = part_i[(size_t)r * n_chunks + c];
        if (sm_better(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (sm_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;    // a row of NaN or -inf everywhere gives token 0
}

// Scratch: part_v float32 and part_i int32, each n_rows * gi_sample_chunks(vocab) entries.
extern "C" int gi_sample_chunks(int vocab) { return (vocab + SM_CHUNK - 1) / SM_CHUNK; }

extern "C" int gi_sample(const float* logits, long long row_stride, int n_rows, int vocab,
                         const float* temperature, const long long* streams, const int* counters,
                         unsigned long long seed, float* part_v, int* part_i, int* out, void* stream) {
    GI_REQUIRE(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "gi_sample: sizes");
    GI_REQUIRE(n_rows <= 65535, "gi_sample: %d rows in one call is beyond 65535", n_rows);
    if (n_rows == 0) return 0;
    const int n_chunks = gi_sample_chunks(vocab);
    gi_launch(sample_partial_kernel, dim3(n_chunks, n_rows), dim3(SM_THREADS), 0, (cudaStream_t)stream, 
        logits, row_stride, vocab, temperature, streams, counters, seed, part_v, part_i);
    gi_launch(sample_final_kernel, dim3(n_rows), dim3(32), 0, (cudaStream_t)stream, part_v, part_i, n_chunks, out);
    return gi_check_launch("gi_sample");
}

// The generator itself, for callers that want to check a draw on the host.
extern "C" float gi_sample_uniform(unsigned long long seed, long long stream, int counter, int index) {
    return gi_uniform(seed, (unsigned long long)stream, (unsigned long long)counter, (unsigned long long)index);
}

// The last step of the generator alone: the uniform a given 64-bit hash turns into (for tests of its two ends).
extern "C" float gi_sample_uniform_from_hash(unsigned long long h) { return gi_uniform_from_hash(h); }
