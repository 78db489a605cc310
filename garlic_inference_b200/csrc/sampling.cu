// Next-token choice from float32 logits: greedy (temperature <= 0) or a draw
// from softmax(logits / temperature), one block per row, one pass over the row.
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

__host__ __device__ __forceinline__ unsigned long long gi_mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// uniform in (0, 1) from the generator's 24 high bits
__host__ __device__ __forceinline__ float gi_uniform(unsigned long long seed, unsigned long long stream,
                                                     unsigned long long counter, unsigned long long index) {
    unsigned long long h = gi_mix64(seed);
    h = gi_mix64(h ^ stream);
    h = gi_mix64(h ^ counter);
    h = gi_mix64(h ^ index);
    return ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

#define SM_THREADS 512

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const long long* __restrict__ streams,
              const int* __restrict__ counters, unsigned long long seed, int* __restrict__ out) {
    __shared__ float best_v[SM_THREADS / 32];
    __shared__ int best_i[SM_THREADS / 32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const unsigned long long stream = streams ? (unsigned long long)streams[r] : 0ull;
    const unsigned long long counter = counters ? (unsigned long long)counters[r] : 0ull;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += SM_THREADS) {
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
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SM_THREADS / 32; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        out[r] = bi == 0x7fffffff ? 0 : bi;   // a row of NaN or -inf everywhere gives token 0
    }
}

extern "C" int gi_sample(const float* logits, long long row_stride, int n_rows, int vocab,
                         const float* temperature, const long long* streams, const int* counters,
                         unsigned long long seed, int* out, void* stream) {
    GI_REQUIRE(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "gi_sample: sizes");
    if (n_rows == 0) return 0;
    sample_kernel<<<n_rows, SM_THREADS, 0, (cudaStream_t)stream>>>(logits, row_stride, vocab, temperature, streams,
                                                                   counters, seed, out);
    return gi_check_launch("gi_sample");
}

// The generator itself, for callers that want to check a draw on the host.
extern "C" float gi_sample_uniform(unsigned long long seed, long long stream, int counter, int index) {
    return gi_uniform(seed, (unsigned long long)stream, (unsigned long long)counter, (unsigned long long)index);
}
