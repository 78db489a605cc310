// Random weights made on the device: out[i] = mean + std * z_i, where z_i is a standard normal variate that
// depends only on (key, i).  The key is a hash of the seed and the tensor's name, made by the caller.
//
// z_i is the sum of twelve 16-bit fields of three hashes of (key, i), centred and scaled: an Irwin-Hall
// variate with mean 0 and variance (65536^2 - 1) / 65536^2, cut at +-6.  Everything up to the last two
// operations is integer arithmetic and the scale is a power of two, so a host program that does the same
// steps in float32 (one multiplication, one addition, neither fused) gets the same bits: a model folder
// written on the CPU and a model initialised here hold identical tensors.  Upstream has no random weights.
#include "common.cuh"

#define RI_THREADS 256

__host__ __device__ __forceinline__ int ri_sum12(unsigned long long key, unsigned long long i) {
    int s = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const unsigned long long h = gi_mix64(key ^ (3ull * i + (unsigned long long)j));
        s += (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) + (int)(h >> 48);
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(RI_THREADS)
random_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, float mean, float std) {
    gi_pdl_start();
    const long long stride = (long long)gridDim.x * RI_THREADS;
    for (long long i = (long long)blockIdx.x * RI_THREADS + threadIdx.x; i < n; i += stride) {
        // twelve fields of mean 32767.5 each: twice the sum minus 786420 is an exact integer below 2^21
        const float z = (float)(2 * ri_sum12(key, (unsigned long long)i) - 786420) * (1.0f / 131072.0f);
        out[i] = from_f32<T>(__fadd_rn(mean, __fmul_rn(std, z)));
    }
}

// out: n elements of `dtype` (GI_DTYPE_F32 or GI_DTYPE_BF16) on the device.
extern "C" int gi_random_normal(void* out, int dtype, long long n, unsigned long long key, float mean, float std,
                                void* stream) {
    GI_REQUIRE(n >= 0, "gi_random_normal: %lld elements", n);
    GI_REQUIRE(dtype == GI_DTYPE_F32 || dtype == GI_DTYPE_BF16, "gi_random_normal: dtype code %d", dtype);
    if (n == 0) return 0;
    const long long blocks = (n + RI_THREADS - 1) / RI_THREADS;
    const dim3 grid((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16));
    if (dtype == GI_DTYPE_F32)
        gi_launch(random_normal_kernel<float>, grid, dim3(RI_THREADS), 0, (cudaStream_t)stream, (float*)out, n, key, mean, std);
    else
        gi_launch(random_normal_kernel<bf16>, grid, dim3(RI_THREADS), 0, (cudaStream_t)stream, (bf16*)out, n, key, mean, std);
    return gi_check_launch("gi_random_normal");
}

// The integer part of the generator for one element, for host programs that check their own copy of it.
extern "C" int gi_random_sum12(unsigned long long key, unsigned long long index) { return ri_sum12(key, index); }
