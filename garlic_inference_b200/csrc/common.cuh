// Shared helpers of the kernels: element types, conversions, warp reductions,
// and the error channel of the C entry points.
//
// Every entry point is `extern "C" int gi_<name>(..., void* stream)`.  It
// returns 0 when the kernel was launched, and a non-zero code otherwise; the
// text of the last failure on the calling thread is read with
// gi_last_error().  Sizes that a kernel cannot take are refused here with a
// message, never computed wrongly.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GI_DTYPE_F32 0
#define GI_DTYPE_BF16 1

#define GI_ERR_ARGUMENT 1000001   // a size or dtype the kernel refuses

#ifdef __cplusplus
extern "C" {
#endif
const char* gi_last_error(void);
#ifdef __cplusplus
}
#endif

void gi_set_error(const char* fmt, ...);
int gi_check_launch(const char* what);

#define GI_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            gi_set_error(__VA_ARGS__);        \
            return GI_ERR_ARGUMENT;           \
        }                                     \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// weight vectors (norm weights) may be stored in either type, whatever the activations are
__device__ __forceinline__ float load_w(const void* w, int w_dtype, int i) {
    return w_dtype == GI_DTYPE_F32 ? ((const float*)w)[i] : __bfloat162float(((const bf16*)w)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block in a fixed order (lane tree, then warps in index order), so
// that the result depends only on the block size and the data.
__device__ __forceinline__ float block_sum(float v, float* smem /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < n_warps; ++w) t += smem[w];
        smem[32] = t;
    }
    __syncthreads();
    return smem[32];
}
