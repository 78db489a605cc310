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

// Programmatic dependent launch.  Every kernel of this library starts with gi_pdl_start(): when the
// launches carry the attribute below, it lets the next kernel of the stream be launched while this one
// still runs (its blocks then sit in their own gi_pdl_start until this grid has finished and its writes
// are visible).  Nothing may be read or written before it.  Without the attribute both instructions do
// nothing.  Measured on a B200 inside the recorded decode step of Qwen3-8B sizes, with the kernels
// requesting before the wait what no kernel of the step writes (weights, tables, the cache of earlier
// steps): batch 8 +7 %, batch 1 +11 %, batch 64 +1 %.  The engine asks for it (gi_set_pdl) while it records
// decode steps, and nowhere else; GARLIC_B200_PDL=0 or =1 in the environment overrides that for the process.
__device__ __forceinline__ void gi_pdl_start() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// The two halves apart, for kernels that have something to do that depends on no earlier kernel (fetching
// weights): gi_pdl_launch_dependents() first, then that work, then gi_pdl_wait() before anything an
// earlier kernel wrote is read and before anything is written.
__device__ __forceinline__ void gi_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void gi_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// kernel<<<grid, block, smem, stream>>>(args...), with the attribute that allows the overlap above when
// gi_pdl_enabled().
bool gi_pdl_enabled();
template <typename... KArgs, typename... Args>
static inline void gi_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gi_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);      // errors surface in gi_check_launch
}

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
