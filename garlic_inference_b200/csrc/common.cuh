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
// Raises `kernel`'s limit of dynamic shared memory to `bytes` on the current device; remembered per kernel and
// device only once it has succeeded, so a second device, or a call after a failed one, sets it again.
int gi_reserve_smem(const void* kernel, size_t bytes, const char* who);

#define GI_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            gi_set_error(__VA_ARGS__);        \
            return GI_ERR_ARGUMENT;           \
        }                                     \
    } while (0)

typedef __nv_bfloat16 bf16;

// A timeline of a recorded step, for builds made with -DGI_TIMELINE -DGI_TU=<file stem> (csrc/build.py does
// that when GARLIC_B200_TIMELINE=1; the ordinary build has none of it).  Thread 0 of block 0 of every kernel
// notes %globaltimer twice: when it starts (mark 0, with the launch's size) and when the kernel before it in the
// stream has finished (mark 1, after griddepcontrol.wait).  Both marks are taken in launch order, so entry i of
// either list belongs to the i-th kernel, and the time between the second marks of two neighbours is what the
// earlier one costs the chain.  Layout of the buffer (unsigned 64-bit): [0] and [1] count the marks, entry i is
// [4 + 4 i + {0: start ns, 1: released ns, 2: blocks << 16 | threads}].  Every file has its own copy of the
// pointer, set through gi_tl_set_<file stem>().
#ifdef GI_TIMELINE
#define GI_TL_ENTRIES 4096
static __device__ unsigned long long* gi_tl_buf = nullptr;
#define GI_TL_CAT2(a, b) a##b
#define GI_TL_CAT(a, b) GI_TL_CAT2(a, b)
extern "C" void GI_TL_CAT(gi_tl_set_, GI_TU)(void* p) { cudaMemcpyToSymbol(gi_tl_buf, &p, sizeof(p)); }
__device__ __forceinline__ void gi_tl_mark(int which) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && gi_tl_buf) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const unsigned long long i = atomicAdd(gi_tl_buf + which, 1ULL);
        if (i < GI_TL_ENTRIES) {
            gi_tl_buf[4 + 4 * i + which] = t;
            if (which == 0)
                gi_tl_buf[4 + 4 * i + 2] = ((unsigned long long)(gridDim.x * gridDim.y * gridDim.z) << 16) | blockDim.x;
        }
    }
}
#else
__device__ __forceinline__ void gi_tl_mark(int) {}
#endif

// Programmatic dependent launch.  Every kernel of this library starts with gi_pdl_start(): when the
// launches carry the attribute below, it lets the next kernel of the stream be launched while this one
// still runs (its blocks then sit in their own gi_pdl_start until this grid has finished and its writes
// are visible).  Nothing may be read or written before it.  Without the attribute both instructions do
// nothing.  Measured on a B200 inside the recorded decode step of Qwen3-8B sizes, with the kernels
// requesting before the wait what no kernel of the step writes (weights, tables, the cache of earlier
// steps): batch 8 +7 %, batch 1 +11 %, batch 64 +1 %.  The engine asks for it (gi_set_pdl) while it records
// decode steps, and nowhere else; GARLIC_B200_PDL=0 or =1 in the environment overrides that for the process.
__device__ __forceinline__ void gi_pdl_start() {
    gi_tl_mark(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    gi_tl_mark(1);
}
// The two halves apart, for kernels that have something to do that depends on no earlier kernel (fetching
// weights): gi_pdl_launch_dependents() first, then that work, then gi_pdl_wait() before anything an
// earlier kernel wrote is read and before anything is written.
__device__ __forceinline__ void gi_pdl_launch_dependents() {
    gi_tl_mark(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void gi_pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    gi_tl_mark(1);
}

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

// The hash behind every counter-based random number of this library (sampling draws, random weights): the
// splitmix64 finaliser.  Integer arithmetic only, so host and device agree bit for bit.
__host__ __device__ __forceinline__ unsigned long long gi_mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
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
