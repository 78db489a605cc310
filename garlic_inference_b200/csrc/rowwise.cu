// Row-wise kernels: token embedding, residual add + RMSNorm, SwiGLU, casts.
//
// The residual stream is float32 in both precisions of the engine; T is the
// activation type (float or bfloat16).  Norms and the residual sum are
// computed in float32 and rounded once.
//
// Upstream counterparts: embedding rows (src/src-cuda/embedding.cu:29-53),
// RMSNorm and add+RMSNorm (src/src-cuda/norm.cu:3-101), SiLU then a product
// as two kernels (src/src-cuda/activations/silu.cu:35-67,
// src/src-cuda/mat-ops/simple-ops/hadamard.cu:48-67).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32.  An id outside [0, vocab) writes zeros.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int vocab, int hidden) {
    gi_pdl_start();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]);
}

extern "C" int gi_embedding(const int* ids, const void* table, int table_dtype, float* out,
                            int n_tokens, int vocab, int hidden, void* stream) {
    GI_REQUIRE(n_tokens >= 0 && vocab > 0 && hidden > 0, "gi_embedding: sizes must be positive");
    if (n_tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == GI_DTYPE_F32)
        gi_launch(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, ids, (const float*)table, out, vocab, hidden);
    else if (table_dtype == GI_DTYPE_BF16)
        gi_launch(embedding_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, ids, (const bf16*)table, out, vocab, hidden);
    else
        GI_REQUIRE(false, "gi_embedding: table dtype %d is neither float32 nor bfloat16", table_dtype);
    return gi_check_launch("gi_embedding");
}

// ------------------------------------------------------- residual add + RMSNorm
// For output row r (input row i = rows ? rows[r] : r):
//   s = residual[i] (+ delta[i] when delta is given)        float32
//   if write_residual: residual[i] = s
//   out[r] = s * rsqrt(mean(s^2) + eps) * weight            rounded once to T
// The block size depends on `dim` alone, so a row's result does not depend on
// how many rows are in the launch.
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ delta, float* __restrict__ residual,
                                   const void* __restrict__ weight, int w_dtype, T* __restrict__ out,
                                   const int* __restrict__ rows, int dim, float eps, int write_residual) {
    gi_pdl_start();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + i * dim;
    const T* del = delta ? delta + i * dim : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float s = res[c];
        if (del) s += to_f32(del[c]);
        if (write_residual && del) res[c] = s;
        ss += s * s;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)dim + eps);
    T* o = out + (size_t)r * dim;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float s = res[c];
        if (del && !write_residual) s += to_f32(del[c]);
        o[c] = from_f32<T>(s * inv * load_w(weight, w_dtype, c));
    }
}

// The same with the row held in registers: one read of the inputs, four elements per thread and load.
// Taken when dim is a multiple of 4 and at most 8,192; the thread count depends on dim alone.
#define NORM_VEC_MAX_IT 8
__device__ __forceinline__ float4 load4_f32(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4_act(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4_act(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4_act(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4_act(bf16* p, float4 v) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}
__device__ __forceinline__ float4 load4_w(const void* w, int w_dtype, int c) {
    return w_dtype == GI_DTYPE_F32 ? load4_f32((const float*)w + c) : load4_act((const bf16*)w + c);
}

// EARLY_W: the weight is fetched into registers before the wait for the kernel that makes delta (it is
// nobody's output).  That pays for a few rows, where the kernel is one chain of latencies; for thousands
// of rows the registers cost more in occupancy than the early fetch gives (13.6 vs 20.1 us at 2,048 rows).
template <typename T, int EARLY_W>
__global__ void add_rmsnorm_vec_kernel(const T* __restrict__ delta, float* __restrict__ residual,
                                       const void* __restrict__ weight, int w_dtype, T* __restrict__ out,
                                       const int* __restrict__ rows, int dim, float eps, int write_residual) {
    gi_pdl_launch_dependents();
    __shared__ float red[33];
    const int r = blockIdx.x;
    float4 w4[EARLY_W ? NORM_VEC_MAX_IT : 1];
    if (EARLY_W) {
#pragma unroll
        for (int it = 0; it < NORM_VEC_MAX_IT; ++it) {
            const int c = (it * blockDim.x + threadIdx.x) * 4;
            if (c < dim) w4[it] = load4_w(weight, w_dtype, c);
        }
        // The residual was last written several kernels ago and the weights streamed since have pushed it out
        // of L2: its lines are asked back into L2 now (a hint, nothing is read yet, so it does not matter
        // whether that earlier kernel has finished).
        if (!rows) {
            const float* line = residual + (size_t)r * dim + threadIdx.x * 32;
            if (threadIdx.x * 32 < dim) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
        }
    }
    gi_pdl_wait();
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + i * dim;
    const T* del = delta ? delta + i * dim : nullptr;
    float4 v[NORM_VEC_MAX_IT];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NORM_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            float4 s = load4_f32(res + c);
            if (del) {
                const float4 d4 = load4_act(del + c);
                s.x += d4.x; s.y += d4.y; s.z += d4.z; s.w += d4.w;
                if (write_residual) *reinterpret_cast<float4*>(res + c) = s;
            }
            v[it] = s;
            ss += s.x * s.x;                     // the same order of additions whatever the batch is
            ss += s.y * s.y;
            ss += s.z * s.z;
            ss += s.w * s.w;
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)dim + eps);
    T* o = out + (size_t)r * dim;
#pragma unroll
    for (int it = 0; it < NORM_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            const float4 w = EARLY_W ? w4[EARLY_W ? it : 0] : load4_w(weight, w_dtype, c);
            store4_act(o + c, make_float4(v[it].x * inv * w.x, v[it].y * inv * w.y, v[it].z * inv * w.z, v[it].w * inv * w.w));
        }
    }
}

extern "C" int gi_add_rmsnorm(const void* delta, float* residual, const void* weight, int w_dtype,
                              void* out, int act_dtype, const int* rows, int n_rows, int dim,
                              float eps, int write_residual, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0, "gi_add_rmsnorm: sizes must be positive");
    GI_REQUIRE(w_dtype == GI_DTYPE_F32 || w_dtype == GI_DTYPE_BF16, "gi_add_rmsnorm: weight dtype %d", w_dtype);
    GI_REQUIRE(!(rows && write_residual), "gi_add_rmsnorm: gathered rows cannot write the residual back");
    if (n_rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = ((uintptr_t)residual % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                         ((uintptr_t)delta % 16 == 0);
    if (dim % 4 == 0 && dim <= 256 * 4 * NORM_VEC_MAX_IT && aligned) {
        int threads = ((dim / 4 + 31) / 32) * 32;
        threads = threads > 256 ? 256 : threads;
        const bool early = n_rows <= 256;
#define LAUNCH_NORM(T, E) gi_launch(add_rmsnorm_vec_kernel<T, E>, dim3(n_rows), dim3(threads), 0, s, (const T*)delta, residual, \
                                    weight, w_dtype, (T*)out, rows, dim, eps, write_residual)
        if (act_dtype == GI_DTYPE_F32) { if (early) LAUNCH_NORM(float, 1); else LAUNCH_NORM(float, 0); }
        else if (act_dtype == GI_DTYPE_BF16) { if (early) LAUNCH_NORM(bf16, 1); else LAUNCH_NORM(bf16, 0); }
#undef LAUNCH_NORM
        else
            GI_REQUIRE(false, "gi_add_rmsnorm: activation dtype %d", act_dtype);
        return gi_check_launch("gi_add_rmsnorm");
    }
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : (dim >= 128 ? 128 : 32));
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (const float*)delta, residual, weight, w_dtype,
                                                             (float*)out, rows, dim, eps, write_residual);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, (const bf16*)delta, residual, weight, w_dtype,
                                                            (bf16*)out, rows, dim, eps, write_residual);
    else
        GI_REQUIRE(false, "gi_add_rmsnorm: activation dtype %d", act_dtype);
    return gi_check_launch("gi_add_rmsnorm");
}

// residual[i] += delta[i] (float32 sum), for arrangements that need the stream itself.
template <typename T>
__global__ void residual_add_kernel(const T* __restrict__ delta, float* __restrict__ residual, size_t n) {
    gi_pdl_start();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) residual[i] += to_f32(delta[i]);
}

extern "C" int gi_residual_add(const void* delta, int act_dtype, float* residual, long long n, void* stream) {
    GI_REQUIRE(n >= 0, "gi_residual_add: negative size");
    if (n == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 4096 ? (n + threads - 1) / threads : 4096);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(residual_add_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)delta, residual, (size_t)n);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)delta, residual, (size_t)n);
    else
        GI_REQUIRE(false, "gi_residual_add: activation dtype %d", act_dtype);
    return gi_check_launch("gi_residual_add");
}

// ------------------------------------------------------------------- SwiGLU
// gate_up is [n, 2*inter]: the gate in the first `inter` columns, the up
// projection in the last.  out[n, inter] = silu(gate) * up, in float32, rounded once.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
    gi_pdl_start();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t row = i / inter;
        const int c = (int)(i - row * inter);
        const float g = to_f32(gate_up[row * 2 * inter + c]);
        const float u = to_f32(gate_up[row * 2 * inter + inter + c]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

// bfloat16, 8 columns a thread (inter must be a multiple of 8)
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int inter,
                                     size_t total_vec) {
    gi_pdl_start();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int vec_per_row = inter / 8;
    for (; i < total_vec; i += stride) {
        const size_t row = i / vec_per_row;
        const int c = (int)(i - row * vec_per_row) * 8;
        const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + c);
        const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(g2[k]);
            const float2 u = __bfloat1622float2(u2[k]);
            o2[k] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + row * inter + c) = ov;
    }
}

extern "C" int gi_swiglu(const void* gate_up, void* out, int act_dtype, int n_rows, int inter, void* stream) {
    GI_REQUIRE(n_rows >= 0 && inter > 0, "gi_swiglu: sizes must be positive");
    if (n_rows == 0) return 0;
    const size_t total = (size_t)n_rows * inter;
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_BF16 && inter % 8 == 0) {
        const size_t nv = total / 8;
        const int blocks = (int)((nv + threads - 1) / threads < 65535 ? (nv + threads - 1) / threads : 65535);
        gi_launch(swiglu_bf16x8_kernel, dim3(blocks), dim3(threads), 0, s, (const bf16*)gate_up, (bf16*)out, inter, nv);
        return gi_check_launch("gi_swiglu");
    }
    const int blocks = (int)((total + threads - 1) / threads < 65535 ? (total + threads - 1) / threads : 65535);
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, inter, total);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)gate_up, (bf16*)out, inter, total);
    else
        GI_REQUIRE(false, "gi_swiglu: activation dtype %d", act_dtype);
    return gi_check_launch("gi_swiglu");
}

// -------------------------------------------------------------------- casts
template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
    gi_pdl_start();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = from_f32<D>(to_f32(src[i]));
}

extern "C" int gi_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream) {
    GI_REQUIRE(n >= 0, "gi_cast: negative size");
    if (n == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 65535 ? (n + threads - 1) / threads : 65535);
    cudaStream_t s = (cudaStream_t)stream;
    if (src_dtype == GI_DTYPE_F32 && dst_dtype == GI_DTYPE_BF16)
        gi_launch(cast_kernel<float, bf16>, dim3(blocks), dim3(threads), 0, s, (const float*)src, (bf16*)dst, (size_t)n);
    else if (src_dtype == GI_DTYPE_BF16 && dst_dtype == GI_DTYPE_F32)
        gi_launch(cast_kernel<bf16, float>, dim3(blocks), dim3(threads), 0, s, (const bf16*)src, (float*)dst, (size_t)n);
    else
        GI_REQUIRE(false, "gi_cast: from dtype %d to dtype %d", src_dtype, dst_dtype);
    return gi_check_launch("gi_cast");
}
