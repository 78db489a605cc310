// bfloat16 matrix product for a handful of rows (decoding at small batch):
// out[M,N] = x[M,K] . W[N,K]^T with M <= 8.  The step reads every weight once,
// so the kernel is written for memory bandwidth: one warp per weight row, 16-byte
// loads that bypass L1 for the weights, four loads in flight per lane, float32
// accumulation, x read through L1 (all warps of an SM share it).
//
// Upstream calls a library product whatever M is (src/src-cuda/mat-ops/gemm/gemm.cu:22-41).
#include "common.cuh"

#define GV_WARPS 8

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <int M>
__device__ __forceinline__ void fma8(const uint4& w, const bf16* __restrict__ x, int K, int k, float (&acc)[M]) {
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w);
    float2 wf[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wf[i] = __bfloat1622float2(w2[i]);
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K + k));
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 xf = __bfloat1622float2(x2[i]);
            acc[m] = fmaf(wf[i].x, xf.x, acc[m]);
            acc[m] = fmaf(wf[i].y, xf.y, acc[m]);
        }
    }
}

template <int M, typename OutT>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ out, int N, int K) {
    gi_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GV_WARPS + warp;
    if (n >= N) return;
    const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)n * K);
    const int nvec = K / 8;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    // The row is walked in groups of 128 vectors (four loads per lane), from a group that differs from row to
    // row, wrapping around: warps that all begin at the start of their rows ask the same few memory channels at
    // the same time.  The order of a row's sum is fixed by the row's number.
    const int groups = nvec / 128;
    const int g0 = groups > 0 ? (int)(((unsigned)n * 13u) % (unsigned)groups) : 0;
    int v = g0 * 128 + lane;
    // W is nobody's output: the first loads go out before the wait for the kernel that makes x
    uint4 h0, h1, h2, h3;
    if (groups > 0) {
        h0 = ld_stream(wrow + v), h1 = ld_stream(wrow + v + 32);
        h2 = ld_stream(wrow + v + 64), h3 = ld_stream(wrow + v + 96);
    }
    gi_pdl_wait();
    for (int j = 0; j < groups; ++j) {
        const int cur = v;
        const uint4 w0 = h0, w1 = h1, w2 = h2, w3 = h3;
        if (j + 1 < groups) {                    // the next group's loads go out before this one is multiplied
            v = (g0 + j + 1 < groups ? g0 + j + 1 : g0 + j + 1 - groups) * 128 + lane;
            h0 = ld_stream(wrow + v), h1 = ld_stream(wrow + v + 32);
            h2 = ld_stream(wrow + v + 64), h3 = ld_stream(wrow + v + 96);
        }
        fma8<M>(w0, x, K, cur * 8, acc);
        fma8<M>(w1, x, K, (cur + 32) * 8, acc);
        fma8<M>(w2, x, K, (cur + 64) * 8, acc);
        fma8<M>(w3, x, K, (cur + 96) * 8, acc);
    }
    for (v = groups * 128 + lane; v < nvec; v += 32) {
        const uint4 w0 = ld_stream(wrow + v);
        fma8<M>(w0, x, K, v * 8, acc);
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float s = warp_sum(acc[m]);
        if (lane == 0) out[(size_t)m * N + n] = from_f32<OutT>(s);
    }
}

template <typename OutT>
static int launch_gemv(const bf16* x, const bf16* W, OutT* out, int M, int N, int K, cudaStream_t s) {
    const int blocks = (N + GV_WARPS - 1) / GV_WARPS;
    switch (M) {
        case 1: gi_launch(gemv_bf16_kernel<1, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 2: gi_launch(gemv_bf16_kernel<2, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 3: gi_launch(gemv_bf16_kernel<3, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 4: gi_launch(gemv_bf16_kernel<4, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 5: gi_launch(gemv_bf16_kernel<5, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 6: gi_launch(gemv_bf16_kernel<6, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 7: gi_launch(gemv_bf16_kernel<7, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        case 8: gi_launch(gemv_bf16_kernel<8, OutT>, dim3(blocks), dim3(GV_WARPS * 32), 0, s, x, W, out, N, K); break;
        default: GI_REQUIRE(false, "gi_gemv_bf16: %d rows; this kernel takes 1 to 8", M);
    }
    return gi_check_launch("gi_gemv_bf16");
}

// out_dtype: GI_DTYPE_BF16 or GI_DTYPE_F32.  x, W and out are dense row-major.
extern "C" int gi_gemv_bf16(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K,
                            void* stream) {
    GI_REQUIRE(M >= 1 && M <= 8, "gi_gemv_bf16: %d rows; this kernel takes 1 to 8", M);
    GI_REQUIRE(N > 0 && K > 0, "gi_gemv_bf16: sizes must be positive");
    GI_REQUIRE(K % 8 == 0, "gi_gemv_bf16: inner size %d is no multiple of 8 (rows must start on 16 bytes)", K);
    GI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0), "gi_gemv_bf16: operands must start on 16 bytes");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == GI_DTYPE_BF16) return launch_gemv<bf16>((const bf16*)x, (const bf16*)W, (bf16*)out, M, N, K, s);
    if (out_dtype == GI_DTYPE_F32) return launch_gemv<float>((const bf16*)x, (const bf16*)W, (float*)out, M, N, K, s);
    GI_REQUIRE(false, "gi_gemv_bf16: output dtype %d", out_dtype);
}

// One row of x against a gate and an up projection at once: W is [2 I, K] (the gate rows first), a warp takes
// gate row n and up row I + n with eight 16-byte loads in flight per lane, and writes silu(gate) * up
// (each factor rounded to bfloat16 as a stored product would be, then the SwiGLU kernel's arithmetic).
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_swiglu_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, bf16* __restrict__ out, int inter, int K) {
    gi_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GV_WARPS + warp;
    if (n >= inter) return;
    const uint4* grow = reinterpret_cast<const uint4*>(W + (size_t)n * K);
    const uint4* urow = reinterpret_cast<const uint4*>(W + (size_t)(inter + n) * K);
    const int nvec = K / 8;
    float ga[1] = {0.f}, ua[1] = {0.f};
    // each row from the group its own number gives it, as in the kernel above (the same sums, bit for bit)
    const int groups = nvec / 128;
    const int gs = groups > 0 ? (int)(((unsigned)n * 13u) % (unsigned)groups) : 0;
    const int us = groups > 0 ? (int)(((unsigned)(inter + n) * 13u) % (unsigned)groups) : 0;
    int gv = gs * 128 + lane, uv = us * 128 + lane;
    uint4 g0, g1, g2, g3, u0, u1, u2, u3;
    // W is nobody's output: the first loads go out before the wait for the kernel that makes x
    if (groups > 0) {
        g0 = ld_stream(grow + gv), g1 = ld_stream(grow + gv + 32), g2 = ld_stream(grow + gv + 64), g3 = ld_stream(grow + gv + 96);
        u0 = ld_stream(urow + uv), u1 = ld_stream(urow + uv + 32), u2 = ld_stream(urow + uv + 64), u3 = ld_stream(urow + uv + 96);
    }
    gi_pdl_wait();
    for (int j = 0; j < groups; ++j) {
        const int gc = gv, uc = uv;
        const uint4 a0 = g0, a1 = g1, a2 = g2, a3 = g3, b0 = u0, b1 = u1, b2 = u2, b3 = u3;
        if (j + 1 < groups) {
            gv = (gs + j + 1 < groups ? gs + j + 1 : gs + j + 1 - groups) * 128 + lane;
            uv = (us + j + 1 < groups ? us + j + 1 : us + j + 1 - groups) * 128 + lane;
            g0 = ld_stream(grow + gv), g1 = ld_stream(grow + gv + 32), g2 = ld_stream(grow + gv + 64), g3 = ld_stream(grow + gv + 96);
            u0 = ld_stream(urow + uv), u1 = ld_stream(urow + uv + 32), u2 = ld_stream(urow + uv + 64), u3 = ld_stream(urow + uv + 96);
        }
        fma8<1>(a0, x, K, gc * 8, ga); fma8<1>(a1, x, K, (gc + 32) * 8, ga);
        fma8<1>(a2, x, K, (gc + 64) * 8, ga); fma8<1>(a3, x, K, (gc + 96) * 8, ga);
        fma8<1>(b0, x, K, uc * 8, ua); fma8<1>(b1, x, K, (uc + 32) * 8, ua);
        fma8<1>(b2, x, K, (uc + 64) * 8, ua); fma8<1>(b3, x, K, (uc + 96) * 8, ua);
    }
    for (int v = groups * 128 + lane; v < nvec; v += 32) {
        const uint4 gw = ld_stream(grow + v), uw = ld_stream(urow + v);
        fma8<1>(gw, x, K, v * 8, ga);
        fma8<1>(uw, x, K, v * 8, ua);
    }
    const float gate = warp_sum(ga[0]), up = warp_sum(ua[0]);
    if (lane == 0) {
        const float gf = __bfloat162float(__float2bfloat16_rn(gate)), uf = __bfloat162float(__float2bfloat16_rn(up));
        out[n] = __float2bfloat16_rn(gf / (1.f + expf(-gf)) * uf);
    }
}

// out[1, I] = silu(x . Wg^T) * (x . Wu^T) for one row x and W = [Wg; Wu] of two_inter = 2 I rows.
extern "C" int gi_gemv_swiglu_bf16(const void* x, const void* W, void* out, int two_inter, int K, void* stream) {
    GI_REQUIRE(two_inter > 0 && two_inter % 2 == 0 && K > 0, "gi_gemv_swiglu_bf16: W must hold a gate and an up half (%d rows)", two_inter);
    GI_REQUIRE(K % 8 == 0, "gi_gemv_swiglu_bf16: inner size %d is no multiple of 8 (rows must start on 16 bytes)", K);
    GI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0), "gi_gemv_swiglu_bf16: operands must start on 16 bytes");
    const int inter = two_inter / 2;
    gi_launch(gemv_swiglu_bf16_kernel, dim3((inter + GV_WARPS - 1) / GV_WARPS), dim3(GV_WARPS * 32), 0, (cudaStream_t)stream,
              (const bf16*)x, (const bf16*)W, (bf16*)out, inter, K);
    return gi_check_launch("gi_gemv_swiglu_bf16");
}
