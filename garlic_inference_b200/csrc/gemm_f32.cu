// True float32 matrix product for the 32-bit engine: C[M,N] = A[M,K] . W[N,K]^T
// with float32 FMA on the CUDA cores, never a tensor-core or reduced-precision
// mode.  Each output element is one accumulator summed over k in ascending
// order, so a row's result is the same bits whatever M is: whole prompts,
// single tokens and batches agree exactly.
//
// Upstream multiplies with a library in the checkpoint's type only
// (src/src-cuda/mat-ops/gemm/gemm.cu:22-41, y = x W^T with W [out, in]); it has
// no 32-bit path.
#include "common.cuh"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, long long lda, long long ldc) {
    gi_pdl_start();
    __shared__ float As[SG_BK][SG_BM + 4];
    __shared__ float Ws[SG_BK][SG_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + 256 * i;
            const int r = idx >> 4, kk = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

extern "C" int gi_sgemm_nt(const float* A, const float* W, float* C, int M, int N, int K, long long lda,
                           long long ldc, void* stream) {
    GI_REQUIRE(M >= 0 && N > 0 && K > 0, "gi_sgemm_nt: sizes must be positive");
    GI_REQUIRE(lda >= K && ldc >= N, "gi_sgemm_nt: row strides shorter than the rows");
    if (M == 0) return 0;
    const long long gy = (M + SG_BM - 1) / SG_BM;
    GI_REQUIRE(gy <= 65535, "gi_sgemm_nt: %d rows in one product is beyond %d", M, 65535 * SG_BM);
    dim3 grid((N + SG_BN - 1) / SG_BN, (unsigned)gy);
    gi_launch(sgemm_nt_kernel, grid, dim3(256), 0, (cudaStream_t)stream, A, W, C, M, N, K, lda, ldc);
    return gi_check_launch("gi_sgemm_nt");
}
