// bfloat16 product for decode batches: out[M,N] = x[M,K] . W[N,K]^T with 1 <= M <= 16.
//
// At these sizes the step is bound by reading W once, but a plain GEMV has
// too much arithmetic and activation traffic per weight byte once M grows, so
// the product runs on the tensor cores with the operands swapped: 16 rows of W
// are the 16-row operand of mma.sync m16n8k16 and the batch is the 8-wide one.
//
//  * The mma sums over its 16 k-slots in any order, so each thread feeds its
//    own 16 k of a 64-wide chunk into the slots it owns, for the W rows and
//    for x alike: no thread ever needs another thread's data.  Each thread
//    therefore streams its pieces with cp.async through a queue of its own in
//    shared memory, several chunks deep, and the warps never wait for each
//    other while they stream.  W bypasses L1; x (at most 16 rows) goes
//    through it.
//  * A CTA has 8 warps: WR groups of 16 rows times WK interleaved shares of K,
//    added up in shared memory at the end.
//  * K is also split across the CTAs of a thread-block cluster.  Their partial
//    sums meet in distributed shared memory: every CTA of the cluster adds up
//    one share of the tile, reading its peers' partials in rank order, so the
//    result is the same from run to run and no scratch memory or second
//    kernel is needed.
//
// Upstream calls a library product whatever M is (src/src-cuda/mat-ops/gemm/gemm.cu:22-41).
#include "common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define SK_DEPTH 4          // chunks of 64 k a thread has in flight or in use

// 16 bytes global -> shared, zero-filled when `valid` is false.  .cg keeps the weights out of L1 (they are
// read once); .ca lets L1 hold the activations, which every warp reads again.
__device__ __forceinline__ void sk_cp_async_cg(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sk_cp_async_ca(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sk_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 k of this thread for the W rows g and g+8 and for NT batch rows, multiplied into acc
template <int NT>
__device__ __forceinline__ void sk_step(float (&acc)[NT][4], const uint4& lo0, const uint4& lo1, const uint4& hi0,
                                        const uint4& hi1, const uint4 (&x0)[NT], const uint4 (&x1)[NT]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        sk_mma(acc[nt], lo0.x, hi0.x, lo0.y, hi0.y, x0[nt].x, x0[nt].y);
        sk_mma(acc[nt], lo0.z, hi0.z, lo0.w, hi0.w, x0[nt].z, x0[nt].w);
        sk_mma(acc[nt], lo1.x, hi1.x, lo1.y, hi1.y, x1[nt].x, x1[nt].y);
        sk_mma(acc[nt], lo1.z, hi1.z, lo1.w, hi1.w, x1[nt].z, x1[nt].w);
    }
}

// GLU: W is [2 I, K], a gate projection in its first I rows and an up projection in its last I.  A CTA then
// takes R / 2 gate rows and the R / 2 up rows that belong to them, and writes silu(gate) * up, [M, I]
// bfloat16: each factor rounded to bfloat16 as a stored product would be, then the SwiGLU kernel's float32
// arithmetic: the product followed by that kernel, up to the order in which a CTA walks K.
template <int NT, int WR, int WK, bool GLU>
__global__ void __launch_bounds__(SK_THREADS)
skinny_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, void* __restrict__ out, int out_f32,
                   int M, int N, int K, int k_slice) {
    static_assert(WR * WK == SK_WARPS, "8 warps");
    gi_pdl_launch_dependents();
    constexpr int MP = 8 * NT;                   // padded batch
    constexpr int R = 16 * WR;                   // W rows per CTA
    constexpr int CH = 4;                        // 16-byte pieces of W a thread brings in per chunk
    extern __shared__ __align__(16) unsigned char sk_smem[];
    uint4* ring = reinterpret_cast<uint4*>(sk_smem);                     // [SK_DEPTH][CH][threads]: each thread's own queue
    float* red = reinterpret_cast<float*>(ring + SK_DEPTH * CH * SK_THREADS);   // [WK][MP][R]
    float* part = red + WK * MP * R;                                     // [MP][R], read by the cluster's other CTAs

    cg::cluster_group cluster = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int wr = warp % WR, wk = warp / WR;
    const int row0 = blockIdx.x * R;
    const int k_begin = blockIdx.y * k_slice, k_end = min(K, k_begin + k_slice);

    // the rows of W behind local rows wr * 16 + g and + 8
    auto w_row = [&](int local) {
        if (!GLU) return min(row0 + local, N - 1);
        constexpr int half = R / 2;
        const int inter = N / 2;
        return local < half ? min((int)blockIdx.x * half + local, inter - 1)
                            : min(inter + (int)blockIdx.x * half + local - half, N - 1);
    };
    const bf16* wa = W + (size_t)w_row(wr * 16 + g) * K;
    const bf16* wb = W + (size_t)w_row(wr * 16 + g + 8) * K;
    const bf16* xr[NT];
    bool xok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        xok[nt] = nt * 8 + g < M;
        xr[nt] = x + (size_t)min(nt * 8 + g, M - 1) * K;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;

    // This warp's chunks of 64 k are wk, wk + WK, ...; inside a chunk a thread takes the 8 k at 8 t and
    // the 8 k at 32 + 8 t, so that each copy of a warp reads 64 contiguous bytes (two whole sectors) of
    // 8 rows.  The chunk count depends on the warp alone: mma.sync needs all 32 lanes, so a chunk that
    // K cuts short is still multiplied by every lane, the lanes beyond K getting zeros.
    // Every thread keeps SK_DEPTH - 1 chunks in flight in a queue of its own in shared memory
    // (cp.async into slots that only it reads back), so the bytes in flight do not depend on
    // registers or on the other warps, and nothing but the copy itself is ever waited for.
    const int k_first = k_begin + wk * 64;
    const int n_chunks = k_first < k_end ? (k_end - k_first + WK * 64 - 1) / (WK * 64) : 0;
    // Every CTA walks its chunks from another start (and wraps around).  CTAs that all begin at k = 0 ask the
    // same few memory channels at the same time, row after row 8 KB apart: measured, the rotation takes the
    // gate/up product of the benchmark model at 8 rows from 37.7 to 35.8 us and the head from 214 to 192 us.
    // The order of the sum over k is fixed per CTA, so a result is the same from run to run.
    const int rot = n_chunks > 0 ? (int)((blockIdx.x * 13u + blockIdx.y * 5u) % (unsigned)n_chunks) : 0;
    auto issue = [&](int i) {
        if (i < n_chunks) {
            const int ir = i + rot < n_chunks ? i + rot : i + rot - n_chunks;
            const int k = k_first + ir * WK * 64 + t * 8;
            const bool in0 = k + 8 <= k_end, in1 = k + 40 <= k_end;
            uint4* slot = ring + (size_t)(i % SK_DEPTH) * CH * SK_THREADS + threadIdx.x;
            sk_cp_async_cg(slot + 0 * SK_THREADS, wa + (in0 ? k : 0), in0);
            sk_cp_async_cg(slot + 1 * SK_THREADS, wa + (in1 ? k + 32 : 0), in1);
            sk_cp_async_cg(slot + 2 * SK_THREADS, wb + (in0 ? k : 0), in0);
            sk_cp_async_cg(slot + 3 * SK_THREADS, wb + (in1 ? k + 32 : 0), in1);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");   // an empty group when nothing is left: the count stays uniform
    };
    // x comes from L1/L2 into registers one chunk ahead (a chunk takes far longer than that read)
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    auto load_x = [&](int i, uint4 (&x0)[NT], uint4 (&x1)[NT]) {
        const int ir = i + rot < n_chunks ? i + rot : i + rot - n_chunks;
        const int k = k_first + ir * WK * 64 + t * 8;
        const bool in0 = i < n_chunks && k + 8 <= k_end, in1 = i < n_chunks && k + 40 <= k_end;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            x0[nt] = in0 && xok[nt] ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + k)) : zero4;
            x1[nt] = in1 && xok[nt] ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + k + 32)) : zero4;
        }
    };
#pragma unroll
    for (int i = 0; i < SK_DEPTH - 1; ++i) issue(i);
    gi_pdl_wait();                               // W is nobody's output: its first chunks are on their way by now
    uint4 x0[NT], x1[NT];
    load_x(0, x0, x1);
    for (int i = 0; i < n_chunks; ++i) {
        issue(i + SK_DEPTH - 1);
        uint4 nx0[NT], nx1[NT];
        load_x(i + 1, nx0, nx1);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SK_DEPTH - 1) : "memory");
        const uint4* slot = ring + (size_t)(i % SK_DEPTH) * CH * SK_THREADS + threadIdx.x;
        const uint4 lo0 = slot[0 * SK_THREADS], lo1 = slot[1 * SK_THREADS];
        const uint4 hi0 = slot[2 * SK_THREADS], hi1 = slot[3 * SK_THREADS];
        sk_step<NT>(acc, lo0, lo1, hi0, hi1, x0, x1);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { x0[nt] = nx0[nt]; x1[nt] = nx1[nt]; }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");

    // the warps' shares of K meet in shared memory: red[wk][m][r], r fastest
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int m = nt * 8 + 2 * t, r = wr * 16 + g;
        red[(wk * MP + m) * R + r] = acc[nt][0];
        red[(wk * MP + m + 1) * R + r] = acc[nt][1];
        red[(wk * MP + m) * R + r + 8] = acc[nt][2];
        red[(wk * MP + m + 1) * R + r + 8] = acc[nt][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < MP * R; i += SK_THREADS) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WK; ++w) v += red[w * MP * R + i];
        part[i] = v;
    }
    const unsigned n_ranks = cluster.num_blocks(), rank = cluster.block_rank();
    if (n_ranks > 1) cluster.sync(); else __syncthreads();
    // every CTA of the cluster finishes one share of the tile, adding the partials in rank order
    if (GLU) {
        constexpr int half = R / 2;
        const int inter = N / 2;
        const int share = (MP * half + n_ranks - 1) / n_ranks;
        const int i_end = min(MP * half, (int)(rank + 1) * share);
        for (int i = rank * share + threadIdx.x; i < i_end; i += SK_THREADS) {
            const int m = i / half, r = i % half;
            float gate = 0.f, up = 0.f;
            for (unsigned c = 0; c < n_ranks; ++c) {
                const float* p = n_ranks > 1 ? cluster.map_shared_rank(part, c) : part;
                gate += p[m * R + r];
                up += p[m * R + r + half];
            }
            const int col = blockIdx.x * half + r;
            if (m < M && col < inter) {
                const float gf = __bfloat162float(__float2bfloat16_rn(gate)), uf = __bfloat162float(__float2bfloat16_rn(up));
                reinterpret_cast<bf16*>(out)[(size_t)m * inter + col] = __float2bfloat16_rn(gf / (1.f + expf(-gf)) * uf);
            }
        }
    } else {
        const int share = (MP * R + n_ranks - 1) / n_ranks;
        const int i_end = min(MP * R, (int)(rank + 1) * share);
        for (int i = rank * share + threadIdx.x; i < i_end; i += SK_THREADS) {
            float v = 0.f;
            for (unsigned c = 0; c < n_ranks; ++c) v += n_ranks > 1 ? cluster.map_shared_rank(part, c)[i] : part[i];
            const int m = i / R, row = row0 + i % R;
            if (m < M && row < N) {
                if (out_f32) reinterpret_cast<float*>(out)[(size_t)m * N + row] = v;
                else reinterpret_cast<bf16*>(out)[(size_t)m * N + row] = __float2bfloat16_rn(v);
            }
        }
    }
    if (n_ranks > 1) cluster.sync();            // nobody leaves while a peer still reads its partial
}

template <int NT, int WR, int WK, bool GLU>
static int launch_skinny(const bf16* x, const bf16* W, void* out, int out_f32, int M, int N, int K, int n_split,
                         cudaStream_t stream) {
    constexpr int MP = 8 * NT, R = 16 * WR, KC = 64 * WK;
    const size_t smem = (size_t)SK_DEPTH * 4 * SK_THREADS * 16 + (size_t)(WK + 1) * MP * R * sizeof(float);
    if (int rc = gi_reserve_smem((const void*)skinny_gemm_kernel<NT, WR, WK, GLU>, smem, "gi_gemm_skinny_bf16")) return rc;
    const int k_slice = ((K + n_split - 1) / n_split + KC - 1) / KC * KC;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(GLU ? (N / 2 + R / 2 - 1) / (R / 2) : (N + R - 1) / R, n_split, 1);
    cfg.blockDim = dim3(SK_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = n_split;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gi_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<NT, WR, WK, GLU>, x, W, out, out_f32, M, N, K, k_slice);
    if (e != cudaSuccess) { gi_set_error("gi_gemm_skinny_bf16: launch: %s", cudaGetErrorString(e)); return (int)e; }
    return gi_check_launch("gi_gemm_skinny_bf16");
}

// n_split: CTAs of a cluster that share K (1 to 8); 0 lets the entry point choose.
// wide: 0 = 32 rows of W per CTA, 1 = 64 rows, -1 lets the entry point choose.
// glu: 0 = out[M, N]; 1 = W holds a gate and an up half and out is silu(gate) * up, [M, N / 2] bfloat16.
static int skinny_entry(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K, int n_split,
                        int wide, int glu, void* stream) {
    GI_REQUIRE(M >= 1 && M <= 16, "gi_gemm_skinny_bf16: %d rows; this kernel takes 1 to 16", M);
    GI_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gi_gemm_skinny_bf16: inner size %d must be a positive multiple of 8", K);
    GI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0), "gi_gemm_skinny_bf16: operands must start on 16 bytes");
    GI_REQUIRE(out_dtype == GI_DTYPE_BF16 || out_dtype == GI_DTYPE_F32, "gi_gemm_skinny_bf16: output dtype %d", out_dtype);
    GI_REQUIRE(n_split >= 0 && n_split <= 8, "gi_gemm_skinny_bf16: a cluster of %d CTAs; 1 to 8 are possible", n_split);
    GI_REQUIRE(wide >= -1 && wide <= 1, "gi_gemm_skinny_bf16: wide must be -1, 0 or 1");
    GI_REQUIRE(!glu || (N % 2 == 0 && out_dtype == GI_DTYPE_BF16),
               "gi_gemm_skinny_swiglu_bf16: W must hold a gate and an up half (%d rows) and the output be bfloat16", N);
    // Every CTA streams at the pace its own loads in flight allow, so the launch should fit the GPU in one
    // wave of equal CTAs (3 fit an SM) or be many waves long.  Among the shapes that fit in one wave, the
    // choice goes to slices of K of equal length (measured at 8 rows inside a decode step: hidden 4096 to 4096
    // as 2 slices of 2048 is 2.4 us faster than as 3 slices of 1536, 1536 and 1024), then to the most CTAs,
    // then to slices of at most 2048 (12288 to 4096 in 6 slices over 64-row tiles is 0.9 us faster than in 3
    // slices over 32-row tiles), then to the narrower tile.
    const int slots = 148 * 3;
    const bool pick_wide = wide < 0, pick_split = n_split == 0;
    if (pick_wide || pick_split) {
        long long best = -1;
        int best_wide = pick_wide ? 0 : wide, best_split = pick_split ? 1 : n_split;
        for (int w = 0; w <= 1; ++w) {
            if (!pick_wide && w != wide) continue;
            const int R = w ? 64 : 32, KC = w ? 128 : 256;
            const long long tiles = glu ? (N / 2 + R / 2 - 1) / (R / 2) : (N + R - 1) / R;
            for (int ns = 1; ns <= 8; ++ns) {
                if (!pick_split && ns != n_split) continue;
                if (tiles * ns > slots || (ns > 1 && K / ns < 2 * KC)) continue;
                const bool even = K % (ns * KC) == 0;
                const int slice = (K + ns - 1) / ns;
                const long long score = (even ? 1LL << 40 : 0) + ((tiles * ns) << 8) + (slice <= 2048 ? 2 : 0) + (w ? 0 : 1);
                if (score > best) best = score, best_wide = w, best_split = ns;
            }
        }
        if (best < 0) {                          // no shape fits in one wave: many waves of whole rows
            if (pick_wide) best_wide = (N + 31) / 32 > slots && (N + 63) / 64 <= 8 * slots ? 1 : 0;
            if (pick_split) best_split = 1;
        }
        wide = best_wide, n_split = best_split;
    }
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    const int f32 = out_dtype == GI_DTYPE_F32;
    cudaStream_t s = (cudaStream_t)stream;
#define GI_SK(NT, WR, WK) (glu ? launch_skinny<NT, WR, WK, true>(xp, wp, out, f32, M, N, K, n_split, s) \
                               : launch_skinny<NT, WR, WK, false>(xp, wp, out, f32, M, N, K, n_split, s))
    if (M <= 8) return wide ? GI_SK(1, 4, 2) : GI_SK(1, 2, 4);
    return wide ? GI_SK(2, 4, 2) : GI_SK(2, 2, 4);
#undef GI_SK
}

extern "C" int gi_gemm_skinny_bf16(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K,
                                   int n_split, int wide, void* stream) {
    return skinny_entry(x, W, out, out_dtype, M, N, K, n_split, wide, 0, stream);
}

// out[M, I] = silu(x . Wg^T) * (x . Wu^T) for W = [Wg; Wu] of two_inter = 2 I rows: the gate/up product of a
// SwiGLU feed-forward at decode batches with the activation in the kernel's last step.
extern "C" int gi_gemm_skinny_swiglu_bf16(const void* x, const void* W, void* out, int M, int two_inter, int K,
                                          int n_split, int wide, void* stream) {
    return skinny_entry(x, W, out, GI_DTYPE_BF16, M, two_inter, K, n_split, wide, 1, stream);
}
