// bfloat16 product for many rows (prompts): out[M,N] = x[M,K] . W[N,K]^T on the fifth-generation
// tensor cores.
//
// One CTA per SM walks over 128 x 256 tiles of the output.  Its six warps have three jobs:
//   warp 0, one lane:  TMA.  For every 64-wide slice of K it brings the 128 x 64 tile of x and the
//                      256 x 64 tile of W into one of four shared-memory stages (tensor maps with the
//                      128-byte swizzle, which is the layout the tensor core reads) and arms the
//                      stage's "full" mbarrier with the byte count.
//   warp 1, one lane:  MMA.  It waits for a stage, issues four tcgen05.mma (128 x 256 x 16 each) that
//                      accumulate in tensor memory (256 columns of float32, allocated by this warp),
//                      and commits them to the stage's "empty" mbarrier so the TMA lane may refill it;
//                      after the last slice it commits to the tile's "accumulator full" mbarrier.  There
//                      are two accumulators (2 x 256 = all 512 columns), so the next tile's products run
//                      while the epilogue drains the last one.
//   warps 2..5:        epilogue.  Each reads its 32 lanes of tensor memory with tcgen05.ld, 32 columns
//                      at a time, rounds to the output type, stores, and hands the accumulator back.
// Rows of x beyond M and columns beyond N or K are zero-filled by the TMA unit and never stored.
//
// Every wait on an mbarrier is bounded.  When a wait runs out the kernel records a code in
// *error_flag, all roles leave their loops, the copies still in flight are waited for (bounded again),
// tensor memory is freed and the kernel returns; the output is then unspecified.
//
// Upstream calls a library product for every size (src/src-cuda/mat-ops/gemm/gemm.cu:22-41).
#include "common.cuh"

#include <cuda.h>

#define TG_BM 128
#define TG_BN 256
#define TG_BK 64
#define TG_STAGES 4
#define TG_THREADS 192
#define TG_A_BYTES (TG_BM * TG_BK * 2)
#define TG_B_BYTES (TG_BN * TG_BK * 2)
#define TG_TMEM_COLS 512          // two float32 accumulators of 256 columns
#define TG_SPIN_LIMIT (1 << 22)

#define TG_ERR_PRODUCER 11
#define TG_ERR_MMA 12
#define TG_ERR_EPILOGUE 13

struct TgControl {
    unsigned long long full[TG_STAGES];
    unsigned long long empty[TG_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned int tmem_base;
    int abort;
};

__device__ __forceinline__ uint32_t tg_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tg_mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tg_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tg_mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tg_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tg_mbar_try(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(tg_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role gave up.
__device__ __forceinline__ bool tg_mbar_wait(void* bar, uint32_t parity, volatile int* abort) {
    for (int i = 0; i < TG_SPIN_LIMIT; ++i) {
        if (tg_mbar_try(bar, parity)) return true;
        if ((i & 255) == 255 && *abort) return false;
    }
    return false;
}
__device__ __forceinline__ void tg_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tg_smem(dst)), "l"(map), "r"(tg_smem(bar)), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the 128-byte
// swizzle in groups of 8 rows (1,024 bytes apart): start address, leading offset 1 (unused with a
// swizzle), stride offset 1,024 bytes, descriptor version 1, layout type 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t tg_smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tg_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tg_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tg_smem(bar)) : "memory");
}
__device__ __forceinline__ void tg_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 columns of one output row from tensor-memory registers, rounded to the output type
template <int OUT_F32>
__device__ __forceinline__ void tg_store_row(void* out, const uint32_t (&r)[32], int row, int col, int M, int N) {
    if (row >= M || col >= N) return;
    if (OUT_F32) {
        float* dst = reinterpret_cast<float*>(out) + (size_t)row * N + col;
        if (col + 32 <= N && (N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
            for (int j = 0; j < 32 && col + j < N; ++j) dst[j] = __uint_as_float(r[j]);
        }
    } else {
        bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * N + col;
        if (col + 32 <= N && (N & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = v;
            }
        } else {
            for (int j = 0; j < 32 && col + j < N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
        }
    }
}

// 32 columns of silu(gate) * up of one row: both factors rounded to bfloat16 as a stored product would be,
// then the SwiGLU kernel's float32 arithmetic, rounded once
__device__ __forceinline__ void tg_store_swiglu(bf16* out, const uint32_t (&g)[32], const uint32_t (&u)[32], int row, int col,
                                                int M, int inter) {
    if (row >= M || col >= inter) return;
    bf16* dst = out + (size_t)row * inter + col;
    const bool whole = col + 32 <= inter && (inter & 7) == 0;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            float v[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float gf = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j + e + h])));
                const float uf = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j + e + h])));
                v[h] = gf / (1.f + expf(-gf)) * uf;
            }
            __nv_bfloat162 p = __floats2bfloat162_rn(v[0], v[1]);
            packed[e >> 1] = *reinterpret_cast<uint32_t*>(&p);
        }
        if (whole) {
            *reinterpret_cast<uint4*>(dst + j) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col + j + e < inter) {
                    const uint32_t w = packed[e >> 1];
                    const unsigned short half = (e & 1) ? (unsigned short)(w >> 16) : (unsigned short)(w & 0xffff);
                    reinterpret_cast<unsigned short*>(dst)[j + e] = half;
                }
        }
    }
}

template <int OUT_F32>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, int M, int N, int K, int* __restrict__ error_flag) {
    gi_pdl_start();
    extern __shared__ unsigned char tg_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)tg_raw + 1023) & ~(uintptr_t)1023);   // the swizzle wants 1,024-byte tiles
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + TG_STAGES * TG_A_BYTES;
    TgControl* ctl = reinterpret_cast<TgControl*>(smem + TG_STAGES * (TG_A_BYTES + TG_B_BYTES));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + TG_BM - 1) / TG_BM, n_tiles = (N + TG_BN - 1) / TG_BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_tiles = (K + TG_BK - 1) / TG_BK;
    volatile int* abort = &ctl->abort;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TG_STAGES; ++s) { tg_mbar_init(&ctl->full[s], 1); tg_mbar_init(&ctl->empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tg_mbar_init(&ctl->acc_full[b], 1); tg_mbar_init(&ctl->acc_empty[b], 4); }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                             // this warp owns the tensor memory: allocates it now, frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tg_smem(&ctl->tmem_base)), "r"(TG_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctl->tmem_base;

    // A CTA walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...; tile t covers rows (t % m_tiles) and
    // columns (t / m_tiles), so the CTAs that run together share a few W tiles (L2 holds them) and all of x.
    if (warp == 0) {
        if (lane == 0) {
            int it = 0, armed = 0;               // slices so far over all tiles; slices whose copies were issued
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int m0 = (t % m_tiles) * TG_BM, n0 = (t / m_tiles) * TG_BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % TG_STAGES;
                    if (!tg_mbar_wait(&ctl->empty[s], ((it / TG_STAGES) & 1) ^ 1, abort)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_PRODUCER); }
                        ok = false;
                        break;
                    }
                    tg_mbar_expect_tx(&ctl->full[s], TG_A_BYTES + TG_B_BYTES);
                    tg_tma_load_2d(a_tiles + s * TG_A_BYTES, &map_x, kt * TG_BK, m0, &ctl->full[s]);
                    tg_tma_load_2d(b_tiles + s * TG_B_BYTES, &map_w, kt * TG_BK, n0, &ctl->full[s]);
                    armed = it + 1;
                }
            }
            if (*abort) {                        // let the copies still in flight land before the CTA leaves
                int never = 0;
                for (int i = max(0, armed - TG_STAGES); i < armed; ++i)
                    tg_mbar_wait(&ctl->full[i % TG_STAGES], (i / TG_STAGES) & 1, &never);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bfloat16 a and b, both K-major, N = 256, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TG_BN >> 3) << 17) | ((uint32_t)(TG_BM >> 4) << 24);
            int it = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
                const int buf = local & 1;       // two accumulators: the epilogue drains one while the other fills
                if (!tg_mbar_wait(&ctl->acc_empty[buf], ((local >> 1) & 1) ^ 1, abort)) {
                    if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_MMA); }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + buf * TG_BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % TG_STAGES;
                    if (!tg_mbar_wait(&ctl->full[s], (it / TG_STAGES) & 1, abort)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_MMA); }
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = tg_smem(a_tiles + s * TG_A_BYTES), b_addr = tg_smem(b_tiles + s * TG_B_BYTES);
#pragma unroll
                    for (int k = 0; k < TG_BK / 16; ++k)     // 16 elements = 32 bytes further along K inside the swizzled row
                        tg_mma(acc, tg_smem_desc(a_addr + k * 32), tg_smem_desc(b_addr + k * 32), idesc, (kt | k) != 0);
                    tg_commit(&ctl->empty[s]);               // arrives when these products have read the stage
                }
                if (ok) tg_commit(&ctl->acc_full[buf]);      // arrives when every product of the tile is done
            }
        }
    } else {
        const int q = warp & 3;                          // a warp reads the 32 lanes of tensor memory of its quarter
        int local = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
            const int buf = local & 1;
            const bool ready = tg_mbar_wait(&ctl->acc_full[buf], (local >> 1) & 1, abort);
            if (!ready) {
                if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_EPILOGUE); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m0 = (t % m_tiles) * TG_BM, n0 = (t / m_tiles) * TG_BN;
            const int row = m0 + q * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < TG_BN / 32; ++c) {
                uint32_t r[32];
                tg_ld32(tmem + ((uint32_t)(q * 32) << 16) + buf * TG_BN + c * 32, r);
                tg_store_row<OUT_F32>(out, r, row, n0 + c * 32, M, N);
            }
            // this warp has drained its part of the accumulator: the MMA lane may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tg_smem(&ctl->acc_empty[buf])) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TG_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------ pairs of CTAs
// The same product with two CTAs of a cluster on one 256 x 256 tile (tcgen05 `cta_group::2`).  Each CTA
// loads its 128 rows of x and its 128 of the tile's 256 rows of W (the pair's tensor cores exchange the
// halves of W between them, so every CTA fills and reads half the shared memory per product of the
// single-CTA kernel above), holds the accumulator of its 128 output rows in its own tensor memory, and
// stores them.  Only the CTA of even rank issues products.  The barriers across the pair:
//   full[s]       in the even CTA: armed there with the bytes of both CTAs; the TMA copies of both CTAs
//                 complete on it (the odd CTA's copies name the even CTA's barrier).
//   empty[s]      in both CTAs: the even CTA's commit arrives on both (multicast).
//   acc_full[b]   in both CTAs: likewise.
//   acc_empty[b]  in the even CTA: the epilogue warps of both CTAs arrive on it (8 arrivals).
#define TP_BN_HALF 128
#define TP_STAGES 6
#define TP_B_BYTES (TP_BN_HALF * TG_BK * 2)
#define TP_PEER_MASK 0xFEFFFFFFu             // clears the bit that tells the two CTAs of a pair apart in a shared::cluster address

struct TpControl {
    unsigned long long full[TP_STAGES];
    unsigned long long empty[TP_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned int tmem_base;
    int abort;
};

__device__ __forceinline__ void tp_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar_in_even_cta) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tg_smem(dst)), "l"(map), "r"(tg_smem(bar_in_even_cta) & TP_PEER_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tp_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair when the products issued so far are done
__device__ __forceinline__ void tp_commit_both(void* bar) {
    const unsigned short both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(tg_smem(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void tp_arrive_in_even_cta(void* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(tg_smem(bar) & TP_PEER_MASK) : "memory");
}
__device__ __forceinline__ void tp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// SWIGLU: W is [2 I, K], a gate projection in its first I rows and an up projection in its last I; the
// even CTA of the pair loads 128 gate rows and the odd CTA the 128 up rows that belong to them, so the
// accumulator holds a gate in columns 0..127 and its up in columns 128..255, and the epilogue writes
// silu(gate) * up, [M, I] bfloat16 (each factor rounded to bfloat16 first, then the SwiGLU kernel's
// arithmetic: the same bits as the product followed by that kernel).
template <int OUT_F32, int SWIGLU>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         void* __restrict__ out, int M, int N, int K, int* __restrict__ error_flag) {
    gi_pdl_start();
    extern __shared__ unsigned char tg_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)tg_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + TP_STAGES * TG_A_BYTES;
    TpControl* ctl = reinterpret_cast<TpControl*>(smem + TP_STAGES * (TG_A_BYTES + TP_B_BYTES));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = blockIdx.x & 1;             // clusters of two along x: the rank in the pair
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int inter = N / 2;                     // SWIGLU only
    const int m_tiles = (M + 2 * TG_BM - 1) / (2 * TG_BM);
    const int n_tiles = SWIGLU ? (inter + TP_BN_HALF - 1) / TP_BN_HALF : (N + TG_BN - 1) / TG_BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_tiles = (K + TG_BK - 1) / TG_BK;
    volatile int* abort = &ctl->abort;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TP_STAGES; ++s) { tg_mbar_init(&ctl->full[s], 1); tg_mbar_init(&ctl->empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tg_mbar_init(&ctl->acc_full[b], 1); tg_mbar_init(&ctl->acc_empty[b], 8); }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                             // the same warp of both CTAs allocates the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tg_smem(&ctl->tmem_base)), "r"(TG_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    tp_cluster_sync();                           // the other CTA's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, armed = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += n_pairs) {
                const int m0 = (t % m_tiles) * 2 * TG_BM + rank * TG_BM;
                const int n0 = SWIGLU ? (t / m_tiles) * TP_BN_HALF + rank * inter : (t / m_tiles) * TG_BN + rank * TP_BN_HALF;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % TP_STAGES;
                    if (!tg_mbar_wait(&ctl->empty[s], ((it / TP_STAGES) & 1) ^ 1, abort)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_PRODUCER); }
                        ok = false;
                        break;
                    }
                    if (rank == 0) tg_mbar_expect_tx(&ctl->full[s], 2 * (TG_A_BYTES + TP_B_BYTES));
                    tp_tma_load_2d(a_tiles + s * TG_A_BYTES, &map_x, kt * TG_BK, m0, &ctl->full[s]);
                    tp_tma_load_2d(b_tiles + s * TP_B_BYTES, &map_w, kt * TG_BK, n0, &ctl->full[s]);
                    armed = it + 1;
                }
            }
            if (*abort && rank == 0) {           // let the copies still in flight land before the CTA leaves
                int never = 0;
                for (int i = max(0, armed - TP_STAGES); i < armed; ++i)
                    tg_mbar_wait(&ctl->full[i % TP_STAGES], (i / TP_STAGES) & 1, &never);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // float32 accumulate, bfloat16 a and b, both K-major, N = 256, M = 256 over the pair
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TG_BN >> 3) << 17) | ((uint32_t)((2 * TG_BM) >> 4) << 24);
            int it = 0, local = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += n_pairs, ++local) {
                const int buf = local & 1;
                if (!tg_mbar_wait(&ctl->acc_empty[buf], ((local >> 1) & 1) ^ 1, abort)) {
                    if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_MMA); }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + buf * TG_BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % TP_STAGES;
                    if (!tg_mbar_wait(&ctl->full[s], (it / TP_STAGES) & 1, abort)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_MMA); }
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = tg_smem(a_tiles + s * TG_A_BYTES), b_addr = tg_smem(b_tiles + s * TP_B_BYTES);
#pragma unroll
                    for (int k = 0; k < TG_BK / 16; ++k)
                        tp_mma(acc, tg_smem_desc(a_addr + k * 32), tg_smem_desc(b_addr + k * 32), idesc, (kt | k) != 0);
                    tp_commit_both(&ctl->empty[s]);
                }
                if (ok) tp_commit_both(&ctl->acc_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        int local = 0;
        for (int t = pair; t < total_tiles; t += n_pairs, ++local) {
            const int buf = local & 1;
            const bool ready = tg_mbar_wait(&ctl->acc_full[buf], (local >> 1) & 1, abort);
            if (!ready) {
                if (!*abort) { *abort = 1; atomicExch(error_flag, TG_ERR_EPILOGUE); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m0 = (t % m_tiles) * 2 * TG_BM + rank * TG_BM;
            const int row = m0 + q * 32 + lane;
            const uint32_t acc = tmem + ((uint32_t)(q * 32) << 16) + buf * TG_BN;
            if (SWIGLU) {
                const int col0 = (t / m_tiles) * TP_BN_HALF;
#pragma unroll 1
                for (int c = 0; c < TP_BN_HALF / 32; ++c) {
                    uint32_t g[32], u[32];
                    tg_ld32(acc + c * 32, g);
                    tg_ld32(acc + TP_BN_HALF + c * 32, u);
                    tg_store_swiglu(reinterpret_cast<bf16*>(out), g, u, row, col0 + c * 32, M, inter);
                }
            } else {
                const int n0 = (t / m_tiles) * TG_BN;
#pragma unroll 1
                for (int c = 0; c < TG_BN / 32; ++c) {
                    uint32_t r[32];
                    tg_ld32(acc + c * 32, r);
                    tg_store_row<OUT_F32>(out, r, row, n0 + c * 32, M, N);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tp_arrive_in_even_cta(&ctl->acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    tp_cluster_sync();                           // neither CTA frees tensor memory or leaves while the other still works
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TG_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*tg_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static tg_encode_fn tg_encoder() {
    static tg_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (tg_encode_fn)p;
    }
    return fn;
}

// A [rows, K] row-major bfloat16 matrix as a 2-D tensor map with boxes of 64 x box_rows and the 128-byte swizzle.
static int tg_make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    tg_encode_fn enc = tg_encoder();
    GI_REQUIRE(enc != nullptr, "gi_gemm_tcgen05_bf16: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TG_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GI_REQUIRE(r == CUDA_SUCCESS, "gi_gemm_tcgen05_bf16: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

#include <stdlib.h>
#include <string.h>
// GARLIC_B200_GEMM_PAIRS=0 keeps every product on the single-CTA kernel.
static bool gi_tcgen05_pairs_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("GARLIC_B200_GEMM_PAIRS");
        on = (v && strcmp(v, "0") == 0) ? 0 : 1;
    }
    return on == 1;
}

// error_flag: an int on the device that the kernel sets when one of its bounded waits runs out (0 = fine).
extern "C" int gi_gemm_tcgen05_bf16(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K,
                                    int* error_flag, void* stream) {
    GI_REQUIRE(M > 0 && N > 0 && K > 0, "gi_gemm_tcgen05_bf16: sizes must be positive");
    GI_REQUIRE(K % 8 == 0, "gi_gemm_tcgen05_bf16: inner size %d is no multiple of 8 (rows must be a multiple of 16 bytes for TMA)", K);
    GI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)out % 16 == 0),
               "gi_gemm_tcgen05_bf16: operands must start on 16 bytes");
    GI_REQUIRE(out_dtype == GI_DTYPE_BF16 || out_dtype == GI_DTYPE_F32, "gi_gemm_tcgen05_bf16: output dtype %d", out_dtype);
    GI_REQUIRE(error_flag != nullptr, "gi_gemm_tcgen05_bf16: an error flag on the device is required");
    int n_sm = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    }
    const int f32 = out_dtype == GI_DTYPE_F32;
    CUtensorMap map_x, map_w;
    if (int rc = tg_make_map(&map_x, x, M, K, TG_BM)) return rc;
    if (M > TG_BM && n_sm >= 2 && gi_tcgen05_pairs_enabled()) {
        // more than one tile of rows: pairs of CTAs on 256 x 256 tiles
        const long long tiles = (long long)((M + 2 * TG_BM - 1) / (2 * TG_BM)) * ((N + TG_BN - 1) / TG_BN);
        GI_REQUIRE(tiles < 1073741823LL, "gi_gemm_tcgen05_bf16: too many tiles");
        if (int rc = tg_make_map(&map_w, W, N, K, TP_BN_HALF)) return rc;
        const size_t smem = (size_t)TP_STAGES * (TG_A_BYTES + TP_B_BYTES) + sizeof(TpControl) + 1024;
        static bool attr_done[2] = {false, false};
        if (!attr_done[f32]) {
            cudaError_t e = f32 ? cudaFuncSetAttribute((const void*)gemm_tcgen05_pair_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                : cudaFuncSetAttribute((const void*)gemm_tcgen05_pair_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) { gi_set_error("gi_gemm_tcgen05_bf16: shared memory: %s", cudaGetErrorString(e)); return (int)e; }
            attr_done[f32] = true;
        }
        const long long pairs = tiles < n_sm / 2 ? tiles : n_sm / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
        cfg.blockDim = dim3(TG_THREADS, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = gi_pdl_enabled() ? 2 : 1;
        cudaError_t e = f32 ? cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<1, 0>, map_x, map_w, out, M, N, K, error_flag)
                            : cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<0, 0>, map_x, map_w, out, M, N, K, error_flag);
        if (e != cudaSuccess) { gi_set_error("gi_gemm_tcgen05_bf16: launch: %s", cudaGetErrorString(e)); return (int)e; }
        return gi_check_launch("gi_gemm_tcgen05_bf16");
    }
    const long long tiles = (long long)((M + TG_BM - 1) / TG_BM) * ((N + TG_BN - 1) / TG_BN);
    GI_REQUIRE(tiles < 2147483647LL, "gi_gemm_tcgen05_bf16: too many tiles");
    if (int rc = tg_make_map(&map_w, W, N, K, TG_BN)) return rc;
    const size_t smem = (size_t)TG_STAGES * (TG_A_BYTES + TG_B_BYTES) + sizeof(TgControl) + 1024;
    static bool attr_done[2] = {false, false};
    if (!attr_done[f32]) {
        cudaError_t e = f32 ? cudaFuncSetAttribute((const void*)gemm_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute((const void*)gemm_tcgen05_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { gi_set_error("gi_gemm_tcgen05_bf16: shared memory: %s", cudaGetErrorString(e)); return (int)e; }
        attr_done[f32] = true;
    }
    dim3 grid((unsigned)(tiles < n_sm ? tiles : n_sm));      // one CTA per SM, each walks its share of the tiles
    if (f32) gi_launch(gemm_tcgen05_kernel<1>, grid, dim3(TG_THREADS), smem, (cudaStream_t)stream, map_x, map_w, out, M, N, K, error_flag);
    else gi_launch(gemm_tcgen05_kernel<0>, grid, dim3(TG_THREADS), smem, (cudaStream_t)stream, map_x, map_w, out, M, N, K, error_flag);
    return gi_check_launch("gi_gemm_tcgen05_bf16");
}

// out[M, I] = silu(x . Wg^T) * (x . Wu^T) for W = [Wg; Wu] of 2 I rows: the gate/up product of a SwiGLU
// feed-forward with the activation in its epilogue, on pairs of CTAs.  bfloat16 in and out.
extern "C" int gi_gemm_tcgen05_swiglu_bf16(const void* x, const void* W, void* out, int M, int two_inter, int K,
                                           int* error_flag, void* stream) {
    GI_REQUIRE(M > 0 && two_inter > 0 && K > 0, "gi_gemm_tcgen05_swiglu_bf16: sizes must be positive");
    GI_REQUIRE(two_inter % 2 == 0, "gi_gemm_tcgen05_swiglu_bf16: W has %d rows, which cannot be a gate and an up half", two_inter);
    GI_REQUIRE(K % 8 == 0, "gi_gemm_tcgen05_swiglu_bf16: inner size %d is no multiple of 8 (rows must be a multiple of 16 bytes for TMA)", K);
    GI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)out % 16 == 0),
               "gi_gemm_tcgen05_swiglu_bf16: operands must start on 16 bytes");
    GI_REQUIRE(error_flag != nullptr, "gi_gemm_tcgen05_swiglu_bf16: an error flag on the device is required");
    int n_sm = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    }
    GI_REQUIRE(n_sm >= 2, "gi_gemm_tcgen05_swiglu_bf16: needs two SMs");
    const int inter = two_inter / 2;
    const long long tiles = (long long)((M + 2 * TG_BM - 1) / (2 * TG_BM)) * ((inter + TP_BN_HALF - 1) / TP_BN_HALF);
    GI_REQUIRE(tiles < 1073741823LL, "gi_gemm_tcgen05_swiglu_bf16: too many tiles");
    CUtensorMap map_x, map_w;
    if (int rc = tg_make_map(&map_x, x, M, K, TG_BM)) return rc;
    if (int rc = tg_make_map(&map_w, W, two_inter, K, TP_BN_HALF)) return rc;
    const size_t smem = (size_t)TP_STAGES * (TG_A_BYTES + TP_B_BYTES) + sizeof(TpControl) + 1024;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute((const void*)gemm_tcgen05_pair_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { gi_set_error("gi_gemm_tcgen05_swiglu_bf16: shared memory: %s", cudaGetErrorString(e)); return (int)e; }
        attr_done = true;
    }
    const long long pairs = tiles < n_sm / 2 ? tiles : n_sm / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(TG_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gi_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<0, 1>, map_x, map_w, out, M, two_inter, K, error_flag);
    if (e != cudaSuccess) { gi_set_error("gi_gemm_tcgen05_swiglu_bf16: launch: %s", cudaGetErrorString(e)); return (int)e; }
    return gi_check_launch("gi_gemm_tcgen05_swiglu_bf16");
}
