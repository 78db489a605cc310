// bfloat16 product for decode batches on the fifth-generation tensor cores, with the weight matrix
// cut evenly over the SMs: out[M,N] = x[M,K] . W[N,K]^T for 1 <= M <= 64.
//
// A decode step is bound by reading W once, so what matters is that every SM streams the same share
// of W without a pause.  The work is the list of (128 rows of W) x (64 of K) blocks, tile after tile;
// CTA c of G (one per SM) takes the blocks [c U / G, (c + 1) U / G) of the U blocks in that order, whatever
// the shape is.  Its range is at most the tail of one tile, some whole tiles, and the head of one tile:
//   warp 0, one lane:  TMA.  Block after block, 128 x 64 of W (16 KB) and the BN x 64 of x that go with
//                      it (BN = 16, 32 or 64 rows, the batch rounded up; rows beyond M zero-filled) into a
//                      ring of shared-memory stages (nine or ten; four to six when every CTA takes one whole
//                      tile, see the entry point).
//   warp 1, one lane:  MMA.  The operands are swapped: the 128 rows of W are the 128-row operand of
//                      tcgen05.mma, the batch is the BN-wide one; a tile's part accumulates in one of two
//                      accumulators of BN columns in tensor memory.
//   warps 2..5:        epilogue.  A whole tile is stored; the tail of a tile (its head belongs to the CTA
//                      before) goes as float32 to this CTA's slot of a work space, followed by a flag;
//                      the head of a tile (the CTA's last part) waits for the flags of the CTAs after it that
//                      hold the rest, adds their parts in CTA order and stores.  Those CTAs write their part
//                      first of all, so the wait at the very end is short, and the sum has one order.
// A CTA waits only for CTAs with larger numbers, and only for what they do first, before any wait of
// their own: there is no cycle.  All G CTAs are resident at once (G <= number of SMs, one CTA fits an SM).
// Every wait is bounded all the same: when one runs out a code goes to *error_flag, the roles leave their
// loops, copies in flight are waited for, tensor memory is freed and the kernel returns.
//
// Upstream calls a library product whatever M is (src/src-cuda/mat-ops/gemm/gemm.cu:22-41).
#include "common.cuh"

#include <cuda.h>

#define SKT_ROWS 128                    // rows of W per tile
#define SKT_BK 64
#define SKT_MAX_BN 64                   // the widest batch (padded) a launch takes; narrower ones use 16 or 32
#define SKT_MAX_STAGES 10               // the cut-evenly mode, one CTA per SM: 10 stages of 18 or 20 KB, 9 of 24 KB
#define SKT_THREADS 192
#define SKT_W_BYTES (SKT_ROWS * SKT_BK * 2)
#define SKT_SPIN_LIMIT (1 << 22)
#define SKT_MAX_CTAS 256
#define SKT_SLOT_FLOATS (SKT_MAX_BN * SKT_ROWS)      // a CTA's slot of the work space, whatever the batch
// stages of the ring: as many as fit one CTA per SM, or two CTAs per SM (the mode of one whole tile per CTA)
constexpr int skt_stages(int bn, bool whole_tiles) {
    return whole_tiles ? (bn == 16 ? 6 : bn == 32 ? 5 : 4) : (bn == 64 ? 9 : 10);
}

#define SKT_ERR_PRODUCER 31
#define SKT_ERR_MMA 32
#define SKT_ERR_EPILOGUE 33
#define SKT_ERR_PARTIAL 34

struct SktControl {
    unsigned long long full[SKT_MAX_STAGES];
    unsigned long long empty[SKT_MAX_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned int tmem_base;
    int abort;
};

__device__ __forceinline__ uint32_t skt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void skt_mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(skt_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void skt_mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(skt_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool skt_mbar_try(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(skt_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool skt_mbar_wait(void* bar, uint32_t parity, volatile int* abort) {
    for (int i = 0; i < SKT_SPIN_LIMIT; ++i) {
        if (skt_mbar_try(bar, parity)) return true;
        if ((i & 255) == 255 && *abort) return false;
    }
    return false;
}
__device__ __forceinline__ void skt_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(skt_smem(dst)), "l"(map), "r"(skt_smem(bar)), "r"(x), "r"(y) : "memory");
}
// K-major tile with rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1,024 bytes apart
__device__ __forceinline__ uint64_t skt_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void skt_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void skt_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(skt_smem(bar)) : "memory");
}
__device__ __forceinline__ void skt_ld16(uint32_t taddr, float (&r)[16]) {
    uint32_t u[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
                   "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
}
// The four epilogue warps among themselves: a barrier that also tells whether any of the 128 threads has
// `pred`, so that they all leave a loop together when a wait of one of them ran out.
__device__ __forceinline__ bool skt_epilogue_any(bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
                 "bar.red.or.pred p, 1, 128, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(r) : "r"((uint32_t)pred) : "memory");
    return r != 0;
}

// The part of the work a CTA does next: blocks [ka, kb) of tile `tile`.
struct SktSegment { int tile, ka, kb; };
__device__ __forceinline__ SktSegment skt_segment(long long u, long long u1, int kb_per_tile) {
    SktSegment s;
    s.tile = (int)(u / kb_per_tile);
    s.ka = (int)(u - (long long)s.tile * kb_per_tile);
    const long long left = u1 - u;
    s.kb = (int)(s.ka + left < kb_per_tile ? s.ka + left : kb_per_tile);
    return s;
}

template <int OUT_F32, int SKT_STAGES, int BN>
__global__ void __launch_bounds__(SKT_THREADS, 1)
gemm_streamk_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                            void* __restrict__ out, float* __restrict__ partials, int* __restrict__ flags,
                            int M, int N, int K, int* __restrict__ error_flag, int unanswered_limit) {
    constexpr int SKT_X_BYTES = BN * SKT_BK * 2;
    constexpr int SKT_TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;       // two accumulators of BN columns
    gi_pdl_launch_dependents();
    extern __shared__ unsigned char skt_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)skt_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* w_tiles = smem;
    unsigned char* x_tiles = smem + SKT_STAGES * SKT_W_BYTES;
    SktControl* ctl = reinterpret_cast<SktControl*>(x_tiles + SKT_STAGES * SKT_X_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_per_tile = (K + SKT_BK - 1) / SKT_BK;
    const int n_tiles = (N + SKT_ROWS - 1) / SKT_ROWS;
    const long long units = (long long)n_tiles * kb_per_tile;
    const int G = gridDim.x, c = blockIdx.x;
    const long long u0 = units * c / G, u1 = units * (c + 1) / G;
    volatile int* abort = &ctl->abort;

    // The start is kept short: the lane that issues the copies sets up the barriers itself and goes straight to
    // its copies (their descriptors asked for first of all); the other warps meet it at a named barrier only to
    // see the barriers initialised and, among themselves, the tensor memory allocated.
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < SKT_STAGES; ++s) { skt_mbar_init(&ctl->full[s], 1); skt_mbar_init(&ctl->empty[s], 1); }
        for (int b = 0; b < 2; ++b) { skt_mbar_init(&ctl->acc_full[b], 1); skt_mbar_init(&ctl->acc_empty[b], 4); }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    uint32_t tmem = 0;
    if (warp == 0) {
        __syncwarp();
        asm volatile("bar.arrive 2, 192;" ::: "memory");             // the barriers are set up; does not wait
    } else {
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(skt_smem(&ctl->tmem_base)), "r"(SKT_TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync 2, 192;" ::: "memory");
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem = ctl->tmem_base;
    }

    if (warp == 0) {
        if (lane == 0) {
            // W is nobody's output: its first blocks are asked for before the wait for the kernel that makes x,
            // into stages whose x part follows after the wait
            int it = 0, armed = 0;
            bool ok = true, waited = false;
            int pending_x[SKT_STAGES];           // k block of the x part still to be asked for, per stage (-1: none)
            int n_pending = 0;
            for (long long u = u0; u < u1 && ok;) {
                const SktSegment sg = skt_segment(u, u1, kb_per_tile);
                for (int kt = sg.ka; kt < sg.kb; ++kt, ++it) {
                    const int s = it % SKT_STAGES;
                    if (it >= SKT_STAGES && !waited) {           // the ring is full of W: now x is needed
                        gi_pdl_wait();
                        waited = true;
                        for (int p = 0; p < n_pending; ++p)
                            skt_tma_load_2d(x_tiles + p * SKT_X_BYTES, &map_x, pending_x[p] * SKT_BK, 0, &ctl->full[p]);
                        n_pending = 0;
                    }
                    if (!skt_mbar_wait(&ctl->empty[s], ((it / SKT_STAGES) & 1) ^ 1, abort)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, SKT_ERR_PRODUCER); }
                        ok = false;
                        break;
                    }
                    skt_mbar_expect_tx(&ctl->full[s], SKT_W_BYTES + SKT_X_BYTES);
                    skt_tma_load_2d(w_tiles + s * SKT_W_BYTES, &map_w, kt * SKT_BK, sg.tile * SKT_ROWS, &ctl->full[s]);
                    if (waited) skt_tma_load_2d(x_tiles + s * SKT_X_BYTES, &map_x, kt * SKT_BK, 0, &ctl->full[s]);
                    else pending_x[n_pending++] = kt;            // stage s == n_pending - 1 while it < SKT_STAGES
                    armed = it + 1;
                }
                u += sg.kb - sg.ka;
            }
            if (!waited) {
                gi_pdl_wait();
                for (int p = 0; p < n_pending; ++p)
                    skt_tma_load_2d(x_tiles + p * SKT_X_BYTES, &map_x, pending_x[p] * SKT_BK, 0, &ctl->full[p]);
            }
            if (*abort) {                        // let the copies still in flight land before the CTA leaves
                int never = 0;
                for (int i = max(0, armed - SKT_STAGES); i < armed; ++i)
                    skt_mbar_wait(&ctl->full[i % SKT_STAGES], (i / SKT_STAGES) & 1, &never);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // float32 accumulate, bfloat16 operands, both K-major, N = BN (the batch), M = 128 (rows of W)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(SKT_ROWS >> 4) << 24);
            int it = 0, local = 0;
            bool ok = true;
            for (long long u = u0; u < u1 && ok; ++local) {
                const SktSegment sg = skt_segment(u, u1, kb_per_tile);
                const int buf = local & 1;
                if (!skt_mbar_wait(&ctl->acc_empty[buf], ((local >> 1) & 1) ^ 1, abort)) {
                    if (!*abort) { *abort = 1; atomicExch(error_flag, SKT_ERR_MMA); }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + buf * BN;
                for (int kt = sg.ka; kt < sg.kb; ++kt, ++it) {
                    const int s = it % SKT_STAGES;
                    if (!skt_mbar_wait(&ctl->full[s], (it / SKT_STAGES) & 1, abort)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, SKT_ERR_MMA); }
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t w_addr = skt_smem(w_tiles + s * SKT_W_BYTES), x_addr = skt_smem(x_tiles + s * SKT_X_BYTES);
#pragma unroll
                    for (int k = 0; k < SKT_BK / 16; ++k)
                        skt_mma(acc, skt_desc(w_addr + k * 32), skt_desc(x_addr + k * 32), idesc, (kt != sg.ka) | (k != 0));
                    skt_commit(&ctl->empty[s]);
                }
                if (ok) skt_commit(&ctl->acc_full[buf]);
                u += sg.kb - sg.ka;
            }
        }
    } else {
        gi_pdl_wait();                                   // this warp writes: after everything before it in the stream
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        int local = 0;
        bool ok = true;
        for (long long u = u0; u < u1 && ok; ++local) {
            const SktSegment sg = skt_segment(u, u1, kb_per_tile);
            const int buf = local & 1;
            if (skt_epilogue_any(!skt_mbar_wait(&ctl->acc_full[buf], (local >> 1) & 1, abort))) {
                if (!*abort) { *abort = 1; atomicExch(error_flag, SKT_ERR_EPILOGUE); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float v[BN];
#pragma unroll
            for (int part = 0; part < BN / 16; ++part) {
                float piece[16];
                skt_ld16(tmem + ((uint32_t)(q * 32) << 16) + buf * BN + part * 16, piece);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[part * 16 + i] = piece[i];
            }
            // the accumulator is in registers: the MMA lane may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(skt_smem(&ctl->acc_empty[buf])) : "memory");

            if (sg.ka > 0) {
                // the tail of a tile whose head another CTA holds: float32 to this CTA's slot, then the flag
                float* slot = partials + (size_t)c * SKT_SLOT_FLOATS;
#pragma unroll
                for (int m = 0; m < BN; ++m) slot[m * SKT_ROWS + row_in_tile] = v[m];
                __threadfence();
                skt_epilogue_any(false);
                // (unanswered_limit > 0 is the test of the wait below: the flag is held back, so the wait must run out)
                if (threadIdx.x == 64 && unanswered_limit == 0)
                    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flags + c), "r"(1) : "memory");
            } else {
                if (sg.kb < kb_per_tile) {
                    // the head of a tile: the CTAs after this one hold the rest, each as the first thing it did
                    long long covered = (long long)sg.tile * kb_per_tile + sg.kb;
                    const long long tile_end = (long long)(sg.tile + 1) * kb_per_tile;
                    // which CTAs: c + 1 .. c + n_after; all their flags are waited for at once (one round trip, not n)
                    int n_after = 0;
                    for (long long cov = covered; cov < tile_end; ++n_after) {
                        const long long e2 = units * (c + 1 + n_after + 1) / G;
                        cov = e2 < tile_end ? e2 : tile_end;
                    }
                    int missing = 0;
                    const int spin_limit = unanswered_limit > 0 ? unanswered_limit : SKT_SPIN_LIMIT;
                    for (int j = (int)(threadIdx.x - 64); j < n_after; j += 128) {
                        int seen = 0;
                        for (int i = 0; i < spin_limit && !seen; ++i) {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flags + c + 1 + j) : "memory");
                            if (!seen && (i & 255) == 255 && *abort) break;
                        }
                        missing |= !seen;
                    }
                    if (skt_epilogue_any(missing != 0)) {
                        if (!*abort) { *abort = 1; atomicExch(error_flag, SKT_ERR_PARTIAL); }
                        ok = false;
                    } else {
                        __threadfence();                                 // the flags were seen by other threads of the CTA
                        for (int j = 0; j < n_after; ++j) {              // added in CTA order: one order of summation
                            const float* slot = partials + (size_t)(c + 1 + j) * SKT_SLOT_FLOATS;
#pragma unroll
                            for (int m = 0; m < BN; ++m) v[m] += __ldcg(slot + m * SKT_ROWS + row_in_tile);
                        }
                        skt_epilogue_any(false);                         // all four warps have read the slots
                        for (int j = (int)(threadIdx.x - 64); j < n_after; j += 128) flags[c + 1 + j] = 0;   // for the next launch
                    }
                }
                if (ok) {
                    const int row = sg.tile * SKT_ROWS + row_in_tile;
                    if (row < N) {
                        if (OUT_F32) {
                            float* o = reinterpret_cast<float*>(out);
#pragma unroll
                            for (int m = 0; m < BN; ++m)
                                if (m < M) o[(size_t)m * N + row] = v[m];
                        } else {
                            bf16* o = reinterpret_cast<bf16*>(out);
#pragma unroll
                            for (int m = 0; m < BN; ++m)
                                if (m < M) o[(size_t)m * N + row] = __float2bfloat16_rn(v[m]);
                        }
                    }
                }
            }
            u += sg.kb - sg.ka;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(SKT_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*skt_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static skt_encode_fn skt_encoder() {
    static skt_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (skt_encode_fn)p;
    }
    return fn;
}

static int skt_make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    skt_encode_fn enc = skt_encoder();
    GI_REQUIRE(enc != nullptr, "gi_gemm_streamk_bf16: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {SKT_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GI_REQUIRE(r == CUDA_SUCCESS, "gi_gemm_streamk_bf16: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

#include <stdlib.h>
#include <string.h>
// GARLIC_B200_STREAMK_WHOLE_TILES=0 keeps every shape in the cut-evenly mode.
static bool gi_streamk_whole_tiles_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("GARLIC_B200_STREAMK_WHOLE_TILES");
        on = (v && strcmp(v, "0") == 0) ? 0 : 1;
    }
    return on == 1;
}

// Floats of work space and ints of flags the entry point below wants (for any shape): one slot and one flag
// per CTA.  The flags must be zero before the first call; every call that ends without an error leaves them
// zero.  After a call that recorded an error (a wait that ran out) the flags are undefined: CTAs that had
// announced their partial sums were never answered.  Zero them before the next call.
extern "C" long long gi_gemm_streamk_workspace_floats(void) { return (long long)SKT_MAX_CTAS * SKT_SLOT_FLOATS; }
extern "C" int gi_gemm_streamk_flags(void) { return SKT_MAX_CTAS; }

// For the test of the bounded wait: with a limit above zero the CTAs that hold the tail of a cut tile write their
// partial sums but hold back the flag that announces them, and the CTA that holds the tile's head waits at most
// `limit` polls for it.  The wait runs out, the CTA records code 34 in *error_flag, skips its tile and returns;
// nothing else of the kernel changes, no copy or product is in flight for the waiting warps, and the flags stay
// zero.  0 (the default) is the product as it is used.
static int g_skt_unanswered_limit = 0;
extern "C" void gi_gemm_streamk_test_unanswered_flags(int limit) { g_skt_unanswered_limit = limit > 0 ? limit : 0; }

template <int OUT_F32, bool WHOLE, int BN>
static int skt_launch(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, float* partials, int* flags, int M, int N,
                      int K, long long g, int* error_flag, cudaStream_t stream) {
    constexpr int stages = skt_stages(BN, WHOLE);
    const size_t smem = (size_t)stages * (SKT_W_BYTES + BN * SKT_BK * 2) + sizeof(SktControl) + 1024;
    if (int rc = gi_reserve_smem((const void*)gemm_streamk_tcgen05_kernel<OUT_F32, stages, BN>, smem, "gi_gemm_streamk_bf16")) return rc;
    gi_launch(gemm_streamk_tcgen05_kernel<OUT_F32, stages, BN>, dim3((unsigned)g), dim3(SKT_THREADS), smem, stream, map_w, map_x,
              out, partials, flags, M, N, K, error_flag, g_skt_unanswered_limit);
    return gi_check_launch("gi_gemm_streamk_bf16");
}

extern "C" int gi_gemm_streamk_bf16(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K,
                                    float* partials, int* flags, int* error_flag, void* stream) {
    GI_REQUIRE(M >= 1 && M <= SKT_MAX_BN, "gi_gemm_streamk_bf16: %d rows; this kernel takes 1 to %d", M, SKT_MAX_BN);
    GI_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gi_gemm_streamk_bf16: inner size %d must be a positive multiple of 8", K);
    GI_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0), "gi_gemm_streamk_bf16: operands must start on 16 bytes");
    GI_REQUIRE(out_dtype == GI_DTYPE_BF16 || out_dtype == GI_DTYPE_F32, "gi_gemm_streamk_bf16: output dtype %d", out_dtype);
    GI_REQUIRE(partials != nullptr && flags != nullptr && error_flag != nullptr,
               "gi_gemm_streamk_bf16: work space, flags and an error flag on the device are required");
    int n_sm = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    }
    const long long n_tiles = (N + SKT_ROWS - 1) / SKT_ROWS;
    const long long units = n_tiles * ((K + SKT_BK - 1) / SKT_BK);
    // Two ways to share W out.  When there are between one and two tiles of 128 rows per SM, every CTA takes one
    // whole tile, two CTAs to an SM: nothing is cut, nothing merged, and with enough bytes in flight per CTA the
    // memory system serves all of them at the same pace however they are spread over the SMs.  Otherwise the
    // blocks are cut evenly over one CTA per SM and the cut tiles merged (the kernel's main text).
    const bool whole_tiles = n_tiles >= n_sm && n_tiles <= 2LL * n_sm && gi_streamk_whole_tiles_enabled();
    long long g = whole_tiles ? n_tiles : (units < n_sm ? units : n_sm);   // cut mode: all CTAs resident at once, they wait for one another
    if (!whole_tiles && g > SKT_MAX_CTAS) g = SKT_MAX_CTAS;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap map_w, map_x;
    if (int rc = skt_make_map(&map_w, W, N, K, SKT_ROWS)) return rc;
    if (int rc = skt_make_map(&map_x, x, M, K, bn)) return rc;
    const int f32 = out_dtype == GI_DTYPE_F32;
    cudaStream_t s = (cudaStream_t)stream;
#define SKT_GO(F, WH, B) return skt_launch<F, WH, B>(map_w, map_x, out, partials, flags, M, N, K, g, error_flag, s)
#define SKT_PICK_BN(F, WH) { if (bn == 16) SKT_GO(F, WH, 16); if (bn == 32) SKT_GO(F, WH, 32); SKT_GO(F, WH, 64); }
    if (f32) { if (whole_tiles) SKT_PICK_BN(1, true) else SKT_PICK_BN(1, false) }
    else { if (whole_tiles) SKT_PICK_BN(0, true) else SKT_PICK_BN(0, false) }
#undef SKT_PICK_BN
#undef SKT_GO
}
