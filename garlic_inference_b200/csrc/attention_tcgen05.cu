// bfloat16 flash attention for prompts on the fifth-generation tensor cores: head_dim 128, cache pages
// that are a multiple of 64 tokens.
//
// A work item is 128 consecutive queries of one sequence and one query head; its CTA walks the keys of the
// sequence's cache 64 at a time.  The grid is persistent, two CTAs to an SM (one's softmax runs under the
// other's products), and every CTA takes several items, a long one with a short one (see the kernel):
//   warp 0, one lane:  TMA.  The item's query tile; per key tile the 64 keys and 64 values of the tile's
//                      page (the pools are 2-D tensor maps [all rows, head_dim]; a tile never crosses a
//                      page), into rings of two stages each for keys and for values, 128-byte swizzled.
//   warp 1, one lane:  MMA.  S = Q K^T (128 x 64, float32) into one of two buffers in tensor memory, one
//                      tile ahead of the softmax; when the softmax warps have written the probabilities
//                      over the scores as bfloat16, O += P V (128 x 128) with P read from tensor memory
//                      and V from shared memory.  O stays in tensor memory for all tiles of an item.
//   warps 2..5:        softmax.  Thread i owns query row i: it reads its row of S from tensor memory,
//                      scales and masks it (causal, window), and writes exp2(s - ref).  `ref` follows
//                      the row's running maximum lazily: only when the maximum has grown by more than
//                      FT_LAZY (in powers of two) are ref, the running sum and the row of O in tensor
//                      memory rescaled; until then probabilities up to 2^FT_LAZY are simply accumulated,
//                      which float32 holds exactly as well.  No shuffles, no shared memory, and O is
//                      read once, at the end of the item.  The barriers' phases run on from item to item.
//
// Scores, softmax and the output sum are float32; probabilities are rounded to bfloat16 for the second
// product.  Every wait on an mbarrier is bounded: when one runs out, a code goes to *error_flag, all
// roles leave their loops, copies in flight are waited for, tensor memory is freed, and the kernel
// returns (the output is then unspecified).
//
// Upstream hands attention to a library (src/src-cuda/attention/fattn.cu:74-140).
#include "common.cuh"

#include <cuda.h>
#include <math.h>

#define FT_BM 128
#define FT_BN 64
#define FT_D 128
#define FT_STAGES 2
#define FT_THREADS 192
#define FT_Q_BYTES (FT_BM * FT_D * 2)          // two 128 x 64 swizzled halves
#define FT_KV_BYTES (FT_BN * FT_D * 2)         // two 64 x 64 swizzled halves, keys; the same for values
#define FT_TMEM_COLS 256
#define FT_COL_S 0                             // S: two buffers of 64 float32 columns; P (64 bfloat16 = 32 columns)
                                               // overwrites the start of its S
#define FT_COL_O 128                           // O: 128 float32 columns
#define FT_LAZY 8.f                            // growth of a row's maximum (log2) that triggers a rescale
#define FT_SPIN_LIMIT (1 << 22)

#define FT_ERR_PRODUCER 21
#define FT_ERR_MMA 22
#define FT_ERR_SOFTMAX 23
#define FT_ERR_PAGE 24

struct FtControl {
    unsigned long long q_full, q_empty;
    unsigned long long o_free;
    unsigned long long k_full[FT_STAGES], k_empty[FT_STAGES];
    unsigned long long v_full[FT_STAGES], v_empty[FT_STAGES];
    unsigned long long s_full[2];
    unsigned long long p_ready[2];
    unsigned long long o_done;
    unsigned int tmem_base;
    int abort;
};

__device__ __forceinline__ uint32_t ft_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ft_mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ft_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void ft_mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ft_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ft_mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ft_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ft_mbar_try(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(ft_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool ft_mbar_wait(void* bar, uint32_t parity, volatile int* abort) {
    for (int i = 0; i < FT_SPIN_LIMIT; ++i) {
        if (ft_mbar_try(bar, parity)) return true;
        if ((i & 255) == 255 && *abort) return false;
    }
    return false;
}
__device__ __forceinline__ void ft_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(ft_smem(dst)), "l"(map), "r"(ft_smem(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand (rows of 128 bytes = 64 elements along the contraction, 128-byte swizzle, groups of 8
// rows 1,024 bytes apart): used for Q and K in S = Q K^T.
__device__ __forceinline__ uint64_t ft_desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand: V as the second factor of P V.  Rows are keys (the contraction), 128 bytes = 64 output
// columns wide, 128-byte swizzle; groups of 8 keys are 1,024 bytes apart (stride offset), the second block
// of 64 output columns lies `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t ft_desc_mnmajor(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void ft_mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ft_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ft_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ft_smem(bar)) : "memory");
}
__device__ __forceinline__ float ft_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void ft_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t u[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
                   "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
                   "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
                   "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void ft_st32(uint32_t taddr, const uint32_t (&u)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
                   "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
                   "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]),
                   "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// tiles[t] = {slot, first row of q, rows in the tile (<= 128), position of the first row}
//
// The grid is persistent: at most two CTAs per SM walk the list of (tile, head) items, CTA c of G taking the
// items c, 2G - 1 - c, 2G + c, 4G - 1 - c, ... : with the tiles sorted by the keys they walk, longest first
// (the engine sorts them), every CTA gets a long item with a short one and they finish together.
struct FtItem { int slot, row0, n_rows, pos0, h, kvh, kt_lo, n_tiles; };

__global__ void __launch_bounds__(FT_THREADS, 2)
flash_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                             const int4* __restrict__ tiles, int n_q_tiles, bf16* __restrict__ out, int n_q, int n_kv,
                             int page_size, int max_pages, int n_pool_pages, int window, float scale_log2,
                             int* __restrict__ error_flag) {
    gi_pdl_start();
    extern __shared__ unsigned char ft_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)ft_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = smem;                                        // [2 halves][128 rows][128 bytes]
    unsigned char* k_tiles = smem + FT_Q_BYTES;                          // [stages][2 halves][64 rows][128 bytes]
    unsigned char* v_tiles = k_tiles + FT_STAGES * FT_KV_BYTES;
    FtControl* ctl = reinterpret_cast<FtControl*>(v_tiles + FT_STAGES * FT_KV_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long n_items = (long long)n_q_tiles * n_q;
    const int G = gridDim.x, c = blockIdx.x;
    // item of round `round` of this CTA: 1 = there is one, 0 = none in this round, -1 = no more rounds
    auto item_at = [&](int round, FtItem& it) -> int {
        if ((long long)round * G >= n_items) return -1;
        const long long t = (round & 1) ? (long long)(round + 1) * G - 1 - c : (long long)round * G + c;
        if (t >= n_items) return 0;
        const int4 ti = tiles[t / n_q];
        it.slot = ti.x, it.row0 = ti.y, it.n_rows = ti.z, it.pos0 = ti.w;
        it.h = (int)(t % n_q), it.kvh = it.h / (n_q / n_kv);
        const int hi = it.pos0 + it.n_rows - 1;
        const int lo = window > 0 ? max(0, it.pos0 - window + 1) : 0;
        it.kt_lo = lo / FT_BN;
        it.n_tiles = (it.slot < 0 || it.n_rows <= 0) ? 0 : hi / FT_BN - it.kt_lo + 1;
        return it.n_tiles > 0 ? 1 : 0;
    };
    volatile int* abort = &ctl->abort;

    if (threadIdx.x == 0) {
        ft_mbar_init(&ctl->q_full, 1);
        ft_mbar_init(&ctl->q_empty, 1);
        ft_mbar_init(&ctl->o_free, 4);
        for (int s = 0; s < FT_STAGES; ++s) {
            ft_mbar_init(&ctl->k_full[s], 1); ft_mbar_init(&ctl->k_empty[s], 1);
            ft_mbar_init(&ctl->v_full[s], 1); ft_mbar_init(&ctl->v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) { ft_mbar_init(&ctl->s_full[b], 1); ft_mbar_init(&ctl->p_ready[b], 4); }
        ft_mbar_init(&ctl->o_done, 1);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(ft_smem(&ctl->tmem_base)), "r"(FT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            // Keys and values have rings of their own: the keys of a tile are free again as soon as its
            // scores are computed (a tile ahead of the softmax), the values only after P V.  Keys of tile
            // it + 1 go out before the values of tile it, in the order in which the stages come free.
            int qn = 0, g0 = 0;                          // items and key tiles done so far: the barriers' phases go on
            int armed_q = 0, armed_k = 0, armed_v = 0;
            bool ok = true;
            FtItem im;
            for (int round = 0; ok; ++round) {
                const int have = item_at(round, im);
                if (have < 0) break;
                if (have == 0) continue;
                // the query tile may be overwritten when the last scores of the item before are computed
                if (!ft_mbar_wait(&ctl->q_empty, (qn & 1) ^ 1, abort)) { ok = false; break; }
                ft_mbar_expect_tx(&ctl->q_full, FT_Q_BYTES);
                ft_tma_load_2d(q_tile, &map_q, im.h * FT_D, im.row0, &ctl->q_full);
                ft_tma_load_2d(q_tile + FT_Q_BYTES / 2, &map_q, im.h * FT_D + 64, im.row0, &ctl->q_full);
                armed_q = qn + 1;
                const int* bt_row = block_table + (size_t)im.slot * max_pages;
                auto tile_row = [&](int it) {
                    const int key0 = (im.kt_lo + it) * FT_BN;
                    const int lp = key0 / page_size;
                    int page = lp < max_pages ? bt_row[lp] : -1;
                    if (page < 0 || page >= n_pool_pages) { atomicExch(error_flag, FT_ERR_PAGE); page = 0; }
                    return (page * n_kv + im.kvh) * page_size + (key0 - lp * page_size);
                };
                auto load = [&](int it, bool keys) -> bool {
                    const int g = g0 + it, s = g % FT_STAGES;
                    unsigned long long* empty = keys ? &ctl->k_empty[s] : &ctl->v_empty[s];
                    unsigned long long* full = keys ? &ctl->k_full[s] : &ctl->v_full[s];
                    if (!ft_mbar_wait(empty, ((g / FT_STAGES) & 1) ^ 1, abort)) return false;
                    const int row = tile_row(it);
                    unsigned char* dst = (keys ? k_tiles : v_tiles) + s * FT_KV_BYTES;
                    ft_mbar_expect_tx(full, FT_KV_BYTES);
                    ft_tma_load_2d(dst, keys ? &map_k : &map_v, 0, row, full);
                    ft_tma_load_2d(dst + FT_KV_BYTES / 2, keys ? &map_k : &map_v, 64, row, full);
                    (keys ? armed_k : armed_v) = g + 1;
                    return true;
                };
                ok = load(0, true);
                for (int it = 0; it < im.n_tiles && ok; ++it) {
                    if (it + 1 < im.n_tiles) ok = load(it + 1, true);
                    if (ok) ok = load(it, false);
                }
                g0 += im.n_tiles;
                ++qn;
            }
            if (!ok && !*abort) { *abort = 1; atomicExch(error_flag, FT_ERR_PRODUCER); }
            if (*abort) {                                // no copy may be in flight when the CTA leaves
                int never = 0;
                if (armed_q > 0) ft_mbar_wait(&ctl->q_full, (armed_q - 1) & 1, &never);
                for (int i = max(0, armed_k - FT_STAGES); i < armed_k; ++i)
                    ft_mbar_wait(&ctl->k_full[i % FT_STAGES], (i / FT_STAGES) & 1, &never);
                for (int i = max(0, armed_v - FT_STAGES); i < armed_v; ++i)
                    ft_mbar_wait(&ctl->v_full[i % FT_STAGES], (i / FT_STAGES) & 1, &never);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // S = Q K^T: float32 accumulate, bfloat16 operands, both K-major, N = 64, M = 128
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FT_BN >> 3) << 17) | ((uint32_t)(FT_BM >> 4) << 24);
            // P V: the same with the second operand MN-major (bit 16), N = 128
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(FT_D >> 3) << 17) | ((uint32_t)(FT_BM >> 4) << 24);
            const uint32_t q_addr = ft_smem(q_tile);
            int qn = 0, g0 = 0;
            bool ok = true;
            FtItem im;
            for (int round = 0; ok; ++round) {
                const int have = item_at(round, im);
                if (have < 0) break;
                if (have == 0) continue;
                if (!ft_mbar_wait(&ctl->q_full, qn & 1, abort)) { ok = false; break; }
                auto issue_s = [&](int it) -> bool {
                    const int g = g0 + it, s = g % FT_STAGES;
                    if (!ft_mbar_wait(&ctl->k_full[s], (g / FT_STAGES) & 1, abort)) return false;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t k_addr = ft_smem(k_tiles + s * FT_KV_BYTES);
#pragma unroll
                    for (int k = 0; k < FT_D / 16; ++k) {
                        const uint32_t qa = q_addr + (k >> 2) * (FT_Q_BYTES / 2) + (k & 3) * 32;
                        const uint32_t ka = k_addr + (k >> 2) * (FT_KV_BYTES / 2) + (k & 3) * 32;
                        ft_mma_ss(tmem + FT_COL_S + (g & 1) * FT_BN, ft_desc_kmajor(qa), ft_desc_kmajor(ka), idesc_s, k != 0);
                    }
                    ft_commit(&ctl->s_full[g & 1]);
                    ft_commit(&ctl->k_empty[s]);
                    if (it + 1 == im.n_tiles) ft_commit(&ctl->q_empty);      // the item's last scores: the query tile is free
                    return true;
                };
                ok = issue_s(0);
                for (int it = 0; it < im.n_tiles && ok; ++it) {
                    const int g = g0 + it, s = g % FT_STAGES;
                    // The scores of the next tile, into the other buffer, while the softmax warps work on this
                    // one.  The products run in the order they are issued, so this one starts after P V of the
                    // tile before, which read its probabilities from that buffer.
                    if (it + 1 < im.n_tiles && !(ok = issue_s(it + 1))) break;
                    if (!ft_mbar_wait(&ctl->p_ready[g & 1], (g >> 1) & 1, abort) ||
                        !ft_mbar_wait(&ctl->v_full[s], (g / FT_STAGES) & 1, abort)) { ok = false; break; }
                    // the first P V of an item overwrites O: the softmax warps have read the item before out of it
                    if (it == 0 && !ft_mbar_wait(&ctl->o_free, (qn & 1) ^ 1, abort)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t v_addr = ft_smem(v_tiles + s * FT_KV_BYTES);
#pragma unroll
                    for (int k = 0; k < FT_BN / 16; ++k)     // 16 keys = two groups of 8 rows = 2,048 bytes further
                        ft_mma_ts(tmem + FT_COL_O, tmem + FT_COL_S + (g & 1) * FT_BN + k * 8,
                                  ft_desc_mnmajor(v_addr + k * 2048, FT_KV_BYTES / 2), idesc_o, (it | k) != 0);
                    ft_commit(&ctl->o_done);
                    ft_commit(&ctl->v_empty[s]);
                }
                g0 += im.n_tiles;
                ++qn;
            }
            if (!ok && !*abort) { *abort = 1; atomicExch(error_flag, FT_ERR_MMA); }
        }
    } else {
        const int q = warp & 3;
        const int r = q * 32 + lane;                     // this thread's query row = its lane of tensor memory
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        bool ok = true;
        // tensor memory is read and written by whole warps: a wait that gives up does so for the whole warp
        auto wait_warp = [&](void* bar, uint32_t parity) {
            const bool w = ft_mbar_wait(bar, parity, abort);
            return __all_sync(0xffffffffu, w);
        };
        int g0 = 0;
        FtItem im;
        for (int round = 0; ok; ++round) {
            const int have = item_at(round, im);
            if (have < 0) break;
            if (have == 0) continue;
            const int pos = im.pos0 + r;
            float ref = -INFINITY, l = 0.f;              // exponentials are taken against `ref`; l is the sum of them
            for (int it = 0; it < im.n_tiles; ++it) {
                const int g = g0 + it, b = g & 1;
                if (!wait_warp(&ctl->s_full[b], (g >> 1) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int key0 = (im.kt_lo + it) * FT_BN;
                float s[FT_BN];                          // raw scores: the scale is folded into the exponent below
                {
                    float a[32], c2[32];
                    ft_ld32(lane_base + FT_COL_S + b * FT_BN, a);
                    ft_ld32(lane_base + FT_COL_S + b * FT_BN + 32, c2);
#pragma unroll
                    for (int j = 0; j < 32; ++j) { s[j] = a[j]; s[32 + j] = c2[j]; }
                }
                // tiles that every row of the CTA sees whole need no mask
                if (key0 + FT_BN - 1 > im.pos0 || (window > 0 && key0 <= im.pos0 + FT_BM - 1 - window)) {
#pragma unroll
                    for (int j = 0; j < FT_BN; ++j) {
                        const int key = key0 + j;
                        const bool seen = key <= pos && (window <= 0 || key > pos - window);
                        s[j] = seen ? s[j] : -INFINITY;
                    }
                }
                float mx4[4] = {s[0], s[1], s[2], s[3]}; // four chains instead of one of 63 dependent steps
#pragma unroll
                for (int j = 4; j < FT_BN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // the scale is positive
                if (it == 0) {
                    ref = mx;                            // nothing accumulated yet: nothing to rescale
                } else {
                    // O must not change under the rescale: P V of the tile before has to be done (it has been
                    // for long, as a rule).  Waited for every tile, so that the barrier's phases are seen in order.
                    if (!wait_warp(&ctl->o_done, (g - 1) & 1)) { ok = false; break; }
                    const bool grow = mx > ref + FT_LAZY;    // also a row that sees its first key (ref = -inf)
                    if (__any_sync(0xffffffffu, grow)) { // tensor memory is read and written by whole warps
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const float corr = grow ? exp2f(ref - mx) : 1.f;
#pragma unroll
                        for (int c4 = 0; c4 < FT_D / 32; ++c4) {
                            float o[32];
                            uint32_t u[32];
                            ft_ld32(lane_base + FT_COL_O + c4 * 32, o);
#pragma unroll
                            for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(o[j] * corr);
                            ft_st32(lane_base + FT_COL_O + c4 * 32, u);
                        }
                        l *= corr;
                        if (grow) ref = mx;
                    }
                }
                const float neg_use = ref == -INFINITY ? 0.f : -ref; // a row that has seen no key yet stays all zero
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[32];
#pragma unroll
                for (int j = 0; j < FT_BN; j += 2) {
                    // one multiply-add and one ex2 per score; results below 2^-126 are flushed to zero
                    const float p0 = ft_ex2(fmaf(s[j], scale_log2, neg_use)), p1 = ft_ex2(fmaf(s[j + 1], scale_log2, neg_use));
                    sum4[(j >> 1) & 3] += p0 + p1;
                    __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                    pk[j >> 1] = *reinterpret_cast<uint32_t*>(&v);
                }
                l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                ft_st32(lane_base + FT_COL_S + b * FT_BN, pk);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) ft_mbar_arrive(&ctl->p_ready[b]);
            }
            if (ok && !wait_warp(&ctl->o_done, (g0 + im.n_tiles - 1) & 1)) ok = false;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + ((size_t)(im.row0 + r) * n_q + im.h) * FT_D;
#pragma unroll
            for (int c4 = 0; c4 < FT_D / 32; ++c4) {
                float o[32];
                ft_ld32(lane_base + FT_COL_O + c4 * 32, o);      // by whole warps, rows beyond the tile too
                if (r < im.n_rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv);
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
                        v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                        v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                        *reinterpret_cast<uint4*>(dst + c4 * 32 + i) = v;
                    }
                }
            }
            // O is in registers: the first P V of the next item may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) ft_mbar_arrive(&ctl->o_free);
            g0 += im.n_tiles;
        }
        if (!ok && !*abort) { *abort = 1; atomicExch(error_flag, FT_ERR_SOFTMAX); }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(FT_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*ft_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static ft_encode_fn ft_encoder() {
    static ft_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (ft_encode_fn)p;
    }
    return fn;
}

// [rows, cols] row-major bfloat16 as a 2-D map with boxes of 64 columns x box_rows rows, 128-byte swizzle
static int ft_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    ft_encode_fn enc = ft_encoder();
    GI_REQUIRE(enc != nullptr, "gi_attention_prefill_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GI_REQUIRE(r == CUDA_SUCCESS, "gi_attention_prefill_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

// tiles: int32 [n_tiles, 4] = {slot, first q row, rows (<= 128), position of the first row}.
// Takes head_dim 128 and page sizes that are a multiple of 64; everything else is refused.
extern "C" int gi_attention_prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                            const int* tiles, int n_tiles, void* out, int n_tokens, int n_q, int n_kv,
                                            int d, int page_size, int max_pages, int n_pool_pages, int window,
                                            float scale, int* error_flag, void* stream) {
    GI_REQUIRE(d == FT_D, "gi_attention_prefill_tcgen05: head_dim %d; this kernel takes 128", d);
    GI_REQUIRE(page_size > 0 && page_size % FT_BN == 0, "gi_attention_prefill_tcgen05: page size %d is no multiple of 64", page_size);
    GI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0 && n_q <= 65535, "gi_attention_prefill_tcgen05: %d query heads, %d key/value heads", n_q, n_kv);
    GI_REQUIRE(max_pages > 0 && window >= 0 && n_tiles >= 0 && n_tokens >= 0, "gi_attention_prefill_tcgen05: sizes");
    GI_REQUIRE(error_flag != nullptr, "gi_attention_prefill_tcgen05: an error flag on the device is required");
    GI_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
               ((uintptr_t)out % 16 == 0) && ((uintptr_t)tiles % 16 == 0), "gi_attention_prefill_tcgen05: operands must start on 16 bytes");
    if (n_tiles == 0 || n_tokens == 0) return 0;
    CUtensorMap map_q, map_k, map_v;
    if (int rc = ft_make_map(&map_q, q, n_tokens, (long long)n_q * d, FT_BM)) return rc;
    const long long pool_rows = (long long)n_pool_pages * n_kv * page_size;
    if (int rc = ft_make_map(&map_k, k_pool, pool_rows, d, FT_BN)) return rc;
    if (int rc = ft_make_map(&map_v, v_pool, pool_rows, d, FT_BN)) return rc;
    const size_t smem = (size_t)FT_Q_BYTES + 2 * FT_STAGES * FT_KV_BYTES + sizeof(FtControl) + 1024;
    if (int rc = gi_reserve_smem((const void*)flash_prefill_tcgen05_kernel, smem, "gi_attention_prefill_tcgen05")) return rc;
    int n_sm = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    }
    const long long items = (long long)n_tiles * n_q;
    const long long grid = items < 2LL * n_sm ? items : 2LL * n_sm;      // two CTAs fit an SM
    gi_launch(flash_prefill_tcgen05_kernel, dim3((unsigned)grid), dim3(FT_THREADS), smem, (cudaStream_t)stream, map_q, map_k,
              map_v, block_table, (const int4*)tiles, n_tiles, (bf16*)out, n_q, n_kv, page_size, max_pages, n_pool_pages,
              window, scale * 1.4426950408889634f, error_flag);
    return gi_check_launch("gi_attention_prefill_tcgen05");
}
