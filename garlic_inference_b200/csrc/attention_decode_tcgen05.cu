// bfloat16 attention for decode steps on the fifth-generation tensor cores: head_dim 128, cache pages that
// are a multiple of 64 tokens, at most 16 query heads per key/value head.
//
// One CTA takes one sequence, one key/value head and one slice of that sequence's keys.  The query heads
// that share the key/value head are the rows of one 128-row operand (rows beyond the group hold whatever
// shared memory held: every output row depends on its own row alone, and those rows are never stored):
//   warp 0, one lane:  TMA.  The group's queries once (16 rows); per 64 keys the keys and the values of the
//                      tile's page (2-D tensor maps over the pools, 128-byte swizzle) into rings of three
//                      stages each.  No thread computes an address per element: that was what bound the
//                      mma.sync kernel of this library at small batches.
//   warp 1, one lane:  MMA.  S = Q K^T (128 x 64) into one of two buffers in tensor memory, a tile ahead of
//                      the softmax; O += P V (128 x 128) with P read from tensor memory; O stays there.
//   warp 4:            softmax.  Lane r owns query head r of the group (lanes beyond the group idle along):
//                      reads its row of S, masks the edges (position, window), writes exp2(s - ref) over S as
//                      bfloat16; ref follows the running maximum lazily as in the prompt kernel.
// At the end lane r writes its unnormalised row of O with (ref, sum) to the slice's place in the scratch
// buffers; the combine kernel of the mma.sync path merges the slices.  With one slice there is nothing to
// merge: the row goes to the output, normalised, and no second kernel runs.
//
// Every wait on an mbarrier is bounded; when one runs out a code goes to *error_flag, all roles leave their
// loops, copies in flight are waited for, tensor memory is freed and the kernel returns.
//
// Upstream hands attention to a library (src/src-cuda/attention/fattn.cu:74-140).
#include "common.cuh"

#include <cuda.h>
#include <math.h>

#define FD_BM 128
#define FD_BN 64
#define FD_D 128
#define FD_QROWS 16                            // rows of the query tile that are loaded (the group is at most this)
#define FD_STAGES 3
#define FD_THREADS 160                         // warps 2 and 3 only pad: tensor memory lanes 0..31 belong to a warp with index % 4 == 0
#define FD_Q_HALF (FD_QROWS * 128)            // one 16 x 64 swizzled half of the queries.  The 128-row operand reads on
                                               // past it into the key and value stages: rows nobody looks at
#define FD_Q_BYTES (2 * FD_Q_HALF)
#define FD_KV_BYTES (FD_BN * FD_D * 2)
#define FD_TMEM_COLS 256
#define FD_COL_S 0
#define FD_COL_O 128
#define FD_LAZY 8.f
#define FD_SPIN_LIMIT (1 << 22)

#define FD_ERR_PRODUCER 41
#define FD_ERR_MMA 42
#define FD_ERR_SOFTMAX 43
#define FD_ERR_PAGE 44

struct FdControl {
    unsigned long long q_full;
    unsigned long long k_full[FD_STAGES], k_empty[FD_STAGES];
    unsigned long long v_full[FD_STAGES], v_empty[FD_STAGES];
    unsigned long long s_full[2];
    unsigned long long p_ready[2];
    unsigned long long o_done;
    unsigned int tmem_base;
    int abort;
};

__device__ __forceinline__ uint32_t fd_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fd_mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fd_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fd_mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fd_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fd_mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fd_smem(bar)) : "memory");
}
__device__ __forceinline__ bool fd_mbar_try(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(fd_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool fd_mbar_wait(void* bar, uint32_t parity, volatile int* abort) {
    for (int i = 0; i < FD_SPIN_LIMIT; ++i) {
        if (fd_mbar_try(bar, parity)) return true;
        if ((i & 255) == 255 && *abort) return false;
    }
    return false;
}
__device__ __forceinline__ void fd_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(fd_smem(dst)), "l"(map), "r"(fd_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t fd_desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t fd_desc_mnmajor(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void fd_mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fd_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fd_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(fd_smem(bar)) : "memory");
}
__device__ __forceinline__ float fd_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void fd_ld32(uint32_t taddr, float (&r)[32]) {
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
__device__ __forceinline__ void fd_st32(uint32_t taddr, const uint32_t (&u)[32]) {
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

// grid (slices, key/value heads, sequences)
__global__ void __launch_bounds__(FD_THREADS, 2)
decode_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                      const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, float* __restrict__ part_o,
                      float* __restrict__ part_ml, bf16* __restrict__ out, int n_q, int n_kv, int page_size, int max_pages, int n_pool_pages,
                      int window, float scale_log2, int n_splits, int* __restrict__ error_flag) {
    gi_pdl_launch_dependents();
    extern __shared__ unsigned char fd_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)fd_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = smem;                                        // [2 halves][16 rows][128 bytes]
    unsigned char* k_tiles = smem + FD_Q_BYTES;
    unsigned char* v_tiles = k_tiles + FD_STAGES * FD_KV_BYTES;
    FdControl* ctl = reinterpret_cast<FdControl*>(v_tiles + FD_STAGES * FD_KV_BYTES);

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int grp = n_q / n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // positions and slots are set before the step's first kernel: read before the wait below
    const int slot = tok_slot[b], pos = tok_pos[b];
    const int kv_len = pos + 1;
    const int lo = window > 0 ? max(0, kv_len - window) : 0;
    const int kt_lo = lo / FD_BN;
    const int nt_all = slot < 0 ? 0 : (kv_len - kt_lo * FD_BN + FD_BN - 1) / FD_BN;
    const int per = (nt_all + n_splits - 1) / n_splits;
    const int t0 = split * per, n_tiles = max(0, min(nt_all, t0 + per) - t0);
    const size_t row_base = (size_t)b * n_q + (size_t)kvh * grp;         // the group's first row of q and of the partials
    volatile int* abort = &ctl->abort;

    if (n_tiles == 0) {                                                  // nothing for this slice: an empty partial
        gi_pdl_wait();
        if (n_splits == 1) {                                             // no slices: the output itself, zeros
            for (int i = threadIdx.x; i < grp * FD_D; i += FD_THREADS) out[row_base * FD_D + i] = __float2bfloat16_rn(0.f);
        } else if (threadIdx.x < grp) {
            float* ml = part_ml + ((row_base + threadIdx.x) * n_splits + split) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        return;
    }
    if (threadIdx.x == 0) {
        fd_mbar_init(&ctl->q_full, 1);
        for (int s = 0; s < FD_STAGES; ++s) {
            fd_mbar_init(&ctl->k_full[s], 1); fd_mbar_init(&ctl->k_empty[s], 1);
            fd_mbar_init(&ctl->v_full[s], 1); fd_mbar_init(&ctl->v_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) { fd_mbar_init(&ctl->s_full[i], 1); fd_mbar_init(&ctl->p_ready[i], 1); }
        fd_mbar_init(&ctl->o_done, 1);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(fd_smem(&ctl->tmem_base)), "r"(FD_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctl->tmem_base;

    // the lane that issues the copies
    const int* bt_row = block_table + (size_t)slot * max_pages;
    auto tile_row = [&](int it) {
        const int key0 = (kt_lo + t0 + it) * FD_BN;
        const int lp = key0 / page_size;
        int page = lp < max_pages ? bt_row[lp] : -1;
        if (page < 0 || page >= n_pool_pages) { atomicExch(error_flag, FD_ERR_PAGE); page = 0; }
        return (page * n_kv + kvh) * page_size + (key0 - lp * page_size);
    };
    int armed_k = 0, armed_v = 0;
    auto load = [&](int it, bool keys) -> bool {
        const int s = it % FD_STAGES;
        unsigned long long* empty = keys ? &ctl->k_empty[s] : &ctl->v_empty[s];
        unsigned long long* full = keys ? &ctl->k_full[s] : &ctl->v_full[s];
        if (!fd_mbar_wait(empty, ((it / FD_STAGES) & 1) ^ 1, abort)) return false;
        const int row = tile_row(it);
        unsigned char* dst = (keys ? k_tiles : v_tiles) + s * FD_KV_BYTES;
        fd_mbar_expect_tx(full, FD_KV_BYTES);
        fd_tma_load_2d(dst, keys ? &map_k : &map_v, 0, row, full);
        fd_tma_load_2d(dst + FD_KV_BYTES / 2, keys ? &map_k : &map_v, 64, row, full);
        (keys ? armed_k : armed_v) = it + 1;
        return true;
    };
    int next_k = 0, next_v = 0;
    bool copies_ok = true;
    if (warp == 0 && lane == 0) {
        // Tiles that end before this step's token hold keys and values of earlier steps only, and the block
        // table is set before the step's first kernel: the first ring of them goes out before the wait (their
        // stages are free, so nothing here waits for a product that needs q).
        auto settled = [&](int it) { return (kt_lo + t0 + it + 1) * FD_BN <= pos; };
        while (copies_ok && next_k < min(n_tiles, FD_STAGES) && settled(next_k)) copies_ok = load(next_k++, true);
        while (copies_ok && next_v < min(n_tiles, FD_STAGES) && settled(next_v)) copies_ok = load(next_v++, false);
    }
    gi_pdl_wait();                               // q and the newest key come from the kernel before this one

    if (warp == 0) {
        if (lane == 0) {
            fd_mbar_expect_tx(&ctl->q_full, FD_Q_BYTES);
            fd_tma_load_2d(q_tile, &map_q, 0, (int)row_base, &ctl->q_full);
            fd_tma_load_2d(q_tile + FD_Q_HALF, &map_q, 64, (int)row_base, &ctl->q_full);
            bool ok = copies_ok;
            for (int it = 0; it < n_tiles && ok; ++it) {         // keys one tile ahead of the values
                while (ok && next_k < n_tiles && next_k <= it + 1) ok = load(next_k++, true);
                while (ok && next_v <= it) ok = load(next_v++, false);
            }
            if (!ok && !*abort) { *abort = 1; atomicExch(error_flag, FD_ERR_PRODUCER); }
            if (*abort) {                                // no copy may be in flight when the CTA leaves
                int never = 0;
                fd_mbar_wait(&ctl->q_full, 0, &never);
                for (int i = max(0, armed_k - FD_STAGES); i < armed_k; ++i)
                    fd_mbar_wait(&ctl->k_full[i % FD_STAGES], (i / FD_STAGES) & 1, &never);
                for (int i = max(0, armed_v - FD_STAGES); i < armed_v; ++i)
                    fd_mbar_wait(&ctl->v_full[i % FD_STAGES], (i / FD_STAGES) & 1, &never);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FD_BN >> 3) << 17) | ((uint32_t)(FD_BM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(FD_D >> 3) << 17) | ((uint32_t)(FD_BM >> 4) << 24);
            const uint32_t q_addr = fd_smem(q_tile);
            bool ok = fd_mbar_wait(&ctl->q_full, 0, abort);
            auto issue_s = [&](int it) -> bool {
                const int s = it % FD_STAGES;
                if (!fd_mbar_wait(&ctl->k_full[s], (it / FD_STAGES) & 1, abort)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_addr = fd_smem(k_tiles + s * FD_KV_BYTES);
#pragma unroll
                for (int k = 0; k < FD_D / 16; ++k) {
                    const uint32_t qa = q_addr + (k >> 2) * FD_Q_HALF + (k & 3) * 32;
                    const uint32_t ka = k_addr + (k >> 2) * (FD_KV_BYTES / 2) + (k & 3) * 32;
                    fd_mma_ss(tmem + FD_COL_S + (it & 1) * FD_BN, fd_desc_kmajor(qa), fd_desc_kmajor(ka), idesc_s, k != 0);
                }
                fd_commit(&ctl->s_full[it & 1]);
                fd_commit(&ctl->k_empty[s]);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int it = 0; it < n_tiles && ok; ++it) {
                const int s = it % FD_STAGES;
                if (it + 1 < n_tiles && !(ok = issue_s(it + 1))) break;
                if (!fd_mbar_wait(&ctl->p_ready[it & 1], (it >> 1) & 1, abort) ||
                    !fd_mbar_wait(&ctl->v_full[s], (it / FD_STAGES) & 1, abort)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_addr = fd_smem(v_tiles + s * FD_KV_BYTES);
#pragma unroll
                for (int k = 0; k < FD_BN / 16; ++k)
                    fd_mma_ts(tmem + FD_COL_O, tmem + FD_COL_S + (it & 1) * FD_BN + k * 8,
                              fd_desc_mnmajor(v_addr + k * 2048, FD_KV_BYTES / 2), idesc_o, (it | k) != 0);
                fd_commit(&ctl->o_done);
                fd_commit(&ctl->v_empty[s]);
            }
            if (!ok && !*abort) { *abort = 1; atomicExch(error_flag, FD_ERR_MMA); }
        }
    } else if (warp == 4) {
        const int r = lane;                              // query head r of the group = lane r of tensor memory
        const bool mine = r < grp;
        const uint32_t lane_base = tmem;                 // lanes 0..31
        float ref = -INFINITY, l = 0.f;
        bool ok = true;
        auto wait_warp = [&](void* bar, uint32_t parity) {
            const bool w = fd_mbar_wait(bar, parity, abort);
            return __all_sync(0xffffffffu, w);
        };
        for (int it = 0; it < n_tiles; ++it) {
            const int bsel = it & 1;
            if (!wait_warp(&ctl->s_full[bsel], (it >> 1) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int key0 = (kt_lo + t0 + it) * FD_BN;
            float s[FD_BN];
            {
                float a[32], c[32];
                fd_ld32(lane_base + FD_COL_S + bsel * FD_BN, a);
                fd_ld32(lane_base + FD_COL_S + bsel * FD_BN + 32, c);
#pragma unroll
                for (int j = 0; j < 32; ++j) { s[j] = a[j]; s[32 + j] = c[j]; }
            }
            if (key0 + FD_BN - 1 > pos || key0 < lo) {   // the tile with the newest key, or the window's edge
#pragma unroll
                for (int j = 0; j < FD_BN; ++j) {
                    const int key = key0 + j;
                    s[j] = (key <= pos && key >= lo) ? s[j] : -INFINITY;
                }
            }
            float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int j = 4; j < FD_BN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            if (!mine || !(mx == mx)) mx = -INFINITY;    // rows beyond the group hold anything at all: keep them quiet
            if (it == 0) {
                ref = mx;
            } else {
                if (!wait_warp(&ctl->o_done, (it - 1) & 1)) { ok = false; break; }
                const bool grow = mx > ref + FD_LAZY;
                if (__any_sync(0xffffffffu, grow)) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const float corr = grow ? exp2f(ref - mx) : 1.f;
#pragma unroll
                    for (int c4 = 0; c4 < FD_D / 32; ++c4) {
                        float o[32];
                        uint32_t u[32];
                        fd_ld32(lane_base + FD_COL_O + c4 * 32, o);
#pragma unroll
                        for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(o[j] * corr);
                        fd_st32(lane_base + FD_COL_O + c4 * 32, u);
                    }
                    l *= corr;
                    if (grow) ref = mx;
                }
            }
            const float neg_use = ref == -INFINITY ? 0.f : -ref;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int j = 0; j < FD_BN; j += 2) {
                const float p0 = fd_ex2(fmaf(s[j], scale_log2, neg_use)), p1 = fd_ex2(fmaf(s[j + 1], scale_log2, neg_use));
                sum4[(j >> 1) & 3] += p0 + p1;
                __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                pk[j >> 1] = *reinterpret_cast<uint32_t*>(&v);
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            fd_st32(lane_base + FD_COL_S + bsel * FD_BN, pk);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) fd_mbar_arrive(&ctl->p_ready[bsel]);
        }
        if (ok && !wait_warp(&ctl->o_done, (n_tiles - 1) & 1)) ok = false;
        if (!ok && !*abort) { *abort = 1; atomicExch(error_flag, FD_ERR_SOFTMAX); }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* dst = part_o + ((row_base + r) * n_splits + split) * FD_D;
            bf16* whole = out + (row_base + r) * FD_D;                   // without slices the output is written here
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
            for (int c4 = 0; c4 < FD_D / 32; ++c4) {
                float o[32];
                fd_ld32(lane_base + FD_COL_O + c4 * 32, o);              // by the whole warp
                if (mine && n_splits > 1) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(dst + c4 * 32 + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                } else if (mine) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv);
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
                        v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                        v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                        *reinterpret_cast<uint4*>(whole + c4 * 32 + i) = v;
                    }
                }
            }
            if (mine && n_splits > 1) {
                float* ml = part_ml + ((row_base + r) * n_splits + split) * 2;
                ml[0] = l > 0.f ? ref : -INFINITY;       // a slice in which this row saw no key counts as empty
                ml[1] = l;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(FD_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*fd_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static fd_encode_fn fd_encoder() {
    static fd_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (fd_encode_fn)p;
    }
    return fn;
}

static int fd_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    fd_encode_fn enc = fd_encoder();
    GI_REQUIRE(enc != nullptr, "gi_attention_decode_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GI_REQUIRE(r == CUDA_SUCCESS, "gi_attention_decode_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

// The slices' partial results: part_o float32 [n_seqs * n_q * n_splits * 128] (unnormalised), part_ml float32
// [n_seqs * n_q * n_splits * 2] (reference in powers of two, sum); gi_attention_decode_combine merges them.
// With n_splits == 1 the kernel writes out [n_seqs, n_q * 128] bfloat16 itself and the scratch is not touched.
// Takes head_dim 128, page sizes that are a multiple of 64 and groups of at most 16 query heads.
extern "C" int gi_attention_decode_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                           const int* tok_pos, const int* tok_slot, float* part_o, float* part_ml,
                                           void* out, int n_seqs, int n_q, int n_kv, int d, int page_size, int max_pages,
                                           int n_pool_pages, int window, float scale, int n_splits, int* error_flag,
                                           void* stream) {
    GI_REQUIRE(d == FD_D, "gi_attention_decode_tcgen05: head_dim %d; this kernel takes 128", d);
    GI_REQUIRE(page_size > 0 && page_size % FD_BN == 0, "gi_attention_decode_tcgen05: page size %d is no multiple of 64", page_size);
    GI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0 && n_q / n_kv <= FD_QROWS,
               "gi_attention_decode_tcgen05: %d query heads on %d key/value heads; at most 16 per key/value head", n_q, n_kv);
    GI_REQUIRE(n_seqs >= 0 && n_seqs <= 65535 && n_kv <= 65535 && n_splits >= 1 && max_pages > 0 && window >= 0,
               "gi_attention_decode_tcgen05: sizes");
    GI_REQUIRE(error_flag != nullptr, "gi_attention_decode_tcgen05: an error flag on the device is required");
    GI_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
               ((uintptr_t)part_o % 16 == 0) && ((uintptr_t)out % 16 == 0), "gi_attention_decode_tcgen05: operands must start on 16 bytes");
    GI_REQUIRE(out != nullptr && (n_splits == 1 || (part_o != nullptr && part_ml != nullptr)), "gi_attention_decode_tcgen05: buffers");
    if (n_seqs == 0) return 0;
    CUtensorMap map_q, map_k, map_v;
    if (int rc = fd_make_map(&map_q, q, (long long)n_seqs * n_q, d, FD_QROWS)) return rc;
    const long long pool_rows = (long long)n_pool_pages * n_kv * page_size;
    if (int rc = fd_make_map(&map_k, k_pool, pool_rows, d, FD_BN)) return rc;
    if (int rc = fd_make_map(&map_v, v_pool, pool_rows, d, FD_BN)) return rc;
    const size_t smem = (size_t)FD_Q_BYTES + 2 * FD_STAGES * FD_KV_BYTES + sizeof(FdControl) + 1024;
    if (int rc = gi_reserve_smem((const void*)decode_tcgen05_kernel, smem, "gi_attention_decode_tcgen05")) return rc;
    gi_launch(decode_tcgen05_kernel, dim3(n_splits, n_kv, n_seqs), dim3(FD_THREADS), smem, (cudaStream_t)stream, map_q, map_k,
              map_v, block_table, tok_pos, tok_slot, part_o, part_ml, (bf16*)out, n_q, n_kv, page_size, max_pages, n_pool_pages, window,
              scale * 1.4426950408889634f, n_splits, error_flag);
    return gi_check_launch("gi_attention_decode_tcgen05");
}
