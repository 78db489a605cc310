// bfloat16 attention over the paged cache on the tensor cores: a flash-style
// kernel for steps that bring several tokens per sequence (prompts) and a
// split-KV kernel for decode steps, with its combine kernel.
//
// Both compute, per query,  o = softmax_j(q . k_j * scale) v_j  over the keys
// j <= pos of the query's own sequence (and j > pos - window when window > 0),
// query head h reading key/value head h / (n_q / n_kv); scores, softmax and
// the accumulation are float32, the probabilities are rounded to bfloat16 for
// the second product.  Upstream hands all of this to a library
// (src/src-cuda/attention/fattn.cu:74-140).
//
// Tiles: 64 keys at a time, read through the block table row by row (a tile
// may span pages of any size), staged in shared memory with cp.async in two
// stages, rows padded by 16 bytes so that ldmatrix is free of bank conflicts
// for every head size.  Products are mma.sync m16n8k16.
//   prefill: one CTA = 64 consecutive queries of one sequence and one query
//            head; 4 warps of 16 queries; every warp visits all keys.
//   decode:  one CTA = one sequence, one key/value head, one slice of the
//            keys; the rows of the product are the n_q / n_kv query heads of
//            the group (at most 16); the 4 warps take 16 keys each of every
//            tile, each streaming them through a queue of its own, and are
//            merged at the end.  Each slice writes a partial
//            (max, sum, unnormalised output) to scratch memory; the combine
//            kernel merges the slices.  The number of slices is a launch
//            parameter; which keys a slice covers follows from the sequence's
//            length on the device, so a recorded launch stays valid as the
//            sequence grows.
// Head sizes: multiples of 16 up to 128.
#include "common.cuh"
#include <math.h>

#define AT_THREADS 128
#define AT_BN 64            // keys per tile
#define AT_BM 64            // queries per prefill CTA
#define AT_DEC_DEPTH 2      // stages of a warp's queue in the decode kernel

// ------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;                     // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Element offset of row j of a sequence inside a pool (for key/value head kvh), or -1 when j is not below
// key_end or its page is not mapped.  No branch around the table read, so that a thread's reads for
// several rows are issued together instead of one after the other.
__device__ __forceinline__ long long kv_row_offset(const int* __restrict__ bt_row, int j, int key_end, int n_kv, int kvh,
                                                   int page_size, int max_pages, int n_pool_pages, int D) {
    const int lp = j / page_size;
    const bool in = j >= 0 && j < key_end && lp < max_pages;
    const int page = __ldg(bt_row + (in ? lp : 0));
    const bool ok = in && page >= 0 && page < n_pool_pages;
    return ok ? (((long long)page * n_kv + kvh) * page_size + (j - lp * page_size)) * D : -1;
}

// Stage one tile of 64 keys (rows key0 .. key0+63 of the sequence) of keys and values into shared memory.
// Rows at or beyond key_end, and rows whose page is not mapped, are zero-filled.
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* sK, bf16* sV, const bf16* __restrict__ k_pool,
                                             const bf16* __restrict__ v_pool, const int* __restrict__ bt_row,
                                             int key0, int key_end, int n_kv, int kvh, int page_size,
                                             int max_pages, int n_pool_pages) {
    constexpr int LD = D + 8, CH = D / 8, PASSES = AT_BN * CH / AT_THREADS;
    long long off[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; ++p)
        off[p] = kv_row_offset(bt_row, key0 + (threadIdx.x + p * AT_THREADS) / CH, key_end, n_kv, kvh, page_size,
                               max_pages, n_pool_pages, D);
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const int i = threadIdx.x + p * AT_THREADS;
        const int r = i / CH, c = i % CH;
        const bool valid = off[p] >= 0;
        const size_t o = valid ? (size_t)off[p] + c * 8 : 0;
        cp_async_16(sK + r * LD + c * 8, k_pool + o, valid);
        cp_async_16(sV + r * LD + c * 8, v_pool + o, valid);
    }
}

// A fragments (16 rows x D) of a row-major tile in shared memory, kept in registers.
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t (&a)[D / 16][4], const bf16* tile /* 16 rows, stride D+8 */) {
    constexpr int LD = D + 8;
    const int lane = threadIdx.x & 31, mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(a[kk], tile + ((mat & 1) * 8 + r) * LD + kk * 16 + (mat >> 1) * 8);
}

// S[16 x 8*NT] += Q[16 x D] . K[keys x D]^T for NT key n-tiles starting at row `krow0` of the staged keys.
template <int D, int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const uint32_t (&a)[D / 16][4], const bf16* sK, int krow0) {
    constexpr int LD = D + 8;
    const int lane = threadIdx.x & 31, mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, sK + (krow0 + np * 16 + (mat >> 1) * 8 + r) * LD + kk * 16 + (mat & 1) * 8);
            mma_16816(s[2 * np], a[kk], b[0], b[1]);
            mma_16816(s[2 * np + 1], a[kk], b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x 16*KS] . V[keys x D] for KS key k-steps starting at row `vrow0` of the staged values.
template <int D, int KS>
__device__ __forceinline__ void pv_product(float (&o)[D / 8][4], const uint32_t (&p)[KS][4], const bf16* sV, int vrow0) {
    constexpr int LD = D + 8;
    const int lane = threadIdx.x & 31, mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, sV + (vrow0 + ks * 16 + (mat & 1) * 8 + r) * LD + dp * 16 + (mat >> 1) * 8);
            mma_16816(o[2 * dp], p[ks], b[0], b[1]);
            mma_16816(o[2 * dp + 1], p[ks], b[2], b[3]);
        }
    }
}

// One online-softmax update of a warp's 16 rows over NT*8 scores (already scaled to the log2 domain and
// masked with -inf): rescales o, updates (m, l) and leaves bfloat16 probabilities in p.
template <int D, int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                               uint32_t (&p)[NT / 2][4]) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
    }
    float corr[2], use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        use[h] = m_new == -INFINITY ? 0.f : m_new;        // a row with no key yet: everything stays 0
        corr[h] = exp2f(m[h] - use[h]);
        m[h] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float p0 = exp2f(s[nt][0] - use[0]), p1 = exp2f(s[nt][1] - use[0]);
        const float p2 = exp2f(s[nt][2] - use[1]), p3 = exp2f(s[nt][3] - use[1]);
        sum[0] += p0 + p1;
        sum[1] += p2 + p3;
        p[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
        p[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l[0] = l[0] * corr[0] + sum[0];                        // per-thread partial sums; the quad is added up at the end
    l[1] = l[1] * corr[1] + sum[1];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }
}

// ------------------------------------------------------------------------------ prefill
// tiles[t] = {slot, first row of q, rows in the tile (<= 64), position of the first row}
template <int D>
__global__ void __launch_bounds__(AT_THREADS)
flash_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                     const int* __restrict__ block_table, const int4* __restrict__ tiles, bf16* __restrict__ out,
                     int n_q, int n_kv, int page_size, int max_pages, int n_pool_pages, int window, float scale_log2) {
    gi_pdl_start();
    constexpr int LD = D + 8;
    extern __shared__ __align__(16) unsigned char at_smem[];
    bf16* sQ = reinterpret_cast<bf16*>(at_smem);
    bf16* sK = sQ + AT_BM * LD;
    bf16* sV = sK + 2 * AT_BN * LD;

    const int4 ti = tiles[blockIdx.x];
    const int slot = ti.x, row0 = ti.y, n_rows = ti.z, pos0 = ti.w;
    const int h = blockIdx.y, kvh = h / (n_q / n_kv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (slot < 0 || n_rows <= 0) return;
    const int* bt_row = block_table + (size_t)slot * max_pages;

    const int hi = pos0 + n_rows - 1;                                   // last position of the tile
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;          // first key any row of the tile sees
    const int kt_lo = lo / AT_BN, n_tiles = hi / AT_BN - kt_lo + 1;

    {   // the queries of the tile, rows beyond n_rows zero-filled
        constexpr int CH = D / 8;
#pragma unroll
        for (int p = 0; p < AT_BM * CH / AT_THREADS; ++p) {
            const int i = threadIdx.x + p * AT_THREADS;
            const int r = i / CH, c = i % CH;
            const bool valid = r < n_rows;
            const bf16* src = q + ((size_t)(row0 + (valid ? r : 0)) * n_q + h) * D + c * 8;
            cp_async_16(sQ + r * LD + c * 8, src, valid);
        }
    }
    load_kv_tile<D>(sK, sV, k_pool, v_pool, bt_row, kt_lo * AT_BN, hi + 1, n_kv, kvh, page_size, max_pages, n_pool_pages);
    cp_async_commit();

    uint32_t a[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int p_row[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};      // positions of this thread's rows
    const int p_warp_max = pos0 + warp * 16 + 15;

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        if (it + 1 < n_tiles) {
            load_kv_tile<D>(sK + (st ^ 1) * AT_BN * LD, sV + (st ^ 1) * AT_BN * LD, k_pool, v_pool, bt_row,
                            (kt_lo + it + 1) * AT_BN, hi + 1, n_kv, kvh, page_size, max_pages, n_pool_pages);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) load_a_frags<D>(a, sQ + warp * 16 * LD);
        const int key0 = (kt_lo + it) * AT_BN;
        const bool warp_sees = key0 <= p_warp_max && (window <= 0 || key0 + AT_BN - 1 > pos0 + warp * 16 - window);
        if (warp_sees) {
            float s[AT_BN / 8][4];
            qk_product<D, AT_BN / 8>(s, a, sK + st * AT_BN * LD, 0);
#pragma unroll
            for (int nt = 0; nt < AT_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + 2 * t + (e & 1);
                    const int p = p_row[e >> 1];
                    const bool ok = j <= p && (window <= 0 || j > p - window);
                    s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
                }
            }
            uint32_t pf[AT_BN / 16][4];
            softmax_update<D, AT_BN / 8>(s, m, l, o, pf);
            pv_product<D, AT_BN / 16>(o, pf, sV + st * AT_BN * LD, 0);
        }
        __syncthreads();
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = warp * 16 + g + hh * 8;
        if (r >= n_rows) continue;
        const float inv = l[hh] > 0.f ? 1.f / l[hh] : 0.f;
        bf16* dst = out + ((size_t)(row0 + r) * n_q + h) * D;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt)
            *reinterpret_cast<uint32_t*>(dst + dt * 8 + 2 * t) = pack_bf16(o[dt][hh * 2] * inv, o[dt][hh * 2 + 1] * inv);
    }
}

// ------------------------------------------------------------------------------ decode (split-KV)
// part_o  [n_seqs, n_q, n_splits, D]  float32 unnormalised outputs
// part_ml [n_seqs, n_q, n_splits, 2]  float32 (max in the log2 domain, sum)
template <int D>
__global__ void __launch_bounds__(AT_THREADS)
decode_splitkv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                      const int* __restrict__ block_table, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_slot, float* __restrict__ part_o, float* __restrict__ part_ml,
                      int n_q, int n_kv, int page_size, int max_pages, int n_pool_pages, int window,
                      float scale_log2, int n_splits) {
    gi_pdl_launch_dependents();
    constexpr int LD = D + 8, CH = D / 8;
    constexpr int STAGE = 2 * 16 * LD;                           // elements of one warp's stage: 16 keys, 16 values
    extern __shared__ __align__(16) unsigned char at_smem[];
    bf16* sQ = reinterpret_cast<bf16*>(at_smem);                // 16 rows
    bf16* sKV = sQ + 16 * LD;                                    // [4 warps][AT_DEC_DEPTH][keys | values][16][LD]

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int grp = n_q / n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int slot = tok_slot[b], pos = tok_pos[b];
    const int kv_len = pos + 1;
    const int lo = window > 0 ? max(0, kv_len - window) : 0;
    const int lo_al = lo / AT_BN * AT_BN;
    const int nt_all = slot < 0 ? 0 : (kv_len - lo_al + AT_BN - 1) / AT_BN;
    const int per = (nt_all + n_splits - 1) / n_splits;
    const int t0 = split * per, t1 = min(nt_all, t0 + per);
    float* my_ml = part_ml + (((size_t)b * n_q + kvh * grp) * n_splits + split) * 2;
    gi_pdl_wait();                               // positions and slots above are set before the step's first kernel
    if (t0 >= t1) {                                              // nothing for this slice: an empty partial
        if (threadIdx.x < grp) {
            my_ml[(size_t)threadIdx.x * n_splits * 2] = -INFINITY;
            my_ml[(size_t)threadIdx.x * n_splits * 2 + 1] = 0.f;
        }
        return;
    }
    const int* bt_row = block_table + (size_t)slot * max_pages;

    for (int i = threadIdx.x; i < 16 * (D / 8); i += AT_THREADS) {
        const int r = i / (D / 8), c = i % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < grp) v = *reinterpret_cast<const uint4*>(q + ((size_t)b * n_q + kvh * grp + r) * D + c * 8);
        *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
    }

    // Each warp streams its own 16 keys (and values) of every 64-key tile through a queue of its own,
    // AT_DEC_DEPTH stages deep: the warps never wait for each other while the cache is read.
    bf16* ring = sKV + warp * AT_DEC_DEPTH * STAGE;
    const int n_it = t1 - t0;
    auto issue = [&](int i) {
        if (i < n_it) {
            bf16* st = ring + (i % AT_DEC_DEPTH) * STAGE;
            const int key0 = lo_al + (t0 + i) * AT_BN + warp * 16;
            long long off[16 * CH / 32];
#pragma unroll
            for (int p = 0; p < 16 * CH / 32; ++p)
                off[p] = kv_row_offset(bt_row, key0 + (lane + p * 32) / CH, kv_len, n_kv, kvh, page_size, max_pages,
                                       n_pool_pages, D);
#pragma unroll
            for (int p = 0; p < 16 * CH / 32; ++p) {
                const int idx = lane + p * 32;
                const int r = idx / CH, c = idx % CH;
                const bool valid = off[p] >= 0;
                const size_t o = valid ? (size_t)off[p] + c * 8 : 0;
                cp_async_16(st + r * LD + c * 8, k_pool + o, valid);
                cp_async_16(st + 16 * LD + r * LD + c * 8, v_pool + o, valid);
            }
        }
        cp_async_commit();                                       // an empty group when nothing is left: the count stays uniform
    };
#pragma unroll
    for (int i = 0; i < AT_DEC_DEPTH - 1; ++i) issue(i);

    uint32_t a[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    __syncthreads();                                             // the queries are in shared memory
    load_a_frags<D>(a, sQ);

    for (int i = 0; i < n_it; ++i) {
        issue(i + AT_DEC_DEPTH - 1);
        cp_async_wait<AT_DEC_DEPTH - 1>();
        __syncwarp();                                            // every lane's copies of stage i have landed
        const bf16* st = ring + (i % AT_DEC_DEPTH) * STAGE;
        const int key0 = lo_al + (t0 + i) * AT_BN + warp * 16;  // this warp's 16 keys of the tile
        if (key0 <= pos && key0 + 15 >= lo) {
            float s[2][4];
            qk_product<D, 2>(s, a, st, 0);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + 2 * t + (e & 1);
                    s[nt][e] = (j <= pos && j >= lo) ? s[nt][e] * scale_log2 : -INFINITY;
                }
            uint32_t pf[1][4];
            softmax_update<D, 2>(s, m, l, o, pf);
            pv_product<D, 1>(o, pf, st + 16 * LD, 0);
        }
        __syncwarp();                                            // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
    __syncthreads();                                             // all warps are done with their queues
    // merge the four warps (each saw other keys) through shared memory, reusing the tile buffers
    float* mO = reinterpret_cast<float*>(sKV);                   // [4][16][D]
    float* mM = mO + 4 * 16 * D;                                 // [4][16]
    float* mL = mM + 4 * 16;                                     // [4][16]
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = g + hh * 8;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            mO[(warp * 16 + r) * D + dt * 8 + 2 * t] = o[dt][hh * 2];
            mO[(warp * 16 + r) * D + dt * 8 + 2 * t + 1] = o[dt][hh * 2 + 1];
        }
        if (t == 0) { mM[warp * 16 + r] = m[hh]; mL[warp * 16 + r] = l[hh]; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < grp * D; i += AT_THREADS) {
        const int r = i / D, dim = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mM[w * 16 + r]);
        float acc = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(mM[w * 16 + r] - M);       // 0 for a warp that saw no key
                acc += f * mO[(w * 16 + r) * D + dim];
                L += f * mL[w * 16 + r];
            }
        }
        part_o[(((size_t)b * n_q + kvh * grp + r) * n_splits + split) * D + dim] = acc;
        if (dim == 0) {
            my_ml[(size_t)r * n_splits * 2] = M;
            my_ml[(size_t)r * n_splits * 2 + 1] = L;
        }
    }
}

template <int D>
__global__ void __launch_bounds__(128)
decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                      int n_splits) {
    gi_pdl_start();
    const size_t row = blockIdx.x;                               // sequence * n_q + head
    const float* ml = part_ml + row * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
    for (int dim = threadIdx.x; dim < D; dim += blockDim.x) {
        float acc = 0.f, L = 0.f;
        if (M != -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float ms = ml[2 * s];
                if (ms == -INFINITY) continue;                   // an empty slice: its output was never written
                const float f = exp2f(ms - M);
                acc += f * part_o[(row * n_splits + s) * D + dim];
                L += f * ml[2 * s + 1];
            }
        }
        out[row * D + dim] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
}

// ------------------------------------------------------------------------------ entry points
#define AT_DISPATCH_D(d, CALL)                                                                                 \
    switch (d) {                                                                                               \
        case 16: { CALL(16); break; }                                                                          \
        case 32: { CALL(32); break; }                                                                          \
        case 48: { CALL(48); break; }                                                                          \
        case 64: { CALL(64); break; }                                                                          \
        case 80: { CALL(80); break; }                                                                          \
        case 96: { CALL(96); break; }                                                                          \
        case 112: { CALL(112); break; }                                                                        \
        case 128: { CALL(128); break; }                                                                        \
        default: GI_REQUIRE(false, "attention (tensor cores): head_dim %d must be a multiple of 16 up to 128", d); \
    }

static int check_common(const char* who, int n_q, int n_kv, int d, int page_size, int max_pages, int window) {
    GI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "%s: %d query heads are no multiple of %d key/value heads", who, n_q, n_kv);
    GI_REQUIRE(d > 0 && d % 16 == 0 && d <= 128, "%s: head_dim %d must be a multiple of 16 up to 128", who, d);
    GI_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "%s: page size, table width and window", who);
    return 0;
}

// Raises a kernel's dynamic shared memory limit, once per kernel and device.
template <int D, int WHICH>
static int set_smem(const void* kernel, size_t bytes) { return gi_reserve_smem(kernel, bytes, "attention"); }

// tiles: int32 [n_tiles, 4] = {slot, first q row, rows (<= 64), position of the first row}
extern "C" int gi_attention_prefill_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                         const int* tiles, int n_tiles, void* out, int n_q, int n_kv, int d,
                                         int page_size, int max_pages, int n_pool_pages, int window, float scale,
                                         void* stream) {
    if (int rc = check_common("gi_attention_prefill_bf16", n_q, n_kv, d, page_size, max_pages, window)) return rc;
    GI_REQUIRE(n_tiles >= 0 && n_q <= 65535, "gi_attention_prefill_bf16: tile or head count");
    if (n_tiles == 0) return 0;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(n_tiles, n_q);
#define CALL(DD)                                                                                               \
    {                                                                                                          \
        const size_t smem = (size_t)(AT_BM + 4 * AT_BN) * (DD + 8) * sizeof(bf16);                             \
        if (int rc = set_smem<DD, 0>((const void*)flash_prefill_kernel<DD>, smem)) return rc;                     \
        gi_launch(flash_prefill_kernel<DD>, grid, dim3(AT_THREADS), smem, (cudaStream_t)stream,                             \
            (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, (const int4*)tiles,         \
            (bf16*)out, n_q, n_kv, page_size, max_pages, n_pool_pages, window, scale_log2);                    \
    }
    AT_DISPATCH_D(d, CALL)
#undef CALL
    return gi_check_launch("gi_attention_prefill_bf16");
}

// Scratch: part_o float32 [n_seqs * n_q * n_splits * d], part_ml float32 [n_seqs * n_q * n_splits * 2].
extern "C" int gi_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                        const int* tok_pos, const int* tok_slot, void* out, float* part_o,
                                        float* part_ml, int n_seqs, int n_q, int n_kv, int d, int page_size,
                                        int max_pages, int n_pool_pages, int window, float scale, int n_splits,
                                        void* stream) {
    if (int rc = check_common("gi_attention_decode_bf16", n_q, n_kv, d, page_size, max_pages, window)) return rc;
    GI_REQUIRE(n_q / n_kv <= 16, "gi_attention_decode_bf16: %d query heads per key/value head; this kernel takes up to 16", n_q / n_kv);
    GI_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_kv <= 65535 && n_seqs >= 0 && n_seqs <= 65535,
               "gi_attention_decode_bf16: %d slices, %d key/value heads, %d sequences", n_splits, n_kv, n_seqs);
    if (n_seqs == 0) return 0;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(n_splits, n_kv, n_seqs);
#define CALL(DD)                                                                                               \
    {                                                                                                          \
        size_t smem = (size_t)(16 + 4 * AT_DEC_DEPTH * 32) * (DD + 8) * sizeof(bf16);                          \
        const size_t merge = (size_t)16 * (DD + 8) * sizeof(bf16) + (size_t)(4 * 16 * DD + 128) * sizeof(float); \
        if (merge > smem) smem = merge;                                                                        \
        if (int rc = set_smem<DD, 1>((const void*)decode_splitkv_kernel<DD>, smem)) return rc;                    \
        gi_launch(decode_splitkv_kernel<DD>, grid, dim3(AT_THREADS), smem, (cudaStream_t)stream,                            \
            (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, tok_pos, tok_slot, part_o,  \
            part_ml, n_q, n_kv, page_size, max_pages, n_pool_pages, window, scale_log2, n_splits);             \
        gi_launch(decode_combine_kernel<DD>, dim3(n_seqs * n_q), dim3(DD < 128 ? (DD < 32 ? 32 : DD) : 128), 0, (cudaStream_t)stream,  \
            part_o, part_ml, (bf16*)out, n_splits);                                                            \
    }
    AT_DISPATCH_D(d, CALL)
#undef CALL
    return gi_check_launch("gi_attention_decode_bf16");
}

// Merges the slices' partial results of a split-KV decode kernel (this file's or the tcgen05 one):
// part_o float32 [rows * n_splits * d] unnormalised, part_ml float32 [rows * n_splits * 2] = (maximum in
// powers of two, sum); out bfloat16 [rows, d] for rows = sequences * query heads.
extern "C" int gi_attention_decode_combine(const float* part_o, const float* part_ml, void* out, int rows, int d,
                                           int n_splits, void* stream) {
    GI_REQUIRE(rows >= 0 && n_splits >= 1, "gi_attention_decode_combine: sizes");
    GI_REQUIRE(d >= 16 && d <= 128 && d % 16 == 0, "gi_attention_decode_combine: head_dim %d", d);
    if (rows == 0) return 0;
#define CALL(DD)                                                                                                 \
    gi_launch(decode_combine_kernel<DD>, dim3(rows), dim3(DD < 128 ? (DD < 32 ? 32 : DD) : 128), 0, (cudaStream_t)stream, \
              part_o, part_ml, (bf16*)out, n_splits);
    AT_DISPATCH_D(d, CALL)
#undef CALL
    return gi_check_launch("gi_attention_decode_combine");
}
