// Per-head RMSNorm of q and k, rotary position encoding, and the write of the
// new keys and values into the paged cache, in one pass over the projection
// output.
//
// Upstream does this as two RMSNorm launches over head_dim, two rotation
// launches, three transposes, a cache-append kernel and a length-increment
// kernel (src/models/qwen3/qwen3.cpp:149-168, src/src-cuda/rope.cu:109-131,
// src/src-cuda/kvcache.cu:7-45).  The arithmetic is theirs: the norm over
// the whole head with the weight as it is, then rotate-half
//   y[i]        = x[i] cos - x[i+r/2] sin
//   y[i + r/2]  = x[i+r/2] cos + x[i] sin        for i < r/2,  r = rotary_dim
// with dimensions beyond r passed through.  All of it is float32, rounded once.
//
// Layouts: qkv [n_tokens, (n_q + 2 n_kv) * d] (q heads, then k heads, then v
// heads); q_out [n_tokens, n_q, d]; cache pools [n_pages, n_kv, page_size, d];
// block_table [n_slots, max_pages] maps a slot's logical page to a pool page;
// cos/sin [max_positions, r/2] float32.  A token whose slot is negative is
// padding: its q is still written, nothing goes to the cache.
#include "common.cuh"

#include <type_traits>

#define ROPE_WARPS 4

template <typename T>
__global__ void qk_norm_rope_append_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const void* __restrict__ q_w, const void* __restrict__ k_w, int w_dtype, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rotary_dim,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, const int* __restrict__ block_table,
    int n_tokens, int n_q, int n_kv, int d, int page_size, int max_pages, int n_pool_pages,
    int max_positions, int append, int* __restrict__ status) {
    gi_pdl_start();
    extern __shared__ float head_buf[];            // ROPE_WARPS * d floats
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_here = append ? n_q + 2 * n_kv : n_q;
    const long long item = (long long)blockIdx.x * ROPE_WARPS + warp;
    if (item >= (long long)n_tokens * heads_here) return;
    const int t = (int)(item / heads_here);
    const int h = (int)(item - (long long)t * heads_here);
    const int row_w = (n_q + 2 * n_kv) * d;
    const T* src = qkv + (size_t)t * row_w + (size_t)h * d;
    float* buf = head_buf + warp * d;

    const bool is_q = h < n_q;
    const bool is_k = !is_q && h < n_q + n_kv;
    const int kvh = is_q ? 0 : (is_k ? h - n_q : h - n_q - n_kv);

    // destination
    T* dst;
    const int pos = tok_pos[t];
    if (is_q) {
        dst = q_out + ((size_t)t * n_q + h) * d;
    } else {
        const int slot = tok_slot[t];
        if (slot < 0) return;
        const int lp = pos / page_size;
        if (pos < 0 || lp >= max_pages) { if (lane == 0) atomicExch(status, 1); return; }
        const int page = block_table[(size_t)slot * max_pages + lp];
        if (page < 0 || page >= n_pool_pages) { if (lane == 0) atomicExch(status, 2); return; }
        T* pool = is_k ? k_pool : v_pool;
        dst = pool + (((size_t)page * n_kv + kvh) * page_size + (pos - lp * page_size)) * d;
    }

    if (!is_q && !is_k) {                          // values: copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }

    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float x = to_f32(src[i]);
        buf[i] = x;
        ss += x * x;
    }
    const void* w = is_q ? q_w : k_w;
    float inv = 1.f;
    if (w) inv = rsqrtf(warp_sum(ss) / (float)d + eps);
    __syncwarp();
    if (pos < 0 || pos >= max_positions) { if (lane == 0) atomicExch(status, 3); return; }
    const int half = rotary_dim / 2;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    for (int i = lane; i < d; i += 32) {
        float y;
        if (i < rotary_dim) {
            const int j = i < half ? i : i - half;
            const float a = w ? buf[j] * inv * load_w(w, w_dtype, j) : buf[j];
            const float b = w ? buf[j + half] * inv * load_w(w, w_dtype, j + half) : buf[j + half];
            // upstream rounds the normed value to the activation type before it rotates;
            // here it stays float32 until the single rounding at the end
            y = i < half ? a * cs[j] - b * sn[j] : b * cs[j] + a * sn[j];
        } else {
            y = w ? buf[i] * inv * load_w(w, w_dtype, i) : buf[i];
        }
        dst[i] = from_f32<T>(y);
    }
}

// A lane's N consecutive elements as the widest words that divide them (16, 8 or 4 bytes): one or two
// instructions instead of N.  The address must be aligned to that word (the entry point checks the bases).
template <typename T, int N>
struct RopeWords {
    static constexpr int bytes = N * (int)sizeof(T);
    static constexpr int W = bytes % 16 == 0 ? 16 : (bytes % 8 == 0 ? 8 : 4);
    static_assert(bytes % 4 == 0, "an even number of elements");
    typedef typename std::conditional<W == 16, uint4, typename std::conditional<W == 8, uint2, uint32_t>::type>::type word;
    union Both { word w[bytes / W]; T e[N]; __device__ Both() {} };
};
template <typename T, int N>
__device__ __forceinline__ void rope_load(T (&r)[N], const T* p) {
    typedef RopeWords<T, N> R;
    typename R::Both u;
#pragma unroll
    for (int i = 0; i < R::bytes / R::W; ++i) u.w[i] = reinterpret_cast<const typename R::word*>(p)[i];
#pragma unroll
    for (int i = 0; i < N; ++i) r[i] = u.e[i];
}
template <typename T, int N>
__device__ __forceinline__ void rope_store(T* p, const T (&r)[N]) {
    typedef RopeWords<T, N> R;
    typename R::Both u;
#pragma unroll
    for (int i = 0; i < N; ++i) u.e[i] = r[i];
#pragma unroll
    for (int i = 0; i < R::bytes / R::W; ++i) reinterpret_cast<typename R::word*>(p)[i] = u.w[i];
}

// The same for heads whose size is a multiple of 64 (up to 256) with the whole head rotated: a lane
// holds EPL = d/32 consecutive elements, so that loads and stores are contiguous over the warp and the
// rotation partner of lane l (the element half a head away) sits in lane l ^ 16.  A warp takes
// ROPE_GROUP consecutive heads of one token: their loads go out together, and the token's position,
// slot, page and rotation table are read once for all of them (prompts: 4 heads, a third less time at
// 2,048 tokens; decode steps: 1 head, where more warps matter more than fewer loads).
template <typename T, int EPL, int ROPE_GROUP>
__global__ void qk_norm_rope_append_vec_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const void* __restrict__ q_w, const void* __restrict__ k_w, int w_dtype, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, const int* __restrict__ block_table,
    int n_tokens, int n_q, int n_kv, int page_size, int max_pages, int n_pool_pages,
    int max_positions, int append, int* __restrict__ status) {
    gi_pdl_launch_dependents();
    constexpr int d = EPL * 32, half = d / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_here = append ? n_q + 2 * n_kv : n_q;
    const int groups = (heads_here + ROPE_GROUP - 1) / ROPE_GROUP;
    const long long item = (long long)blockIdx.x * ROPE_WARPS + warp;
    if (item >= (long long)n_tokens * groups) return;
    const int t = (int)(item / groups);
    const int h0 = (int)(item - (long long)t * groups) * ROPE_GROUP;
    // Positions, slots, the block table and the rotation table are set before the step's first kernel and
    // change in none of them: they are read before the wait for the kernel that makes qkv.
    const int pos = tok_pos[t];
    // where this token's keys and values go, if any head of the group is one
    T* k_dst = nullptr;
    T* v_dst = nullptr;
    bool cache_ok = false;
    int bad = 0;
    if (h0 + ROPE_GROUP > n_q && append) {
        const int slot = tok_slot[t];
        if (slot >= 0) {
            const int lp = pos / page_size;
            if (pos < 0 || lp >= max_pages) {
                bad = 1;
            } else {
                const int page = block_table[(size_t)slot * max_pages + lp];
                if (page < 0 || page >= n_pool_pages) {
                    bad = 2;
                } else {
                    const size_t row = (size_t)page * n_kv * page_size + (pos - lp * page_size);
                    k_dst = k_pool + row * d + lane * EPL;
                    v_dst = v_pool + row * d + lane * EPL;
                    cache_ok = true;
                }
            }
        }
    }
    const bool pos_ok = pos >= 0 && pos < max_positions;
    float cs[EPL], sn[EPL];
    if (pos_ok) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            cs[e] = cos_t[(size_t)pos * half + (lane & 15) * EPL + e];
            sn[e] = sin_t[(size_t)pos * half + (lane & 15) * EPL + e];
        }
    }
    gi_pdl_wait();
    if (bad && lane == 0) atomicExch(status, bad);
    const T* src = qkv + (size_t)t * (n_q + 2 * n_kv) * d + lane * EPL;
    T raw[ROPE_GROUP][EPL];
#pragma unroll
    for (int g = 0; g < ROPE_GROUP; ++g)
        if (h0 + g < heads_here) rope_load<T, EPL>(raw[g], src + (size_t)(h0 + g) * d);
#pragma unroll
    for (int g = 0; g < ROPE_GROUP; ++g) {
        const int h = h0 + g;
        if (h >= heads_here) break;                  // the same for the whole warp
        const bool is_q = h < n_q;
        const bool is_k = !is_q && h < n_q + n_kv;
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * n_q + h) * d + lane * EPL;
        } else {
            if (!cache_ok) continue;                 // padding, or an index outside the cache (reported above)
            const int kvh = is_k ? h - n_q : h - n_q - n_kv;
            dst = (is_k ? k_dst : v_dst) + (size_t)kvh * page_size * d;
        }
        if (!is_q && !is_k) {                        // values: copy
            rope_store<T, EPL>(dst, raw[g]);
            continue;
        }
        float x[EPL];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { x[e] = to_f32(raw[g][e]); ss += x[e] * x[e]; }
        const void* w = is_q ? q_w : k_w;
        if (w) {
            const float inv = rsqrtf(warp_sum(ss) / (float)d + eps);
#pragma unroll
            for (int e = 0; e < EPL; ++e) x[e] = x[e] * inv * load_w(w, w_dtype, lane * EPL + e);
        }
        if (!pos_ok) { if (lane == 0) atomicExch(status, 3); continue; }
        T y[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            y[e] = from_f32<T>(lane < 16 ? x[e] * cs[e] - other * sn[e] : x[e] * cs[e] + other * sn[e]);
        }
        rope_store<T, EPL>(dst, y);
    }
}

extern "C" int gi_qk_norm_rope_append(
    const void* qkv, void* q_out, void* k_pool, void* v_pool, int act_dtype,
    const void* q_w, const void* k_w, int w_dtype, float eps,
    const float* cos_t, const float* sin_t, int rotary_dim,
    const int* tok_pos, const int* tok_slot, const int* block_table,
    int n_tokens, int n_q, int n_kv, int d, int page_size, int max_pages, int n_pool_pages,
    int max_positions, int append, int* status, void* stream) {
    GI_REQUIRE(n_tokens >= 0 && n_q > 0 && n_kv > 0 && d > 0, "gi_qk_norm_rope_append: sizes must be positive");
    GI_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
               "gi_qk_norm_rope_append: rotary_dim %d must be even and at most head_dim %d", rotary_dim, d);
    GI_REQUIRE(d <= 1024, "gi_qk_norm_rope_append: head_dim %d is beyond 1024", d);
    GI_REQUIRE(page_size > 0 && max_pages > 0, "gi_qk_norm_rope_append: page sizes must be positive");
    GI_REQUIRE((q_w == nullptr) == (k_w == nullptr), "gi_qk_norm_rope_append: q and k norm weights go together");
    if (n_tokens == 0) return 0;
    const int heads_here = append ? n_q + 2 * n_kv : n_q;
    const long long items = (long long)n_tokens * heads_here;
    const long long blocks = (items + ROPE_WARPS - 1) / ROPE_WARPS;
    GI_REQUIRE(blocks < 2147483647LL, "gi_qk_norm_rope_append: too many (token, head) pairs");
    const size_t smem = (size_t)ROPE_WARPS * d * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) &&
                         ((uintptr_t)v_pool % 16 == 0);
    if (d % 64 == 0 && d <= 256 && rotary_dim == d && aligned) {
        const int group = n_tokens >= 256 ? 4 : 1;
        const long long vec_items = (long long)n_tokens * ((heads_here + group - 1) / group);
        const long long vec_blocks = (vec_items + ROPE_WARPS - 1) / ROPE_WARPS;
#define LAUNCH_VEC_G(T, EPL, G)                                                                                 \
    gi_launch(qk_norm_rope_append_vec_kernel<T, EPL, G>, dim3((int)vec_blocks), dim3(ROPE_WARPS * 32), 0, s,    \
              (const T*)qkv, (T*)q_out, (T*)k_pool, (T*)v_pool, q_w, k_w, w_dtype, eps, cos_t, sin_t, tok_pos,  \
              tok_slot, block_table, n_tokens, n_q, n_kv, page_size, max_pages, n_pool_pages, max_positions,    \
              append, status)
#define LAUNCH_VEC(T, EPL)                                                                                      \
    do { if (group == 4) LAUNCH_VEC_G(T, EPL, 4); else LAUNCH_VEC_G(T, EPL, 1); } while (0)
#define LAUNCH_VEC_T(T)                                                                                         \
    switch (d / 32) {                                                                                           \
        case 2: LAUNCH_VEC(T, 2); break;                                                                        \
        case 4: LAUNCH_VEC(T, 4); break;                                                                        \
        case 6: LAUNCH_VEC(T, 6); break;                                                                        \
        default: LAUNCH_VEC(T, 8); break;                                                                       \
    }
        if (act_dtype == GI_DTYPE_F32) { LAUNCH_VEC_T(float) }
        else if (act_dtype == GI_DTYPE_BF16) { LAUNCH_VEC_T(bf16) }
        else GI_REQUIRE(false, "gi_qk_norm_rope_append: activation dtype %d", act_dtype);
#undef LAUNCH_VEC_T
#undef LAUNCH_VEC
#undef LAUNCH_VEC_G
        return gi_check_launch("gi_qk_norm_rope_append");
    }
#define LAUNCH(T)                                                                                     \
    gi_launch(qk_norm_rope_append_kernel<T>, dim3((int)blocks), dim3(ROPE_WARPS * 32), smem, s,                          \
        (const T*)qkv, (T*)q_out, (T*)k_pool, (T*)v_pool, q_w, k_w, w_dtype, eps, cos_t, sin_t,       \
        rotary_dim, tok_pos, tok_slot, block_table, n_tokens, n_q, n_kv, d, page_size, max_pages,     \
        n_pool_pages, max_positions, append, status)
    if (act_dtype == GI_DTYPE_F32) LAUNCH(float);
    else if (act_dtype == GI_DTYPE_BF16) LAUNCH(bf16);
    else GI_REQUIRE(false, "gi_qk_norm_rope_append: activation dtype %d", act_dtype);
#undef LAUNCH
    return gi_check_launch("gi_qk_norm_rope_append");
}
