// Attention over the paged cache for any number of new tokens per sequence,
// float32 or bfloat16, any head_dim that is a multiple of 8 up to 512.
//
// This is the engine's exact path: the float32 engine uses it for prompts and
// for decoding alike, and the bfloat16 engine uses it for head sizes its
// tensor-core kernels do not take.  One block computes one (token, query
// head).  Keys are visited in chunks of 32 aligned to absolute positions
// (chunk c = keys 32c..32c+31), chunk c by warp c mod 4, and the four partial
// results are merged in warp order: the result at a position therefore does
// not depend on how the tokens were cut into steps, on the batch, or on where
// the pages lie.
//
//   o = softmax_j( q . k_j * scale ) v_j   over keys j <= pos, and j > pos - window
//                                           when window > 0
// Query head h reads key/value head h / (n_q / n_kv).  Scores, softmax and the
// weighted sum are float32.  Upstream hands this to a library
// (src/src-cuda/attention/fattn.cu:74-86: scale 1/sqrt(head_dim), causal mask
// aligned to the last key, float32 intermediates).
#include "common.cuh"
#include <math.h>

#define AG_WARPS 4

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; typedef float4 type; };
template <> struct Vec<bf16> { static constexpr int N = 8; typedef uint4 type; };

__device__ __forceinline__ float dot_vec(const float4& k, const float* q) {
    return k.x * q[0] + k.y * q[1] + k.z * q[2] + k.w * q[3];
}
__device__ __forceinline__ float dot_vec(const uint4& k, const float* q) {
    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&k);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(k2[i]);
        s += f.x * q[2 * i] + f.y * q[2 * i + 1];
    }
    return s;
}

template <typename T, int DPL>
__global__ void __launch_bounds__(AG_WARPS * 32)
attn_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                    const int* __restrict__ block_table, const int* __restrict__ tok_pos,
                    const int* __restrict__ tok_slot, T* __restrict__ out, int n_q, int n_kv, int d,
                    int page_size, int max_pages, int n_pool_pages, int window, float scale,
                    int* __restrict__ status) {
    gi_pdl_start();
    extern __shared__ float smem[];
    float* q_s = smem;                       // d
    float* acc_s = smem + d;                 // AG_WARPS * d
    float* m_s = acc_s + AG_WARPS * d;       // AG_WARPS
    float* l_s = m_s + AG_WARPS;             // AG_WARPS

    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* o = out + ((size_t)t * n_q + h) * d;
    const int slot = tok_slot[t];
    const int pos = tok_pos[t];
    if (slot < 0 || pos < 0 || pos / page_size >= max_pages) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<T>(0.f);
        if (slot >= 0 && threadIdx.x == 0) atomicExch(status, 4);
        return;
    }
    const int kvh = h / (n_q / n_kv);
    const T* qrow = q + ((size_t)t * n_q + h) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) q_s[i] = to_f32(qrow[i]) * scale;
    __syncthreads();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)slot * max_pages;
    float m = -INFINITY, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int r = 0; r < DPL; ++r) acc[r] = 0.f;

    constexpr int VN = Vec<T>::N;
    typedef typename Vec<T>::type vec_t;
    for (int c = lo / 32 + warp; c <= pos / 32; c += AG_WARPS) {
        const int j = c * 32 + lane;
        const bool valid = j >= lo && j <= pos;
        long long row = -1;                  // element offset of this lane's key/value row
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= n_pool_pages) {
                atomicExch(status, 5);
            } else {
                row = (((long long)page * n_kv + kvh) * page_size + (j % page_size)) * d;
                const vec_t* kr = reinterpret_cast<const vec_t*>(k_pool + row);
                float a = 0.f;
                for (int i = 0; i < d / VN; ++i) a += dot_vec(kr[i], q_s + i * VN);
                s = a;
            }
        }
        const float cmax = warp_max(s);
        if (cmax == -INFINITY) continue;
        const float m_new = fmaxf(m, cmax);
        const float corr = expf(m - m_new);              // 0 when m is -inf
        const float p = row >= 0 ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < DPL; ++r) acc[r] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (rj < 0) continue;
            const T* vr = v_pool + rj;
#pragma unroll
            for (int r = 0; r < DPL; ++r) {
                const int i = lane + 32 * r;
                if (i < d) acc[r] += pj * to_f32(vr[i]);
            }
        }
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int r = 0; r < DPL; ++r) {
        const int i = lane + 32 * r;
        if (i < d) acc_s[warp * d + i] = acc[r];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < AG_WARPS; ++w) M = fmaxf(M, m_s[w]);
    float L = 0.f;
    for (int w = 0; w < AG_WARPS; ++w) L += (m_s[w] == -INFINITY ? 0.f : expf(m_s[w] - M) * l_s[w]);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < AG_WARPS; ++w)
            if (m_s[w] != -INFINITY) v += expf(m_s[w] - M) * acc_s[w * d + i];
        o[i] = from_f32<T>(L > 0.f ? v / L : 0.f);
    }
}

template <typename T>
static int launch_generic(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                          const int* tok_pos, const int* tok_slot, void* out, int n_tokens, int n_q, int n_kv,
                          int d, int page_size, int max_pages, int n_pool_pages, int window, float scale,
                          int* status, cudaStream_t s) {
    dim3 grid(n_tokens, n_q);
    const size_t smem = ((size_t)d * (1 + AG_WARPS) + 2 * AG_WARPS) * sizeof(float);
#define AG_LAUNCH(DPL)                                                                               \
    gi_launch(attn_generic_kernel<T, DPL>, grid, dim3(AG_WARPS * 32), smem, s,                                     \
        (const T*)q, (const T*)k_pool, (const T*)v_pool, block_table, tok_pos, tok_slot, (T*)out,     \
        n_q, n_kv, d, page_size, max_pages, n_pool_pages, window, scale, status)
    if (d <= 32) AG_LAUNCH(1);
    else if (d <= 64) AG_LAUNCH(2);
    else if (d <= 128) AG_LAUNCH(4);
    else if (d <= 256) AG_LAUNCH(8);
    else AG_LAUNCH(16);
#undef AG_LAUNCH
    return gi_check_launch("gi_attention_generic");
}

extern "C" int gi_attention_generic(const void* q, const void* k_pool, const void* v_pool, int act_dtype,
                                    const int* block_table, const int* tok_pos, const int* tok_slot,
                                    void* out, int n_tokens, int n_q, int n_kv, int d, int page_size,
                                    int max_pages, int n_pool_pages, int window, float scale, int* status,
                                    void* stream) {
    GI_REQUIRE(n_tokens >= 0 && n_q > 0 && n_kv > 0 && d > 0, "gi_attention_generic: sizes must be positive");
    GI_REQUIRE(n_q % n_kv == 0, "gi_attention_generic: %d query heads are no multiple of %d key/value heads", n_q, n_kv);
    GI_REQUIRE(d % 8 == 0 && d <= 512, "gi_attention_generic: head_dim %d must be a multiple of 8, at most 512", d);
    GI_REQUIRE(n_q <= 65535, "gi_attention_generic: %d query heads is beyond 65535", n_q);
    GI_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "gi_attention_generic: page size, table width and window");
    if (n_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        return launch_generic<float>(q, k_pool, v_pool, block_table, tok_pos, tok_slot, out, n_tokens, n_q, n_kv, d,
                                     page_size, max_pages, n_pool_pages, window, scale, status, s);
    if (act_dtype == GI_DTYPE_BF16)
        return launch_generic<bf16>(q, k_pool, v_pool, block_table, tok_pos, tok_slot, out, n_tokens, n_q, n_kv, d,
                                    page_size, max_pages, n_pool_pages, window, scale, status, s);
    GI_REQUIRE(false, "gi_attention_generic: activation dtype %d", act_dtype);
}
