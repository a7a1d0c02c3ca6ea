// Plain attention over the paged cache: one warp per (query row, head), keys
// one after another with a running maximum and sum.  It serves prefill and
// decode alike, in 32-bit storage (the true 32-bit path) and in bfloat16
// storage (the path to compare the tensor-core kernels with).  A row's result
// depends only on its own sequence's cache contents and position: the same
// code runs however the tokens are cut into steps or batched.
//
// For a query at position p of head h (kv head h / group): keys j in
// [max(0, p - window + 1), p];  s_j = (q . K_j) * scale;  online softmax
// m' = max(m, s), l = l e^(m-m') + e^(s-m'), acc = acc e^(m-m') + e^(s-m') V_j;
// out = acc / l   (src/kernels_cuda/attention_online.cuh:64-102; the window
// rule is src/model/config.rs:1184-1185: i - j < window).
//
// Orders, which a host mirror repeats bit for bit: the dot product as a fused
// multiply-add chain per lane over elements lane, lane + 32, ..., then the
// lanes' butterfly, then times scale; l = fma(l, corr, p);
// acc = fma(acc, corr, p * v) with the product rounded first; the exponential
// is `exact_expf`.
#include "common.cuh"
#include "exact_math.cuh"
#include "paged.cuh"

namespace {

using namespace rfx;

constexpr int MAX_PER_LANE = 16;  // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(128)
attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                       const T* __restrict__ v_pages, PagedKV cache,
                       const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                       T* __restrict__ out, int nq, int window, float scale) {
    pdl_prologue();
    const int d = cache.head_dim;
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= nq) return;
    const int kvh = h / (nq / cache.n_kv_heads);
    const int pos = row_pos[r], slot = row_slot[r];
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qrow = q + ((size_t)r * nq + h) * d;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = i * 32 + lane;
        qv[i] = e < d ? ld<T>(qrow, e) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int j = lo; j <= pos; ++j) {
        const size_t off = kv_offset(cache, slot, j, kvh);
        const T* kp = k_pages + off;
        const T* vp = v_pages + off;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (e < d) dot = fmaf(qv[i], ld<T>(kp, e), dot);
        }
        const float s = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = exact_expf(m - m_new);  // 0 at the first key (m = -inf)
        const float p = exact_expf(s - m_new);
        l = fmaf(l, corr, p);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (e < d) acc[i] = fmaf(acc[i], corr, __fmul_rn(p, ld<T>(vp, e)));
        }
        m = m_new;
    }
    T* orow = out + ((size_t)r * nq + h) * d;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = i * 32 + lane;
        if (e < d) st<T>(orow, e, acc[i] / l);
    }
}

}  // namespace

extern "C" int rfx_attention_plain(const void* q, const void* k_pages, const void* v_pages, int dt,
                                   const int* page_table, int max_pages, int page_size,
                                   const int* row_pos, const int* row_slot, void* out, int R,
                                   int nq, int nkv, int head_dim, int window, float scale,
                                   void* stream) {
    if (R <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * MAX_PER_LANE) return RFX_ERR_UNSUPPORTED;
    if (nkv <= 0 || nq % nkv != 0) return RFX_ERR_BAD_ARG;
    PagedKV cache{page_table, max_pages, page_size, nkv, head_dim};
    dim3 grid(R, (nq + 3) / 4);
    if (grid.y > 65535) return RFX_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(attention_plain_kernel<float>, grid, 128, 0, s, (const float*)q,
                   (const float*)k_pages, (const float*)v_pages, cache, row_pos, row_slot,
                   (float*)out, nq, window, scale);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(attention_plain_kernel<__nv_bfloat16>, grid, 128, 0, s, (const __nv_bfloat16*)q,
                   (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, cache, row_pos,
                   row_slot, (__nv_bfloat16*)out, nq, window, scale);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
