// Prefill attention on tensor cores: causal (optionally windowed)
// grouped-query attention of a packed batch of sequences over the paged cache.
//
// A CTA serves one (sequence, kv head, tile of query positions).  Its 128 MMA
// rows are (position, head of the kv head's group) pairs, position-major, so
// the K/V pages of that kv head are read once for all heads of the group
// (the reference's tiled kernel packs rows x group heads the same way with CUDA
// cores: src/kernels_cuda/attention_tiled.cuh:73-296).  Each of the 8 warps owns
// 16 rows; pages of 64 keys stream through double-buffered shared-memory tiles
// and every warp runs the online-softmax update on the whole page.  Keys come
// from the cache, which already holds this step's rows, so a prompt that
// arrives in chunks or continues an earlier step needs nothing special.
#include "attn_mma.cuh"
#include "common.cuh"
#include "paged.cuh"

namespace {

using namespace attn;
using rfx::PagedKV;

constexpr int PAGE = 64;
constexpr int PF_THREADS = 256;
constexpr int PF_ROWS = 128;

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages, PagedKV cache,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_new, const int* __restrict__ seq_row0,
                         __nv_bfloat16* __restrict__ out, int nq, int bq, int window,
                         float scale_log2) {
    constexpr int LD = D + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [128][LD]
    __nv_bfloat16* kbuf = qs + PF_ROWS * LD;                          // [2][PAGE][LD]
    __nv_bfloat16* vbuf = kbuf + 2 * PAGE * LD;

    rfx::pdl_prologue();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.y, kvh = blockIdx.z;
    const int n_new = seq_new[seq];
    // Tiles late in a sequence see the most keys: they are handed out first, so
    // the longest CTAs do not start last (src/kernels_cuda/attention_tiled.cuh
    // orders its row tiles the same way).
    const int q0 = (gridDim.x - 1 - blockIdx.x) * bq;  // first query of the tile, within this step's rows
    if (q0 >= n_new) return;
    const int g = nq / cache.n_kv_heads;
    const int slot = seq_slot[seq], start = seq_start[seq], row0 = seq_row0[seq];
    const int n_pos = min(bq, n_new - q0);
    const int n_rows = n_pos * g;  // valid MMA rows of the tile
    const int pos_first = start + q0, pos_last = pos_first + n_pos - 1;
    const int lo_tile = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;

    for (int i = tid; i < PF_ROWS * (D / 8); i += PF_THREADS) {
        const int row = i / (D / 8), c = i % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n_rows) {
            const int p = row / g, h = row % g;
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + q0 + p) * nq + kvh * g + h) * D + c * 8);
        }
        *reinterpret_cast<uint4*>(qs + row * LD + c * 8) = v;
    }

    const int* table = cache.page_table + (size_t)slot * cache.max_pages;
    auto issue = [&](int pg, int page, int buf) {
        const size_t off = ((size_t)page * cache.n_kv_heads + kvh) * PAGE * D;
        const int valid = min(PAGE, pos_last + 1 - pg * PAGE);
        load_tile_async<D>(kbuf + buf * PAGE * LD, k_pages + off, PAGE, valid, tid, PF_THREADS);
        load_tile_async<D>(vbuf + buf * PAGE * LD, v_pages + off, PAGE, valid, tid, PF_THREADS);
        cp_async_commit();
    };

    // this thread's two rows: warp * 16 + lane / 4 and + 8
    int row_pos[2], row_lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + (lane >> 2) + 8 * h;
        const int p = pos_first + min(row / g, n_pos - 1);
        row_pos[h] = row < n_rows ? p : -1;  // rows beyond the tile see nothing
        row_lo[h] = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    }
    const int warp_row0 = warp * 16;
    const int warp_pos_max = pos_first + min((min(warp_row0 + 15, n_rows - 1)) / g, n_pos - 1);
    const int warp_pos_min = pos_first + min(warp_row0 / g, n_pos - 1);
    const int warp_lo = (window > 0 && warp_pos_min + 1 > window) ? warp_pos_min + 1 - window : 0;
    const bool warp_active = warp_row0 < n_rows;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;

    const int pg0 = lo_tile / PAGE, pg1 = pos_last / PAGE + 1;
    // page ids are read one iteration ahead of their loads
    issue(pg0, table[pg0], 0);
    int page_ahead = pg0 + 1 < pg1 ? table[pg0 + 1] : 0;
    for (int pg = pg0; pg < pg1; ++pg) {
        const int buf = (pg - pg0) & 1;
        if (pg + 1 < pg1) {
            const int page_now = page_ahead;
            if (pg + 2 < pg1) page_ahead = table[pg + 2];
            issue(pg + 1, page_now, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int base = pg * PAGE;
        // skip pages wholly after this warp's last query or before its window
        if (warp_active && base <= warp_pos_max && base + PAGE > warp_lo) {
            auto visible = [&](int key, int h) {
                const int j = base + key;
                return j <= row_pos[h] && j >= row_lo[h];
            };
            attend_tile<D, 8>(qs + warp_row0 * LD, kbuf + buf * PAGE * LD, vbuf + buf * PAGE * LD, 0,
                              scale_log2, visible, m, l, acc);
        }
        __syncthreads();
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp_row0 + (lane >> 2) + 8 * h;
        if (row >= n_rows) continue;
        const int p = row / g, hd = row % g;
        const float inv = 1.0f / l[h];
        __nv_bfloat16* o = out + ((size_t)(row0 + q0 + p) * nq + kvh * g + hd) * D + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(acc[n][2 * h] * inv, acc[n][2 * h + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(o + n * 8) = v;
        }
    }
}

template <int D>
int launch_prefill(const void* q, const void* k_pages, const void* v_pages, const PagedKV& cache,
                   const int* seq_slot, const int* seq_start, const int* seq_new,
                   const int* seq_row0, void* out, int S, int max_new, int nq, int window,
                   float scale, cudaStream_t s) {
    constexpr int LD = D + 8;
    const int g = nq / cache.n_kv_heads;
    if (g > PF_ROWS) return RFX_ERR_UNSUPPORTED;
    const int bq = PF_ROWS / g;
    const size_t smem = (size_t)(PF_ROWS + 4 * PAGE) * LD * 2;
    auto kernel = attention_prefill_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((max_new + bq - 1) / bq, S, cache.n_kv_heads);
    if (grid.y > 65535 || grid.z > 65535) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(kernel, grid, PF_THREADS, smem, s, (const __nv_bfloat16*)q,
               (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, cache, seq_slot, seq_start,
               seq_new, seq_row0, (__nv_bfloat16*)out, nq, bq, window, scale * 1.4426950408889634f);
    return 0;
}

}  // namespace

// bfloat16 q and out [rows, nq, D] packed by sequence; seq_* describe the S
// sequences of the step (slot, positions already cached, rows in this step,
// first row).  The cache must already hold this step's keys and values.
// head_dim: multiples of 16 up to 256; group size nq / nkv up to 128; page 64.
extern "C" int rfx_attention_prefill(const void* q, const void* k_pages, const void* v_pages,
                                     const int* page_table, int max_pages, int page_size,
                                     const int* seq_slot, const int* seq_start, const int* seq_new,
                                     const int* seq_row0, void* out, int S, int max_new, int nq,
                                     int nkv, int head_dim, int window, float scale, void* stream) {
    if (S <= 0 || max_new <= 0) return 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0) return RFX_ERR_BAD_ARG;
    PagedKV cache{page_table, max_pages, page_size, nkv, head_dim};
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_CASE(DD)                                                                              \
    case DD:                                                                                      \
        return launch_prefill<DD>(q, k_pages, v_pages, cache, seq_slot, seq_start, seq_new,       \
                                  seq_row0, out, S, max_new, nq, window, scale, s);
    switch (head_dim) {
        RFX_CASE(16) RFX_CASE(32) RFX_CASE(48) RFX_CASE(64) RFX_CASE(80) RFX_CASE(96)
        RFX_CASE(112) RFX_CASE(128) RFX_CASE(144) RFX_CASE(160) RFX_CASE(176) RFX_CASE(192)
        RFX_CASE(208) RFX_CASE(224) RFX_CASE(240) RFX_CASE(256)
        default:
            return RFX_ERR_UNSUPPORTED;
    }
#undef RFX_CASE
}
