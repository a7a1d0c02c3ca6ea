// Decode attention on tensor cores: one query position per row, split over
// the keys.
//
// A CTA serves one (row, kv head, tile of up to 8 query heads of that kv
// head's group, split of the key range).  The keys are the rows of the MMA
// tiles and the query heads that share the kv head its 8 columns
// (attn_mma.cuh: attend_keys16), so each K/V page is read once for the whole
// group (the reference's decode kernel does the same with CUDA cores:
// src/kernels_cuda/attention_decode.cuh:34-176).  Pages of 64 keys stream
// through a three-stage ring of shared-memory tiles; warp w takes keys
// [16 w, 16 w + 16) of every page with its own running (max, sum, acc), and
// the four warps are merged at the end.  With more than one split the splits
// either form a thread-block cluster that merges its partials over distributed
// shared memory, or write unnormalised partials (acc, max, sum) to scratch for
// a second kernel that combines them in split order
// (src/kernels_cuda/attention_online.cu:51-78).  Softmax runs in 32-bit on
// base-2 exponentials: p = 2^((s - m) * scale * log2 e).
#include <cooperative_groups.h>

#include <mutex>

#include "attn_mma.cuh"
#include "common.cuh"
#include "noalloc.h"
#include "paged.cuh"

namespace {

namespace cg = cooperative_groups;
using namespace attn;
using rfx::PagedKV;

// Optional timeline for tuning: when a buffer is set (rfx_attention_decode_trace),
// thread 0 of every CTA stores %globaltimer at chosen moments of its life in the
// record of its launch: 0 entry, 1 the kernel before is done, 2 query rows loaded,
// 3 last page done, 4 the warps merged, 5 past the cluster's barrier, 6 exit.
struct DecTraceRec {
    unsigned long long t[8];
};
static __device__ DecTraceRec* g_dtrace = nullptr;
static __device__ int g_dtrace_ctas = 0;  // records per launch
static __device__ int g_dtrace_launches = 0;
int g_dtrace_next = 0;  // launch counter: the record a launch writes
__device__ __forceinline__ void dtrace_mark(int launch, int which) {
    if (g_dtrace == nullptr || launch >= g_dtrace_launches || threadIdx.x != 0) return;
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta >= g_dtrace_ctas) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_dtrace[(size_t)launch * g_dtrace_ctas + cta].t[which] = t;
}

constexpr int PAGE = 64;
constexpr int DEC_THREADS = 128;
constexpr int DEC_STAGES = 3;  // pages in flight per CTA
constexpr int MAX_RANKS = 16;  // 8 is the portable cluster size; 16 where the device places one

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, PagedKV cache,
                        const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int nq,
                        int n_htiles, int n_splits, int window, float scale_log2, int cluster_merge,
                        int trace_id) {
    constexpr int LD = D + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [16][LD], rows 0..7 used
    __nv_bfloat16* kbuf = qs + 16 * LD;                               // [STAGES][PAGE][LD]
    __nv_bfloat16* vbuf = kbuf + DEC_STAGES * PAGE * LD;              // [STAGES][PAGE][LD]
    // with the splits merged inside a cluster: what the other ranks send
    float* recv_m = reinterpret_cast<float*>(vbuf + DEC_STAGES * PAGE * LD);  // [ranks][16]
    float* recv_l = recv_m + MAX_RANKS * 16;                                  // [ranks][16]
    float* recv_a = recv_l + MAX_RANKS * 16;                                  // [ranks][slice]

    rfx::pdl_launch_dependents();
    dtrace_mark(trace_id, 0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = blockIdx.x;
    const int kvh = blockIdx.y / n_htiles, ht = blockIdx.y % n_htiles;
    const int split = blockIdx.z;
    const int g = nq / cache.n_kv_heads;
    const int h0 = kvh * g + ht * 8;  // a tile holds up to eight query heads: the MMA's columns
    const int nh = min(8, g - ht * 8);
    const int pos = row_pos[r], slot = row_slot[r];
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_page = lo / PAGE, last_page = pos / PAGE;
    const int n_pg = last_page - first_page + 1;
    const int pps = (n_pg + n_splits - 1) / n_splits;
    const int pg0 = first_page + split * pps;
    const int pg1 = min(last_page + 1, pg0 + pps);

    const int* table = cache.page_table + (size_t)slot * cache.max_pages;
    auto issue = [&](int pg, int page, int buf) {
        const size_t off = ((size_t)page * cache.n_kv_heads + kvh) * PAGE * D;
        const int valid = min(PAGE, pos + 1 - pg * PAGE);
        load_tile_async<D>(kbuf + buf * PAGE * LD, k_pages + off, PAGE, valid, tid, DEC_THREADS);
        load_tile_async<D>(vbuf + buf * PAGE * LD, v_pages + off, PAGE, valid, tid, DEC_THREADS);
        cp_async_commit();
    };

    // this thread's heads are 2 (lane % 4) and 2 (lane % 4) + 1 (attn_mma.cuh: attend_keys16)
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[D / 16][4];
#pragma unroll
    for (int n = 0; n < D / 16; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    uint32_t qf[D / 16][2];
    load_query_fragments<D>(qs, qf);  // whatever the tile holds: the dry pass only needs operands

    // a ring of DEC_STAGES pages: one commit group per page, empty groups past the end
    // The page id of a load is read one iteration before the load is issued, so
    // the page-table read never stalls the loop.
    int pages_first[DEC_STAGES];
#pragma unroll
    for (int i = 0; i < DEC_STAGES; ++i) pages_first[i] = pg0 + i < pg1 ? table[pg0 + i] : 0;
    // Pages before the one that holds this row's own position were written by
    // earlier steps: their loads start before the wait on the preceding kernel,
    // which writes only the new key, value and query.  Positions, slots and the
    // page table are the step's inputs, uploaded before the step's kernels.
    int issued = 0;
#pragma unroll
    for (int i = 0; i < DEC_STAGES - 1; ++i) {
        if (issued == i && pg0 + i < pg1 && pg0 + i < last_page) {
            issue(pg0 + i, pages_first[i], i);
            ++issued;
        }
    }
    // The loop's first pass is a dry one, still before the wait: it runs the tile
    // code on whatever the last ring buffer holds with every key masked, so that
    // the instructions are in the cache when the real pages come; its results
    // are thrown away.  Then the wait, the query rows, and the real passes.
    int page_ahead = pages_first[DEC_STAGES - 1];
#pragma unroll 1
    for (int pg = pg0 - 1;;) {
        const bool dry = pg < pg0;
        const int buf = dry ? DEC_STAGES - 1 : (pg - pg0) % DEC_STAGES;
        if (!dry) {
            cp_async_wait<DEC_STAGES - 2>();  // page pg has landed (this thread's part)
            __syncthreads();                  // everyone's part; and buffer (pg - 1) is free
            const int nxt = pg + DEC_STAGES - 1;
            const int page_now = page_ahead;
            if (nxt + 1 < pg1) page_ahead = table[nxt + 1];
            if (nxt < pg1) issue(nxt, page_now, (nxt - pg0) % DEC_STAGES);
            else cp_async_commit();
        }
        const int base = pg * PAGE;
        const int lo_eff = dry ? 0x7fffffff : lo;
        auto visible = [&](int key) { return base + key >= lo_eff && base + key <= pos; };
        attend_keys16<D>(qf, kbuf + buf * PAGE * LD, vbuf + buf * PAGE * LD, warp * 16, scale_log2, visible,
                         m, l, acc);
        if (dry) {
            m[0] = m[1] = -INFINITY;
            l[0] = l[1] = 0.0f;
#pragma unroll
            for (int n = 0; n < D / 16; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
            // After the wait on the kernel before: first the loads of the pages that
            // had to wait for it (the one with this row's own position), then the query
            // rows, whose latency those loads then cover.
            rfx::pdl_wait();
            dtrace_mark(trace_id, 1);
#pragma unroll
            for (int i = 0; i < DEC_STAGES - 1; ++i) {
                if (i >= issued) {
                    if (pg0 + i < pg1) issue(pg0 + i, pages_first[i], i);
                    else cp_async_commit();
                }
            }
            // the query heads of this tile; rows beyond the group are zero
            __syncthreads();  // every warp has read the tile for its dry pass
            for (int i = tid; i < 8 * (D / 8); i += DEC_THREADS) {
                const int row = i / (D / 8), c = i % (D / 8);
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row < nh) v = *reinterpret_cast<const uint4*>(q + ((size_t)r * nq + h0 + row) * D + c * 8);
                *reinterpret_cast<uint4*>(qs + row * LD + c * 8) = v;
            }
            __syncthreads();
            load_query_fragments<D>(qs, qf);
            dtrace_mark(trace_id, 2);
        }
        ++pg;
        if (pg >= pg1) break;
    }
    cp_async_wait<0>();
    __syncthreads();  // all warps are done with the tiles before they are reused below
    dtrace_mark(trace_id, 3);

    // a head's sum lies in the eight lanes that share lane % 4
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        l[j] += __shfl_xor_sync(0xffffffffu, l[j], 4);
        l[j] += __shfl_xor_sync(0xffffffffu, l[j], 8);
        l[j] += __shfl_xor_sync(0xffffffffu, l[j], 16);
    }
    // merge the four warps: each holds (m, l, acc) over its quarter of the keys
    float* red = reinterpret_cast<float*>(kbuf);  // [4][8][D] acc, then [4][8] m, [4][8] l
    float* red_m = red + 4 * 8 * D;
    float* red_l = red_m + 4 * 8;
    {
        const int g0 = lane >> 2, c = lane & 3;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int head = 2 * c + j;
            if (head < nh) {  // columns beyond the group's heads hold nothing
                float* dst = red + (size_t)(warp * 8 + head) * D + g0;
#pragma unroll
                for (int i = 0; i < D / 16; ++i) {
                    dst[16 * i] = acc[i][j];
                    dst[16 * i + 8] = acc[i][2 + j];
                }
                if (g0 == 0) {
                    red_m[warp * 8 + head] = m[j];
                    red_l[warp * 8 + head] = l[j];
                }
            }
        }
    }
    __syncthreads();
    const int total = nh * D;
    const int slice = (total + n_splits - 1) / n_splits;  // elements of the tile's output a rank merges
    for (int i = tid; i < total; i += DEC_THREADS) {
        const int row = i / D, e = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 8 + row]);
        float L = 0.0f, A = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(red_m[w * 8 + row] - M);
                L += red_l[w * 8 + row] * f;
                A += red[(size_t)(w * 8 + row) * D + e] * f;
            }
        }
        const size_t head = (size_t)r * nq + h0 + row;
        if (n_splits == 1) {
            out[head * D + e] = __float2bfloat16_rn(A / L);
        } else if (!cluster_merge) {
            float* p = partial + (head * n_splits + split) * (D + 2);
            p[e] = A;
            if (e == 0) {
                p[D] = M;
                p[D + 1] = L;
            }
        } else {
            // element i of the tile's output belongs to rank i / slice: send the
            // partial there, and its (max, sum) to every rank
            cg::cluster_group cluster = cg::this_cluster();
            const int owner = i / slice, off = i % slice;
            cluster.map_shared_rank(recv_a, owner)[(size_t)split * slice + off] = A;
            if (e == 0) {
                for (int dst = 0; dst < n_splits; ++dst) {
                    cluster.map_shared_rank(recv_m, dst)[split * 16 + row] = M;
                    cluster.map_shared_rank(recv_l, dst)[split * 16 + row] = L;
                }
            }
        }
    }
    dtrace_mark(trace_id, 4);
    if (n_splits > 1 && cluster_merge) {
        // One cluster barrier, then every rank merges its slice in rank order with
        // the combine kernel's arithmetic (the same bits) and writes it.  Nobody
        // reads another rank's memory after the barrier.
        cg::this_cluster().sync();
        dtrace_mark(trace_id, 5);
        for (int off = tid; off < slice; off += DEC_THREADS) {
            const int i = split * slice + off;
            if (i >= total) break;
            const int row = i / D, e = i % D;
            float M = -INFINITY;
            for (int sidx = 0; sidx < n_splits; ++sidx) M = fmaxf(M, recv_m[sidx * 16 + row]);
            float L = 0.0f, A = 0.0f;
            for (int sidx = 0; sidx < n_splits; ++sidx) {
                const float ms = recv_m[sidx * 16 + row];
                const float f = ms == -INFINITY ? 0.0f : exp2f(ms - M);
                L = __fadd_rn(L, __fmul_rn(recv_l[sidx * 16 + row], f));
                A += recv_a[(size_t)sidx * slice + off] * f;
            }
            const float inv = 1.0f / L;
            out[((size_t)r * nq + h0 + row) * D + e] = __float2bfloat16_rn(A * inv);
        }
    }
    dtrace_mark(trace_id, 6);
}

// out[head] = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in order.
// The splits' weights 2^(m_s - M) / L are computed once into shared memory.
constexpr int MAX_SPLITS = 64;
__global__ void attention_combine_kernel(const float* __restrict__ partial,
                                         __nv_bfloat16* __restrict__ out, int D, int n_splits) {
    __shared__ float wgt[MAX_SPLITS];
    __shared__ float lw[MAX_SPLITS];
    __shared__ float inv_l;
    rfx::pdl_launch_dependents();
    const size_t head = blockIdx.x;
    const float* p = partial + head * n_splits * (D + 2);
    // Two passes over the same code: a dry one before the wait on the attention
    // kernel (it reads zeros in place of the partials and stores nothing; it
    // brings the instructions into the cache), then the work.
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
        const bool dry = pass == 0;
        if (!dry) rfx::pdl_wait();
        if (threadIdx.x < 32) {
            float ms[MAX_SPLITS / 32], ls[MAX_SPLITS / 32];
            float M = -INFINITY;
#pragma unroll
            for (int i = 0; i < MAX_SPLITS / 32; ++i) {
                const int sidx = threadIdx.x + 32 * i;
                const bool in = sidx < n_splits && !dry;
                ms[i] = in ? p[sidx * (D + 2) + D] : -INFINITY;
                ls[i] = in ? p[sidx * (D + 2) + D + 1] : 0.0f;
                M = fmaxf(M, ms[i]);
            }
            M = rfx::warp_max(M);
#pragma unroll
            for (int i = 0; i < MAX_SPLITS / 32; ++i) {
                const float e = ms[i] == -INFINITY ? 0.0f : exp2f(ms[i] - M);
                wgt[threadIdx.x + 32 * i] = e;
                lw[threadIdx.x + 32 * i] = ls[i] * e;
            }
            __syncwarp();
            if (threadIdx.x == 0) {  // in split order, by one lane: the same bits every time
                float L = 0.0f;
                for (int sidx = 0; sidx < n_splits; ++sidx) L += lw[sidx];
                inv_l = 1.0f / L;
            }
        }
        __syncthreads();
        const float inv = inv_l;
        for (int e = threadIdx.x; e < D; e += blockDim.x) {
            float A = 0.0f;
#pragma unroll 4
            for (int sidx = 0; sidx < n_splits; ++sidx) A += (dry ? 0.0f : p[sidx * (D + 2) + e]) * wgt[sidx];
            if (!dry) out[head * D + e] = __float2bfloat16_rn(A * inv);
        }
        __syncthreads();  // wgt, lw and inv_l are written again by the next pass
    }
}

template <int D>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, const PagedKV& cache,
                  const int* row_pos, const int* row_slot, void* out, float* partial, int R, int nq,
                  int n_splits, int window, float scale, int cluster_merge, cudaStream_t s) {
    constexpr int LD = D + 8;
    const int g = nq / cache.n_kv_heads;
    const int n_htiles = (g + 7) / 8;
    const int tile_heads = g < 8 ? g : 8;
    size_t smem = (size_t)(16 + 2 * DEC_STAGES * PAGE) * LD * 2;
    const size_t red = (size_t)(4 * 16 * D + 2 * 4 * 16) * 4;
    if (red > (size_t)2 * DEC_STAGES * PAGE * LD * 2) return RFX_ERR_UNSUPPORTED;
    if (cluster_merge) {
        smem += (size_t)(2 * MAX_RANKS * 16 + tile_heads * D) * 4;
        if (smem > 227 * 1024) return RFX_ERR_UNSUPPORTED;
    }
    auto kernel = attention_decode_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(R, cache.n_kv_heads * n_htiles, n_splits);
    if (cluster_merge && n_splits > 8) {
        // a cluster of 16 is beyond the portable size: allowed per kernel, and used
        // only if the device can place one with this much shared memory (asked once)
        static int placeable = -1;
        if (placeable < 0) {
            placeable = 0;
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(1, 1, 16);
                cfg.blockDim = dim3(DEC_THREADS);
                cfg.dynamicSmemBytes = smem;
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = 1;
                at[0].val.clusterDim.y = 1;
                at[0].val.clusterDim.z = 16;
                cfg.attrs = at;
                cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0) placeable = 1;
            }
            cudaGetLastError();  // a refusal is an answer, not an error to carry on
        }
        if (!placeable) return RFX_ERR_UNSUPPORTED;
    }
    e = rfx::launch(kernel, grid, dim3(DEC_THREADS), smem, s, cluster_merge ? n_splits : 1,
                    (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                    cache, row_pos, row_slot, (__nv_bfloat16*)out, partial, nq, n_htiles, n_splits, window,
                    scale * 1.4426950408889634f, cluster_merge, g_dtrace_next++);
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1 && !cluster_merge)
        RFX_LAUNCH(attention_combine_kernel, R * nq, D <= 128 ? 64 : 128, 0, s, (const float*)partial,
                   (__nv_bfloat16*)out, D, n_splits);
    return 0;
}

int decode_entry(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                 int max_pages, int page_size, const int* row_pos, const int* row_slot, void* out,
                 float* partial, int R, int nq, int nkv, int head_dim, int n_splits, int window,
                 float scale, int cluster_merge, void* stream) {
    if (R <= 0) return 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0 || n_splits < 1) return RFX_ERR_BAD_ARG;
    if (n_splits > 1 && !partial && !cluster_merge) return RFX_ERR_BAD_ARG;
    if (cluster_merge && n_splits != 2 && n_splits != 4 && n_splits != 8 && n_splits != 16) return RFX_ERR_UNSUPPORTED;
    if (n_splits > MAX_SPLITS) return RFX_ERR_UNSUPPORTED;
    if (n_splits > 65535 || (long long)nkv * ((nq / nkv + 7) / 8) > 65535) return RFX_ERR_UNSUPPORTED;
    PagedKV cache{page_table, max_pages, page_size, nkv, head_dim};
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_CASE(DD)                                                                            \
    case DD:                                                                                    \
        return launch_decode<DD>(q, k_pages, v_pages, cache, row_pos, row_slot, out, partial, R, \
                                 nq, n_splits, window, scale, cluster_merge, s);
    switch (head_dim) {
        RFX_CASE(16) RFX_CASE(32) RFX_CASE(48) RFX_CASE(64) RFX_CASE(80) RFX_CASE(96)
        RFX_CASE(112) RFX_CASE(128) RFX_CASE(144) RFX_CASE(160) RFX_CASE(176) RFX_CASE(192)
        RFX_CASE(208) RFX_CASE(224) RFX_CASE(240) RFX_CASE(256)
        default:
            return RFX_ERR_UNSUPPORTED;
    }
#undef RFX_CASE
}

}  // namespace

// bfloat16 q [R, nq, D], paged K/V, one query position per row.  `partial` is
// scratch of R * nq * n_splits * (D + 2) floats, needed when n_splits > 1.
// head_dim: multiples of 16 up to 256; the page size must be 64.
extern "C" int rfx_attention_decode(const void* q, const void* k_pages, const void* v_pages,
                                    const int* page_table, int max_pages, int page_size,
                                    const int* row_pos, const int* row_slot, void* out,
                                    float* partial, int R, int nq, int nkv, int head_dim,
                                    int n_splits, int window, float scale, void* stream) {
    return decode_entry(q, k_pages, v_pages, page_table, max_pages, page_size, row_pos, row_slot, out,
                        partial, R, nq, nkv, head_dim, n_splits, window, scale, 0, stream);
}

// The same with 2, 4, 8 or (where the device places such a cluster) 16 splits that
// form a thread-block cluster: every rank
// sends its partial to the rank that owns that slice of the output over
// distributed shared memory, one cluster barrier, and the owners merge in rank
// order with the combine kernel's arithmetic.  No scratch, no second kernel.
// RFX_ERR_UNSUPPORTED for other split counts or sizes that leave no shared
// memory for the exchange: the caller then takes the entry point above.
extern "C" int rfx_attention_decode_cluster(const void* q, const void* k_pages, const void* v_pages,
                                            const int* page_table, int max_pages, int page_size,
                                            const int* row_pos, const int* row_slot, void* out, int R,
                                            int nq, int nkv, int head_dim, int n_splits, int window,
                                            float scale, void* stream) {
    return decode_entry(q, k_pages, v_pages, page_table, max_pages, page_size, row_pos, row_slot, out,
                        nullptr, R, nq, nkv, head_dim, n_splits, window, scale, 1, stream);
}

// ---------------------------------------------------------------------------
// The same kernel behind an entry point that allocates nothing (noalloc.h).
// Its split partials live in this file-scope device array instead of a buffer
// the caller allocates.  In host code the array's name is only a stand-in for
// the device symbol, never a device address, so the address is asked for once
// per device, with that device current, and that pointer is what the kernel
// gets.
namespace {

static __device__ __align__(256) float g_noalloc_partial[RFX_NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mu;

// Device address of the array on the current device; looked up on the first
// call per device.
int noalloc_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return RFX_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_partial);
        if (e != cudaSuccess) return (int)e;
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}

}  // namespace

// Tuning aid: give the decode attention kernel a device buffer of launches * ctas
// records of eight 64-bit time stamps; the next launch writes record 0.  Null turns
// it off.
extern "C" int rfx_attention_decode_trace(void* buffer, int launches, int ctas) {
    g_dtrace_next = 0;
    DecTraceRec* p = (DecTraceRec*)buffer;
    cudaError_t e = cudaMemcpyToSymbol(g_dtrace, &p, sizeof(p));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_dtrace_ctas, &ctas, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_dtrace_launches, &launches, sizeof(int));
    return (int)e;
}

extern "C" long long rfx_attention_decode_noalloc_capacity(void) {
    return (long long)RFX_NOALLOC_SCRATCH_FLOATS;
}

extern "C" int rfx_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                            const int* page_table, int max_pages, int page_size,
                                            const int* row_pos, const int* row_slot, void* out, int R,
                                            int nq, int nkv, int head_dim, int n_splits, int window,
                                            float scale, void* stream) {
    if (R <= 0) return 0;
    if (n_splits < 1 || nq <= 0 || head_dim <= 0) return RFX_ERR_BAD_ARG;
    const long long need = (long long)R * nq * n_splits * (head_dim + 2);
    if (n_splits > 1 && need > (long long)RFX_NOALLOC_SCRATCH_FLOATS) return RFX_ERR_SCRATCH;
    float* scratch = nullptr;
    const int st = noalloc_scratch(&scratch);
    if (st != 0) return st;
    // every split writes its whole partial (empty splits write max = -inf, sum = 0)
    // before the combine reads it, so nothing in the array has to start at zero
    return rfx_attention_decode(q, k_pages, v_pages, page_table, max_pages, page_size, row_pos,
                                row_slot, out, scratch, R, nq, nkv, head_dim, n_splits, window, scale,
                                stream);
}
