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
//
// A page's key and value tiles come by TMA where the head size is a multiple
// of 64 and the caller says how many pages the store has: one thread issues
// D / 64 box loads per tile (128-byte swizzle, which the fragment loads undo)
// and a barrier counts the bytes.  Copying the same page in 16-byte pieces from
// all threads (the general form, any head size) costs about as many issue
// cycles as the page's tile code itself.
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <tuple>

#include "attn_mma.cuh"
#include "common.cuh"
#include "noalloc.h"
#include "paged.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

namespace {

namespace cg = cooperative_groups;
using namespace attn;
using rfx::PagedKV;

// Optional timeline for tuning: when a buffer is set (rfx_attention_decode_trace),
// thread 0 of every CTA stores %globaltimer at chosen moments of its life in the
// record of its launch: 0 entry, 1 the kernel before is done, 2 query rows loaded,
// 3 last page done, 4 the warps merged, 5 past the cluster's barrier, 6 exit;
// slots 7 to 9 are not times but cycles of thread 0: spent waiting for pages to
// land, issuing the loads of later pages, and in the tile code.
struct DecTraceRec {
    unsigned long long t[12];
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

__device__ __forceinline__ void dtrace_value(int launch, int which, long long v) {
    if (g_dtrace == nullptr || launch >= g_dtrace_launches || threadIdx.x != 0) return;
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta >= g_dtrace_ctas) return;
    g_dtrace[(size_t)launch * g_dtrace_ctas + cta].t[which] = (unsigned long long)v;
}

constexpr int PAGE = 64;
constexpr int DEC_THREADS = 128;
constexpr int DEC_STAGES = 3;  // pages in flight per CTA
constexpr int MAX_RANKS = 16;  // 8 is the portable cluster size; 16 where the device places one

// TMA: the page tiles come by tensor-map loads (D a multiple of 64) and lie
// swizzled, [D / 64][PAGE][64]; else by 16-byte copies into padded rows.
template <int D, bool TMA>
__global__ void __launch_bounds__(DEC_THREADS + 32)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, PagedKV cache,
                        const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int nq,
                        int n_htiles, int n_splits, int window, float scale_log2, int cluster_merge,
                        int trace_id, int* __restrict__ err) {
    constexpr int LD = D + 8;
    constexpr int TILE = TMA ? PAGE * D : PAGE * LD;  // elements of a page's key (or value) tile
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // the tiles first (1024-byte aligned for the swizzled form), then the query rows
    uint8_t* tiles = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                      ~(uintptr_t)1023)
                         : smem_raw;
    __nv_bfloat16* kbuf = reinterpret_cast<__nv_bfloat16*>(tiles);  // [STAGES] tiles
    __nv_bfloat16* vbuf = kbuf + DEC_STAGES * TILE;                  // [STAGES] tiles
    __nv_bfloat16* qs = vbuf + DEC_STAGES * TILE;                    // [16][LD], rows 0..7 used
    // with the splits merged inside a cluster: what the other ranks send
    float* recv_m = reinterpret_cast<float*>(qs + 16 * LD);  // [ranks][16]
    float* recv_l = recv_m + MAX_RANKS * 16;                 // [ranks][16]
    float* recv_a = recv_l + MAX_RANKS * 16;                 // [ranks][slice]
    __shared__ __align__(8) uint64_t full_bar[DEC_STAGES];   // TMA: a stage's bytes have landed
    __shared__ __align__(8) uint64_t empty_bar[DEC_STAGES];  // TMA: the four warps are done with the stage
    constexpr int NT = TMA ? DEC_THREADS + 32 : DEC_THREADS;  // TMA: a fifth warp that issues the loads

    rfx::pdl_launch_dependents();
    if (TMA) {
        if (threadIdx.x == 0) {
            for (int i = 0; i < DEC_STAGES; ++i) {
                sm100::mbar_init(&full_bar[i], 1);
                sm100::mbar_init(&empty_bar[i], 4);
            }
            sm100::fence_barrier_init();
            sm100::prefetch_tensormap(&map_k);
            sm100::prefetch_tensormap(&map_v);
        }
        __syncthreads();
    }
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
        if constexpr (TMA) {
            if (tid == DEC_THREADS) {
                // the buffer's last readers were ordinary loads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                const int y = (page * cache.n_kv_heads + kvh) * PAGE;  // the tile's first row in the store
                sm100::mbar_expect_tx(&full_bar[buf], 2 * TILE * 2);
#pragma unroll
                for (int kb = 0; kb < D / 64; ++kb) {
                    sm100::tma_load_2d(kbuf + buf * TILE + kb * PAGE * 64, &map_k, &full_bar[buf], kb * 64, y);
                    sm100::tma_load_2d(vbuf + buf * TILE + kb * PAGE * 64, &map_v, &full_bar[buf], kb * 64, y);
                }
            }
        } else {
            const size_t off = ((size_t)page * cache.n_kv_heads + kvh) * PAGE * D;
            const int valid = min(PAGE, pos + 1 - pg * PAGE);
            load_tile_async<D>(kbuf + buf * TILE, k_pages + off, PAGE, valid, tid, DEC_THREADS);
            load_tile_async<D>(vbuf + buf * TILE, v_pages + off, PAGE, valid, tid, DEC_THREADS);
            cp_async_commit();
        }
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

    // a ring of DEC_STAGES pages (16-byte copies: one commit group per page, empty
    // groups past the end; TMA: a barrier per stage).  The page id of a load is read
    // one iteration before the load is issued, so the page-table read never stalls
    // the loop.
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
    // First a dry pass, still before the wait: the tile code runs on whatever the
    // last ring buffer holds with every key masked, so that the instructions are in
    // the cache when the real pages come; its results are thrown away.  Then the
    // wait, the query rows, and the real passes.
    const bool tracing = g_dtrace != nullptr && tid == 0;
    long long waited = 0, issuing = 0, attending = 0;
    auto reset = [&]() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.0f;
#pragma unroll
        for (int n = 0; n < D / 16; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    };
    if constexpr (TMA) {
        // Four warps walk the pages, each at its own pace; a fifth one only issues the
        // loads.  A page's barrier says its bytes have landed, a buffer's second barrier
        // that the four warps are done with it; nothing else orders them page by page.
        if (warp < 4) {
            auto nothing = [&](int) { return false; };
            attend_keys16<D, true>(qf, kbuf + (DEC_STAGES - 1) * TILE, vbuf + (DEC_STAGES - 1) * TILE, warp * 16,
                                   scale_log2, nothing, m, l, acc);
            reset();
            // the dry pass is this buffer's first use: done with it
            __syncwarp();
            if (lane == 0) sm100::mbar_arrive(&empty_bar[DEC_STAGES - 1]);
        }
        rfx::pdl_wait();
        dtrace_mark(trace_id, 1);
        if (warp == 4) {
            if (lane == 0) {
                // the pages that had to wait for the kernel before (the one with this row's
                // own position), then the rest as their buffers come free
#pragma unroll
                for (int i = 0; i < DEC_STAGES - 1; ++i)
                    if (i >= issued && pg0 + i < pg1) issue(pg0 + i, pages_first[i], i);
                int pg = pg0 + DEC_STAGES - 1;
                int page_next = pg < pg1 ? table[pg] : 0;
                for (; pg < pg1; ++pg) {
                    const int i = pg - pg0, buf = i % DEC_STAGES;
                    const int page = page_next;
                    if (pg + 1 < pg1) page_next = table[pg + 1];
                    // the four warps are done with what the buffer held: the page before
                    // this one in it, or, in the last buffer, the dry pass first
                    const int uses = i / DEC_STAGES + (buf == DEC_STAGES - 1 ? 1 : 0);  // of the buffer so far
                    if (uses > 0 && !sm100::mbar_wait(&empty_bar[buf], (uint32_t)((uses - 1) & 1)) && err)
                        atomicExch(err, 32);
                    issue(pg, page, buf);
                }
            }
            __syncwarp();
        } else {
            // the query heads of this tile; rows beyond the group are zero
            asm volatile("bar.sync 1, 128;" ::: "memory");  // every walking warp has read the query tile
            for (int i = tid; i < 8 * (D / 8); i += DEC_THREADS) {
                const int row = i / (D / 8), c = i % (D / 8);
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row < nh) v = *reinterpret_cast<const uint4*>(q + ((size_t)r * nq + h0 + row) * D + c * 8);
                *reinterpret_cast<uint4*>(qs + row * LD + c * 8) = v;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            load_query_fragments<D>(qs, qf);
            dtrace_mark(trace_id, 2);
#pragma unroll 1
            for (int pg = pg0; pg < pg1; ++pg) {
                const int i = pg - pg0, buf = i % DEC_STAGES;
                const long long c0 = tracing ? clock64() : 0;
                // page pg has landed; a wait that runs out is reported and the walk goes on
                if (!sm100::mbar_wait(&full_bar[buf], (uint32_t)((i / DEC_STAGES) & 1)) && err) atomicExch(err, 31);
                // The whole page came, rows past the sequence's end too, which nothing ever
                // wrote: zero those value rows, since 0 * NaN is not 0 (their keys are masked)
                const int valid = pos + 1 - pg * PAGE;
                if (valid < PAGE) {
                    __nv_bfloat16* vt = vbuf + buf * TILE;
                    for (int e = tid; e < (PAGE - valid) * (D / 8); e += DEC_THREADS) {
                        const int row = valid + e / (D / 8), c = e % (D / 8);
                        *reinterpret_cast<uint4*>(vt + (c / 8) * PAGE * 64 + row * 64 + (c % 8) * 8) =
                            make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four walking warps
                }
                const long long c2 = tracing ? clock64() : 0;
                if (tracing) waited += c2 - c0;
                const int base = pg * PAGE;
                auto visible = [&](int key) { return base + key >= lo && base + key <= pos; };
                attend_keys16<D, true>(qf, kbuf + buf * TILE, vbuf + buf * TILE, warp * 16, scale_log2, visible, m,
                                       l, acc);
                __syncwarp();
                if (lane == 0) sm100::mbar_arrive(&empty_bar[buf]);
                if (tracing) attending += clock64() - c2;
            }
        }
    } else {
        int page_ahead = pages_first[DEC_STAGES - 1];
#pragma unroll 1
        for (int pg = pg0 - 1;;) {
            const bool dry = pg < pg0;
            const int buf = dry ? DEC_STAGES - 1 : (pg - pg0) % DEC_STAGES;
            if (!dry) {
                const long long c0 = tracing ? clock64() : 0;
                cp_async_wait<DEC_STAGES - 2>();  // page pg has landed (this thread's part)
                __syncthreads();                  // everyone's part; and buffer (pg - 1) is free
                const long long c1 = tracing ? clock64() : 0;
                if (tracing) waited += c1 - c0;
                const int nxt = pg + DEC_STAGES - 1;
                const int page_now = page_ahead;
                if (nxt + 1 < pg1) page_ahead = table[nxt + 1];
                if (nxt < pg1) issue(nxt, page_now, (nxt - pg0) % DEC_STAGES);
                else cp_async_commit();
                if (tracing) issuing += clock64() - c1;
            }
            const long long c2 = tracing ? clock64() : 0;
            const int base = pg * PAGE;
            const int lo_eff = dry ? 0x7fffffff : lo;
            auto visible = [&](int key) { return base + key >= lo_eff && base + key <= pos; };
            attend_keys16<D, false>(qf, kbuf + buf * TILE, vbuf + buf * TILE, warp * 16, scale_log2, visible, m, l,
                                    acc);
            if (tracing && !dry) attending += clock64() - c2;
            if (dry) {
                reset();
                // After the wait on the kernel before: first the loads of the pages that had
                // to wait for it (the one with this row's own position), then the query rows,
                // whose latency those loads then cover.
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
    }
    __syncthreads();  // all warps are done with the tiles before they are reused below
    dtrace_mark(trace_id, 3);
    if (tracing) {
        dtrace_value(trace_id, 7, waited);
        dtrace_value(trace_id, 8, issuing);
        dtrace_value(trace_id, 9, attending);
    }

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
    if (warp < 4) {
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
    for (int i = tid; i < total; i += NT) {
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
        for (int off = tid; off < slice; off += NT) {
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

// Tensor maps of a key or value store, made once per (pointer, pages).
const CUtensorMap* store_map(const void* base, long long rows, int D) {
    struct Key {
        const void* p;
        long long rows;
        int d;
        bool operator<(const Key& o) const { return std::tie(p, rows, d) < std::tie(o.p, o.rows, o.d); }
    };
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{base, rows, D};
    auto it = cache.find(key);
    if (it != cache.end()) return &it->second;
    CUtensorMap m;
    if (!rfx::tma::make_map_rows64(&m, base, rows, D, PAGE)) return nullptr;
    return &cache.emplace(key, m).first->second;
}

template <int D, bool TMA>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, long long pool_pages,
                  const PagedKV& cache, const int* row_pos, const int* row_slot, void* out, float* partial,
                  int R, int nq, int n_splits, int window, float scale, int cluster_merge, int* err,
                  cudaStream_t s) {
    constexpr int LD = D + 8;
    const int g = nq / cache.n_kv_heads;
    const int n_htiles = (g + 7) / 8;
    const int tile_heads = g < 8 ? g : 8;
    const size_t ring = (size_t)2 * DEC_STAGES * PAGE * (TMA ? D : LD) * 2;
    size_t smem = ring + (size_t)16 * LD * 2 + (TMA ? 1024 : 0);
    const size_t red = (size_t)(4 * 16 * D + 2 * 4 * 16) * 4;
    if (red > ring) return RFX_ERR_UNSUPPORTED;
    if (cluster_merge) smem += (size_t)(2 * MAX_RANKS * 16 + tile_heads * D) * 4;
    if (smem > 227 * 1024) return RFX_ERR_UNSUPPORTED;
    CUtensorMap none{};
    const CUtensorMap *mk = &none, *mv = &none;
    if (TMA) {
        const long long rows = pool_pages * cache.n_kv_heads * PAGE;
        mk = store_map(k_pages, rows, D);
        mv = store_map(v_pages, rows, D);
        if (!mk || !mv) return RFX_ERR_UNSUPPORTED;
    }
    auto kernel = attention_decode_kernel<D, TMA>;
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
                cfg.blockDim = dim3(TMA ? DEC_THREADS + 32 : DEC_THREADS);
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
    e = rfx::launch(kernel, grid, dim3(TMA ? DEC_THREADS + 32 : DEC_THREADS), smem, s,
                    cluster_merge ? n_splits : 1, *mk, *mv,
                    (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                    cache, row_pos, row_slot, (__nv_bfloat16*)out, partial, nq, n_htiles, n_splits, window,
                    scale * 1.4426950408889634f, cluster_merge, g_dtrace_next++, err);
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1 && !cluster_merge)
        RFX_LAUNCH(attention_combine_kernel, R * nq, D <= 128 ? 64 : 128, 0, s, (const float*)partial,
                   (__nv_bfloat16*)out, D, n_splits);
    return 0;
}

int decode_entry(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                 int max_pages, int page_size, const int* row_pos, const int* row_slot, void* out,
                 float* partial, int R, int nq, int nkv, int head_dim, int n_splits, int window,
                 float scale, int cluster_merge, long long pool_pages, int* err, void* stream) {
    if (R <= 0) return 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0 || n_splits < 1) return RFX_ERR_BAD_ARG;
    if (n_splits > 1 && !partial && !cluster_merge) return RFX_ERR_BAD_ARG;
    if (cluster_merge && n_splits != 2 && n_splits != 4 && n_splits != 8 && n_splits != 16) return RFX_ERR_UNSUPPORTED;
    if (n_splits > MAX_SPLITS) return RFX_ERR_UNSUPPORTED;
    if (n_splits > 65535 || (long long)nkv * ((nq / nkv + 7) / 8) > 65535) return RFX_ERR_UNSUPPORTED;
    PagedKV cache{page_table, max_pages, page_size, nkv, head_dim};
    cudaStream_t s = (cudaStream_t)stream;
    // page tiles by TMA: head sizes that are whole 64-column boxes, a store whose
    // size the caller gave, 16-byte aligned (REFLEX_B200_DECODE_TMA=0: a tuning aid)
    static const bool tma_on = [] {
        const char* e = getenv("REFLEX_B200_DECODE_TMA");
        return !(e && e[0] == '0');
    }();
    const bool tma = tma_on && pool_pages > 0 && head_dim % 64 == 0 &&
                     ((reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0 &&
                     pool_pages * nkv * PAGE < 2147483647LL;
#define RFX_GO(DD, T)                                                                                     \
    launch_decode<DD, T>(q, k_pages, v_pages, pool_pages, cache, row_pos, row_slot, out, partial, R, nq, \
                         n_splits, window, scale, cluster_merge, err, s)
#define RFX_CASE(DD)                                        \
    case DD:                                                \
        if (DD % 64 == 0 && tma) {                          \
            const int st = RFX_GO(DD, (DD % 64 == 0));      \
            if (st != RFX_ERR_UNSUPPORTED) return st;       \
        }                                                   \
        return RFX_GO(DD, false);
    switch (head_dim) {
        RFX_CASE(16) RFX_CASE(32) RFX_CASE(48) RFX_CASE(64) RFX_CASE(80) RFX_CASE(96)
        RFX_CASE(112) RFX_CASE(128) RFX_CASE(144) RFX_CASE(160) RFX_CASE(176) RFX_CASE(192)
        RFX_CASE(208) RFX_CASE(224) RFX_CASE(240) RFX_CASE(256)
        default:
            return RFX_ERR_UNSUPPORTED;
    }
#undef RFX_CASE
#undef RFX_GO
}

}  // namespace

// bfloat16 q [R, nq, D], paged K/V, one query position per row.  `partial` is
// scratch of R * nq * n_splits * (D + 2) floats, needed when n_splits > 1.
// head_dim: multiples of 16 up to 256; the page size must be 64.
// `pool_pages`: pages of the key (and value) store that `k_pages` points to, if the
// caller knows (else 0): with it, head sizes 64, 128, 192 and 256 take their pages by
// TMA.  `err` (may be null): a device word that receives a non-zero code if a bounded
// wait ran out.
extern "C" int rfx_attention_decode(const void* q, const void* k_pages, const void* v_pages,
                                    const int* page_table, int max_pages, int page_size,
                                    const int* row_pos, const int* row_slot, void* out,
                                    float* partial, int R, int nq, int nkv, int head_dim,
                                    int n_splits, int window, float scale, long long pool_pages,
                                    int* err, void* stream) {
    return decode_entry(q, k_pages, v_pages, page_table, max_pages, page_size, row_pos, row_slot, out,
                        partial, R, nq, nkv, head_dim, n_splits, window, scale, 0, pool_pages, err, stream);
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
                                            float scale, long long pool_pages, int* err, void* stream) {
    return decode_entry(q, k_pages, v_pages, page_table, max_pages, page_size, row_pos, row_slot, out,
                        nullptr, R, nq, nkv, head_dim, n_splits, window, scale, 1, pool_pages, err, stream);
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
// records of twelve 64-bit words (time stamps and cycle counts); the next launch writes record 0.  Null turns
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
                                0, nullptr, stream);
}
