// Decode attention with everything between the q/k/v product and the output
// product in one launch: per-head RMSNorm of q and k, rotary position encoding,
// the new key and value into the paged cache, attention over the cache, and the
// merge of the key-range splits.
//
// The reference's decode step runs these as separate kernels
// (src/model/decode_step.rs:232-311: norm pair, rope, kv store, attention,
// combine); at one token per sequence each of them is a few microseconds of
// launch and hand-off around almost no work, so here they are one.
//
// A CTA serves one (row, kv head, tile of up to 8 query heads of the group,
// split of the key range), as in attention_decode.cu.  The splits of one
// (row, kv head, tile) form a thread-block cluster: every rank sends its
// unnormalised partial (acc, max, sum) to the rank that owns that slice of the
// output over distributed shared memory, one cluster barrier, and each owner
// merges its slice in rank order and writes it.  No scratch in global memory,
// no second kernel.
//
// The rank whose key range ends at the row's own position makes the new key
// (norm, rotation) and value, writes them to the cache (the CTA of head tile 0
// only) and patches them into its shared-memory tile, so nothing is read back
// from global memory within the step.
//
// Formulas are those of qkv_post.cu (norm, rotation: src/kernels_cuda/
// decode_ops.cu:40-71, rope.cu:9-37) and attention_decode.cu (online softmax,
// src/kernels_cuda/attention_online.cu:51-78), evaluated in the same order, so
// the result equals the separate kernels' bit for bit given the same number of
// splits.
#include <cooperative_groups.h>

#include "attn_mma.cuh"
#include "common.cuh"
#include "paged.cuh"

namespace {

namespace cg = cooperative_groups;
using namespace attn;
using rfx::PagedKV;

constexpr int PAGE = 64;
constexpr int THREADS = 128;
constexpr int STAGES = 3;     // pages in flight per CTA
constexpr int MAX_RANKS = 8;  // portable cluster size

// Optional timeline for tuning: when a buffer is set (rfx_attention_fused_trace),
// thread 0 of each CTA stores %globaltimer at up to sixteen places; the last launch wins.
static __device__ unsigned long long* g_trace = nullptr;
static __device__ int g_trace_ctas = 0;
__device__ __forceinline__ void trace_mark(int which) {
    if (g_trace == nullptr || threadIdx.x != 0) return;
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (cta >= g_trace_ctas) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_trace[(size_t)cta * 16 + which] = t;
}

struct FusedArgs {
    const float* qkv;  // [R, row_stride]: q heads, then (nkv_in > 0) k heads, v heads
    int row_stride;
    int nkv_in;  // n_kv_heads when this run writes the cache, else 0 (q only)
    const float* q_w;
    const float* k_w;
    float eps, w_offset;
    const float* rope_denom;
    int rotary_dim;
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    PagedKV cache;
    const int* row_pos;
    const int* row_slot;
    __nv_bfloat16* out;
    int nq, n_htiles, n_splits, window;
    float scale_log2;
    int tile_heads;   // most query heads of a tile: min(16, group)
    int use_scratch;  // the rotation's pairs do not share a lane
};

// One warp: norm (optional; `w` holds this lane's weights) and rotation
// (optional) of one head vector `raw` (32-bit), result rounded to bfloat16 into `dst_s` (shared) and, if given,
// `dst_g` (global).  `scratch` holds D floats of this warp, or is null when
// half the rotation is a multiple of 32 elements (pairs then share a lane).
template <int D>
__device__ __forceinline__ void head_vector(const float (&raw)[(D + 31) / 32], bool has_w,
                                            const float (&w)[(D + 31) / 32], float eps,
                                            float w_offset, bool rotate, int rotary_dim,
                                            const float* cs_tab, const float* sn_tab, float* scratch,
                                            __nv_bfloat16* dst_s, __nv_bfloat16* dst_g, int lane) {
    constexpr int PER = (D + 31) / 32;
    float v[PER];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        v[i] = raw[i];
        ss = fmaf(v[i], v[i], ss);
    }
    if (has_w) {
        const float rinv = 1.0f / sqrtf(rfx::warp_sum(ss) / (float)D + eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) v[i] = (v[i] * rinv) * (w_offset + w[i]);
    }
    const int half = rotary_dim / 2;
    if (rotate && half > 0 && scratch == nullptr) {
        // half a rotation is a whole number of 32-element steps: the partner of
        // element (i, lane) is element (i +- half / 32, lane), in this lane
        const int hs = half >> 5;
        float u[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) u[i] = v[i];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * 32 + lane;
            if (e < rotary_dim) {
                const bool low = e < half;
                const int pi = low ? i + hs : i - hs;
                float other = 0.0f;
#pragma unroll
                for (int j = 0; j < PER; ++j)
                    if (j == pi) other = u[j];
                const int fi = low ? e : e - half;
                const float sn = sn_tab[fi], cs = cs_tab[fi];
                v[i] = low ? u[i] * cs - other * sn : other * sn + u[i] * cs;
            }
        }
    } else if (rotate && half > 0) {
        __syncwarp();
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * 32 + lane;
            if (e < D) scratch[e] = v[i];
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * 32 + lane;
            if (e < rotary_dim) {
                const int fi = e < half ? e : e - half;
                const float sn = sn_tab[fi], cs = cs_tab[fi];
                v[i] = e < half ? v[i] * cs - scratch[e + half] * sn : scratch[e - half] * sn + v[i] * cs;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        if (e < D) {
            const __nv_bfloat16 b = __float2bfloat16_rn(v[i]);
            dst_s[e] = b;
            if (dst_g) dst_g[e] = b;
        }
    }
}

template <int D>
__global__ void __launch_bounds__(THREADS) attention_decode_fused_kernel(const FusedArgs a) {
    constexpr int LD = D + 8;
    constexpr int PER = (D + 31) / 32;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [16][LD]
    __nv_bfloat16* kbuf = qs + 16 * LD;                               // [STAGES][PAGE][LD]
    __nv_bfloat16* vbuf = kbuf + STAGES * PAGE * LD;                  // [STAGES][PAGE][LD]
    __nv_bfloat16* knew = vbuf + STAGES * PAGE * LD;                  // [D]
    __nv_bfloat16* vnew = knew + D;                                   // [D]
    float* cs_tab = reinterpret_cast<float*>(vnew + D);               // [D / 2]
    float* sn_tab = cs_tab + D / 2;                                   // [D / 2]
    float* recv_m = sn_tab + D / 2;                                   // [ranks][16]
    float* recv_l = recv_m + MAX_RANKS * 16;                          // [ranks][16]
    float* recv_a = recv_l + MAX_RANKS * 16;                          // [ranks][slice] = heads of a tile x D
    float* scratch_all = recv_a + a.tile_heads * D;                   // [4][D], only if use_scratch

    trace_mark(0);
    rfx::pdl_launch_dependents();
    const PagedKV& cache = a.cache;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = blockIdx.x;
    const int kvh = blockIdx.y / a.n_htiles, ht = blockIdx.y % a.n_htiles;
    const int split = blockIdx.z, n_splits = a.n_splits;
    const int g = a.nq / cache.n_kv_heads;
    const int h0 = kvh * g + ht * 8;  // a tile holds up to eight query heads: the MMA's columns
    const int nh = min(8, g - ht * 8);
    const int pos = a.row_pos[r], slot = a.row_slot[r];
    const int window = a.window;
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_page = lo / PAGE, last_page = pos / PAGE;
    const int n_pg = last_page - first_page + 1;
    const int pps = (n_pg + n_splits - 1) / n_splits;
    const int pg0 = first_page + split * pps;
    const int pg1 = min(last_page + 1, pg0 + pps);
    const bool has_new = a.nkv_in > 0;                  // this run makes the row's key and value
    const bool tail = pg0 < pg1 && pg1 == last_page + 1;  // this rank's range ends at the row's position

    const int* table = cache.page_table + (size_t)slot * cache.max_pages;
    auto issue = [&](int pg, int page, int buf) {
        const size_t off = ((size_t)page * cache.n_kv_heads + kvh) * PAGE * D;
        // the row's own key and value do not come from global memory when this run makes them
        const int valid = min(PAGE, pos + (has_new ? 0 : 1) - pg * PAGE);
        load_tile_async<D>(kbuf + buf * PAGE * LD, a.k_pages + off, PAGE, valid, tid, THREADS);
        load_tile_async<D>(vbuf + buf * PAGE * LD, a.v_pages + off, PAGE, valid, tid, THREADS);
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

    int pages_first[STAGES];
#pragma unroll
    for (int i = 0; i < STAGES; ++i) pages_first[i] = pg0 + i < pg1 ? table[pg0 + i] : 0;
    // Pages before the one that holds the row's position were written by earlier
    // steps: their loads start before the wait on the preceding kernel.
    int issued = 0;
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (issued == i && pg0 + i < pg1 && pg0 + i < last_page) {
            issue(pg0 + i, pages_first[i], i);
            ++issued;
        }
    }
    // What does not depend on the preceding kernel, before the wait on it: the
    // rotation of this position, the norm weights, the zero rows of the query tile.
    const int half = a.rotary_dim / 2;
    const bool rotate = a.rope_denom != nullptr;
    if (rotate) {
        for (int i = tid; i < half; i += THREADS) {
            const float theta = (float)pos / a.rope_denom[i];
            sincosf(theta, &sn_tab[i], &cs_tab[i]);
        }
    }
    float wq[PER], wk[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        wq[i] = (a.q_w && e < D) ? a.q_w[e] : 0.0f;
        wk[i] = (a.k_w && e < D) ? a.k_w[e] : 0.0f;
    }
    for (int i = tid; i < (8 - nh) * (D / 8); i += THREADS) {
        const int rr = nh + i / (D / 8), c = i % (D / 8);
        *reinterpret_cast<uint4*>(qs + rr * LD + c * 8) = make_uint4(0, 0, 0, 0);
    }
    float* scratch = a.use_scratch ? scratch_all + warp * D : nullptr;

    // The loop's first pass is a dry one, still before the wait: it runs the
    // tile code on whatever the last ring buffer holds with every key masked, so
    // that the instructions are in the cache when the real pages come; its
    // results are thrown away.  Then the wait, this row's vectors, and the
    // real passes.
    int page_ahead = pages_first[STAGES - 1];
#pragma unroll 1
    for (int pg = pg0 - 1;;) {
        const bool dry = pg < pg0;
        const int buf = dry ? STAGES - 1 : (pg - pg0) % STAGES;
        if (!dry) {
            cp_async_wait<STAGES - 2>();  // page pg has landed (this thread's part)
            __syncthreads();              // everyone's part; and buffer (pg - 1) is free
            if (pg - pg0 < 4) trace_mark(8 + 2 * (pg - pg0));
            const int nxt = pg + STAGES - 1;
            const int page_now = page_ahead;
            if (nxt + 1 < pg1) page_ahead = table[nxt + 1];
            if (nxt < pg1) issue(nxt, page_now, (nxt - pg0) % STAGES);
            else cp_async_commit();
            if (has_new && pg == last_page) {  // the row's own key and value, made below
                const int rowi = pos - pg * PAGE;
                for (int i = tid; i < 2 * (D / 8); i += THREADS) {
                    const int c = i % (D / 8);
                    if (i < D / 8)
                        *reinterpret_cast<uint4*>(kbuf + (buf * PAGE + rowi) * LD + c * 8) =
                            *reinterpret_cast<const uint4*>(knew + c * 8);
                    else
                        *reinterpret_cast<uint4*>(vbuf + (buf * PAGE + rowi) * LD + c * 8) =
                            *reinterpret_cast<const uint4*>(vnew + c * 8);
                }
                __syncthreads();
            }
        }
        const int base = pg * PAGE;
        const int lo_eff = dry ? 0x7fffffff : lo;
        auto visible = [&](int key) { return base + key >= lo_eff && base + key <= pos; };
        attend_keys16<D>(qf, kbuf + buf * PAGE * LD, vbuf + buf * PAGE * LD, warp * 16, a.scale_log2, visible,
                         m, l, acc);
        if (!dry && pg - pg0 < 4) trace_mark(9 + 2 * (pg - pg0));
        if (dry) {
            m[0] = m[1] = -INFINITY;
            l[0] = l[1] = 0.0f;
#pragma unroll
            for (int n = 0; n < D / 16; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
            trace_mark(7);
            rfx::pdl_wait();
            trace_mark(1);

            // ---- this row's vectors: raw loads first, so their latency overlaps
            // tasks of the CTA: query heads 0 .. nh-1, then (tail rank) the key, the value
            const int n_tasks = nh + ((has_new && tail) ? 2 : 0);
            constexpr int MAX_T = 3;  // (8 + 2 + 3) / 4
            float raw[MAX_T][PER];
            const float* row = a.qkv + (size_t)r * a.row_stride;
#pragma unroll
            for (int j = 0; j < MAX_T; ++j) {
                const int t = warp + 4 * j;
                const float* src = row;
                if (t < nh) src += (size_t)(h0 + t) * D;
                else if (t == nh) src += (size_t)(a.nq + kvh) * D;
                else src += (size_t)(a.nq + a.nkv_in + kvh) * D;
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int e = i * 32 + lane;
                    raw[j][i] = (t < n_tasks && e < D) ? src[e] : 0.0f;
                }
            }
            __syncthreads();  // the rotation table
#pragma unroll
            for (int j = 0; j < MAX_T; ++j) {
                const int t = warp + 4 * j;
                if (t >= n_tasks) continue;
                if (t < nh) {
                    head_vector<D>(raw[j], a.q_w != nullptr, wq, a.eps, a.w_offset, rotate, a.rotary_dim,
                                   cs_tab, sn_tab, scratch, qs + t * LD, nullptr, lane);
                } else if (t == nh) {
                    __nv_bfloat16* dst = ht == 0 ? a.k_pages + rfx::kv_offset(cache, slot, pos, kvh) : nullptr;
                    head_vector<D>(raw[j], a.k_w != nullptr, wk, a.eps, a.w_offset, rotate, a.rotary_dim,
                                   cs_tab, sn_tab, scratch, knew, dst, lane);
                } else {
                    __nv_bfloat16* dst = ht == 0 ? a.v_pages + rfx::kv_offset(cache, slot, pos, kvh) : nullptr;
                    head_vector<D>(raw[j], false, wk, 0.0f, 0.0f, false, 0, cs_tab, sn_tab, scratch, vnew,
                                   dst, lane);
                }
            }
            // (the next pass's __syncthreads makes knew and vnew visible to all warps)
            __syncthreads();
            load_query_fragments<D>(qs, qf);
            trace_mark(2);
#pragma unroll
            for (int i = 0; i < STAGES - 1; ++i) {
                if (i >= issued) {
                    if (pg0 + i < pg1) issue(pg0 + i, pages_first[i], i);
                    else cp_async_commit();
                }
            }
        }
        ++pg;
        if (pg >= pg1) break;
    }
    cp_async_wait<0>();
    __syncthreads();  // all warps are done with the tiles (and, with no page, qs is complete)
    trace_mark(3);

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
    if (n_splits == 1) {
        for (int i = tid; i < total; i += THREADS) {
            const int rr = i / D, e = i % D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 8 + rr]);
            float L = 0.0f, A = 0.0f;
            if (M != -INFINITY) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float f = exp2f(red_m[w * 8 + rr] - M);
                    L += red_l[w * 8 + rr] * f;
                    A += red[(size_t)(w * 8 + rr) * D + e] * f;
                }
            }
            a.out[((size_t)r * a.nq + h0 + rr) * D + e] = __float2bfloat16_rn(A / L);
        }
        trace_mark(5);
        return;
    }

    // ---- the cluster's merge: element i of the tile's output belongs to rank
    // i / slice; every rank sends its partial there, and its (max, sum) to all.
    cg::cluster_group cluster = cg::this_cluster();
    const int slice = (total + n_splits - 1) / n_splits;
    for (int i = tid; i < total; i += THREADS) {
        const int rr = i / D, e = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 8 + rr]);
        float L = 0.0f, A = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(red_m[w * 8 + rr] - M);
                L += red_l[w * 8 + rr] * f;
                A += red[(size_t)(w * 8 + rr) * D + e] * f;
            }
        }
        const int owner = i / slice, off = i % slice;
        cluster.map_shared_rank(recv_a, owner)[(size_t)split * slice + off] = A;
        if (e == 0) {
            for (int dst = 0; dst < n_splits; ++dst) {
                cluster.map_shared_rank(recv_m, dst)[split * 16 + rr] = M;
                cluster.map_shared_rank(recv_l, dst)[split * 16 + rr] = L;
            }
        }
    }
    trace_mark(6);
    cluster.sync();  // every rank's stores have landed; no rank is read from after this
    trace_mark(4);
    for (int off = tid; off < slice; off += THREADS) {
        const int i = split * slice + off;
        if (i >= total) break;
        const int rr = i / D, e = i % D;
        float M = -INFINITY;
        for (int s = 0; s < n_splits; ++s) M = fmaxf(M, recv_m[s * 16 + rr]);
        float L = 0.0f, A = 0.0f;
        for (int s = 0; s < n_splits; ++s) {  // in rank order: the same bits every time
            const float ms = recv_m[s * 16 + rr];
            const float f = ms == -INFINITY ? 0.0f : exp2f(ms - M);
            L = __fadd_rn(L, __fmul_rn(recv_l[s * 16 + rr], f));  // product rounded, as the combine kernel's
            A += recv_a[(size_t)s * slice + off] * f;
        }
        const float inv = 1.0f / L;  // as attention_combine_kernel rounds it
        a.out[((size_t)r * a.nq + h0 + rr) * D + e] = __float2bfloat16_rn(A * inv);
    }
    trace_mark(5);
}

template <int D>
int launch_fused(const FusedArgs& a, int R, cudaStream_t s) {
    constexpr int LD = D + 8;
    size_t smem = (size_t)(16 + 2 * STAGES * PAGE) * LD * 2;  // q tile and the page ring
    const size_t red = (size_t)(4 * 16 * D + 2 * 4 * 16) * 4;
    if (red > (size_t)2 * STAGES * PAGE * LD * 2) return RFX_ERR_UNSUPPORTED;
    smem += (size_t)2 * D * 2;                                                    // new key, new value
    smem += (size_t)(D + 2 * MAX_RANKS * 16 + a.tile_heads * D) * 4;              // tables, receive area
    if (a.use_scratch) smem += (size_t)4 * D * 4;
    auto kernel = attention_decode_fused_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(R, a.cache.n_kv_heads * a.n_htiles, a.n_splits);
    e = rfx::launch(kernel, grid, dim3(THREADS), smem, s, a.n_splits, a);
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace

// Tuning aid: sixteen 64-bit timestamps per CTA of the launches that follow
// (null switches it off).
extern "C" int rfx_attention_fused_trace(void* buffer, int ctas) {
    unsigned long long* p = (unsigned long long*)buffer;
    cudaError_t e = cudaMemcpyToSymbol(g_trace, &p, sizeof(p));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_ctas, &ctas, sizeof(int));
    return (int)e;
}

// qkv: float32 [R, (nq + 2 nkv_in) * head_dim], the q/k/v product's rows (one
// query position per row); nkv_in = nkv when this run writes the cache, 0 when
// it only reads what an earlier run wrote (then qkv holds the q heads only).
// q_w, k_w: per-head norm weights or null; rope_denom: the rotation's
// denominators or null.  out: bfloat16 [R, nq, head_dim].  n_splits: 1, 2, 4
// or 8 ranks of a cluster over the key range.  head_dim: multiples of 16 up to
// 256; the page size must be 64.
extern "C" int rfx_attention_decode_fused(const float* qkv, int row_stride, int nkv_in, const float* q_w,
                                          const float* k_w, float eps, float w_offset,
                                          const float* rope_denom, int rotary_dim, void* k_pages,
                                          void* v_pages, const int* page_table, int max_pages,
                                          int page_size, const int* row_pos, const int* row_slot,
                                          void* out, int R, int nq, int nkv, int head_dim, int n_splits,
                                          int window, float scale, void* stream) {
    if (R <= 0) return 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0) return RFX_ERR_BAD_ARG;
    if (n_splits != 1 && n_splits != 2 && n_splits != 4 && n_splits != 8) return RFX_ERR_BAD_ARG;
    if (nkv_in != 0 && nkv_in != nkv) return RFX_ERR_BAD_ARG;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return RFX_ERR_BAD_ARG;
    if (row_stride < (nq + 2 * nkv_in) * head_dim) return RFX_ERR_BAD_ARG;
    if ((long long)nkv * ((nq / nkv + 7) / 8) > 65535) return RFX_ERR_UNSUPPORTED;
    FusedArgs a;
    a.qkv = qkv;
    a.row_stride = row_stride;
    a.nkv_in = nkv_in;
    a.q_w = q_w;
    a.k_w = k_w;
    a.eps = eps;
    a.w_offset = w_offset;
    a.rope_denom = rotary_dim > 0 ? rope_denom : nullptr;
    a.rotary_dim = rotary_dim;
    a.k_pages = (__nv_bfloat16*)k_pages;
    a.v_pages = (__nv_bfloat16*)v_pages;
    a.cache = PagedKV{page_table, max_pages, page_size, nkv, head_dim};
    a.row_pos = row_pos;
    a.row_slot = row_slot;
    a.out = (__nv_bfloat16*)out;
    a.nq = nq;
    a.n_htiles = (nq / nkv + 7) / 8;
    a.n_splits = n_splits;
    a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.tile_heads = nq / nkv < 8 ? nq / nkv : 8;
    a.use_scratch = (a.rope_denom != nullptr && (rotary_dim / 2) % 32 != 0) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_CASE(DD) \
    case DD:         \
        return launch_fused<DD>(a, R, s);
    switch (head_dim) {
        RFX_CASE(16) RFX_CASE(32) RFX_CASE(48) RFX_CASE(64) RFX_CASE(80) RFX_CASE(96)
        RFX_CASE(112) RFX_CASE(128) RFX_CASE(144) RFX_CASE(160) RFX_CASE(176) RFX_CASE(192)
        RFX_CASE(208) RFX_CASE(224) RFX_CASE(240) RFX_CASE(256)
        default:
            return RFX_ERR_UNSUPPORTED;
    }
#undef RFX_CASE
}
