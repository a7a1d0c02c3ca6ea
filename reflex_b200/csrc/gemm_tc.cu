// Tensor-core matrix product for the bfloat16 path:  y[r, n] = sum_k x[r, k] W[n, k].
//
// The weight matrix is the M operand of tcgen05.mma (tiles of 128 weight rows),
// the activation rows are its N operand (16 .. 256 rows a tile), so that a
// decode step's few rows still fill the 128-lane datapath and every weight
// byte is read from HBM exactly once.  Per CTA: one warp issues TMA tile loads
// (128-byte swizzle) into a ring of shared-memory stages, one thread issues the
// MMAs with the accumulator in tensor memory, four warps read the accumulator
// back and store.  With few weight-row tiles the K dimension is split over a
// thread-block cluster of up to 8 CTAs so that all SMs stream weights; the
// partial sums are reduced through distributed shared memory in rank order
// (no scratch in global memory, no atomics, a fixed summation order).
//
// It replaces the reference's warp-per-row f16 GEMV for decode
// (src/kernels_cuda/gemv_f16.cuh:23-69, gemv_fused.cu) and can stand in for
// the library product in prefill.  Every wait on an mbarrier is bounded: when
// it runs out the kernel records where, stops issuing, still frees its tensor
// memory and returns.
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "paged.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

namespace cg = cooperative_groups;

namespace {

using namespace sm100;

constexpr int BM = 128;        // weight rows per tile (MMA M)
constexpr int BK = 64;         // elements along K per stage: 128 bytes of bfloat16
constexpr int MAX_STAGES = 12;
constexpr int THREADS = 192;   // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue
constexpr int A_STAGE_BYTES = BM * BK * 2;

// Optional timeline for tuning: when a buffer is set (rfx_gemm_trace), thread 0 of
// every CTA stores %globaltimer at entry, after the dependency wait, when the
// accumulator is complete and at exit, in the record of its launch.
struct TraceRec {
    unsigned long long t[8];
};
static __device__ TraceRec* g_trace = nullptr;
static __device__ int g_trace_ctas = 0;   // records per launch
static __device__ int g_trace_launches = 0;
__device__ __forceinline__ void trace_mark(int launch, int which) {
    if (g_trace == nullptr || launch >= g_trace_launches) return;
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta >= g_trace_ctas) return;
    g_trace[(size_t)launch * g_trace_ctas + cta].t[which] = global_timer_ns();
}

template <int BN>
struct Shape {
    static constexpr int B_STAGE_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
};

// What the epilogue does besides storing, for the fused decode path:
//  * scale_rows (PRO): the activation rows came in unnormalised (x = h * w_norm,
//    rounded to bfloat16); row r of the result is multiplied by
//    1 / sqrt(sum_p ssq_in[r][p] / H + eps), the RMSNorm factor, which commutes
//    with the product.  The partial sums of squares come from the product that
//    made h (below).
//  * EPI 2: the result is a delta of the residual stream: h[r, n] += acc (32-bit,
//    each element by one thread), hb[r, n] = bfloat16(h * (nw_offset + nw[n])) is
//    the next product's unnormalised input, and ssq_out[r][p] = sum of h^2 over
//    this CTA's rows n is one partial of the next norm's statistic.
// Together they replace the separate add + RMSNorm launch between two products
// (src/kernels_cuda/decode_ops.cu:10-35 is the reference's fused add + norm).
struct Fuse {
    const float* ssq_in;   // [R][n_part_in]
    int n_part_in;
    float inv_h, eps;
    float* h;              // [R, N] residual stream, updated in place
    const float* nw;       // [N] weight of the norm that follows
    float nw_offset;
    __nv_bfloat16* hb;     // [R, N]
    float* ssq_out;        // [R][tiles * ksplit]
    // EPI 3 (below): the q/k/v product of a decode step, finished per head
    const float* q_w;      // per-head norm weights [head_dim]; null: no per-head norm
    const float* k_w;
    float qk_eps, qk_offset;
    const float* rope_denom;  // [head_dim / 2] angle denominators; null: no rotation
    float magnitude;
    const int* row_pos;    // [R]
    const int* row_slot;   // [R]
    __nv_bfloat16* q_out;  // [R, nq * head_dim]
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    rfx::PagedKV cache;
    int nq, nkv_in, head_dim;
};

//  * EPI 3: W is the stacked q/k/v matrix of an attention layer whose head size
//    is 64 or 128, so a 128-row tile holds whole heads.  The split-K partials are
//    exchanged by activation row instead of by weight row: each rank of the
//    cluster ends up with complete head vectors for its share of the rows and
//    finishes them there: per-head RMSNorm of q and k, rotary encoding over the
//    whole head (half-split pairs), q to the workspace, k and v into the paged
//    cache at the row's position.  One launch instead of product + `qkv_post`,
//    and the 32-bit q/k/v rows never go to memory.  Formulas as in qkv_post.cu.

// EPI 0: y = x W^T.  EPI 1: W's rows alternate gate, up (row 2j gate_j, row 2j+1
// up_j) and y[r, j] = silu(gate_j) * up_j, so the SwiGLU activation costs no
// launch and no round trip of the [R, 2I] intermediate
// (src/kernels_cuda/silu_and_mul.cu:7-23 is the reference's separate kernel).
using rfx::silu_mul;
using rfx::silu_mul_for;

using rfx::store2;
using rfx::store4;

// One head vector of a row, spread over a warp (lane l holds elements l, l + 32,
// ...): per-head norm, rotation, store.  `rot`: this row's (cos, sin) pairs;
// `w`: the lane's norm weights (offset added), null for no norm.
template <int D>
__device__ __forceinline__ void finish_head(float* hv, bool rotate_it, const float* w, const float* rot,
                                            float eps, __nv_bfloat16* dst, int lane) {
    constexpr int EPL = D / 32;  // elements per lane
    if (w != nullptr) {
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss = fmaf(hv[i], hv[i], ss);
        ss = rfx::warp_sum(ss);
        const float rinv = 1.0f / sqrtf(ss * (1.0f / (float)D) + eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i) hv[i] = (hv[i] * rinv) * w[i];
    }
    if (rotate_it) {
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) {  // the pair (e, e + D / 2) lies in this lane
            const float2 cs = *reinterpret_cast<const float2*>(rot + 2 * (lane + 32 * i));
            const float lo = hv[i], hi = hv[i + EPL / 2];
            hv[i] = fmaf(hi, -cs.y, lo * cs.x);
            hv[i + EPL / 2] = fmaf(lo, cs.y, hi * cs.x);
        }
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(hv[i]);
}

// The epilogue of EPI 3, run by the four epilogue warps (threads 64 .. 191).
// recv: [BN][BM] floats that receive partial head vectors, by (source rank, row);
// rot: [rows of this rank][head_dim / 2] (cos, sin) pairs, then per row its place
// in the cache.  Everything that does not need the accumulator (the rows'
// rotation, their places in the cache, the lane's norm weights) is made while
// the main loop still runs: positions, slots and the page table are the step's
// inputs, no other kernel's output.
template <int BN, bool PRO>
__device__ __forceinline__ void head_epilogue(float* recv, float* rot, uint32_t tmem_d, uint64_t* tmem_full_bar,
                                              bool have, int ksplit, int z, int r0, int R, const Fuse& f,
                                              const float* rstd_s, int* err, int trace_id) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q4 = warp & 3, m = q4 * 32 + lane, et = threadIdx.x - 64, ew = warp - 2;
    const int D = f.head_dim, half = D / 2;
    const int cw = BN / ksplit;  // activation rows each rank finishes (ksplit divides BN)
    const bool rotate = f.rope_denom != nullptr;
    unsigned long long* place = reinterpret_cast<unsigned long long*>(rot + (size_t)cw * D);  // [cw]
    if (rotate) {
        for (int e = et; e < cw * half; e += 128) {
            const int cl = e / half, i = e - cl * half, r = r0 + z * cw + cl;
            float sv = 0.0f, cv = 1.0f;
            if (r < R) {
                sincosf((float)f.row_pos[r] / f.rope_denom[i], &sv, &cv);  // as qkv_post's bfloat16 forms
                sv *= f.magnitude;
                cv *= f.magnitude;
            }
            rot[2 * e] = cv;
            rot[2 * e + 1] = sv;
        }
    }
    if (et < cw) {
        const int r = r0 + z * cw + et;
        unsigned long long off = 0;
        if (r < R && f.nkv_in > 0) off = rfx::kv_offset(f.cache, f.row_slot[r], f.row_pos[r], 0);
        place[et] = off;  // kv head 0's place; the others lie a (page, head) tile apart
    }
    // this tile's heads and the lane's norm weights for them
    const int n_heads = f.nq + 2 * f.nkv_in;
    const int hpt = BM / D;
    int kind[2] = {3, 3};
    float wv[4] = {1.0f, 1.0f, 1.0f, 1.0f};
    bool normed[2] = {false, false};
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
        const int head = blockIdx.x * hpt + hi;
        if (hi < hpt && head < n_heads) {
            kind[hi] = head < f.nq ? 0 : (head < f.nq + f.nkv_in ? 1 : 2);
            const float* w = kind[hi] == 0 ? f.q_w : (kind[hi] == 1 ? f.k_w : nullptr);
            if (w != nullptr) {
                normed[hi] = true;
                if (D == 128) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) wv[i] = f.qk_offset + w[lane + 32 * i];
                } else {
                    wv[2 * hi] = f.qk_offset + w[lane];
                    wv[2 * hi + 1] = f.qk_offset + w[lane + 32];
                }
            }
        }
    }
    if (have && !mbar_wait(tmem_full_bar, 0)) {
        if (lane == 0) atomicExch(err, 3);
        have = false;
    }
    tc_fence_after_sync();
    if (warp == 2 && lane == 0) trace_mark(trace_id, 2);
    // Row m of the tile, for every activation row (column of the accumulator): to
    // the rank that finishes that activation row, slot [this rank][row][m].
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t lane_base = tmem_d + ((uint32_t)(q4 * 32) << 16);
    uint32_t ahead[16];
    if (have) tmem_ld_16_nowait(lane_base, ahead);
#pragma unroll 1
    for (int c = 0; c < BN / 16; ++c) {
        float v[16];
        if (have) {
            tmem_ld_wait_16(ahead);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(ahead[j]);
            if (c + 1 < BN / 16) tmem_ld_16_nowait(lane_base + (uint32_t)((c + 1) * 16), ahead);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int col = c * 16 + j, owner = col / cw, cl = col - owner * cw;
            if (r0 + col < R) {  // rows past the batch are nobody's
                float* base = ksplit > 1 ? cluster.map_shared_rank(recv, owner) : recv;
                base[(size_t)(z * cw + cl) * BM + m] = v[j];
            }
        }
    }
    tc_fence_before_sync();
    if (ksplit > 1) cluster.sync();
    else asm volatile("bar.sync 1, 128;" ::: "memory");
    // A warp finishes a row at a time: the ranks' partials summed in rank order.
    const size_t kv_head_stride = (size_t)f.cache.page_size * D;
    for (int cl = ew; cl < cw; cl += 4) {
        const int col = z * cw + cl, r = r0 + col;
        if (r >= R) continue;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int p = 0; p < ksplit; ++p) {
            const float* src = recv + (size_t)(p * cw + cl) * BM + lane;
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] += src[32 * i];
        }
        if (PRO) {
            const float fr = rstd_s[col];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] *= fr;
        }
        const float* rrow = rot + (size_t)2 * cl * half;
        const size_t kv0 = (size_t)place[cl];
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            if (kind[hi] > 2) continue;
            const int head = blockIdx.x * hpt + hi;
            __nv_bfloat16* dst;
            if (kind[hi] == 0) dst = f.q_out + ((size_t)r * f.nq + head) * D;
            else if (kind[hi] == 1) dst = f.k_pages + kv0 + (size_t)(head - f.nq) * kv_head_stride;
            else dst = f.v_pages + kv0 + (size_t)(head - f.nq - f.nkv_in) * kv_head_stride;
            const bool rot_it = rotate && kind[hi] < 2;
            if (D == 128) finish_head<128>(v, rot_it, normed[hi] ? wv : nullptr, rrow, f.qk_eps, dst, lane);
            else finish_head<64>(v + 2 * hi, rot_it, normed[hi] ? wv + 2 * hi : nullptr, rrow, f.qk_eps, dst, lane);
        }
    }
}

template <int BN, typename TO, int EPI, bool PRO>
__global__ void __launch_bounds__(THREADS)
gemm_wt_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               TO* __restrict__ y, int R, int N, int K, int ksplit, int stages, int bm,
               int l2_ahead, int trace_id, Fuse fuse, int* __restrict__ err) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ float red_s[128];
    __shared__ float rstd_s[BN];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t tmem_full_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    using S = Shape<BN>;
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) trace_mark(trace_id, 0);
    // a tile is `bm` <= 128 weight rows: the MMA always spans 128 rows of shared
    // memory, rows past bm hold whatever was there and give output rows nobody reads
    const int n0 = blockIdx.x * bm, r0 = blockIdx.y * BN, z = blockIdx.z;
    const uint32_t stage_tx = (uint32_t)bm * BK * 2 + S::B_STAGE_BYTES;
    const int num_kb = (K + BK - 1) / BK;
    const int per = (num_kb + ksplit - 1) / ksplit;
    const int kb0 = z * per;
    const int nkb = max(0, min(num_kb, kb0 + per) - kb0);
    // rows of the tile that each rank of a K-split cluster finishes
    const int mw = (EPI == 1) ? ((((bm + ksplit - 1) / ksplit) + 1) & ~1) : (bm + ksplit - 1) / ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&tmem_full_bar, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, S::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_d = tmem_base_smem;

    // Let the next kernel's CTAs start as soon as every CTA of this one runs.
    rfx::pdl_launch_dependents();

    if (warp == 0) {
        if (elect_one()) {
            // The weights do not depend on the kernel before this one: fill the
            // ring with weight tiles first, then wait for that kernel, then add
            // the activation tiles.  HBM keeps streaming across the launch.
            const int pre = min(nkb, stages);
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&full_bar[i], stage_tx);
                tma_load_2d(tiles + (size_t)i * S::STAGE_BYTES, &map_w, &full_bar[i], (kb0 + i) * BK, n0);
            }
            // ... and while still waiting, pull the next weight tiles into L2: the
            // kernels before this one leave HBM idle for microseconds at a time
            const int ahead = min(nkb, pre + l2_ahead);
            for (int i = pre; i < ahead; ++i) tma_prefetch_l2_2d(&map_w, (kb0 + i) * BK, n0);
            rfx::pdl_wait();
            trace_mark(trace_id, 1);
            for (int i = 0; i < pre; ++i)
                tma_load_2d(tiles + (size_t)i * S::STAGE_BYTES + A_STAGE_BYTES, &map_x, &full_bar[i],
                            (kb0 + i) * BK, r0);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % stages;
                const uint32_t ph = (i / stages) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
                    atomicExch(err, 1);
                    abort_flag = 1;
                    break;
                }
                uint8_t* a = tiles + (size_t)s * S::STAGE_BYTES;
                uint8_t* b = a + A_STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], stage_tx);
                tma_load_2d(a, &map_w, &full_bar[s], (kb0 + i) * BK, n0);
                tma_load_2d(b, &map_x, &full_bar[s], (kb0 + i) * BK, r0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % stages;
                const uint32_t ph = (i / stages) & 1;
                if (!mbar_wait(&full_bar[s], ph)) {
                    atomicExch(err, 2);
                    abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a = smem_u32(tiles + (size_t)s * S::STAGE_BYTES);
                const uint64_t da = umma_desc_k_sw128(a);
                const uint64_t db = umma_desc_k_sw128(a + A_STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)  // 32 bytes along K per MMA: +2 in 16-byte units
                    umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);
            }
            if (ok && nkb > 0) umma_commit(&tmem_full_bar);
        }
        __syncwarp();
    } else {
        // ---- the four epilogue warps (threads 64 .. 191) -------------------------
        rfx::pdl_wait();         // y may still be read by an earlier kernel
        const int q = warp & 3;  // this warp may read TMEM lanes [32 q, 32 q + 32)
        const int m = q * 32 + lane;
        const int et = threadIdx.x - 64;  // 0 .. 127 among the epilogue threads
        constexpr int ET = 128;
        if (PRO) {
            // the rows' norm factors, while the main loop runs: 128 / BN threads
            // share a row's partials (a contiguous run each, read four at a
            // time), then one thread adds their sums in order
            const int t = m, rl = t % BN, grp = t / BN;
            constexpr int G = 128 / BN;
            float sum = 0.0f;
            if (r0 + rl < R) {
                const int np = fuse.n_part_in;
                const float* row = fuse.ssq_in + (size_t)(r0 + rl) * np;
                const int per = (np + G - 1) / G;
                const int p0 = grp * per, p1 = min(np, p0 + per);
                if ((np & 3) == 0 && (per & 3) == 0) {
                    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
                    for (int p = p0; p < p1; p += 4) {
                        const float4 v = *reinterpret_cast<const float4*>(row + p);
                        acc.x += v.x;
                        acc.y += v.y;
                        acc.z += v.z;
                        acc.w += v.w;
                    }
                    sum = (acc.x + acc.y) + (acc.z + acc.w);
                } else {
                    for (int p = p0; p < p1; ++p) sum += row[p];
                }
            }
            red_s[t] = sum;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (t < BN) {
                float total = 0.0f;
#pragma unroll
                for (int gi = 0; gi < G; ++gi) total += red_s[gi * BN + t];
                rstd_s[t] = 1.0f / sqrtf(total * fuse.inv_h + fuse.eps);
            }
        }
        // after the stages: a tile of [BN][BM] floats that receives partial rows from
        // the cluster's ranks (it must not alias the stages: a rank that is done
        // early sends while this CTA may still be streaming)
        float* stage0 = reinterpret_cast<float*>(tiles + (size_t)stages * S::STAGE_BYTES);
        const float* recv = stage0;
        float* sq = reinterpret_cast<float*>(tiles);  // [BN][mw] (split K); this CTA's stages are drained by then
        if constexpr (EPI == 3) {
            head_epilogue<BN, PRO>(stage0, stage0 + BN * BM, tmem_d, &tmem_full_bar, nkb > 0, ksplit, z, r0, R,
                                   fuse, rstd_s, err, trace_id);
        } else {
        // Four neighbouring rows of the tile at a time where the sizes allow it
        // (the slices are whole multiples of four and so are the output's rows):
        // one 16-byte access per rank's partial, per residual, per result.
        const bool quads = (mw & 3) == 0 && (N & 3) == 0 && (bm & 3) == 0;
        const int mq = mw >> 2;
        // Split K, EPI 2: the residual rows this rank will add to and their norm
        // weights are fetched now, long before they are needed.
        constexpr int MAX_IT = (EPI == 2 && BN <= 64) ? (BN * (BM / 8) + ET - 1) / ET : 1;  // two ranks or more
        float4 hv[MAX_IT], nwv[MAX_IT];
        if (EPI == 2 && BN <= 64 && ksplit > 1 && quads) {
#pragma unroll
            for (int it = 0; it < MAX_IT; ++it) {
                hv[it] = nwv[it] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (it * ET >= BN * mq) continue;
                const int e = et + it * ET;
                const int rr = e / mq, ml = 4 * (e % mq), mm = z * mw + ml;
                const int r = r0 + rr, n = n0 + mm;
                if (e < BN * mq && mm < bm && r < R && n < N) {
                    hv[it] = *reinterpret_cast<const float4*>(fuse.h + (size_t)r * N + n);
                    nwv[it] = *reinterpret_cast<const float4*>(fuse.nw + n);
                }
            }
        }

        // Two passes over the same code.  The first is a dry one, while the main
        // loop still runs: it reads no tensor memory, stores nothing and skips the
        // waits; it brings the epilogue's instructions into the cache, which at
        // one pass per launch would otherwise be fetched when every microsecond is
        // on the critical path.  The second is the work.
        bool have = nkb > 0;
#pragma unroll 1
        for (int pass = 0; pass < 2; ++pass) {
            const bool dry = pass == 0;
            if (!dry) {
                if (have && !mbar_wait(&tmem_full_bar, 0)) {
                    if (lane == 0) atomicExch(err, 3);
                    have = false;
                }
                tc_fence_after_sync();
                if (warp == 2 && lane == 0) trace_mark(trace_id, 2);
            }
            const bool load = have && !dry;
            const int chunks = dry ? 1 : BN / 16;
            const uint32_t lane_base = tmem_d + ((uint32_t)(q * 32) << 16);
            if (ksplit > 1) {
                // Split K: this CTA's tile is a partial sum.  Row m of the tile belongs to
                // rank m / mw of the cluster; send it there (remote shared-memory stores,
                // nothing waits on them) into slot [this rank][column][m % mw].
                cg::cluster_group cluster = cg::this_cluster();
                const int owner = m / mw, ml = m % mw;
                float* dst = cluster.map_shared_rank(stage0, owner < ksplit ? owner : 0) + (size_t)z * BN * mw + ml;
                uint32_t ahead[16];
                if (load) tmem_ld_16_nowait(lane_base, ahead);
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    float v[16];
                    if (load) {
                        tmem_ld_wait_16(ahead);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(ahead[j]);
                        if (c + 1 < chunks) tmem_ld_16_nowait(lane_base + (uint32_t)((c + 1) * 16), ahead);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    }
                    if (m < bm && !dry) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) dst[(c * 16 + j) * mw] = v[j];
                    }
                }
                if (!dry) {
                    tc_fence_before_sync();
                    if (threadIdx.x == 64) trace_mark(trace_id, 4);
                    // After one cluster barrier every rank holds all ranks' partial rows
                    // of its share of the tile in its own shared memory: [rank][column]
                    // [row].  Nobody reads remote memory after the barrier, so CTAs may
                    // leave as they finish.
                    cluster.sync();
                    if (threadIdx.x == 64) trace_mark(trace_id, 5);
                }
                // Sum in rank order, then the epilogue.
                if (quads && EPI == 0) {
                    for (int e = et; e < BN * mq; e += ET) {
                        const int rr = e / mq, ml4 = 4 * (e % mq), mm = z * mw + ml4;
                        const int r = r0 + rr, n = n0 + mm;
                        if (mm >= bm || r >= R || n >= N) continue;
                        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                        for (int p = 0; p < 8; ++p) {  // every rank's load in flight at once
                            if (p < ksplit) {
                                const float4 v = *reinterpret_cast<const float4*>(recv + (p * BN + rr) * mw + ml4);
                                acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
                            }
                        }
                        if (PRO) {
                            const float f = rstd_s[rr];
                            acc.x *= f, acc.y *= f, acc.z *= f, acc.w *= f;
                        }
                        if (!dry) store4(y + (size_t)r * N + n, acc);
                    }
                } else if (quads && EPI == 1) {
                    for (int e = et; e < BN * mq; e += ET) {
                        const int rr = e / mq, ml4 = 4 * (e % mq), mm = z * mw + ml4;
                        const int r = r0 + rr, n = n0 + mm;
                        if (mm >= bm || r >= R || n >= N) continue;
                        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);  // gate, up, gate, up
#pragma unroll
                        for (int p = 0; p < 8; ++p) {  // every rank's load in flight at once
                            if (p < ksplit) {
                                const float4 v = *reinterpret_cast<const float4*>(recv + (p * BN + rr) * mw + ml4);
                                acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
                            }
                        }
                        if (PRO) {
                            const float f = rstd_s[rr];
                            acc.x *= f, acc.y *= f, acc.z *= f, acc.w *= f;
                        }
                        const float o0 = silu_mul_for<TO>(acc.x, acc.y), o1 = silu_mul_for<TO>(acc.z, acc.w);
                        if (!dry) store2(y + (size_t)r * (N / 2) + n / 2, o0, o1);
                    }
                } else if (quads && EPI == 2 && BN <= 64) {
                    // A row's slice lies in mq neighbouring lanes; where mq is a power of
                    // two its squares are summed by shuffles, else through shared memory.
                    const bool seg = mq > 0 && (mq & (mq - 1)) == 0 && mq <= 32;
                    const int mq_shift = 31 - __clz(mq > 0 ? mq : 1);
#pragma unroll
                    for (int it = 0; it < MAX_IT; ++it) {
                        if (it * ET >= BN * mq) break;  // the same for every thread
                        const int e = et + it * ET;
                        const bool in = e < BN * mq;
                        const int rr = seg ? e >> mq_shift : e / mq;
                        const int ml4 = 4 * (seg ? e & (mq - 1) : e % mq), mm = z * mw + ml4;
                        const int r = r0 + rr, n = n0 + mm;
                        float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (in && mm < bm && r < R && n < N) {
                            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                            for (int p = 0; p < 8; ++p) {  // every rank's load in flight at once
                                if (p < ksplit) {
                                    const float4 v = *reinterpret_cast<const float4*>(recv + (p * BN + rr) * mw + ml4);
                                    acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
                                }
                            }
                            t = make_float4(hv[it].x + acc.x, hv[it].y + acc.y, hv[it].z + acc.z, hv[it].w + acc.w);
                            const size_t idx = (size_t)r * N + n;
                            const float4 w4 = nwv[it];
                            const float4 hb4 = make_float4(t.x * (fuse.nw_offset + w4.x), t.y * (fuse.nw_offset + w4.y),
                                                           t.z * (fuse.nw_offset + w4.z), t.w * (fuse.nw_offset + w4.w));
                            if (!dry) {
                                *reinterpret_cast<float4*>(fuse.h + idx) = t;
                                store4(fuse.hb + idx, hb4);
                            }
                        }
                        if (seg) {
                            // the same order every time: pairs inside the quad, then lanes 1, 2, 4, .. apart
                            float ss = (t.x * t.x + t.y * t.y) + (t.z * t.z + t.w * t.w);
                            for (int d = 1; d < mq; d <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
                            if (in && (ml4 == 0) && r < R && !dry)
                                fuse.ssq_out[(size_t)r * (gridDim.x * ksplit) + blockIdx.x * ksplit + z] = ss;
                        } else if (in && !dry) {
                            *reinterpret_cast<float4*>(sq + rr * mw + ml4) =
                                make_float4(t.x * t.x, t.y * t.y, t.z * t.z, t.w * t.w);
                        }
                    }
                    if (!seg) {
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        // this CTA's partial of each row's sum of squares, added in index order
                        if (et < BN && r0 + et < R && !dry) {
                            float tot = 0.0f;
                            for (int i = 0; i < mw; ++i) tot += sq[et * mw + i];
                            fuse.ssq_out[(size_t)(r0 + et) * (gridDim.x * ksplit) + blockIdx.x * ksplit + z] = tot;
                        }
                    }
                } else if (EPI == 0) {
                    for (int e = et; e < BN * mw; e += ET) {
                        const int rr = e / mw, ml1 = e % mw, mm = z * mw + ml1;
                        if (mm >= bm) continue;
                        float acc = 0.0f;
                        for (int p = 0; p < ksplit; ++p) acc += recv[((size_t)p * BN + rr) * mw + ml1];
                        if (PRO) acc *= rstd_s[rr];
                        const int r = r0 + rr;
                        if (r < R && n0 + mm < N && !dry) rfx::st<TO>(y, (size_t)r * N + n0 + mm, acc);
                    }
                } else if (EPI == 1) {
                    const int pw = mw / 2;
                    for (int e = et; e < BN * pw; e += ET) {
                        const int rr = e / pw, ml1 = 2 * (e % pw), mm = z * mw + ml1;
                        if (mm + 1 >= bm) continue;
                        float g = 0.0f, u = 0.0f;
                        for (int p = 0; p < ksplit; ++p) {
                            g += recv[((size_t)p * BN + rr) * mw + ml1];
                            u += recv[((size_t)p * BN + rr) * mw + ml1 + 1];
                        }
                        if (PRO) {
                            g *= rstd_s[rr];
                            u *= rstd_s[rr];
                        }
                        const int r = r0 + rr;
                        if (r < R && n0 + mm + 1 < N && !dry)
                            rfx::st<TO>(y, (size_t)r * (N / 2) + (n0 + mm) / 2, silu_mul_for<TO>(g, u));
                    }
                } else {
                    for (int e = et; e < BN * mw; e += ET) {
                        const int rr = e / mw, ml1 = e % mw, mm = z * mw + ml1;
                        const int r = r0 + rr, n = n0 + mm;
                        float hv1 = 0.0f;
                        if (mm < bm && r < R && n < N && !dry) {
                            float acc = 0.0f;
                            for (int p = 0; p < ksplit; ++p) acc += recv[((size_t)p * BN + rr) * mw + ml1];
                            const size_t idx = (size_t)r * N + n;
                            hv1 = fuse.h[idx] + acc;
                            fuse.h[idx] = hv1;
                            fuse.hb[idx] = __float2bfloat16_rn(hv1 * (fuse.nw_offset + fuse.nw[n]));
                        }
                        if (!dry) sq[rr * mw + ml1] = hv1 * hv1;
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    // this CTA's partial of each row's sum of squares, added in index order
                    if (et < BN && r0 + et < R && !dry) {
                        float tot = 0.0f;
                        for (int i = 0; i < mw; ++i) tot += sq[et * mw + i];
                        fuse.ssq_out[(size_t)(r0 + et) * (gridDim.x * ksplit) + blockIdx.x * ksplit + z] = tot;
                    }
                }
                if (!dry && threadIdx.x == 64) trace_mark(trace_id, 6);
            } else {
                // One CTA has the whole sum: finish straight from the registers.  The
                // next 16 columns are on their way from tensor memory while these are
                // worked on.
                float* sq1 = stage0;  // [BN][BM] squares of the new residual (EPI 2)
                uint32_t ahead[16];
                if (load) tmem_ld_16_nowait(lane_base, ahead);
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    float v[16];
                    if (load) {
                        tmem_ld_wait_16(ahead);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(ahead[j]);
                        if (c + 1 < chunks) tmem_ld_16_nowait(lane_base + (uint32_t)((c + 1) * 16), ahead);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    }
                    if (EPI == 1) {
                        // Rows alternate gate, up: lanes 2i and 2i + 1 hold one feature's
                        // pair.  Of every two columns the even lane finishes the first and
                        // the odd lane the second, after one exchange.
                        const bool even = (m & 1) == 0;
                        const int n = n0 + m;
                        const bool pair_ok = (m | 1) < bm && (n | 1) < N && !dry;
#pragma unroll
                        for (int j = 0; j < 16; j += 2) {
                            float a0 = v[j], a1 = v[j + 1];
                            if (PRO) {
                                a0 *= rstd_s[c * 16 + j];
                                a1 *= rstd_s[c * 16 + j + 1];
                            }
                            const float got = __shfl_xor_sync(0xffffffffu, even ? a1 : a0, 1);
                            const float gate = even ? a0 : got, up = even ? got : a1;
                            const int r = r0 + c * 16 + j + (even ? 0 : 1);
                            const float o = silu_mul_for<TO>(gate, up);
                            if (pair_ok && r < R) rfx::st<TO>(y, (size_t)r * (N / 2) + n / 2, o);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int rr = c * 16 + j, r = r0 + rr, n = n0 + m;
                            float a = v[j];
                            if (PRO) a *= rstd_s[rr];
                            if (EPI == 0) {
                                if (r < R && m < bm && n < N && !dry) rfx::st<TO>(y, (size_t)r * N + n, a);
                            } else {
                                float hv1 = 0.0f;
                                if (r < R && m < bm && n < N && !dry) {
                                    const size_t idx = (size_t)r * N + n;
                                    hv1 = fuse.h[idx] + a;
                                    fuse.h[idx] = hv1;
                                    fuse.hb[idx] = __float2bfloat16_rn(hv1 * (fuse.nw_offset + fuse.nw[n]));
                                }
                                if (!dry) sq1[rr * BM + m] = hv1 * hv1;
                            }
                        }
                    }
                    if (!dry && c == 0 && threadIdx.x == 64) trace_mark(trace_id, 4);
                }
                if (!dry && threadIdx.x == 64) trace_mark(trace_id, 5);
                if (EPI == 2) {
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    // this CTA's partial of each row's sum of squares, added in index order
                    if (m < BN && r0 + m < R && !dry) {
                        float tot = 0.0f;
                        for (int i = 0; i < bm; ++i) tot += sq1[m * BM + i];
                        fuse.ssq_out[(size_t)(r0 + m) * gridDim.x + blockIdx.x] = tot;
                    }
                }
                if (!dry) tc_fence_before_sync();
            }
        }
        }  // EPI != 3
    }
    // the producer and the MMA warp take part in the cluster's barrier too
    if (warp < 2 && ksplit > 1) {
        rfx::pdl_wait();
        cg::this_cluster().sync();
    }

    __syncthreads();
    if (threadIdx.x == 0) trace_mark(trace_id, 3);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_d, S::TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------
// A [rows, cols] row-major bfloat16 matrix, tiles of box_rows x 64 columns,
// 128-byte swizzle, zero fill outside.
static_assert(BK == 64, "the shared map maker cuts 64-column boxes");
bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    return rfx::tma::make_map_rows64(map, base, rows, cols, box_rows);
}

struct MapKey {
    const void* p;
    int rows, cols, box;
    bool operator<(const MapKey& o) const {
        return std::tie(p, rows, cols, box) < std::tie(o.p, o.rows, o.cols, o.box);
    }
};

// Weight maps are made once per (pointer, shape); activation maps per call.
const CUtensorMap* cached_map(const void* base, int rows, int cols, int box_rows) {
    static std::map<MapKey, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{base, rows, cols, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) return &it->second;
    CUtensorMap m;
    if (!make_map(&m, base, rows, cols, box_rows)) return nullptr;
    return &cache.emplace(key, m).first->second;
}

using rfx::sm_count;

int g_trace_next = 0;  // launch counter: the trace record a launch writes

int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

// Tuning aids, read from the environment once, at the first product.
struct Knobs {
    int cps, even, smem_kb, stages, smem_cap_kb, l2pf_mb, max_cta_pct;
};
const Knobs& knobs() {
    static const Knobs k = {env_int("REFLEX_B200_GEMM_CPS", 0),      env_int("REFLEX_B200_GEMM_EVEN", 1),
                            env_int("REFLEX_B200_GEMM_SMEM_KB", 110), env_int("REFLEX_B200_GEMM_STAGES", 0),
                            env_int("REFLEX_B200_GEMM_SMEM_CAP_KB", 112), env_int("REFLEX_B200_GEMM_L2PF_MB", 0),
                            env_int("REFLEX_B200_GEMM_MAX_CTA_PCT", 200)};
    return k;
}

// How a product is cut into CTAs.  Streaming weights at HBM speed needs every SM
// pulling all the time (one SM tops out near 55 GB/s), so the grid is made a
// whole multiple of the SM count with equal work per CTA: `tiles` row tiles of
// `bm` <= 128 weight rows (a tile need not be 128 rows: TMA boxes take any
// height) times a K split of `ks` CTAs that form a cluster.  When no such cut
// exists (small matrices) tiles are 128 rows and K is split while CTAs are few.
struct Cut {
    int bm, tiles, ks;
};

Cut choose_cut(int N, int r_tiles, int num_kb, int ks_req, bool whole_tiles, int bn) {
    if (ks_req > 0) return Cut{BM, (N + BM - 1) / BM, ks_req};
    if (whole_tiles) {  // tiles of exactly 128 rows; K split while CTAs are few
        const int t = (N + BM - 1) / BM;
        int k = 1;
        while (k < 8 && t * r_tiles * k * 2 <= 2 * sm_count() && num_kb >= k * 4) k *= 2;
        return Cut{BM, t, k};
    }
    const int sms = sm_count();
    const int cps_first = knobs().cps;  // tuning aid: CTAs per SM to try first
    for (int pass = 0; pass < 2 && cps_first > 0; ++pass) {
        const int c = cps_first ? (pass == 0 ? cps_first : 3 - cps_first) : (pass == 0 ? 1 : 2);
        if (c < 1 || c > 2) continue;
        int best_ks = 0, best_bm = 0, best_tiles = 0;
        for (int ks = 1; ks <= 8; ks *= 2) {
            const int total = sms * c;
            if (total % (ks * r_tiles)) continue;
            const int tiles = total / (ks * r_tiles);
            const int bm = (N + tiles - 1) / tiles;
            if (bm > BM || bm < 32 || num_kb < 4 * ks) continue;
            if ((N + bm - 1) / bm != tiles) continue;  // the last tiles would be empty
            if (bm > best_bm) {  // the tallest tile reuses each activation tile most
                best_bm = bm;
                best_ks = ks;
                best_tiles = tiles;
            }
        }
        if (best_ks) return Cut{best_bm, best_tiles, best_ks};
    }
    const int tiles = (N + BM - 1) / BM;
    // Between one and two 128-row tiles per SM the SMs that get two CTAs finish
    // late while the rest idle: cut lower tiles instead, two per SM, equal work.
    // (Not with 64 activation rows: a lower tile brings the same activation tile
    // for fewer weight rows, and what an SM can take in is the limit there; measured
    // 2 % of a batch-64 step.)
    if (r_tiles == 1 && tiles > sms && tiles < 2 * sms && knobs().even && bn < 64) {
        int bm = (N + 2 * sms - 1) / (2 * sms);
        bm = (bm + 1) & ~1;
        if (bm >= 32 && bm <= BM) return Cut{bm, (N + bm - 1) / bm, 1};
    }
    int ks = 1;
    const int max_ctas = sms * knobs().max_cta_pct / 100;  // tuning aid: CTAs the K split may make
    while (ks < 8 && tiles * r_tiles * ks * 2 <= max_ctas && num_kb >= ks * 4) ks *= 2;
    return Cut{BM, tiles, ks};
}

template <int BN, typename TO, int EPI, bool PRO>
int launch(const void* x, const void* W, void* y, int R, int N, int K, int ksplit_req, const Fuse& fuse_in,
           int* n_part_out, int* err, cudaStream_t s) {
    using S = Shape<BN>;
    const int r_tiles = (R + BN - 1) / BN;
    const int num_kb = (K + BK - 1) / BK;
    Cut cut = choose_cut(N, r_tiles, num_kb, ksplit_req, EPI == 3, BN);
    if (EPI == 3 && (r_tiles != 1 || BN % cut.ks)) return RFX_ERR_UNSUPPORTED;
    if (EPI == 1 && (cut.bm & 1)) {  // pairs must not straddle tiles
        cut.bm += 1;
        if (cut.bm > BM) return RFX_ERR_UNSUPPORTED;
        cut.tiles = (N + cut.bm - 1) / cut.bm;
    }
    const int ks = cut.ks;
    if (ks != 1 && ks != 2 && ks != 4 && ks != 8) return RFX_ERR_BAD_ARG;
    const CUtensorMap* mw = cached_map(W, N, K, cut.bm);
    CUtensorMap mx;
    if (!mw || !make_map(&mx, x, R, K, BN)) return RFX_ERR_UNSUPPORTED;
    // A ring of about 72 KB: three CTAs fit an SM, so the kernels that follow
    // (launched early, see common.cuh) are resident and prefetch their weights
    // while this one runs; a deeper ring measured slower for that reason.
    int stages = (knobs().smem_kb * 1024) / S::STAGE_BYTES;
    if (stages < 3) stages = 3;
    const int st_env = knobs().stages;  // tuning aid
    if (st_env >= 2) stages = st_env;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    // after the stages, the tile that receives the cluster's partial rows
    constexpr int RECV_BYTES = BN * BM * 4;
    const int cap = knobs().smem_cap_kb * 1024;  // tuning aid
    // EPI 3 keeps its rows' rotation table behind the receive tile: (cos, sin) per row and pair
    // EPI 3 keeps its rows' rotation table and places behind the receive tile
    const int rot_bytes = EPI == 3 ? (BN / ks) * (fuse_in.head_dim * 4 + 8) : 0;
    while (stages > 3 && stages * S::STAGE_BYTES + RECV_BYTES + rot_bytes > cap) --stages;
    if (stages * S::STAGE_BYTES < BN * BM * 4) return RFX_ERR_UNSUPPORTED;  // the squares of EPI 2
    if (n_part_out) *n_part_out = cut.tiles * ks;
    if (EPI == 2 && r_tiles != 1) return RFX_ERR_UNSUPPORTED;
    const size_t smem = (size_t)stages * S::STAGE_BYTES + RECV_BYTES + rot_bytes + 1024;
    auto kernel = gemm_wt_kernel<BN, TO, EPI, PRO>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // L2 prefetch before the dependency wait: up to a budget for the whole grid
    const long long budget = (long long)knobs().l2pf_mb << 20;
    const long long ctas = (long long)cut.tiles * r_tiles * ks;
    int l2_ahead = (int)(budget / (ctas * cut.bm * BK * 2));
    if (r_tiles > 1) l2_ahead = 0;  // prefill-sized calls are not bandwidth-bound
    e = rfx::launch(kernel, dim3(cut.tiles, r_tiles, ks), dim3(THREADS), smem, s, ks, *mw, mx, (TO*)y, R,
                    N, K, ks, stages, cut.bm, l2_ahead, g_trace_next++, fuse_in, err);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

template <typename TO, int EPI, bool PRO>
int dispatch(const void* x, const void* W, void* y, int R, int N, int K, int ksplit, const Fuse& fuse,
             int* n_part_out, int* err, cudaStream_t s) {
    if (R <= 16) return launch<16, TO, EPI, PRO>(x, W, y, R, N, K, ksplit, fuse, n_part_out, err, s);
    if (R <= 32) return launch<32, TO, EPI, PRO>(x, W, y, R, N, K, ksplit, fuse, n_part_out, err, s);
    if (R <= 64) return launch<64, TO, EPI, PRO>(x, W, y, R, N, K, ksplit, fuse, n_part_out, err, s);
    if (EPI >= 2 || PRO) return RFX_ERR_UNSUPPORTED;  // the fused forms are for decode-sized batches
    return launch<128, TO, EPI, PRO>(x, W, y, R, N, K, ksplit, fuse, n_part_out, err, s);
}

int check_common(const void* x, const void* W, int R, int N, int K) {
    if (K <= 0 || K % 8 != 0) return RFX_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15) return RFX_ERR_BAD_ARG;
    if ((N + BM - 1) / BM > 2147483647 || (R + 127) / 128 > 65535) return RFX_ERR_UNSUPPORTED;
    return 0;
}

}  // namespace

// y [R, N] = x [R, K] . W [N, K]^T, bfloat16 inputs, float32 accumulation,
// y float32 or bfloat16.  K must be a multiple of 8 and the pointers 16-byte
// aligned (TMA).  ksplit: 0 = choose, else 1, 2, 4 or 8.  `err` is a device
// word that receives a non-zero code if a bounded wait ran out.
// epilogue 1: W's rows alternate gate/up, N is even, y is [R, N / 2] =
// silu(gate) * up.
// ssq_in (optional, R <= 64): x is unnormalised; row r of the result is scaled by
// 1 / sqrt(sum_p ssq_in[r][p] / norm_h + eps), p < n_part_in.
extern "C" int rfx_gemm_bf16_tc(const void* x, const void* W, void* y, int y_dt, int R, int N,
                                int K, int ksplit, int epilogue, const float* ssq_in, int n_part_in,
                                int norm_h, float eps, int* err, void* stream) {
    if (R <= 0 || N <= 0) return 0;
    if (int c = check_common(x, W, R, N, K)) return c;
    if (epilogue != 0 && epilogue != 1) return RFX_ERR_BAD_ARG;
    if (epilogue == 1 && (N & 1)) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    Fuse f{};
    const bool pro = ssq_in != nullptr;
    if (pro) {
        if (n_part_in <= 0 || norm_h <= 0) return RFX_ERR_BAD_ARG;
        f.ssq_in = ssq_in;
        f.n_part_in = n_part_in;
        f.inv_h = 1.0f / (float)norm_h;
        f.eps = eps;
    }
#define RFX_GO(TO, E, P) return dispatch<TO, E, P>(x, W, y, R, N, K, ksplit, f, nullptr, err, s)
    if (y_dt == RFX_DT_F32) {
        if (epilogue == 0) { if (pro) RFX_GO(float, 0, true); else RFX_GO(float, 0, false); }
        else { if (pro) RFX_GO(float, 1, true); else RFX_GO(float, 1, false); }
    } else if (y_dt == RFX_DT_BF16) {
        if (epilogue == 0) { if (pro) RFX_GO(__nv_bfloat16, 0, true); else RFX_GO(__nv_bfloat16, 0, false); }
        else { if (pro) RFX_GO(__nv_bfloat16, 1, true); else RFX_GO(__nv_bfloat16, 1, false); }
    }
#undef RFX_GO
    return RFX_ERR_BAD_ARG;
}

// The product as a delta of the residual stream, for R <= 64:
//   h [R, N] (float32) += x . W^T;   hb [R, N] = bfloat16(h * (nw_offset + nw[n]));
//   ssq_out[r][p] = this CTA's share of sum_n h[r, n]^2, p < *n_part_out
// (ssq_out must hold at least rfx_gemm_bf16_tc_max_parts(N) * R floats).
extern "C" int rfx_gemm_bf16_tc_residual(const void* x, const void* W, float* h, const float* nw,
                                         float nw_offset, void* hb, float* ssq_out, int* n_part_out,
                                         int R, int N, int K, int ksplit, int* err, void* stream) {
    if (R <= 0 || N <= 0) return 0;
    if (R > 64) return RFX_ERR_UNSUPPORTED;
    if (int c = check_common(x, W, R, N, K)) return c;
    if (!h || !nw || !hb || !ssq_out || !n_part_out) return RFX_ERR_BAD_ARG;
    Fuse f{};
    f.h = h;
    f.nw = nw;
    f.nw_offset = nw_offset;
    f.hb = (__nv_bfloat16*)hb;
    f.ssq_out = ssq_out;
    return dispatch<float, 2, false>(x, W, nullptr, R, N, K, ksplit, f, n_part_out, err, (cudaStream_t)stream);
}

// The q/k/v product of a decode step, finished per head (R <= 64, head_dim 64 or
// 128, the rotation, if any, over the whole head in half-split pairs):
//   q_out [R, nq * head_dim] = rotate(norm(x . Wq^T));  the key rotate(norm(x . Wk^T))
//   and the value x . Wv^T of row r into the paged cache at (row_slot[r], row_pos[r]).
// W is [(nq + 2 nkv_in) * head_dim, K]; nkv_in is nkv, or 0 for a product that
// brings queries only.  ssq_in as in rfx_gemm_bf16_tc.
extern "C" int rfx_gemm_bf16_tc_qkv(const void* x, const void* W, int R, int K, const float* ssq_in,
                                    int n_part_in, int norm_h, float eps, const float* q_w,
                                    const float* k_w, float qk_eps, float qk_offset,
                                    const float* rope_denom, float magnitude, const int* row_pos,
                                    const int* row_slot, void* q_out, void* k_pages, void* v_pages,
                                    const int* page_table, int max_pages, int page_size, int nq,
                                    int nkv_in, int nkv, int head_dim, int* err, void* stream) {
    if (R <= 0) return 0;
    if (R > 64 || (head_dim != 64 && head_dim != 128)) return RFX_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || (nkv_in != 0 && nkv_in != nkv)) return RFX_ERR_BAD_ARG;
    const int N = (nq + 2 * nkv_in) * head_dim;
    if (int c = check_common(x, W, R, N, K)) return c;
    if (!row_pos || !row_slot || !q_out || (nkv_in && (!k_pages || !v_pages || !page_table))) return RFX_ERR_BAD_ARG;
    Fuse f{};
    const bool pro = ssq_in != nullptr;
    if (pro) {
        if (n_part_in <= 0 || norm_h <= 0) return RFX_ERR_BAD_ARG;
        f.ssq_in = ssq_in;
        f.n_part_in = n_part_in;
        f.inv_h = 1.0f / (float)norm_h;
        f.eps = eps;
    }
    f.q_w = q_w;
    f.k_w = k_w;
    f.qk_eps = qk_eps;
    f.qk_offset = qk_offset;
    f.rope_denom = rope_denom;
    f.magnitude = magnitude;
    f.row_pos = row_pos;
    f.row_slot = row_slot;
    f.q_out = (__nv_bfloat16*)q_out;
    f.k_pages = (__nv_bfloat16*)k_pages;
    f.v_pages = (__nv_bfloat16*)v_pages;
    f.cache = rfx::PagedKV{page_table, max_pages, page_size, nkv, head_dim};
    f.nq = nq;
    f.nkv_in = nkv_in;
    f.head_dim = head_dim;
    cudaStream_t s = (cudaStream_t)stream;
    if (pro) return dispatch<__nv_bfloat16, 3, true>(x, W, q_out, R, N, K, 0, f, nullptr, err, s);
    return dispatch<__nv_bfloat16, 3, false>(x, W, q_out, R, N, K, 0, f, nullptr, err, s);
}

// An upper bound of the partials a residual product of N weight rows writes per row.
extern "C" int rfx_gemm_bf16_tc_max_parts(int N) { return ((N + 31) / 32) * 8 + 8 * sm_count() * 2; }

extern "C" int rfx_sm_count() { return sm_count(); }

// Tuning aid: give the product kernel a device buffer of launches * ctas records of
// four 64-bit timestamps; the next launch writes record 0.  Null turns it off.
extern "C" int rfx_gemm_trace(void* buffer, int launches, int ctas) {
    g_trace_next = 0;
    TraceRec* p = (TraceRec*)buffer;
    cudaError_t e = cudaMemcpyToSymbol(g_trace, &p, sizeof(p));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_ctas, &ctas, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_launches, &launches, sizeof(int));
    return (int)e;
}
