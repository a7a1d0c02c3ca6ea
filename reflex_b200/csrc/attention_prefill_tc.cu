// Prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Same problem as attention_prefill.cu (causal, optionally windowed
// grouped-query attention of a packed batch over the paged cache; a CTA =
// one sequence, one kv head, 128 rows that are (position, head of the group)
// pairs), for head sizes 64 and 128.  Per page of 64 keys:
//   S = Q K^T      tcgen05.mma, Q [128 x D] and the K page [64 x D] in shared
//                  memory (TMA, 128-byte swizzle), S [128 x 64] float32 in TMEM;
//   softmax        four warps, one thread per row: tcgen05.ld its row of S,
//                  mask, running max and sum in 32-bit, P as bfloat16 back into
//                  TMEM over the columns S came from (tcgen05.st);
//   O += P V       tcgen05.mma with P from TMEM and the V page as the MN-major
//                  shared-memory operand, O [128 x D] accumulating in TMEM.
// The running maximum is a reference, not the exact maximum: it is raised (and
// the row of O rescaled through tcgen05.ld / tcgen05.st) only when a page's
// maximum passes it by more than 2^8, so rescaling is rare; probabilities are
// 2^(s - reference) <= 2^8 and the final division by the sum, taken with the
// same reference, gives the exact softmax.  S and P are double-buffered so the
// tensor core works on page j + 1 while the softmax warps are on page j.  Warp 0 issues TMA loads, warp 1 issues
// MMAs, warps 2..5 are the softmax rows.  Every mbarrier wait is bounded; on a
// timeout the kernel records it, stops, frees its tensor memory and returns.
// The reference's tiled kernel is the CUDA-core ancestor
// (src/kernels_cuda/attention_tiled.cuh:73-296).
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "paged.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

namespace {

// Optional timeline for tuning: when a buffer is set (rfx_attention_prefill_tc_trace),
// chosen threads store %globaltimer at a few places of a CTA's life (32 slots per
// CTA); the last launch wins.
static __device__ unsigned long long* g_trace = nullptr;
static __device__ int g_trace_ctas = 0;
__device__ __forceinline__ void trace_mark(int which) {
    if (g_trace == nullptr) return;
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (cta >= g_trace_ctas) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_trace[(size_t)cta * 32 + which] = t;
}

// a raw value (cycles spent in a wait, summed) instead of a timestamp
__device__ __forceinline__ void trace_value(int which, long long v) {
    if (g_trace == nullptr) return;
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (cta >= g_trace_ctas) return;
    g_trace[(size_t)cta * 32 + which] = (unsigned long long)v;
}

using namespace sm100;
using rfx::PagedKV;

constexpr int PAGE = 64;
constexpr int ROWS = 128;
constexpr int THREADS = 192;
constexpr int KV_STAGES = 2;  // with 97 KB of shared memory two CTAs share an SM

// 3-D tile load (x innermost)
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
          "r"(x), "r"(y), "r"(z)
        : "memory");
}
// 2^x, hardware approximation (about 2 ulp; the result is rounded to bfloat16)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// MN-major operand, 128-byte swizzle: 64 elements contiguous per k-row, k-rows
// 128 bytes apart, groups of 8 k-rows `sbo` bytes apart, blocks of 64 elements
// along MN `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, A bfloat16 K-major, B bfloat16 MN-major, D float32
__host__ __device__ constexpr uint32_t idesc_b_mn(int M, int N) {
    return umma_idesc_bf16(M, N) | (1u << 16);
}

struct Smem {
    // all tiles 1024-byte aligned
    static constexpr int q_bytes(int D) { return ROWS * D * 2; }
    static constexpr int kv_bytes(int D) { return PAGE * D * 2; }
    static constexpr int total(int D) { return q_bytes(D) + 2 * KV_STAGES * kv_bytes(D) + 1024; }
};

template <int D>
__global__ void __launch_bounds__(THREADS)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                            const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PagedKV cache,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                            const int* __restrict__ seq_new, const int* __restrict__ seq_row0,
                            __nv_bfloat16* __restrict__ out, int nq, int bq, int window,
                            float scale_log2, int* __restrict__ err) {
    static_assert(D == 64 || D == 128, "head sizes 64 and 128");
    constexpr int KB = D / 64;                 // 64-column blocks of a row
    constexpr int KV_BYTES = PAGE * D * 2;
    constexpr uint32_t TMEM_COLS = 256;
    // S: 2 x 64 columns (P_b, 32 columns of packed bfloat16, overwrites the start
    // of S_b once the row has read it), then O: D columns
    constexpr uint32_t S_COL = 0, O_COL = 128;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES],
        v_empty[KV_STAGES], s_full[2], p_full[2], o_full;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;

    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = base;
    uint8_t* k_ring = q_tile + ROWS * D * 2;
    uint8_t* v_ring = k_ring + KV_STAGES * KV_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) trace_mark(0);  // 0 entry, 1 set up, 2 first scores, 3 last page done, 4 output written, 5 exit
    // CTAs are handed out with x fastest: kv heads and sequences vary fastest and
    // the tile slowest, so that the longest tiles of every head start first
    const int kvh = blockIdx.x, seq = blockIdx.y;
    const int n_new = seq_new[seq];
    const int q0 = (gridDim.z - 1 - blockIdx.z) * bq;  // the longest tiles first
    const bool active = q0 < n_new;
    const int g = nq / cache.n_kv_heads;
    const int slot = seq_slot[seq], start = seq_start[seq], row0 = seq_row0[seq];
    const int n_pos = active ? min(bq, n_new - q0) : 0;
    const int n_rows = n_pos * g;
    const int pos_first = start + q0, pos_last = pos_first + n_pos - 1;
    const int lo_tile = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;
    const int pg0 = lo_tile / PAGE, pg1 = active ? pos_last / PAGE + 1 : 0;
    const int n_pages = active ? pg1 - pg0 : 0;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4);
        }
        mbar_init(&o_full, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_smem;
    rfx::pdl_prologue();  // q and this step's keys and values come from the kernel before
    if (threadIdx.x == 0) trace_mark(1);

    if (!active) {
        // nothing to do for this tile; fall through to the teardown
    } else if (warp == 0) {
        if (elect_one()) {
            const int* table = cache.page_table + (size_t)slot * cache.max_pages;
            mbar_expect_tx(&q_full, (uint32_t)(bq * g * 128 * KB));
            for (int kb = 0; kb < KB; ++kb)
                tma_load_3d(q_tile + kb * ROWS * 128, &map_q, &q_full, kb * 64, kvh * g, row0 + q0);
            for (int j = 0; j < n_pages; ++j) {
                const int s = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                const int page = table[pg0 + j];
                const int y = (page * cache.n_kv_heads + kvh) * PAGE;
                if (!mbar_wait(&k_empty[s], ph ^ 1)) { atomicExch(err, 11); abort_flag = 1; break; }
                mbar_expect_tx(&k_full[s], KV_BYTES);
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(k_ring + s * KV_BYTES + kb * PAGE * 128, &map_k, &k_full[s], kb * 64, y);
                if (!mbar_wait(&v_empty[s], ph ^ 1)) { atomicExch(err, 12); abort_flag = 1; break; }
                mbar_expect_tx(&v_full[s], KV_BYTES);
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(v_ring + s * KV_BYTES + kb * PAGE * 128, &map_v, &v_full[s], kb * 64, y);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(ROWS, PAGE);  // S: N = 64 keys
            constexpr uint32_t idesc_o = idesc_b_mn(ROWS, D);          // O: N = D, V is MN-major
            const bool tracing = g_trace != nullptr;
            long long wait_k = 0, wait_p = 0, wait_v = 0, c0 = 0;
            bool ok = mbar_wait(&q_full, 0);
            if (!ok) { atomicExch(err, 13); abort_flag = 1; }
            auto pv = [&](int i) -> bool {
                const int b = i & 1, s = i % KV_STAGES;
                const uint32_t ph2 = (i >> 1) & 1, phs = (i / KV_STAGES) & 1;
                // P_i is delivered after any rescaling of O that page i asked for
                if (tracing) c0 = clock64();
                if (!mbar_wait(&p_full[b], ph2)) { atomicExch(err, 14); return false; }
                if (tracing) { const long long c1 = clock64(); wait_p += c1 - c0; c0 = c1; }
                if (!mbar_wait(&v_full[s], phs)) { atomicExch(err, 15); return false; }
                if (tracing) wait_v += clock64() - c0;
                tc_fence_after_sync();
                const uint32_t va = smem_u32(v_ring + s * KV_BYTES);
#pragma unroll
                for (int k = 0; k < PAGE / 16; ++k) {  // 16 keys per MMA: 8 packed columns of P
                    const uint64_t db = umma_desc_mn_sw128(va + k * 16 * 128, PAGE * 128, 1024);
                    umma_bf16_ts(tmem + O_COL, tmem + S_COL + b * PAGE + k * 8, db, idesc_o,
                                 (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&v_empty[s]);
                umma_commit(&o_full);
                return true;
            };
            for (int j = 0; j < n_pages && ok; ++j) {
                const int b = j & 1, s = j % KV_STAGES;
                const uint32_t phs = (j / KV_STAGES) & 1;
                // S_j reuses the columns of S_{j-2} and P_{j-2}: PV_{j-2} was issued
                // before this and the tensor core runs MMAs in issue order
                if (tracing) c0 = clock64();
                if (!mbar_wait(&k_full[s], phs)) { atomicExch(err, 18); ok = false; break; }
                if (tracing) wait_k += clock64() - c0;
                tc_fence_after_sync();
                const uint32_t qa = smem_u32(q_tile), ka = smem_u32(k_ring + s * KV_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t da = umma_desc_k_sw128(qa + kb * ROWS * 128) + 2 * k;
                        const uint64_t db = umma_desc_k_sw128(ka + kb * PAGE * 128) + 2 * k;
                        umma_bf16(tmem + S_COL + b * PAGE, da, db, idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                umma_commit(&k_empty[s]);
                umma_commit(&s_full[b]);
                if (j > 0) ok = pv(j - 1);
            }
            if (ok && n_pages > 0) ok = pv(n_pages - 1);
            if (!ok) abort_flag = 1;
            if (tracing) {
                trace_value(8, wait_k);
                trace_value(9, wait_p);
                trace_value(10, wait_v);
            }
        }
        __syncwarp();
    } else {
        // softmax rows: this thread owns row t (TMEM lane t) of the tile
        const int qd = warp & 3;
        const int t = qd * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
        const bool row_valid = t < n_rows;
        const int row_p = t / g, row_h = t % g;
        const int row_pos = row_valid ? pos_first + row_p : -1;
        const int row_lo = (window > 0 && row_pos + 1 > window) ? row_pos + 1 - window : 0;
        const int lo_last = (window > 0 && pos_last + 1 > window) ? pos_last + 1 - window : 0;
        constexpr float RAISE = 8.0f;  // raise the reference maximum only past 2^8
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        const bool tracing = g_trace != nullptr && t == 0;
        long long wait_s = 0, c0 = 0;

        for (int j = 0; j < n_pages && ok; ++j) {
            const int b = j & 1;
            const uint32_t ph2 = (j >> 1) & 1;
            if (tracing) c0 = clock64();
            if (!mbar_wait(&s_full[b], ph2)) { atomicExch(err, 22); ok = false; break; }
            if (tracing) wait_s += clock64() - c0;
            tc_fence_after_sync();
            if (t == 0 && j == 0) trace_mark(2);
            uint32_t sr[PAGE];
#pragma unroll
            for (int c = 0; c < PAGE / 16; ++c)
                tmem_ld_16_nowait(tmem + lane_addr + S_COL + b * PAGE + c * 16, sr + c * 16);
            tmem_ld_wait();

            const int basej = (pg0 + j) * PAGE;
            // every key of the page visible to every valid row of the tile: no compares
            const bool all_visible = basej + PAGE - 1 <= pos_first && basej >= lo_last && n_rows == ROWS;
            // four independent chains each for the maximum and the sum: one warp per
            // scheduler has nothing else to hide a dependent chain's latency with
            float s[PAGE];  // raw scores; the scale (positive) goes into the exponent's multiply-add
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (all_visible) {
#pragma unroll
                for (int c = 0; c < PAGE; ++c) s[c] = __uint_as_float(sr[c]);
#pragma unroll
                for (int c = 0; c < PAGE; c += 8)  // two new values per maximum: a three-input instruction
#pragma unroll
                    for (int k = 0; k < 4; ++k) mx4[k] = fmaxf(fmaxf(mx4[k], s[c + 2 * k]), s[c + 2 * k + 1]);
            } else {
#pragma unroll
                for (int c = 0; c < PAGE; ++c) {
                    const int key = basej + c;
                    s[c] = (key <= row_pos && key >= row_lo) ? __uint_as_float(sr[c]) : -INFINITY;
                    mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // the reference maximum moves only when it must
            float corr = 1.0f;
            const bool raise = mx > m + RAISE || (m == -INFINITY && mx != -INFINITY);
            if (raise) {
                corr = (m == -INFINITY) ? 0.0f : ex2(m - mx);
                m = mx;
                l *= corr;
            }
            // rows that have seen no key yet: every s is -inf, shift by 0 gives p = 0
            const float shift = (m == -INFINITY) ? 0.0f : m;
            float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t packed[PAGE / 2];
#pragma unroll
            for (int c = 0; c < PAGE; c += 2) {
                const float e0 = ex2(fmaf(s[c], scale_log2, -shift));
                const float e1 = ex2(fmaf(s[c + 1], scale_log2, -shift));
                rs4[(c >> 1) & 3] += e0 + e1;
                __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                packed[c / 2] = *reinterpret_cast<uint32_t*>(&h);
            }
            l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);

            // rescale this row of O if its reference moved (whole warp together:
            // the TMEM accesses are warp-wide; lanes that did not move scale by 1)
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                if (!mbar_wait(&o_full, (uint32_t)((j - 1) & 1))) { atomicExch(err, 21); ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < D / 16; ++c) {
                    uint32_t o[16];
                    tmem_ld_16_nowait(tmem + lane_addr + O_COL + c * 16, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
                    tmem_st_16(tmem + lane_addr + O_COL + c * 16, o);
                }
                tmem_st_wait();
                tc_fence_before_sync();
            }

            // row t of P into TMEM, over the columns its S came from
            tmem_st_16(tmem + lane_addr + S_COL + b * PAGE, packed);
            tmem_st_16(tmem + lane_addr + S_COL + b * PAGE + 16, packed + 16);
            tmem_st_wait();
            // the last page may hold keys past this tile's last position whose
            // value rows were never written: zero them, 0 * NaN would not be 0
            const int valid_keys = pos_last + 1 - basej;
            if (valid_keys < PAGE) {
                const int sidx = j % KV_STAGES;
                if (!mbar_wait(&v_full[sidx], (j / KV_STAGES) & 1)) { atomicExch(err, 24); ok = false; break; }
                uint8_t* vt = v_ring + sidx * KV_BYTES;
                for (int i = t; i < (PAGE - valid_keys) * KB * 8; i += ROWS) {
                    const int rrow = valid_keys + i / (KB * 8), rem = i % (KB * 8);
                    *reinterpret_cast<uint4*>(vt + (rem / 8) * PAGE * 128 + rrow * 128 + (rem % 8) * 16) =
                        make_uint4(0, 0, 0, 0);
                }
            }
            if (valid_keys < PAGE) fence_async_proxy();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);
        }
        if (t == 0) trace_mark(3);
        if (tracing) trace_value(11, wait_s);
        if (ok && n_pages > 0) {
            if (!mbar_wait(&o_full, (uint32_t)((n_pages - 1) & 1))) { atomicExch(err, 25); ok = false; }
        }
        if (ok && n_pages > 0) {
            tc_fence_after_sync();
            const float inv = 1.0f / l;
            __nv_bfloat16* o = out + ((size_t)(row0 + q0 + row_p) * nq + kvh * g + row_h) * D;
            // two loads of 16 columns in flight: the next one travels while this one is stored
            uint32_t rr[2][16];
            tmem_ld_16_nowait(tmem + lane_addr + O_COL, rr[0]);
#pragma unroll
            for (int c = 0; c < D / 16; ++c) {
                tmem_ld_wait_16(rr[c & 1]);
                if (c + 1 < D / 16) tmem_ld_16_nowait(tmem + lane_addr + O_COL + (c + 1) * 16, rr[(c + 1) & 1]);
                uint32_t(&r)[16] = rr[c & 1];
                if (row_valid) {
                    uint4 v[2];
                    __nv_bfloat162* pv2 = reinterpret_cast<__nv_bfloat162*>(v);
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        pv2[e] = __floats2bfloat162_rn(__uint_as_float(r[2 * e]) * inv, __uint_as_float(r[2 * e + 1]) * inv);
                    *reinterpret_cast<uint4*>(o + c * 16) = v[0];
                    *reinterpret_cast<uint4*>(o + c * 16 + 8) = v[1];
                }
            }
        }
        if (t == 0) trace_mark(4);
        tc_fence_before_sync();
    }

    __syncthreads();
    if (threadIdx.x == 0) trace_mark(5);
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---- host ---------------------------------------------------------------------
using rfx::tma::encode_fn;
using rfx::tma::EncodeTiledFn;

// q [R, nq, D]: dims (D, nq, R), a box of 64 columns x g heads x bq positions
bool make_map_q(CUtensorMap* map, const void* base, int R, int nq, int D, int g, int bq) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)nq, (cuuint64_t)R};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)nq * D * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)g, (cuuint32_t)bq};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
int launch_tc(const void* q, const void* k_pages, const void* v_pages, long long n_pages_total,
              const PagedKV& cache, const int* seq_slot, const int* seq_start, const int* seq_new,
              const int* seq_row0, void* out, int S, int max_new, int R, int nq, int window, float scale,
              int* err, cudaStream_t s) {
    const int g = nq / cache.n_kv_heads;
    if (g > ROWS) return RFX_ERR_UNSUPPORTED;
    const int bq = ROWS / g;
    CUtensorMap mq, mk, mv;
    const long long kv_rows = n_pages_total * cache.n_kv_heads * PAGE;
    if (!make_map_q(&mq, q, R, nq, D, g, bq) || !rfx::tma::make_map_rows64(&mk, k_pages, kv_rows, D, PAGE) ||
        !rfx::tma::make_map_rows64(&mv, v_pages, kv_rows, D, PAGE))
        return RFX_ERR_UNSUPPORTED;
    const size_t smem = Smem::total(D);
    auto kernel = attention_prefill_tc_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    if ((max_new + bq - 1) / bq > 65535 || S > 65535) return RFX_ERR_UNSUPPORTED;
    dim3 grid(cache.n_kv_heads, S, (max_new + bq - 1) / bq);
    if (grid.y > 65535 || grid.z > 65535) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(kernel, grid, THREADS, smem, s, mq, mk, mv, cache, seq_slot, seq_start, seq_new, seq_row0,
               (__nv_bfloat16*)out, nq, bq, window, scale * 1.4426950408889634f, err);
    return 0;
}

}  // namespace

// As rfx_attention_prefill, for head_dim 64 or 128.  `n_pages_total` is the
// number of pages of the K/V store (for the TMA maps), R the number of rows of
// q.  `err` is a device word that receives a code if a bounded wait ran out.
// Tuning aid: 32 64-bit timestamps per CTA of the launches that follow (null
// switches it off).
extern "C" int rfx_attention_prefill_tc_trace(void* buffer, int ctas) {
    unsigned long long* p = (unsigned long long*)buffer;
    cudaError_t e = cudaMemcpyToSymbol(g_trace, &p, sizeof(p));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_ctas, &ctas, sizeof(int));
    return (int)e;
}

extern "C" int rfx_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages,
                                        long long n_pages_total, const int* page_table, int max_pages,
                                        int page_size, const int* seq_slot, const int* seq_start,
                                        const int* seq_new, const int* seq_row0, void* out, int S,
                                        int max_new, int R, int nq, int nkv, int head_dim, int window,
                                        float scale, int* err, void* stream) {
    if (S <= 0 || max_new <= 0 || R <= 0) return 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0) return RFX_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pages) |
         reinterpret_cast<uintptr_t>(v_pages)) & 15)
        return RFX_ERR_BAD_ARG;
    PagedKV cache{page_table, max_pages, page_size, nkv, head_dim};
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64)
        return launch_tc<64>(q, k_pages, v_pages, n_pages_total, cache, seq_slot, seq_start, seq_new,
                             seq_row0, out, S, max_new, R, nq, window, scale, err, s);
    if (head_dim == 128)
        return launch_tc<128>(q, k_pages, v_pages, n_pages_total, cache, seq_slot, seq_start, seq_new,
                              seq_row0, out, S, max_new, R, nq, window, scale, err, s);
    return RFX_ERR_UNSUPPORTED;
}
