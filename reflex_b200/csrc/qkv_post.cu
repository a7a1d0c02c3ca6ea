// After the q/k/v projections, per row and head: per-head RMSNorm of q and k,
// rotary position encoding, then q to the workspace and k, v into the paged
// cache at the row's position.  One launch instead of the reference's five
// (norm x2, rope x2, cache store: src/model/dense.rs:1355-1409; decode:
// src/model/decode_step.rs:232-279).
//
// Formulas.  Norm: y = (x * r) * w, r = 1/sqrt(mean(x^2) + eps), one weight
// vector of head_dim shared by all heads (src/kernels_cuda/decode_ops.cu:40-71).
// Rotary, half-split pairs (i, i + rd/2) for i < rd/2
// (src/kernels_cuda/rope.cu:9-37):  theta = (float)pos / denom[i] with
// denom[i] = base^(2i/rd);  (a, b) <- (a cos - b sin, a sin + b cos).
// With consecutive pairing the pairs are (2i, 2i + 1) instead
// (src/model/config.rs:15-28).  cos and sin are multiplied by `magnitude` (1 for
// the plain encoding; a frequency-scaled encoding's attention factor,
// src/model/kernels.rs:3086-3129).  Elements >= rd stay.  v is stored as
// projected.  All arithmetic is 32-bit; the angle is a 32-bit division; in the
// 32-bit form its sine and cosine come from `exact_sincosf`, whose bits a host
// program can repeat, in the bfloat16 forms from sincosf.
//
// Orders of the 32-bit form (32-bit in, 32-bit out: always the general kernel),
// which a host mirror repeats: a head's sum of squares as a fused multiply-add
// chain per lane over elements lane, lane + 32, ..., then the lanes' butterfly;
// y = (x * r) * (offset + w); the rotation as fma(partner, -+sin, x * cos) with
// the product x * cos rounded first.
#include "common.cuh"
#include "exact_math.cuh"
#include "paged.cuh"

#define RFX_PAIR_HALF 0
#define RFX_PAIR_CONSECUTIVE 1

namespace {

using namespace rfx;

constexpr int MAX_PER_LANE = 16;  // head_dim <= 512

// Sine and cosine of a row's angle.  The 32-bit form takes the routine whose bits
// a host program can repeat (its range reduction runs in double precision, which
// this GPU executes at a small fraction of its 32-bit rate); a result that is
// rounded to bfloat16 takes the library's 32-bit routine, as every bfloat16
// kernel that rotates does, so that prefill and decode rotate alike.
template <typename TO>
__device__ __forceinline__ void row_sincos(float theta, float* sv, float* cv) {
    if constexpr (sizeof(TO) == 2) sincosf(theta, sv, cv);
    else exact_sincosf(theta, sv, cv);
}

template <typename T, int N>
struct alignas(sizeof(T) * N <= 16 ? sizeof(T) * N : 16) Pack {
    T a[N];
};

// Unpacking and packing a lane's elements; 16-bit floats are converted in pairs.
template <typename T, int N>
__device__ __forceinline__ void unpack(const Pack<T, N>& p, float (&v)[N]) {
    if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&p.a[i]));
            v[i] = f.x;
            v[i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = p.a[i];
    }
}
template <typename T, int N>
__device__ __forceinline__ void pack(const float (&v)[N], Pack<T, N>& p) {
    if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int i = 0; i < N; i += 2)
            *reinterpret_cast<__nv_bfloat162*>(&p.a[i]) = __floats2bfloat162_rn(v[i], v[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) p.a[i] = v[i];
    }
}

// The wide form, for head sizes that are a power of two.  A head vector lies in
// LPH neighbouring lanes, PER neighbouring elements each (head_dim = LPH * PER),
// moved with one wide access; a warp takes 32 / LPH heads of one kind (query, key
// or value) at a time, a "unit".  A rotary pair (e, e + rd/2) lies in two lanes of
// the head's group at the same place of their packs and is exchanged by a shuffle
// (rd/2 a multiple of PER).  What a lane needs for every head of the row (its norm
// weights, its sines and cosines, the row's place in the cache) is fetched once
// per block.  The mean is taken by a multiplication with 1/head_dim, which for a
// power of two gives the quotient's bits.
template <typename TI, typename TO, int PER, int LPH>
__global__ void __launch_bounds__(256, 4)
qkv_post_wide_kernel(const TI* __restrict__ qkv, int row_stride, const float* __restrict__ q_w,
                     const float* __restrict__ k_w, float eps, float w_offset,
                     const float* __restrict__ rope_denom, int rotary_dim,
                     const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                     TO* __restrict__ q_out, TO* __restrict__ k_pages, TO* __restrict__ v_pages,
                     PagedKV cache, int nq, int nkv_in, int dry_pass, float magnitude) {
    extern __shared__ float smem[];  // cos[half], sin[half]
    pdl_launch_dependents();
    constexpr int D = PER * LPH;
    constexpr int HPW = 32 / LPH;  // heads a warp takes at a time
    constexpr int CH = 3;          // units whose loads are in flight together
    constexpr float inv_d = 1.0f / (float)D;
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int half = rotary_dim / 2;
    const bool rotate = rope_denom != nullptr && half > 0;
    const int sub = lane / LPH;          // which of the unit's heads
    const int e0 = (lane % LPH) * PER;   // this lane's first element of the head
    const bool turns = rotate && e0 < rotary_dim;  // a pack lies on one side of the rotation
    const bool low = e0 < half;
    const int hl = half / PER;  // lanes in half a rotation
    const int partner = turns ? (low ? lane + hl : lane - hl) : lane;
    // units: the query heads in groups of HPW, then the key heads, then the value heads
    const int uq = (nq + HPW - 1) / HPW, ukv = (nkv_in + HPW - 1) / HPW;
    const int units = uq + 2 * ukv;
    const int stride = gridDim.y * nwarps;
    const int first = blockIdx.y * nwarps + warp;

    // what a lane needs for every head of the row, filled in by `prepare`
    float sn[PER], cs[PER], wq[PER];  // (the few key heads fetch their weights when they come)
    size_t kv0 = 0;
    const size_t kv_head_stride = (size_t)cache.page_size * D;

    // The rotation of the row's position, once for all heads of the block, the
    // norm weights and the row's place in the cache.  Positions are the step's
    // inputs, so none of this waits for the preceding kernel.
    auto prepare = [&]() {
        const int pos = row_pos[r];
        const int slot = row_slot[r];
        float* cs_tab = smem;
        float* sn_tab = cs_tab + half;
        if (rotate) {
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float theta = (float)pos / rope_denom[i];
                float sv, cv;
                row_sincos<TO>(theta, &sv, &cv);
                sn_tab[i] = sv * magnitude;
                cs_tab[i] = cv * magnitude;
            }
        }
        // head 0's place; the other heads lie a tile apart
        kv0 = nkv_in > 0 ? kv_offset(cache, slot, pos, 0) : 0;
#pragma unroll
        for (int i = 0; i < PER; ++i) sn[i] = cs[i] = wq[i] = 0.0f;
        if (q_w) unpack(*reinterpret_cast<const Pack<float, PER>*>(q_w + e0), wq);
#pragma unroll
        for (int i = 0; i < PER; ++i) wq[i] += w_offset;
        __syncthreads();
        if (turns) {
            unpack(*reinterpret_cast<const Pack<float, PER>*>(sn_tab + (low ? e0 : e0 - half)), sn);
            unpack(*reinterpret_cast<const Pack<float, PER>*>(cs_tab + (low ? e0 : e0 - half)), cs);
        }
        if (low) {  // the lower half subtracts the partner's product: the sign goes into the sine
#pragma unroll
            for (int i = 0; i < PER; ++i) sn[i] = -sn[i];
        }
    };

    // kind of unit u (the same for the whole warp) and this lane's head in it
    auto unit_kind = [&](int u) { return u < uq ? 0 : (u < uq + ukv ? 1 : 2); };
    // the loads of up to CH units, from `src_row` (the row of qkv, or the dry source)
    auto fetch = [&](int u0, Pack<TI, PER> (&in)[CH], int (&head)[CH], bool dry, const TI* dry_src) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int u = u0 + c * stride;
            head[c] = -1;  // nothing for this lane
            if (u < units && !(dry && c > 0)) {
                const int k = unit_kind(u);
                const int h = (k == 0 ? u : (k == 1 ? u - uq : u - uq - ukv)) * HPW + sub;
                if (h < (k == 0 ? nq : nkv_in)) {
                    head[c] = h;
                    const int hh = k == 0 ? h : (k == 1 ? nq + h : nq + nkv_in + h);
                    const TI* src = dry ? dry_src : qkv + (size_t)r * row_stride + (size_t)hh * D;
                    in[c] = *reinterpret_cast<const Pack<TI, PER>*>(src + e0);
                }
            }
        }
    };
    auto finish = [&](int u0, const Pack<TI, PER> (&in)[CH], const int (&head)[CH], bool dry) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int u = u0 + c * stride;
            if (u >= units || (dry && c > 0)) break;
            const int k = unit_kind(u);
            float v[PER];
            if (head[c] >= 0) {
                unpack(in[c], v);
            } else {
#pragma unroll
                for (int i = 0; i < PER; ++i) v[i] = 0.0f;
            }
            if (k < 2) {
                if (k == 0 ? q_w != nullptr : k_w != nullptr) {
                    float ss = 0.0f;
#pragma unroll
                    for (int i = 0; i < PER; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
                    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    const float rinv = 1.0f / sqrtf(ss * inv_d + eps);
                    if (k == 0) {
#pragma unroll
                        for (int i = 0; i < PER; ++i) v[i] = (v[i] * rinv) * wq[i];
                    } else {
                        float wk[PER];
                        unpack(*reinterpret_cast<const Pack<float, PER>*>(k_w + e0), wk);
#pragma unroll
                        for (int i = 0; i < PER; ++i) v[i] = (v[i] * rinv) * (w_offset + wk[i]);
                    }
                }
                if (rotate) {
#pragma unroll
                    for (int i = 0; i < PER; ++i) {
                        const float other = __shfl_sync(0xffffffffu, v[i], partner);
                        // low: v cos - other sin;  high: other sin + v cos
                        if (turns) v[i] = fmaf(other, sn[i], v[i] * cs[i]);
                    }
                }
            }
            if (head[c] >= 0 && !dry) {
                TO* dst = (k == 0 ? q_out + ((size_t)r * nq + head[c]) * D
                                  : (k == 1 ? k_pages : v_pages) + kv0 + (size_t)head[c] * kv_head_stride) + e0;
                Pack<TO, PER> o;
                pack(v, o);
                *reinterpret_cast<Pack<TO, PER>*>(dst) = o;
            }
        }
    };

    Pack<TI, PER> in[CH];
    int head[CH];
    int u0 = first;
    const TI* dry_src = reinterpret_cast<const TI*>(q_w ? q_w : k_w);
    if (dry_src && dry_pass) {
        // Decode-sized launches: the row's tables first, then a dry pass before the
        // wait on the preceding kernel.  It takes a norm weight vector for its input
        // (never the other kernel's output), does one unit and stores nothing; it
        // brings the instructions into the cache.
        prepare();
        if (u0 < units) {
            fetch(u0, in, head, true, dry_src);
            finish(u0, in, head, true);
        }
        pdl_wait();
    } else {
        // Many rows: the row's first loads are issued before its tables are made.
        pdl_wait();
        if (u0 < units) fetch(u0, in, head, false, nullptr);
        prepare();
        if (u0 < units) finish(u0, in, head, false);
        u0 += stride * CH;
    }
#pragma unroll 1
    for (; u0 < units; u0 += stride * CH) {
        fetch(u0, in, head, false, nullptr);
        finish(u0, in, head, false);
    }
}

// The general form.  PER: elements of a head vector per lane, head_dim <= 32 * PER;
// lane l holds elements l, l + 32, ... and a rotary pair is exchanged through
// shared memory.  One warp per (row, head).
template <typename TI, typename TO, int PER>
__global__ void __launch_bounds__(256)
qkv_post_kernel(const TI* __restrict__ qkv, int row_stride, const float* __restrict__ q_w,
                const float* __restrict__ k_w, float eps, float w_offset,
                const float* __restrict__ rope_denom, int rotary_dim,
                const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                TO* __restrict__ q_out, TO* __restrict__ k_pages, TO* __restrict__ v_pages,
                PagedKV cache, int nq, int nkv_in, int dry_pass, int pairing, float magnitude) {
    extern __shared__ float smem[];  // [warps][head_dim], then cos[half], sin[half]
    pdl_launch_dependents();
    const int d = cache.head_dim;
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int pos = row_pos[r];
    const int slot = row_slot[r];
    float* buf = smem + warp * d;
    const int half = rotary_dim / 2;
    const int total = nq + 2 * nkv_in;
    // the row's rotation, once for all heads of the block; positions are the
    // step's inputs, so this does not wait for the preceding kernel
    float* cs_tab = smem + nwarps * d;
    float* sn_tab = cs_tab + half;
    const bool rotate = rope_denom != nullptr && half > 0;
    if (rotate) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float theta = (float)pos / rope_denom[i];
            float sv, cv;
            row_sincos<TO>(theta, &sv, &cv);
            sn_tab[i] = sv * magnitude;
            cs_tab[i] = cv * magnitude;
        }
    }
    // where this row's key and value heads go: head 0's place, the others a tile apart
    const size_t kv0 = nkv_in > 0 ? kv_offset(cache, slot, pos, 0) : 0;
    const size_t kv_head_stride = (size_t)cache.page_size * d;
    __syncthreads();
    const int stride = gridDim.y * nwarps;
    auto destination = [&](int hh) -> TO* {
        if (hh < nq) return q_out + ((size_t)r * nq + hh) * d;
        if (hh < nq + nkv_in) return k_pages + kv0 + (size_t)(hh - nq) * kv_head_stride;
        return v_pages + kv0 + (size_t)(hh - nq - nkv_in) * kv_head_stride;
    };

    // Two passes over the same code.  The first, before the wait on the preceding
    // kernel, is a dry one (decode-sized launches only): it takes a norm weight
    // vector for its input (never the other kernel's output), does one head and
    // stores nothing; it brings the instructions into the cache.  The second is
    // the work.
    const TI* dry_src = reinterpret_cast<const TI*>(q_w ? q_w : k_w);
#pragma unroll 1
    for (int pass = (dry_src && dry_pass) ? 0 : 1; pass < 2; ++pass) {
        const bool dry = pass == 0;
        if (!dry) pdl_wait();
        // one warp per (row, head): blockIdx.y walks the heads in groups of nwarps
        for (int hh = blockIdx.y * nwarps + warp; hh < total; hh += stride) {
            if (dry && hh >= stride) break;
            const TI* src = dry ? dry_src : qkv + (size_t)r * row_stride + (size_t)hh * d;
            const bool is_q = hh < nq, is_k = !is_q && hh < nq + nkv_in;
            TO* dst = destination(hh);
            if (!is_q && !is_k) {  // v: stored as projected
                for (int e = lane; e < d; e += 32)
                    if (!dry) st<TO>(dst, e, ld<TI>(src, e));
                continue;
            }
            float v[PER];
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = i * 32 + lane;
                v[i] = e < d ? ld<TI>(src, e) : 0.0f;
                ss = fmaf(v[i], v[i], ss);
            }
            const float* w = is_q ? q_w : k_w;
            if (w) {
                const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int e = i * 32 + lane;
                    if (e < d) v[i] = (v[i] * rinv) * (w_offset + w[e]);
                }
            }
            if (!rotate) {
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int e = i * 32 + lane;
                    if (e < d && !dry) st<TO>(dst, e, v[i]);
                }
                continue;
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = i * 32 + lane;
                if (e < d) buf[e] = v[i];
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = i * 32 + lane;
                if (e >= d) break;
                float o = v[i];
                if (e < rotary_dim) {
                    // the pair's first element takes -sin, its second +sin
                    int fi, other;
                    bool first_of_pair;
                    if (pairing == RFX_PAIR_CONSECUTIVE) {
                        fi = e >> 1;
                        first_of_pair = (e & 1) == 0;
                        other = e ^ 1;
                    } else {
                        first_of_pair = e < half;
                        fi = first_of_pair ? e : e - half;
                        other = first_of_pair ? e + half : e - half;
                    }
                    const float sn = sn_tab[fi], cs = cs_tab[fi];
                    o = fmaf(buf[other], first_of_pair ? -sn : sn, __fmul_rn(v[i], cs));
                }
                if (!dry) st<TO>(dst, e, o);
            }
        }
    }
}

}  // namespace

extern "C" int rfx_qkv_post(const void* qkv, int in_dt, int row_stride, const float* q_w,
                            const float* k_w, float eps, float w_offset, const float* rope_denom,
                            int rotary_dim, const int* row_pos, const int* row_slot, void* q_out,
                            void* k_pages, void* v_pages, int out_dt, const int* page_table,
                            int max_pages, int page_size, int R, int nq, int nkv_in, int nkv,
                            int head_dim, int pairing, float magnitude, void* stream) {
    if (R <= 0) return 0;
    if (pairing != RFX_PAIR_HALF && pairing != RFX_PAIR_CONSECUTIVE) return RFX_ERR_BAD_ARG;
    if (head_dim <= 0 || head_dim > 32 * MAX_PER_LANE) return RFX_ERR_UNSUPPORTED;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return RFX_ERR_BAD_ARG;
    if (nkv_in != 0 && nkv_in != nkv) return RFX_ERR_BAD_ARG;
    PagedKV cache{page_table, max_pages, page_size, nkv, head_dim};
    const int threads = 256;
    const int warps = threads / 32;
    cudaStream_t s = (cudaStream_t)stream;
    // Few rows (decode): a row's heads spread over several blocks, with a dry
    // pass.  Many rows (prefill): one block a row, and no dry pass (the code is
    // warm after the first blocks).
    const bool many = R >= 256;
    const int dry_pass = many ? 0 : 1;
    const int in_size = in_dt == RFX_DT_F32 ? 4 : 2;
    // the wide form: a power of two of elements, 16 bytes of the input a lane where 32 lanes reach
    const bool pow2 = head_dim >= 16 && (head_dim & (head_dim - 1)) == 0;
    int per = 16 / in_size;
    if (pow2 && head_dim / per > 32) per = head_dim / 32;
    const int lph = pow2 ? head_dim / per : 0;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                           reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages) |
                           reinterpret_cast<uintptr_t>(q_w) | reinterpret_cast<uintptr_t>(k_w);
    // (the 32-bit form keeps to the general kernel's one order; so does consecutive pairing)
    const bool rotates = rope_denom != nullptr && rotary_dim > 0;
    const bool wide = pow2 && (!rotates || ((rotary_dim / 2) % per == 0 && pairing == RFX_PAIR_HALF)) &&
                      row_stride % per == 0 && (ptrs & 15) == 0 &&
                      !(in_dt == RFX_DT_F32 && out_dt == RFX_DT_F32);
#define RFX_POST_ARGS(TI, TO)                                                                       \
    (const TI*)qkv, row_stride, q_w, k_w, eps, w_offset, rope_denom, rotary_dim, row_pos, row_slot, \
        (TO*)q_out, (TO*)k_pages, (TO*)v_pages, cache, nq, nkv_in, dry_pass
    if (wide) {
        const int hpw = 32 / lph;
        const int units = (nq + hpw - 1) / hpw + 2 * ((nkv_in + hpw - 1) / hpw);
        const int unit_blocks = many ? 1 : (units + warps - 1) / warps;
        dim3 grid(R, unit_blocks < 65535 ? unit_blocks : 65535);
        const size_t smem = (size_t)rotary_dim * sizeof(float);
#define RFX_WIDE(TI, TO, P, L)                                                                    \
    RFX_LAUNCH((qkv_post_wide_kernel<TI, TO, P, L>), grid, threads, smem, s, RFX_POST_ARGS(TI, TO), magnitude)
#define RFX_WIDE_32(TI, TO)  /* 32-bit input: 4 elements are 16 bytes */   \
    do {                                                                  \
        if (per == 4 && lph == 4) RFX_WIDE(TI, TO, 4, 4);                 \
        else if (per == 4 && lph == 8) RFX_WIDE(TI, TO, 4, 8);            \
        else if (per == 4 && lph == 16) RFX_WIDE(TI, TO, 4, 16);          \
        else if (per == 4 && lph == 32) RFX_WIDE(TI, TO, 4, 32);          \
        else if (per == 8 && lph == 32) RFX_WIDE(TI, TO, 8, 32);          \
        else if (per == 16 && lph == 32) RFX_WIDE(TI, TO, 16, 32);        \
        else return RFX_ERR_UNSUPPORTED;                                  \
    } while (0)
#define RFX_WIDE_16(TI, TO)  /* 16-bit input: 8 elements are 16 bytes */   \
    do {                                                                  \
        if (per == 8 && lph == 2) RFX_WIDE(TI, TO, 8, 2);                 \
        else if (per == 8 && lph == 4) RFX_WIDE(TI, TO, 8, 4);            \
        else if (per == 8 && lph == 8) RFX_WIDE(TI, TO, 8, 8);            \
        else if (per == 8 && lph == 16) RFX_WIDE(TI, TO, 8, 16);          \
        else if (per == 8 && lph == 32) RFX_WIDE(TI, TO, 8, 32);          \
        else if (per == 16 && lph == 32) RFX_WIDE(TI, TO, 16, 32);        \
        else return RFX_ERR_UNSUPPORTED;                                  \
    } while (0)
        if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_BF16) RFX_WIDE_32(float, __nv_bfloat16);
        else if (in_dt == RFX_DT_BF16 && out_dt == RFX_DT_BF16) RFX_WIDE_16(__nv_bfloat16, __nv_bfloat16);
        else return RFX_ERR_BAD_ARG;
#undef RFX_WIDE_32
#undef RFX_WIDE_16
#undef RFX_WIDE
        return 0;
    }
    // the general form: a warp per head, eight heads at a time
    const int head_blocks = many ? 1 : (nq + 2 * nkv_in + warps - 1) / warps;
    const size_t smem = ((size_t)warps * head_dim + rotary_dim) * sizeof(float);
    dim3 grid(R, head_blocks < 65535 ? head_blocks : 65535);
#define RFX_POST(TI, TO)                                                                              \
    do {                                                                                              \
        if (head_dim <= 32) RFX_LAUNCH((qkv_post_kernel<TI, TO, 1>), grid, threads, smem, s, RFX_POST_ARGS(TI, TO), pairing, magnitude);        \
        else if (head_dim <= 64) RFX_LAUNCH((qkv_post_kernel<TI, TO, 2>), grid, threads, smem, s, RFX_POST_ARGS(TI, TO), pairing, magnitude);   \
        else if (head_dim <= 128) RFX_LAUNCH((qkv_post_kernel<TI, TO, 4>), grid, threads, smem, s, RFX_POST_ARGS(TI, TO), pairing, magnitude);  \
        else if (head_dim <= 256) RFX_LAUNCH((qkv_post_kernel<TI, TO, 8>), grid, threads, smem, s, RFX_POST_ARGS(TI, TO), pairing, magnitude);  \
        else RFX_LAUNCH((qkv_post_kernel<TI, TO, 16>), grid, threads, smem, s, RFX_POST_ARGS(TI, TO), pairing, magnitude);                      \
    } while (0)
    if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_F32) RFX_POST(float, float);
    else if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_BF16) RFX_POST(float, __nv_bfloat16);
    else if (in_dt == RFX_DT_BF16 && out_dt == RFX_DT_BF16) RFX_POST(__nv_bfloat16, __nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_POST
#undef RFX_POST_ARGS
    return 0;
}
