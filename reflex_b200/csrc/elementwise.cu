// Embedding gather, RMSNorm with the residual add, SwiGLU.
//
// Statistics and the residual stream are 32-bit in both precisions; only what
// feeds a matrix product is rounded to bfloat16 on the bfloat16 path.
#include "common.cuh"

namespace {

using namespace rfx;

// hidden[r, :] = table[ids[r], :] * scale       (src/model/dense.rs:1959-1967)
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int H, int V, float scale,
                             int* __restrict__ err) {
    // The first kernel of every step.  It does not let its dependents start
    // early: kernels of this step may read, before their own wait, cache pages
    // that earlier steps wrote, so no kernel of this step may run before every
    // kernel of the step before has completed, which this kernel's wait ensures.
    pdl_wait();
    const int r = blockIdx.x;
    const int id = ids[r];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicExch(err, 1 + r);
        for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)r * H + c] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[(size_t)r * H + c] = ld<T>(row, c) * scale;
}

// One block per output row.
//   src = rows ? rows[blockIdx.x] : blockIdx.x
//   t   = x[src] (+ delta[src])                     residual sum in 32-bit
//   if x_out: x_out[src] = t                        (only without `rows`; may be x)
//   if out:   out[blockIdx.x] = t * rsqrt(mean(t^2) + eps) * (w_offset + w)
// The sum of squares runs in an order fixed by the block size, which the host
// derives from H alone, so a row's result does not depend on the batch.
// Formula: src/kernels_cuda/rmsnorm.cuh:14-40, rmsnorm.cu:44-52; the fused add
// is src/kernels_cuda/decode_ops.cu:10-35.
template <typename TD, typename TO>
__global__ void rmsnorm_kernel(const float* x, const TD* __restrict__ delta,
                               float* x_out, const float* __restrict__ w,
                               TO* __restrict__ out, const int* __restrict__ rows, int H,
                               float eps, float w_offset) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float row_buf[];  // H floats
    pdl_prologue();
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + (size_t)src * H;
    float ss = 0.0f;
    const bool vec = (H & 3) == 0;  // rows then start on 16-byte boundaries
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            float4 t = x4[c];
            if (delta) {
                t.x += ld<TD>(delta, (size_t)src * H + 4 * c);
                t.y += ld<TD>(delta, (size_t)src * H + 4 * c + 1);
                t.z += ld<TD>(delta, (size_t)src * H + 4 * c + 2);
                t.w += ld<TD>(delta, (size_t)src * H + 4 * c + 3);
            }
            reinterpret_cast<float4*>(row_buf)[c] = t;
            if (x_out) reinterpret_cast<float4*>(x_out + (size_t)src * H)[c] = t;
            ss = fmaf(t.x, t.x, ss);
            ss = fmaf(t.y, t.y, ss);
            ss = fmaf(t.z, t.z, ss);
            ss = fmaf(t.w, t.w, ss);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float t = xr[c];
            if (delta) t += ld<TD>(delta, (size_t)src * H + c);
            row_buf[c] = t;
            if (x_out) x_out[(size_t)src * H + c] = t;
            ss = fmaf(t, t, ss);
        }
    }
    if (!out) return;
    const float total = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(total / (float)H + eps);
    TO* orow = out + (size_t)blockIdx.x * H;
    if (vec) {
        for (int c = threadIdx.x; c < H / 4; c += blockDim.x) {
            const float4 t = reinterpret_cast<const float4*>(row_buf)[c];
            const float4 ww = reinterpret_cast<const float4*>(w)[c];
            store4(orow + 4 * c, make_float4((t.x * r) * (w_offset + ww.x), (t.y * r) * (w_offset + ww.y),
                                             (t.z * r) * (w_offset + ww.z), (t.w * r) * (w_offset + ww.w)));
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x)
            st<TO>(orow, c, (row_buf[c] * r) * (w_offset + w[c]));
    }
}

// out[r, i] = silu(gate_i) * up_i,  silu(g) = g / (1 + exp(-g))
// (src/kernels_cuda/silu_and_mul.cu:7-23).  A row of `gu` holds the gates in its
// first half and the ups in its second, or (alternating) gate_i at 2i, up_i at 2i+1.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int R, int I,
                              int alternating) {
    pdl_prologue();
    const size_t n = (size_t)R * I;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / I, c = i % I;
        const float g = ld<T>(gu, r * 2 * I + (alternating ? 2 * c : c));
        const float u = ld<T>(gu, r * 2 * I + (alternating ? 2 * c + 1 : I + c));
        st<T>(out, i, silu_mul_for<T>(g, u));
    }
}

// bfloat16, I a multiple of 8: eight outputs a thread and step, 16-byte loads and
// stores, two steps' loads in flight.  With alternating pairs a row's 2I inputs
// and I outputs are contiguous and rows follow one another, so output pack i
// comes from input elements [16 i, 16 i + 16).
__device__ __forceinline__ uint4 swiglu8(const uint4 a, const uint4 b, bool alternating) {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
    if (alternating) {  // a = g0 u0 g1 u1 g2 u2 g3 u3, b = g4 u4 ...
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 p0 = __bfloat1622float2(pa[2 * j]), p1 = __bfloat1622float2(pa[2 * j + 1]);
            const float2 q0 = __bfloat1622float2(pb[2 * j]), q1 = __bfloat1622float2(pb[2 * j + 1]);
            po[j] = __floats2bfloat162_rn(silu_mul_for<__nv_bfloat16>(p0.x, p0.y),
                                          silu_mul_for<__nv_bfloat16>(p1.x, p1.y));
            po[2 + j] = __floats2bfloat162_rn(silu_mul_for<__nv_bfloat16>(q0.x, q0.y),
                                              silu_mul_for<__nv_bfloat16>(q1.x, q1.y));
        }
    } else {  // a = eight gates, b = their ups
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(pa[j]), up = __bfloat1622float2(pb[j]);
            po[j] = __floats2bfloat162_rn(silu_mul_for<__nv_bfloat16>(g.x, up.x),
                                          silu_mul_for<__nv_bfloat16>(g.y, up.y));
        }
    }
    return o;
}

__global__ void __launch_bounds__(256)
swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int R, int I,
                     int alternating) {
    pdl_prologue();
    const size_t n8 = (size_t)R * (I / 8);
    const size_t step = (size_t)gridDim.x * blockDim.x;
    const unsigned i8 = (unsigned)(I / 8);
    auto sources = [&](size_t i, const uint4*& a, const uint4*& b) {
        if (alternating) {
            a = reinterpret_cast<const uint4*>(gu + 16 * i);
            b = a + 1;
        } else {
            const size_t r = i / i8, c = (i - r * i8) * 8;
            a = reinterpret_cast<const uint4*>(gu + r * 2 * I + c);
            b = reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c);
        }
    };
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + step < n8; i += 2 * step) {
        const uint4 *a0, *b0, *a1, *b1;
        sources(i, a0, b0);
        sources(i + step, a1, b1);
        const uint4 va0 = *a0, vb0 = *b0, va1 = *a1, vb1 = *b1;
        *reinterpret_cast<uint4*>(out + 8 * i) = swiglu8(va0, vb0, alternating);
        *reinterpret_cast<uint4*>(out + 8 * (i + step)) = swiglu8(va1, vb1, alternating);
    }
    if (i < n8) {
        const uint4 *a0, *b0;
        sources(i, a0, b0);
        *reinterpret_cast<uint4*>(out + 8 * i) = swiglu8(*a0, *b0, alternating);
    }
}

// y[i] = a[i] + b[i] in 32-bit (src/kernels_cuda/elementwise.cu:8-24)
template <typename T>
__global__ void add_kernel(float* __restrict__ a, const T* __restrict__ b, size_t n) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        a[i] += ld<T>(b, i);
}

// A function of H alone, so that a row's sum of squares is reduced in the same
// order whatever the batch.
int norm_threads(int H) {
    int t = ((H + 15) / 16 + 31) / 32 * 32;  // about four 16-byte loads a thread
    if (t < 32) t = 32;
    if (t > 256) t = 256;
    return t;
}

}  // namespace

extern "C" int rfx_embed(const void* table, int table_dt, const int* ids, int R, int H, int V,
                         float scale, float* out, int* err, void* stream) {
    if (R <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dt == RFX_DT_F32)
        RFX_LAUNCH(embed_kernel<float>, R, threads, 0, s, (const float*)table, ids, out, H, V, scale, err);
    else if (table_dt == RFX_DT_BF16)
        RFX_LAUNCH(embed_kernel<__nv_bfloat16>, R, threads, 0, s, (const __nv_bfloat16*)table, ids, out,
                   H, V, scale, err);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_rmsnorm(const float* x, const void* delta, int delta_dt, float* x_out,
                           const float* w, float eps, float w_offset, void* out, int out_dt,
                           const int* rows, int R_out, int H, void* stream) {
    if (R_out <= 0) return 0;
    if (rows && x_out) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = norm_threads(H);
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
#define RFX_NORM(TD, TO)                                                                       \
    do {                                                                                       \
        if (smem > 48 * 1024) {                                                                \
            cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<TD, TO>,                       \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                 (int)smem);                                   \
            if (e != cudaSuccess) return (int)e;                                               \
        }                                                                                      \
        RFX_LAUNCH((rmsnorm_kernel<TD, TO>), R_out, threads, smem, s, x, (const TD*)delta, x_out, \
                   w, (TO*)out, rows, H, eps, w_offset);                                       \
    } while (0)
    const bool dbf = delta && delta_dt == RFX_DT_BF16;
    if (out_dt == RFX_DT_BF16) {
        if (dbf) RFX_NORM(__nv_bfloat16, __nv_bfloat16);
        else RFX_NORM(float, __nv_bfloat16);
    } else if (out_dt == RFX_DT_F32) {
        if (dbf) RFX_NORM(__nv_bfloat16, float);
        else RFX_NORM(float, float);
    } else {
        return RFX_ERR_BAD_ARG;
    }
#undef RFX_NORM
    return 0;
}

extern "C" int rfx_swiglu(const void* gate_up, void* out, int dt, int R, int I, int alternating,
                          void* stream) {
    if (R <= 0 || I <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)R * I;
    int blocks = (int)((n + 255) / 256);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(swiglu_kernel<float>, blocks, 256, 0, s, (const float*)gate_up, (float*)out, R, I,
                   alternating);
    else if (dt == RFX_DT_BF16 && I % 8 == 0 &&
             ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        int b8 = (int)((n / 8 + 255) / 256);
        if (b8 > sm_count() * 8) b8 = sm_count() * 8;
        RFX_LAUNCH(swiglu_bf16x8_kernel, b8, 256, 0, s, (const __nv_bfloat16*)gate_up,
                   (__nv_bfloat16*)out, R, I, alternating);
    } else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(swiglu_kernel<__nv_bfloat16>, blocks, 256, 0, s, (const __nv_bfloat16*)gate_up,
                   (__nv_bfloat16*)out, R, I, alternating);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_add(float* a, const void* b, int b_dt, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int blocks = (int)((n + 255) / 256);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    if (b_dt == RFX_DT_F32)
        RFX_LAUNCH(add_kernel<float>, blocks, 256, 0, s, a, (const float*)b, (size_t)n);
    else if (b_dt == RFX_DT_BF16)
        RFX_LAUNCH(add_kernel<__nv_bfloat16>, blocks, 256, 0, s, a, (const __nv_bfloat16*)b, (size_t)n);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" const char* rfx_error_string(int code) {
    if (code == RFX_ERR_BAD_ARG) return "bad argument";
    if (code == RFX_ERR_UNSUPPORTED) return "size not supported by this kernel";
    if (code == RFX_ERR_TIMEOUT) return "bounded device wait ran out";
    if (code == RFX_ERR_SCRATCH) return "the call needs more scratch than the built-in array holds";
    return cudaGetErrorString((cudaError_t)code);
}
