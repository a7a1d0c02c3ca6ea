// Matrix products  y[r, n] = sum_k x[r, k] * W[n, k]   (W row-major [out, in],
// the layout of the reference's linear layers: src/kernels_cuda/gemv.cu:1-4).
//
//  * rfx_gemm_f32: the true 32-bit product.  CUDA-core fused multiply-adds
//    only; each output element is reduced over k = 0..K-1 in index order by one
//    thread, so its value does not depend on how many rows the call has or on
//    where the row sits in the batch.
//  * rfx_gemv_bf16: bfloat16 weights and activations for a few rows (decode),
//    32-bit accumulation; a pure weight-streaming kernel with 16-byte loads.
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ y,
                int R, int N, int K) {
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[TK][TN + 1];
    pdl_prologue();
    const int r0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int row = e / TK, kk = e % TK;
            const int k = k0 + kk;
            xs[kk][row] = (r0 + row < R && k < K) ? x[(size_t)(r0 + row) * K + k] : 0.0f;
            ws[kk][row] = (n0 + row < N && k < K) ? W[(size_t)(n0 + row) * K + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty * 4 + i;
        if (r >= R) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[(size_t)r * N + n] = acc[i][j];
        }
    }
}

// One warp per output column n; RT rows of x per pass.  K must be a multiple
// of 8 (16-byte loads); the host refuses other K.
template <int RT, typename TO>
__global__ void __launch_bounds__(256)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                 TO* __restrict__ y, int R, int N, int K) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)n * K);
    const int kv = K / 8;
    for (int r0 = 0; r0 < R; r0 += RT) {
        float acc[RT];
#pragma unroll
        for (int i = 0; i < RT; ++i) acc[i] = 0.0f;
        for (int c = lane; c < kv; c += 32) {
            const uint4 wv = wrow[c];
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
            float wf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(w2[j]);
                wf[2 * j] = f.x;
                wf[2 * j + 1] = f.y;
            }
#pragma unroll
            for (int i = 0; i < RT; ++i) {
                if (r0 + i < R) {
                    const uint4 xv = reinterpret_cast<const uint4*>(x + (size_t)(r0 + i) * K)[c];
                    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(x2[j]);
                        acc[i] = fmaf(wf[2 * j], f.x, acc[i]);
                        acc[i] = fmaf(wf[2 * j + 1], f.y, acc[i]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < RT; ++i) {
            const float total = warp_sum(acc[i]);
            if (lane == 0 && r0 + i < R) st<TO>(y, (size_t)(r0 + i) * N + n, total);
        }
    }
}

// y[j] = x[j, :] . W[ids[j], :]: the head's rows of a handful of token ids only,
// for scoring given continuations (the reference's gathered product,
// src/kernels_cuda/gemv_gather.cu:10-51): kilobytes of the head are read, not
// the whole vocabulary.  One warp per pair.  32-bit: the lanes stage the two
// rows in shared memory, a chunk at a time, and lane 0 runs one fused
// multiply-add chain over k in index order, which gives the bits of
// `gemm_f32_kernel` for the same row and column.  An id outside [0, V) gives
// NaN and sets the error word (the host checks ids before it launches).
constexpr int GATHER_WARPS = 4, GATHER_CHUNK = 512;

__global__ void __launch_bounds__(GATHER_WARPS * 32)
gather_dot_f32_kernel(const float* __restrict__ x, const float* __restrict__ W, const int* __restrict__ ids,
                      float* __restrict__ y, int P, int K, int V, int* __restrict__ err) {
    __shared__ float xs[GATHER_WARPS][GATHER_CHUNK];
    __shared__ float ws[GATHER_WARPS][GATHER_CHUNK];
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * GATHER_WARPS + warp;
    if (j >= P) return;
    const int id = ids[j];
    if (id < 0 || id >= V) {
        if (lane == 0) {
            y[j] = __int_as_float(0x7fc00000);
            atomicExch(err, 1 + j);
        }
        return;
    }
    const float* xr = x + (size_t)j * K;
    const float* wr = W + (size_t)id * K;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += GATHER_CHUNK) {
        const int n = min(GATHER_CHUNK, K - k0);
        for (int i = lane; i < n; i += 32) {
            xs[warp][i] = xr[k0 + i];
            ws[warp][i] = wr[k0 + i];
        }
        __syncwarp();
        if (lane == 0)
            for (int i = 0; i < n; ++i) acc = fmaf(xs[warp][i], ws[warp][i], acc);
        __syncwarp();
    }
    if (lane == 0) y[j] = acc;
}

// bfloat16 rows, 32-bit accumulation: 16-byte loads when K is a multiple of 8.
__global__ void __launch_bounds__(GATHER_WARPS * 32)
gather_dot_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                       const int* __restrict__ ids, float* __restrict__ y, int P, int K, int V,
                       int* __restrict__ err) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * GATHER_WARPS + warp;
    if (j >= P) return;
    const int id = ids[j];
    if (id < 0 || id >= V) {
        if (lane == 0) {
            y[j] = __int_as_float(0x7fc00000);
            atomicExch(err, 1 + j);
        }
        return;
    }
    const __nv_bfloat16* xr = x + (size_t)j * K;
    const __nv_bfloat16* wr = W + (size_t)id * K;
    float acc = 0.0f;
    if ((K & 7) == 0) {
        const uint4* x4 = reinterpret_cast<const uint4*>(xr);
        const uint4* w4 = reinterpret_cast<const uint4*>(wr);
        for (int c = lane; c < K / 8; c += 32) {
            const uint4 xv = x4[c], wv = w4[c];
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __bfloat1622float2(x2[i]), b = __bfloat1622float2(w2[i]);
                acc = fmaf(a.x, b.x, acc);
                acc = fmaf(a.y, b.y, acc);
            }
        }
    } else {
        for (int i = lane; i < K; i += 32) acc = fmaf(__bfloat162float(xr[i]), __bfloat162float(wr[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[j] = acc;
}

}  // namespace

extern "C" int rfx_gather_dot(const void* x, const void* W, int dt, const int* ids, float* y, int P, int K,
                              int V, int* err, void* stream) {
    if (P <= 0) return 0;
    if (K <= 0 || V <= 0) return RFX_ERR_BAD_ARG;
    const int blocks = (P + GATHER_WARPS - 1) / GATHER_WARPS;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(gather_dot_f32_kernel, blocks, GATHER_WARPS * 32, 0, s, (const float*)x, (const float*)W, ids,
                   y, P, K, V, err);
    else if (dt == RFX_DT_BF16) {
        if ((K & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15))
            return RFX_ERR_BAD_ARG;
        RFX_LAUNCH(gather_dot_bf16_kernel, blocks, GATHER_WARPS * 32, 0, s, (const __nv_bfloat16*)x,
                   (const __nv_bfloat16*)W, ids, y, P, K, V, err);
    } else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_gemm_f32(const float* x, const float* W, float* y, int R, int N, int K,
                            void* stream) {
    if (R <= 0 || N <= 0) return 0;
    if (K <= 0) return RFX_ERR_BAD_ARG;
    dim3 grid((N + TN - 1) / TN, (R + TM - 1) / TM);
    if (grid.y > 65535) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(gemm_f32_kernel, grid, 256, 0, (cudaStream_t)stream, x, W, y, R, N, K);
    return 0;
}

extern "C" int rfx_gemv_bf16(const void* x, const void* W, void* y, int y_dt, int R, int N, int K,
                             void* stream) {
    if (R <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0) return RFX_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (N + 7) / 8;
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)W;
#define RFX_GEMV(RT)                                                                             \
    do {                                                                                         \
        if (y_dt == RFX_DT_F32)                                                                  \
            RFX_LAUNCH((gemv_bf16_kernel<RT, float>), blocks, 256, 0, s, xb, wb, (float*)y, R, N, K); \
        else if (y_dt == RFX_DT_BF16)                                                            \
            RFX_LAUNCH((gemv_bf16_kernel<RT, __nv_bfloat16>), blocks, 256, 0, s, xb, wb,         \
                       (__nv_bfloat16*)y, R, N, K);                                              \
        else                                                                                     \
            return RFX_ERR_BAD_ARG;                                                              \
    } while (0)
    if (R == 1) RFX_GEMV(1);
    else if (R == 2) RFX_GEMV(2);
    else if (R <= 4) RFX_GEMV(4);
    else RFX_GEMV(8);
#undef RFX_GEMV
    return 0;
}
