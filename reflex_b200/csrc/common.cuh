// Shared helpers of the sm_100a kernels: status codes, element loads/stores
// that widen to 32-bit, warp and block reductions with a fixed order.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <utility>

#include "exact_math.cuh"

#define RFX_DT_F32 0
#define RFX_DT_BF16 1

// Return codes of the host entry points: 0 ok, a positive cudaError_t, or one
// of these negative values for an argument the kernel refuses.
#define RFX_ERR_BAD_ARG (-1)
#define RFX_ERR_UNSUPPORTED (-2)
#define RFX_ERR_TIMEOUT (-3)
#define RFX_ERR_SCRATCH (-4)

#define RFX_CHECK_LAUNCH()                         \
    do {                                           \
        cudaError_t e__ = cudaGetLastError();      \
        if (e__ != cudaSuccess) return (int)e__;   \
    } while (0)

namespace rfx {

// ---- programmatic dependent launch -------------------------------------------
// Every kernel of the library is launched with programmatic stream
// serialization: the next kernel's CTAs may start while this one drains, run
// whatever does not depend on it (barrier set-up, weight prefetch), and block
// in pdl_wait() until this kernel has completed and its writes are visible.
// Rules every kernel keeps: no global write and no read of another kernel's
// output before pdl_wait(); every kernel executes pdl_wait() (so completion
// stays transitive along the stream).  REFLEX_B200_PDL=0 turns the launch
// attribute off; the device calls are then no-ops.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
    pdl_launch_dependents();
    pdl_wait();
}

inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("REFLEX_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// Streaming multiprocessors of the current device, asked once (148 on a B200).
inline int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// Launch with the library's attributes; cluster_z > 1 asks for a thread-block
// cluster of (1, 1, cluster_z).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, int cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

#define RFX_LAUNCH(kernel, grid, block, smem, stream, ...)                                   \
    do {                                                                                     \
        cudaError_t e__ = rfx::launch(kernel, grid, block, smem, stream, 1, __VA_ARGS__);    \
        if (e__ != cudaSuccess) return (int)e__;                                             \
    } while (0)

template <typename T> __device__ __forceinline__ float ld(const T* p, size_t i);
template <> __device__ __forceinline__ float ld<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
    return __bfloat162float(p[i]);
}

template <typename T> __device__ __forceinline__ void st(T* p, size_t i, float v);
template <> __device__ __forceinline__ void st<float>(float* p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, size_t i, float v) {
    p[i] = __float2bfloat16_rn(v);
}

// four (two) neighbouring results in one access; the address is a multiple of
// their size by the callers' conditions
__device__ __forceinline__ void store4(float* p, const float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4 v) {
    uint2 u;
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ void store2(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// silu(g) * u as the reference writes it (src/kernels_cuda/silu_and_mul.cu:7-23).
// The exponential is `exact_expf`, so a host program can repeat the bits.
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + exact_expf(-g))) * u; }
// The same for a result that is rounded to bfloat16 anyway: the fast exponential
// and division are a few units in the last place of 32 bits off, far below that
// rounding; their limits at large |g| are the function's own (0 and g).
template <typename TO>
__device__ __forceinline__ float silu_mul_for(float g, float u) {
    if constexpr (sizeof(TO) == 2) return __fdividef(g, 1.0f + __expf(-g)) * u;
    else return silu_mul(g, u);
}

// Sum over the 32 lanes in a fixed butterfly order; every lane gets the total.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads.  `scratch` holds 32 floats.  The
// order (lane butterfly, then warps in index order) depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

}  // namespace rfx
