// Random weights as a function of (key, element index) alone: the same bits
// whether a tensor is filled here, on the host (weights/random_init.py restates
// the arithmetic in NumPy), in one piece or in parts.  Every step is an integer
// operation or a single IEEE double operation written out as such (no fused
// multiply-add can form), so host and device agree bit for bit.
//
//   hash(c)   = the splitmix64 finaliser of key + c * 0x9E3779B97F4A7C15
//   normal    : element i takes hashes 3i, 3i+1, 3i+2, cuts each into four 16-bit
//               numbers and sums the twelve: (sum - 12 * 32767.5) / 65536 has mean 0
//               and variance 1 (the sum of twelve uniforms), times the deviation,
//               rounded once to 32-bit
//   uniform   : the top 24 bits u of hash(3i): lo + (hi - lo) * (u + 0.5) / 2^24
//
// A bfloat16 tensor holds the 32-bit draw rounded to nearest even.
#include "common.cuh"

namespace {

using namespace rfx;

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long key, unsigned long long c) {
    unsigned long long z = key + c * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ unsigned int sum16(unsigned long long h) {
    return (unsigned int)(h & 0xFFFF) + (unsigned int)((h >> 16) & 0xFFFF) +
           (unsigned int)((h >> 32) & 0xFFFF) + (unsigned int)(h >> 48);
}

template <typename T>
__global__ void __launch_bounds__(256)
random_fill_kernel(T* __restrict__ out, size_t n, size_t first, unsigned long long key, int kind,
                   double a, double b) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned long long e = first + i;
        double v;
        if (kind == 0) {  // normal: mean a, deviation b
            const unsigned int s = sum16(mix64(key, 3 * e)) + sum16(mix64(key, 3 * e + 1)) +
                                   sum16(mix64(key, 3 * e + 2));
            const double x = __ddiv_rn(__dsub_rn((double)s, 393210.0), 65536.0);
            v = __dadd_rn(a, __dmul_rn(x, b));
        } else {  // uniform in (a, b)
            const unsigned long long u = mix64(key, 3 * e) >> 40;
            const double t = __ddiv_rn(__dadd_rn((double)u, 0.5), 16777216.0);
            v = __dadd_rn(a, __dmul_rn(__dsub_rn(b, a), t));
        }
        st<T>(out, i, (float)v);
    }
}

}  // namespace

// Elements [first, first + n) of the tensor keyed by `key` into out[0 .. n).
extern "C" int rfx_random_fill(void* out, int dt, long long n, long long first, unsigned long long key,
                               int kind, double a, double b, void* stream) {
    if (n <= 0) return 0;
    if (kind != 0 && kind != 1) return RFX_ERR_BAD_ARG;
    long long blocks = (n + 255) / 256;
    const long long cap = (long long)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(random_fill_kernel<float>, (int)blocks, 256, 0, s, (float*)out, (size_t)n, (size_t)first, key,
                   kind, a, b);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(random_fill_kernel<__nv_bfloat16>, (int)blocks, 256, 0, s, (__nv_bfloat16*)out, (size_t)n,
                   (size_t)first, key, kind, a, b);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
