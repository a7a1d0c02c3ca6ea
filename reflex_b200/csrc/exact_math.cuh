// Exponential, sine and cosine whose bits are the same on the host and on the
// device.
//
// CUDA's expf / sincosf and a C library's differ in their last bits, so a host
// program that repeats a kernel's arithmetic step by step (fused multiply-adds
// in the kernel's order) could never be compared with it bit for bit.  These
// routines use only operations that IEEE 754 defines exactly (add, multiply,
// fused multiply-add, round to integer, conversions, and scaling by a power of
// two), written out one by one, so that nvcc and a host compiler (built with
// -ffp-contract=off) produce the same bits.  The true 32-bit path uses them for
// the softmax, SiLU and the rotary angles; the reference's rule for such host
// mirrors is src/model/rmsnorm_tests.rs:1-29 (mul_add in index order, compared
// by to_bits).
//
// Accuracy: exact_expf within 2 units in the last place; exact_sincosf rounds
// a double-precision value whose error is far below half a float's last place.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define RFX_HD __host__ __device__ __forceinline__
#else
#define RFX_HD inline
#endif

namespace rfx {

// 2^e as a float, for -126 <= e <= 127
RFX_HD float exact_pow2(int e) {
    const uint32_t bits = (uint32_t)(e + 127) << 23;
    float f;
#if defined(__CUDA_ARCH__)
    f = __uint_as_float(bits);
#else
    memcpy(&f, &bits, sizeof(f));
#endif
    return f;
}

// e^x.  x = n ln2 + r with n = rint(x / ln2), |r| <= ln2 / 2 (ln2 split in two
// so that n * hi is exact); e^r by its Taylor polynomial of degree 7 (remainder
// below 6e-9); the result scaled by 2^n in two exact-or-once-rounded steps, so
// that subnormal results and overflow come out as IEEE multiplication gives them.
RFX_HD float exact_expf(float x) {
    if (x != x) return x;
    if (!(x > -104.0f)) return 0.0f;       // below half the smallest subnormal, and -inf
    if (x > 89.0f) return INFINITY;
    const float n = rintf(x * 1.4426950408889634f);
    float r = fmaf(n, -0.693145751953125f, x);       // ln2, high part (11 significant bits)
    r = fmaf(n, -1.42860682030941723e-6f, r);        // ln2, low part
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    const int ni = (int)n;
    const int n1 = ni / 2, n2 = ni - n1;
    return (p * exact_pow2(n1)) * exact_pow2(n2);
}

// sin and cos of a 32-bit angle.  The reduction t = k pi/2 + r runs in double
// precision (pi/2 in two parts, each step one fused multiply-add), which is
// accurate for every angle a position below 2^31 can give; sin r and cos r by
// their Taylor polynomials on |r| <= pi/4 (remainders below 5e-17), in double;
// the quadrant picks and signs them; one rounding to 32-bit at the end.
RFX_HD void exact_sincosf(float theta, float* sin_out, float* cos_out) {
    const double t = (double)theta;
    const double k = rint(t * 0.63661977236758134308);
    double r = fma(k, -1.57079632679489655800e+00, t);
    r = fma(k, -6.12323399573676603587e-17, r);
    const double z = r * r;
    // sin r = r (1 + z (-1/3! + z (1/5! + ... + z (1/17!))))
    double s = 1.0 / 355687428096000.0;
    s = fma(s, z, -1.0 / 1307674368000.0);
    s = fma(s, z, 1.0 / 6227020800.0);
    s = fma(s, z, -1.0 / 39916800.0);
    s = fma(s, z, 1.0 / 362880.0);
    s = fma(s, z, -1.0 / 5040.0);
    s = fma(s, z, 1.0 / 120.0);
    s = fma(s, z, -1.0 / 6.0);
    s = fma(s, z, 1.0);
    s = s * r;
    // cos r = 1 + z (-1/2! + z (1/4! + ... + z (1/16!)))
    double c = 1.0 / 20922789888000.0;
    c = fma(c, z, -1.0 / 87178291200.0);
    c = fma(c, z, 1.0 / 479001600.0);
    c = fma(c, z, -1.0 / 3628800.0);
    c = fma(c, z, 1.0 / 40320.0);
    c = fma(c, z, -1.0 / 720.0);
    c = fma(c, z, 1.0 / 24.0);
    c = fma(c, z, -0.5);
    c = fma(c, z, 1.0);
    const int q = (int)((long long)k & 3);
    const double sv = (q == 0) ? s : (q == 1) ? c : (q == 2) ? -s : -c;
    const double cv = (q == 0) ? c : (q == 1) ? -s : (q == 2) ? -c : s;
    *sin_out = (float)sv;
    *cos_out = (float)cv;
}

}  // namespace rfx
