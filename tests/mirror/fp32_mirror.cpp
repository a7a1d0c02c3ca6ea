// A host mirror of the 32-bit kernels' arithmetic, for tests.
//
// Each function repeats, operation by operation and in the same order, what one
// CUDA kernel of the true 32-bit path computes for one output element: the same
// fused multiply-add chains, the same per-lane partial sums and butterfly, the
// same exponential and sine/cosine (restated here from their definitions: IEEE
// operations only).  Built with -ffp-contract=off so that the compiler fuses
// nothing on its own; every fused multiply-add is written out as std::fmaf.
// A test then compares the engine's 32-bit logits with this mirror's bit for
// bit, which is how the reference anchors its RMSNorm kernel
// (src/model/rmsnorm_tests.rs:17-29, 64-72: a host loop with mul_add in index
// order, compared by to_bits; the order rule is src/kernels_cuda/rmsnorm.cuh:1-11).
//
// Whole sequences, no cache, no batches: the engine's results do not depend on
// those, which is what the comparison shows.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

float pow2i(int e) {
    const uint32_t bits = (uint32_t)(e + 127) << 23;
    float f;
    std::memcpy(&f, &bits, sizeof(f));
    return f;
}

// e^x: n = rint(x / ln 2), r = x - n ln2 (ln2 in two parts), Taylor degree 7,
// scaled by 2^n in two steps.
float m_exp(float x) {
    if (x != x) return x;
    if (!(x > -104.0f)) return 0.0f;
    if (x > 89.0f) return INFINITY;
    const float n = std::rint(x * 1.4426950408889634f);
    float r = std::fmaf(n, -0.693145751953125f, x);
    r = std::fmaf(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = std::fmaf(p, r, 1.0f / 720.0f);
    p = std::fmaf(p, r, 1.0f / 120.0f);
    p = std::fmaf(p, r, 1.0f / 24.0f);
    p = std::fmaf(p, r, 1.0f / 6.0f);
    p = std::fmaf(p, r, 0.5f);
    p = std::fmaf(p, r, 1.0f);
    p = std::fmaf(p, r, 1.0f);
    const int ni = (int)n;
    const int n1 = ni / 2, n2 = ni - n1;
    return (p * pow2i(n1)) * pow2i(n2);
}

// sin and cos of a 32-bit angle: reduction by pi/2 (two parts) and Taylor
// polynomials in double, the quadrant's pick, one rounding to 32-bit.
void m_sincos(float theta, float* sn, float* cs) {
    const double t = (double)theta;
    const double k = std::rint(t * 0.63661977236758134308);
    double r = std::fma(k, -1.57079632679489655800e+00, t);
    r = std::fma(k, -6.12323399573676603587e-17, r);
    const double z = r * r;
    double s = 1.0 / 355687428096000.0;
    s = std::fma(s, z, -1.0 / 1307674368000.0);
    s = std::fma(s, z, 1.0 / 6227020800.0);
    s = std::fma(s, z, -1.0 / 39916800.0);
    s = std::fma(s, z, 1.0 / 362880.0);
    s = std::fma(s, z, -1.0 / 5040.0);
    s = std::fma(s, z, 1.0 / 120.0);
    s = std::fma(s, z, -1.0 / 6.0);
    s = std::fma(s, z, 1.0);
    s = s * r;
    double c = 1.0 / 20922789888000.0;
    c = std::fma(c, z, -1.0 / 87178291200.0);
    c = std::fma(c, z, 1.0 / 479001600.0);
    c = std::fma(c, z, -1.0 / 3628800.0);
    c = std::fma(c, z, 1.0 / 40320.0);
    c = std::fma(c, z, -1.0 / 720.0);
    c = std::fma(c, z, 1.0 / 24.0);
    c = std::fma(c, z, -0.5);
    c = std::fma(c, z, 1.0);
    const int q = (int)((long long)k & 3);
    const double sv = (q == 0) ? s : (q == 1) ? c : (q == 2) ? -s : -c;
    const double cv = (q == 0) ? c : (q == 1) ? -s : (q == 2) ? -c : s;
    *sn = (float)sv;
    *cs = (float)cv;
}

// The 32 lanes' butterfly sum: offsets 16, 8, 4, 2, 1; every lane ends with the total.
float butterfly32(float* v) {
    for (int o = 16; o > 0; o >>= 1) {
        float nv[32];
        for (int l = 0; l < 32; ++l) nv[l] = v[l] + v[l ^ o];
        std::memcpy(v, nv, sizeof(nv));
    }
    return v[0];
}

// threads of the norm kernel's block: a function of the width alone
int norm_threads(int H) {
    int t = ((H + 15) / 16 + 31) / 32 * 32;
    if (t < 32) t = 32;
    if (t > 256) t = 256;
    return t;
}

}  // namespace

extern "C" {

float mir_exp(float x) { return m_exp(x); }
void mir_sincos(float theta, float* sn, float* cs) { m_sincos(theta, sn, cs); }

// RMSNorm with the residual add before it: t = x (+ delta); t_out = t;
// out = (t * r) * (w_offset + w), r = 1 / sqrt(sum(t^2) / H + eps).  The sum of
// squares as the kernel's block forms it: thread i takes elements (or groups
// of four when H is a multiple of 4) i, i + threads, ...; lanes' butterfly per
// warp; warps added in index order.  order = 1 sums in plain index order
// instead: a deliberately different order, to show that the comparison sees it.
void mir_rmsnorm(const float* x, const float* delta, float* t_out, const float* w, float eps,
                 float w_offset, float* out, int R, int H, int order) {
    const int T = norm_threads(H);
    std::vector<float> t(H), part(T);
    for (int r = 0; r < R; ++r) {
        for (int c = 0; c < H; ++c) {
            float v = x[(size_t)r * H + c];
            if (delta) v = v + delta[(size_t)r * H + c];
            t[c] = v;
        }
        float total = 0.0f;
        if (order == 1) {
            for (int c = 0; c < H; ++c) total = std::fmaf(t[c], t[c], total);
        } else {
            for (int i = 0; i < T; ++i) {
                float ss = 0.0f;
                if (H % 4 == 0) {
                    for (int c = i; c < H / 4; c += T)
                        for (int j = 0; j < 4; ++j) ss = std::fmaf(t[4 * c + j], t[4 * c + j], ss);
                } else {
                    for (int c = i; c < H; c += T) ss = std::fmaf(t[c], t[c], ss);
                }
                part[i] = ss;
            }
            for (int wp = 0; wp < T / 32; ++wp) total += butterfly32(&part[wp * 32]);
        }
        const float rr = 1.0f / std::sqrt(total / (float)H + eps);
        for (int c = 0; c < H; ++c) {
            if (t_out) t_out[(size_t)r * H + c] = t[c];
            if (out) out[(size_t)r * H + c] = (t[c] * rr) * (w_offset + w[c]);
        }
    }
}

// y[r, n] = sum_k x[r, k] W[n, k]: one fused multiply-add chain over k in index order.
void mir_linear(const float* x, const float* W, float* y, int R, int N, int K) {
    for (int r = 0; r < R; ++r)
        for (int n = 0; n < N; ++n) {
            float acc = 0.0f;
            const float* xr = x + (size_t)r * K;
            const float* wn = W + (size_t)n * K;
            for (int k = 0; k < K; ++k) acc = std::fmaf(xr[k], wn[k], acc);
            y[(size_t)r * N + n] = acc;
        }
}

// Per-head RMSNorm (when w is given) and rotary encoding of heads [T, n, d], in place.
// Norm: lane l sums elements l, l + 32, ... by fused multiply-adds, butterfly,
// r = 1 / sqrt(sum / d + eps), y = (x * r) * (w_offset + w).  Rotation: angle =
// (float)pos / denom[i], cos and sin times magnitude, pair (first, second):
// first = fma(second, -sin, first * cos), second = fma(first, sin, second * cos).
void mir_head_norm_rope(float* heads, const float* w, float eps, float w_offset, const float* denom,
                        int rotary_dim, int pairing, float magnitude, const int* pos, int T, int n,
                        int d) {
    const int half = rotary_dim / 2;
    std::vector<float> sn(half > 0 ? half : 1), cs(half > 0 ? half : 1), v(d), o(d);
    for (int t = 0; t < T; ++t) {
        if (denom && half > 0) {
            for (int i = 0; i < half; ++i) {
                const float theta = (float)pos[t] / denom[i];
                float s, c;
                m_sincos(theta, &s, &c);
                sn[i] = s * magnitude;
                cs[i] = c * magnitude;
            }
        }
        for (int h = 0; h < n; ++h) {
            float* p = heads + ((size_t)t * n + h) * d;
            for (int e = 0; e < d; ++e) v[e] = p[e];
            if (w) {
                float lanes[32];
                for (int l = 0; l < 32; ++l) {
                    float ss = 0.0f;
                    for (int e = l; e < d; e += 32) ss = std::fmaf(v[e], v[e], ss);
                    lanes[l] = ss;
                }
                const float rinv = 1.0f / std::sqrt(butterfly32(lanes) / (float)d + eps);
                for (int e = 0; e < d; ++e) v[e] = (v[e] * rinv) * (w_offset + w[e]);
            }
            for (int e = 0; e < d; ++e) {
                o[e] = v[e];
                if (denom && e < rotary_dim) {
                    int fi, other;
                    bool first;
                    if (pairing == 1) {
                        fi = e >> 1;
                        first = (e & 1) == 0;
                        other = e ^ 1;
                    } else {
                        first = e < half;
                        fi = first ? e : e - half;
                        other = first ? e + half : e - half;
                    }
                    o[e] = std::fmaf(v[other], first ? -sn[fi] : sn[fi], v[e] * cs[fi]);
                }
            }
            for (int e = 0; e < d; ++e) p[e] = o[e];
        }
    }
}

// Causal attention of one whole sequence: query i of head h reads kv head
// h / (nq / nkv) and keys max(0, i - window + 1) .. i, one after another with a
// running maximum: s = butterfly(lane chains of q . k) * scale;
// m' = max(m, s); corr = exp(m - m'); p = exp(s - m'); l = fma(l, corr, p);
// acc = fma(acc, corr, p * v); out = acc / l.
void mir_attention(const float* q, const float* k, const float* v, float* out, int T, int nq,
                   int nkv, int d, int window, float scale) {
    const int g = nq / nkv;
    std::vector<float> acc(d);
    for (int i = 0; i < T; ++i)
        for (int h = 0; h < nq; ++h) {
            const int kh = h / g;
            const float* qv = q + ((size_t)i * nq + h) * d;
            const int lo = (window > 0 && i + 1 > window) ? i + 1 - window : 0;
            float m = -INFINITY, l = 0.0f;
            for (int e = 0; e < d; ++e) acc[e] = 0.0f;
            for (int j = lo; j <= i; ++j) {
                const float* kv = k + ((size_t)j * nkv + kh) * d;
                const float* vv = v + ((size_t)j * nkv + kh) * d;
                float lanes[32];
                for (int ln = 0; ln < 32; ++ln) {
                    float dot = 0.0f;
                    for (int e = ln; e < d; e += 32) dot = std::fmaf(qv[e], kv[e], dot);
                    lanes[ln] = dot;
                }
                const float s = butterfly32(lanes) * scale;
                const float m_new = std::fmax(m, s);
                const float corr = m_exp(m - m_new);
                const float p = m_exp(s - m_new);
                l = std::fmaf(l, corr, p);
                for (int e = 0; e < d; ++e) acc[e] = std::fmaf(acc[e], corr, p * vv[e]);
                m = m_new;
            }
            float* o = out + ((size_t)i * nq + h) * d;
            for (int e = 0; e < d; ++e) o[e] = acc[e] / l;
        }
}

// out = (g / (1 + exp(-g))) * u
void mir_swiglu(const float* g, const float* u, float* out, long long n) {
    for (long long i = 0; i < n; ++i) out[i] = (g[i] / (1.0f + m_exp(-g[i]))) * u[i];
}

}  // extern "C"
