// Choosing the next token on the device from 32-bit logits [B, V].
//
//  * argmax: ties go to the highest index, as the reference's host argmax does
//    (src/model/mod.rs:1371-1380: `max_by` keeps the last maximum).  NaN never
//    wins.  Two stages for a large vocabulary: 64 chunks a row, then the
//    winners of the chunks.
//  * sample: temperature softmax, optional top-k, optional top-p, then an
//    inverse-CDF draw with a uniform number the caller supplies
//    (src/sampling.rs:241-294).  p_i = exp((l_i - max) / T); top-k keeps the k
//    largest p; top-p keeps the shortest prefix, in descending order of p over
//    what top-k left, whose probabilities (normalised over the whole
//    vocabulary) sum to >= top_p; ties at a cut are kept lowest index first.
//    The draw walks the kept entries in index order: the token is the first
//    whose running sum reaches u * (sum of kept p).
//    Both cuts are found by a radix select over the bit patterns of p (p >= 0,
//    so the patterns order like the values), four 8-bit digits, histograms of
//    counts and of mass in shared memory.  `probs` is scratch of B*V floats.
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int SAMPLE_THREADS = 1024;
constexpr int ARGMAX_CHUNKS = 64;

__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bidx) {
    return i >= 0 && v == v && (bidx < 0 || v > bv || (v == bv && i > bidx));
}

// Stage 1: block (row, chunk) scans its chunk of the row; stage 2 (chunks == 1
// input) reduces the per-chunk winners.  `src_idx` is null in stage 1.
__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ vals, const int* __restrict__ src_idx, long long stride,
              int n, int chunk, float* __restrict__ out_val, int* __restrict__ out_idx) {
    __shared__ float sv[8];
    __shared__ int si[8];
    pdl_prologue();
    const float* row = vals + (size_t)blockIdx.x * stride;
    const int lo = blockIdx.y * chunk, hi = min(n, lo + chunk);
    float best = -INFINITY;
    int bi = -1;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        const int id = src_idx ? src_idx[(size_t)blockIdx.x * stride + i] : i;
        if (argmax_better(v, id, best, bi)) {
            best = v;
            bi = id;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (argmax_better(ov, oi, best, bi)) {
            best = ov;
            bi = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        for (int w = 1; w < nw; ++w)
            if (argmax_better(sv[w], si[w], best, bi)) {
                best = sv[w];
                bi = si[w];
            }
        const size_t o = (size_t)blockIdx.x * gridDim.y + blockIdx.y;
        if (out_val) out_val[o] = best;
        out_idx[o] = (bi < 0 && !out_val) ? 0 : bi;
    }
}

struct SelectResult {
    unsigned int bits;   // bit pattern of the value at the cut
    int above;           // entries strictly greater than it
    int ties;            // entries equal to it that are kept
    float mass_above;
};

// Radix select over p[0..V): by count (the `want`-th largest, want >= 1) when
// by_mass is false, else the first entry, in descending order, at which the
// running mass reaches `want_mass`.  All threads of the block call it.
__device__ SelectResult radix_select(const float* __restrict__ p, int V, bool by_mass, int want,
                                     float want_mass, int* hist_n, float* hist_m,
                                     int* sh_state) {
    unsigned int prefix = 0, mask = 0;
    int above = 0;
    float mass_above = 0.0f;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            hist_n[b] = 0;
            hist_m[b] = 0.0f;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = p[i];
            const unsigned int u = __float_as_uint(v);
            if ((u & mask) == prefix) {
                const int b = (u >> shift) & 255;
                atomicAdd(&hist_n[b], 1);
                if (by_mass) atomicAdd(&hist_m[b], v);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int n = above;
            float ms = mass_above;
            int b = 255;
            for (; b > 0; --b) {
                const int nb = hist_n[b];
                if (nb == 0) continue;
                const bool stop = by_mass ? (ms + hist_m[b] >= want_mass) : (n + nb >= want);
                if (stop) break;
                n += nb;
                ms += hist_m[b];
            }
            sh_state[0] = b;
            sh_state[1] = n;
            reinterpret_cast<float*>(sh_state)[2] = ms;
        }
        __syncthreads();
        const int b = sh_state[0];
        above = sh_state[1];
        mass_above = reinterpret_cast<float*>(sh_state)[2];
        prefix |= (unsigned int)b << shift;
        mask |= 255u << shift;
        __syncthreads();
    }
    // entries equal to the cut value
    SelectResult r;
    r.bits = prefix;
    r.above = above;
    r.mass_above = mass_above;
    const float v = __uint_as_float(prefix);
    int n_equal = hist_n[(prefix)&255];  // last digit's bin: all entries equal to the value
    __syncthreads();
    if (by_mass) {
        int need = 1;
        if (v > 0.0f) {
            const float rest = want_mass - mass_above;
            need = (int)ceilf(rest / v);
            if (need < 1) need = 1;
        }
        r.ties = need < n_equal ? need : n_equal;
    } else {
        int need = want - above;
        if (need < 1) need = 1;
        r.ties = need < n_equal ? need : n_equal;
    }
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              float* __restrict__ probs, int* __restrict__ out) {
    __shared__ float scratch[32];
    __shared__ int hist_n[256];
    __shared__ float hist_m[256];
    __shared__ int sh_state[4];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int tie_base[SAMPLE_THREADS];
    __shared__ int sh_pick;

    pdl_prologue();
    const int b = blockIdx.x;
    const float* row = logits + (size_t)b * stride;
    float* p = probs + (size_t)b * V;
    const float T = temperature[b];

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = scratch[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, scratch[w]);
    __syncthreads();

    float part = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float e = expf((row[i] - mx) / T);
        p[i] = e;
        part += e;
    }
    const float total = block_sum(part, scratch);
    __syncthreads();

    // cut: keep the n_keep largest
    int k = top_k ? top_k[b] : 0;
    const float tp = top_p ? top_p[b] : 1.0f;
    int n_keep = (k > 0 && k < V) ? k : V;
    if (top_p && tp < 1.0f) {
        const SelectResult rp = radix_select(p, V, true, 0, tp * total, hist_n, hist_m, sh_state);
        const int n_p = rp.above + rp.ties;
        if (n_p < n_keep) n_keep = n_p;
    }
    unsigned int cut_bits = 0;
    int ties_kept = 0x7fffffff;
    if (n_keep < V) {
        const SelectResult rk = radix_select(p, V, false, n_keep, 0.0f, hist_n, hist_m, sh_state);
        cut_bits = rk.bits;
        ties_kept = n_keep - rk.above;
    }

    // contiguous chunk per thread, so the walk is in index order
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int i0 = threadIdx.x * per;
    const int i1 = min(V, i0 + per);
    int n_tie = 0;
    for (int i = i0; i < i1; ++i)
        if (__float_as_uint(p[i]) == cut_bits) ++n_tie;
    tie_base[threadIdx.x] = n_tie;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            const int n = tie_base[t];
            tie_base[t] = run;
            run += n;
        }
    }
    __syncthreads();
    float cs = 0.0f;
    {
        int seen = tie_base[threadIdx.x];
        for (int i = i0; i < i1; ++i) {
            const unsigned int u = __float_as_uint(p[i]);
            bool keep = u > cut_bits;
            if (u == cut_bits) keep = (seen++ < ties_kept);
            if (keep) cs += p[i];
        }
    }
    chunk_sum[threadIdx.x] = cs;
    __syncthreads();
    if (threadIdx.x == 0) {
        float renorm = 0.0f;
        for (int t = 0; t < (int)blockDim.x; ++t) renorm += chunk_sum[t];
        const float draw = uniform[b] * renorm;
        float acc = 0.0f;
        int pick = -1;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (chunk_sum[t] > 0.0f && draw <= acc + chunk_sum[t]) {
                pick = t;
                break;
            }
            acc += chunk_sum[t];
        }
        if (pick < 0) {  // rounding left the draw above the total: last kept chunk
            for (int t = (int)blockDim.x - 1; t >= 0; --t)
                if (chunk_sum[t] > 0.0f) {
                    pick = t;
                    acc -= 0.0f;
                    break;
                }
            float a2 = 0.0f;
            for (int t = 0; t < pick; ++t) a2 += chunk_sum[t];
            acc = a2;
        }
        sh_pick = pick;
        scratch[0] = acc;
        scratch[1] = draw;
    }
    __syncthreads();
    if ((int)threadIdx.x == sh_pick) {
        float acc = scratch[0];
        const float draw = scratch[1];
        int seen = tie_base[threadIdx.x];
        int chosen = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            const unsigned int u = __float_as_uint(p[i]);
            bool keep = u > cut_bits;
            if (u == cut_bits) keep = (seen++ < ties_kept);
            if (!keep) continue;
            last_kept = i;
            acc += p[i];
            if (draw <= acc) {
                chosen = i;
                break;
            }
        }
        out[b] = chosen >= 0 ? chosen : (last_kept >= 0 ? last_kept : 0);
    }
}

}  // namespace

// `scratch` holds B * ARGMAX_CHUNKS floats followed by as many ints.
extern "C" int rfx_argmax(const float* logits, long long stride, int B, int V, int* out,
                          void* scratch, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (V <= 4096 || !scratch) {
        RFX_LAUNCH(argmax_kernel, dim3(B, 1), 256, 0, s, logits, (const int*)nullptr, stride, V, V,
                   (float*)nullptr, out);
        return 0;
    }
    const int chunks = ARGMAX_CHUNKS;
    const int chunk = (V + chunks - 1) / chunks;
    float* pv = (float*)scratch;
    int* pi = (int*)(pv + (size_t)B * chunks);
    RFX_LAUNCH(argmax_kernel, dim3(B, chunks), 256, 0, s, logits, (const int*)nullptr, stride, V, chunk,
               pv, pi);
    RFX_LAUNCH(argmax_kernel, dim3(B, 1), 64, 0, s, (const float*)pv, (const int*)pi, (long long)chunks,
               chunks, chunks, (float*)nullptr, out);
    return 0;
}

// temperature[B] > 0; top_k[B] (<= 0: off) or NULL; top_p[B] (>= 1: off) or
// NULL; uniform[B] in [0, 1); probs: scratch of B * V floats.
extern "C" int rfx_sample(const float* logits, long long stride, int B, int V,
                          const float* temperature, const int* top_k, const float* top_p,
                          const float* uniform, float* probs, int* out, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !probs) return RFX_ERR_BAD_ARG;
    RFX_LAUNCH(sample_kernel, B, SAMPLE_THREADS, 0, (cudaStream_t)stream, logits, stride, V,
               temperature, top_k, top_p, uniform, probs, out);
    return 0;
}
