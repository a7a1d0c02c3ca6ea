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
//    The cut is one radix select over the bit patterns of p for both rules
//    (below); `probs` is scratch of B*V floats and `work` holds the chunk sums
//    and histograms.
#include "common.cuh"

namespace {

using namespace rfx;

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

// ---- sampling ------------------------------------------------------------------
// A row's vocabulary is cut into chunks of SCHUNK entries (a multiple of it when
// there are many rows), a block each, so that a few rows still fill the GPU; the kernels of one call follow one another:
//   max      chunk maxima
//   exp      row maximum, p = exp((l - max) / T) into `probs`, chunk sums; with a
//            cut, the first histogram
//   select   (twice, with a cut) the bin of the last histogram that holds the
//            cut, then the next histogram over the entries in that bin
//   cut      the cut value and how many entries equal to it are kept; per chunk
//            the sum above the cut and the number of entries equal to it
//   pick     the chunk, then the entry, at which the running sum of the kept
//            entries in index order reaches u * (their sum)
// The cut is a radix select over the bit patterns of p (p >= 0, so the patterns
// order like the values): 11, 11 and 9 bits.  Top-k and top-p cut the same
// descending order, so one select serves both: scanning bins from the top it
// stops at the first where the count reaches k or the mass reaches
// top_p * total, whichever comes first.  Counts are integers and masses are
// 64-bit fixed point (p * 2^43, truncated), so the histograms do not depend on
// the order in which blocks add to them.
constexpr int SCHUNK = 4096;
constexpr int STHREADS = 256;
constexpr int NBINS = 2048;
__host__ __device__ constexpr int pass_shift(int pass) { return pass == 0 ? 20 : (pass == 1 ? 9 : 0); }
__host__ __device__ constexpr int pass_bins(int pass) { return pass == 2 ? 512 : 2048; }
constexpr double MASS_ONE = 8796093022208.0;  // 2^43: a million entries of mass 1 still fit 63 bits

struct SampleRow {
    unsigned int prefix;             // the cut value's bits decided so far
    int above;                       // entries above the chosen bin
    unsigned long long mass_above;   // their mass
    int in_bin;                      // entries in the chosen bin
    int ties_kept;                   // after the last pass: entries equal to the cut that are kept
    unsigned long long want_mass;    // top_p * total, fixed point
    int k_on, p_on;
    int k;
    int pad;
};

struct SampleWork {
    float* cmax;                  // [B][C]
    double* csum;                 // [B][C]
    int* hist_n;                  // [3][B][NBINS]
    unsigned long long* hist_m;   // [3][B][NBINS]
    SampleRow* rows;              // [3][B]: the state after each pass (a launch reads one, writes the next)
    int* tie_cnt;                 // [B][C]
    double* above_sum;            // [B][C]
    size_t pad_hist_bytes;        // the histograms lie first: this many bytes are cleared per call
};

__device__ __forceinline__ unsigned long long mass_of(float p) {
    return (unsigned long long)((double)p * MASS_ONE);
}

__device__ __forceinline__ double block_sum_double(double v, double* scratch8) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += scratch8[w];
    return t;
}

__global__ void __launch_bounds__(STHREADS)
sample_max_kernel(const float* __restrict__ logits, long long stride, int V, SampleWork w, int chunk) {
    __shared__ float sm[STHREADS / 32];
    pdl_prologue();
    const int c = blockIdx.x, b = blockIdx.y, C = gridDim.x;
    const float* row = logits + (size_t)b * stride;
    const int lo = c * chunk, hi = min(V, lo + chunk);
    float mx = -INFINITY;
    for (int i = lo + threadIdx.x; i < hi; i += STHREADS) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < STHREADS / 32; ++i) mx = fmaxf(mx, sm[i]);
        w.cmax[(size_t)b * C + c] = mx;
    }
}

// The histogram of one pass over this block's chunk, added to the row's.  A bin's
// mass is kept in shared memory as two 32-bit halves so that the additions are
// native 32-bit atomics: the low half wraps, and the addition that wrapped it
// (it sees the old value) carries one into the high half.  Integer additions
// commute, so the result does not depend on their order.
template <bool MASS>
__device__ void chunk_histogram(const float* __restrict__ p, int lo, int hi, unsigned int prefix,
                                unsigned int mask, int shift, int bins, int* hn,
                                unsigned int* hm_lo, unsigned int* hm_hi, int* g_n,
                                unsigned long long* g_m) {
    for (int i = threadIdx.x; i < bins; i += STHREADS) {
        hn[i] = 0;
        if (MASS) hm_lo[i] = hm_hi[i] = 0u;
    }
    __syncthreads();
    for (int i = lo + threadIdx.x; i < hi; i += STHREADS) {
        const float v = p[i];
        const unsigned int u = __float_as_uint(v);
        if ((u & mask) == prefix) {
            const int bin = (u >> shift) & (bins - 1);
            atomicAdd(&hn[bin], 1);
            if (MASS) {
                const unsigned long long m = mass_of(v);
                const unsigned int m_lo = (unsigned int)m, m_hi = (unsigned int)(m >> 32);
                const unsigned int old = atomicAdd(&hm_lo[bin], m_lo);
                const unsigned int carry = (old + m_lo < old) ? 1u : 0u;
                if (m_hi + carry) atomicAdd(&hm_hi[bin], m_hi + carry);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += STHREADS) {
        const int n = hn[i];
        if (n) {
            atomicAdd(&g_n[i], n);
            if (MASS) atomicAdd(&g_m[i], ((unsigned long long)hm_hi[i] << 32) | hm_lo[i]);
        }
    }
}

__global__ void __launch_bounds__(STHREADS)
sample_exp_kernel(const float* __restrict__ logits, long long stride, int V,
                  const float* __restrict__ temperature, float* __restrict__ probs, SampleWork w,
                  int cuts, int B, int chunk) {
    __shared__ float sm[STHREADS / 32];
    __shared__ double sd[STHREADS / 32];
    __shared__ int hn[NBINS];
    __shared__ unsigned int hm_lo[NBINS], hm_hi[NBINS];
    pdl_prologue();
    const int c = blockIdx.x, b = blockIdx.y, C = gridDim.x;
    const float* row = logits + (size_t)b * stride;
    float* p = probs + (size_t)b * V;
    const float T = temperature[b];
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < C; i += STHREADS) mx = fmaxf(mx, w.cmax[(size_t)b * C + i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = sm[0];
    for (int i = 1; i < STHREADS / 32; ++i) mx = fmaxf(mx, sm[i]);
    const int lo = c * chunk, hi = min(V, lo + chunk);
    double part = 0.0;
    for (int i = lo + threadIdx.x; i < hi; i += STHREADS) {
        const float e = expf((row[i] - mx) / T);
        p[i] = e;
        part += (double)e;
    }
    const double total = block_sum_double(part, sd);
    if (threadIdx.x == 0) w.csum[(size_t)b * C + c] = total;
    if (cuts) {  // 1: by count only (no row has a top-p), 2: counts and masses
        __syncthreads();
        if (cuts == 1)
            chunk_histogram<false>(p, lo, hi, 0u, 0u, pass_shift(0), pass_bins(0), hn, hm_lo, hm_hi,
                                   w.hist_n + (size_t)b * NBINS, w.hist_m + (size_t)b * NBINS);
        else
            chunk_histogram<true>(p, lo, hi, 0u, 0u, pass_shift(0), pass_bins(0), hn, hm_lo, hm_hi,
                                  w.hist_n + (size_t)b * NBINS, w.hist_m + (size_t)b * NBINS);
    }
}

// Which bin of pass `pass`'s histogram holds the cut.  Every thread of the block
// calls it; all return the same row state (also left in `out` by thread 0 when
// `out` is given).  Bins are walked from the top, eight (or two) a thread.
__device__ SampleRow decide(int pass, int b, int B, int V, const SampleWork& w, const int* top_k,
                            const float* top_p, SampleRow st, int* sh_i, unsigned long long* sh_m,
                            SampleRow* sh_row) {
    const int bins = pass_bins(pass);
    const int per = bins / STHREADS;
    const int* hn = w.hist_n + ((size_t)pass * B + b) * NBINS;
    const unsigned long long* hm = w.hist_m + ((size_t)pass * B + b) * NBINS;
    int cn[NBINS / STHREADS];
    unsigned long long cm[NBINS / STHREADS];
    int tn = 0;
    unsigned long long tm = 0ull;
    for (int q = 0; q < per; ++q) {
        const int j = bins - 1 - (threadIdx.x * per + q);
        cn[q] = hn[j];
        cm[q] = hm[j];
        tn += cn[q];
        tm += cm[q];
    }
    // inclusive scan over the threads (descending bins)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int in = tn;
    unsigned long long im = tm;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, in, o);
        const unsigned long long m2 = __shfl_up_sync(0xffffffffu, im, o);
        if (lane >= o) {
            in += a;
            im += m2;
        }
    }
    __syncthreads();  // sh_* free
    if (lane == 31) {
        sh_i[warp] = in;
        sh_m[warp] = im;
    }
    if (threadIdx.x == 0) sh_i[16] = 0x7fffffff;  // the first stopping position
    __syncthreads();
    int wn = 0, all_n = 0;
    unsigned long long wm = 0ull, all_m = 0ull;
    for (int i = 0; i < STHREADS / 32; ++i) {
        if (i < warp) {
            wn += sh_i[i];
            wm += sh_m[i];
        }
        all_n += sh_i[i];
        all_m += sh_m[i];
    }
    int n = st.above + wn + in - tn;                     // entries above this thread's first bin
    unsigned long long ms = st.mass_above + wm + im - tm;
    if (pass == 0) {
        // the row's parameters, fixed for the later passes
        const int k = top_k ? top_k[b] : 0;
        const float tp = top_p ? top_p[b] : 1.0f;
        st.k_on = (k > 0 && k < V) ? 1 : 0;
        st.k = k;
        st.p_on = (top_p && tp < 1.0f) ? 1 : 0;
        st.want_mass = (unsigned long long)((double)tp * (double)all_m);
    }
    const int n_all = st.above + all_n;  // the last occupied bin always stops the walk
    int my_stop = 0x7fffffff, my_n = 0, my_in = 0;
    unsigned long long my_m = 0ull;
    for (int q = 0; q < per; ++q) {
        if (cn[q] != 0) {
            const bool stop = (st.k_on && n + cn[q] >= st.k) || (st.p_on && ms + cm[q] >= st.want_mass) ||
                              n + cn[q] >= n_all;
            if (stop) {
                my_stop = threadIdx.x * per + q;
                my_n = n;
                my_m = ms;
                my_in = cn[q];
                break;
            }
        }
        n += cn[q];
        ms += cm[q];
    }
    if (my_stop != 0x7fffffff) atomicMin(&sh_i[16], my_stop);
    __syncthreads();
    if (my_stop != 0x7fffffff && sh_i[16] == my_stop) {
        SampleRow r = st;
        r.prefix = st.prefix | ((unsigned int)(bins - 1 - my_stop) << pass_shift(pass));
        r.above = my_n;
        r.mass_above = my_m;
        r.in_bin = my_in;
        *sh_row = r;
    }
    if (threadIdx.x == 0 && sh_i[16] == 0x7fffffff) {  // an empty histogram: nothing to cut
        SampleRow r = st;
        r.in_bin = 0;
        *sh_row = r;
    }
    __syncthreads();
    return *sh_row;
}

template <int PASS>  // 1 or 2: decide on pass PASS - 1, histogram of pass PASS
__global__ void __launch_bounds__(STHREADS)
sample_select_kernel(int V, const int* __restrict__ top_k, const float* __restrict__ top_p,
                     const float* __restrict__ probs, SampleWork w, int B, int chunk) {
    __shared__ int sh_i[17];
    __shared__ unsigned long long sh_m[STHREADS / 32];
    __shared__ SampleRow sh_row;
    pdl_prologue();
    const int c = blockIdx.x, b = blockIdx.y;
    SampleRow st;
    if (PASS == 1) {
        st.prefix = 0u;
        st.above = 0;
        st.mass_above = 0ull;
        st.in_bin = 0;
        st.ties_kept = 0;
        st.want_mass = 0ull;
        st.k_on = st.p_on = st.k = st.pad = 0;
    } else {
        st = w.rows[(size_t)(PASS - 2) * B + b];
    }
    st = decide(PASS - 1, b, B, V, w, top_k, top_p, st, sh_i, sh_m, &sh_row);
    // every block of the row reaches the same state; the row's last block records it
    // for the kernels that follow
    if (c == (int)gridDim.x - 1 && threadIdx.x == 0) w.rows[(size_t)(PASS - 1) * B + b] = st;
    // Only the entries of the chosen bin count now, a few hundred of a row: they go
    // straight into the row's histogram (integer additions: any order, the same result).
    const unsigned int mask = PASS == 1 ? (0x7ffu << 20) : ((0x7ffu << 20) | (0x7ffu << 9));
    const int lo = c * chunk, hi = min(V, lo + chunk);
    const float* p = probs + (size_t)b * V;
    int* g_n = w.hist_n + ((size_t)PASS * B + b) * NBINS;
    unsigned long long* g_m = w.hist_m + ((size_t)PASS * B + b) * NBINS;
    const int shift = pass_shift(PASS), bins = pass_bins(PASS);
    for (int i = lo + threadIdx.x; i < hi; i += STHREADS) {
        const float v = p[i];
        const unsigned int u = __float_as_uint(v);
        if ((u & mask) == st.prefix) {
            const int bin = (u >> shift) & (bins - 1);
            atomicAdd(&g_n[bin], 1);
            atomicAdd(&g_m[bin], mass_of(v));
        }
    }
}

__global__ void __launch_bounds__(STHREADS)
sample_cut_kernel(int V, const int* __restrict__ top_k, const float* __restrict__ top_p,
                  const float* __restrict__ probs, SampleWork w, int B, int chunk) {
    __shared__ int sh_i[17];
    __shared__ unsigned long long sh_m[STHREADS / 32];
    __shared__ SampleRow sh_row;
    __shared__ double sd[STHREADS / 32];
    __shared__ int st_n[STHREADS / 32];
    pdl_prologue();
    const int c = blockIdx.x, b = blockIdx.y, C = gridDim.x;
    SampleRow st = decide(2, b, B, V, w, top_k, top_p, w.rows[(size_t)B + b], sh_i, sh_m, &sh_row);
    // entries equal to the cut value that are kept: what the count still wants,
    // what the mass still wants, and no more than there are
    const unsigned int cut = st.prefix;
    int ties = st.in_bin;
    if (st.k_on) ties = min(ties, max(1, st.k - st.above));
    if (st.p_on) {
        const unsigned long long each = mass_of(__uint_as_float(cut));
        long long need = 1;
        if (each > 0ull && st.want_mass > st.mass_above)
            need = (long long)((st.want_mass - st.mass_above + each - 1ull) / each);
        if (need < 1) need = 1;
        if (need < (long long)ties) ties = (int)need;
    }
    st.ties_kept = ties;
    const float* p = probs + (size_t)b * V;
    const int lo = c * chunk, hi = min(V, lo + chunk);
    int n_tie = 0;
    double above = 0.0;
    for (int i = lo + threadIdx.x; i < hi; i += STHREADS) {
        const float v = p[i];
        const unsigned int u = __float_as_uint(v);
        if (u > cut) above += (double)v;
        else if (u == cut) ++n_tie;
    }
    const double total_above = block_sum_double(above, sd);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n_tie += __shfl_xor_sync(0xffffffffu, n_tie, o);
    if ((threadIdx.x & 31) == 0) st_n[threadIdx.x >> 5] = n_tie;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int i = 0; i < STHREADS / 32; ++i) t += st_n[i];
        w.tie_cnt[(size_t)b * C + c] = t;
        w.above_sum[(size_t)b * C + c] = total_above;
        if (c == C - 1) w.rows[(size_t)2 * B + b] = st;
    }
}

// The draw.  One block a row: the chunk in which the running sum of kept entries
// reaches the draw, then the entry inside it; sums in double, in index order.
__global__ void __launch_bounds__(STHREADS)
sample_pick_kernel(int V, int C, const float* __restrict__ uniform, const float* __restrict__ probs,
                   SampleWork w, int cuts, int B, int chunk, int* __restrict__ out) {
    __shared__ double sh_d[STHREADS / 32 + 2];
    __shared__ int sh_n[STHREADS / 32 + 4];
    pdl_prologue();
    const int b = blockIdx.x;
    const float* p = probs + (size_t)b * V;
    unsigned int cut = 0u;
    int ties_kept = 0x7fffffff;
    if (cuts) {
        const SampleRow st = w.rows[(size_t)2 * B + b];
        cut = st.prefix;
        ties_kept = st.ties_kept;
    }
    const double cut_v = (double)__uint_as_float(cut);
    // the chunks' sums and tie counts, fetched by all threads (up to PICK_C chunks;
    // beyond that thread 0 reads them from where they lie)
    constexpr int PICK_C = 512;
    __shared__ double s_sum[PICK_C];
    __shared__ int s_tie[PICK_C];
    const bool staged = C <= PICK_C;
    if (staged) {
        for (int c = threadIdx.x; c < C; c += STHREADS) {
            s_sum[c] = cuts ? w.above_sum[(size_t)b * C + c] : w.csum[(size_t)b * C + c];
            s_tie[c] = cuts ? w.tie_cnt[(size_t)b * C + c] : 0;
        }
        __syncthreads();
    }
    auto chunk_sum = [&](int c) {
        return staged ? s_sum[c] : (cuts ? w.above_sum[(size_t)b * C + c] : w.csum[(size_t)b * C + c]);
    };
    auto chunk_ties = [&](int c) { return staged ? s_tie[c] : (cuts ? w.tie_cnt[(size_t)b * C + c] : 0); };
    // thread 0: the kept sum of every chunk, in chunk order, and the chunk of the draw
    if (threadIdx.x == 0) {
        double renorm = 0.0;
        int seen = 0;
        for (int c = 0; c < C; ++c) {
            double s = chunk_sum(c);
            if (cuts) {
                const int nt = chunk_ties(c);
                const int kept = max(0, min(nt, ties_kept - seen));
                seen += nt;
                s += (double)kept * cut_v;
            }
            renorm += s;
        }
        const double draw = (double)uniform[b] * renorm;
        double acc = 0.0;
        int pick = -1, last = -1, ties_before = 0, last_ties = 0;
        double last_acc = 0.0;
        seen = 0;
        for (int c = 0; c < C; ++c) {
            double s = chunk_sum(c);
            int nt = 0;
            if (cuts) {
                nt = chunk_ties(c);
                const int kept = max(0, min(nt, ties_kept - seen));
                s += (double)kept * cut_v;
            }
            if (s > 0.0) {
                last = c;
                last_acc = acc;
                last_ties = seen;
                if (draw <= acc + s) {
                    pick = c;
                    ties_before = seen;
                    break;
                }
            }
            acc += s;
            seen += nt;
        }
        if (pick < 0) {  // rounding left the draw above the total: the last chunk that keeps anything
            pick = last;
            acc = last_acc;
            ties_before = last_ties;
        }
        sh_n[STHREADS / 32] = pick;
        sh_n[STHREADS / 32 + 1] = ties_before;
        sh_d[STHREADS / 32] = acc;
        sh_d[STHREADS / 32 + 1] = draw;
    }
    __syncthreads();
    const int pick = sh_n[STHREADS / 32];
    if (pick < 0) {  // nothing kept anywhere (cannot happen: the maximum has p = 1)
        if (threadIdx.x == 0) out[b] = 0;
        return;
    }
    const int ties_before = sh_n[STHREADS / 32 + 1];
    const double acc0 = sh_d[STHREADS / 32], draw = sh_d[STHREADS / 32 + 1];
    // inside the chunk: contiguous entries a thread
    const int per = chunk / STHREADS;
    const int i0 = pick * chunk + threadIdx.x * per, i1 = min(V, i0 + per);
    int my_ties = 0;
    for (int i = i0; i < i1; ++i)
        if (__float_as_uint(p[i]) == cut) ++my_ties;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int it = my_ties;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, it, o);
        if (lane >= o) it += a;
    }
    if (lane == 31) sh_n[warp] = it;
    __syncthreads();
    int seen0 = ties_before + it - my_ties;
    for (int i = 0; i < warp; ++i) seen0 += sh_n[i];
    double mine = 0.0;
    {
        int seen = seen0;
        for (int i = i0; i < i1; ++i) {
            const unsigned int u = __float_as_uint(p[i]);
            bool keep = u > cut;
            if (u == cut) keep = (seen++ < ties_kept);
            if (keep) mine += (double)p[i];
        }
    }
    double inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double a = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += a;
    }
    if (lane == 31) sh_d[warp] = inc;
    if (threadIdx.x == 0) sh_n[STHREADS / 32 + 2] = 0x7fffffff;
    __syncthreads();
    double before = acc0 + inc - mine;
    for (int i = 0; i < warp; ++i) before += sh_d[i];
    // the first thread whose kept entries reach the draw; failing that, the last that keeps any
    if (mine > 0.0 && draw <= before + mine) atomicMin(&sh_n[STHREADS / 32 + 2], (int)threadIdx.x);
    __syncthreads();
    int who = sh_n[STHREADS / 32 + 2];
    if (who == 0x7fffffff) {
        if (threadIdx.x == 0) sh_n[STHREADS / 32 + 3] = -1;
        __syncthreads();
        if (mine > 0.0) atomicMax(&sh_n[STHREADS / 32 + 3], (int)threadIdx.x);
        __syncthreads();
        who = sh_n[STHREADS / 32 + 3];
    }
    if ((int)threadIdx.x == who) {
        double acc = before;
        int seen = seen0;
        int chosen = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            const unsigned int u = __float_as_uint(p[i]);
            bool keep = u > cut;
            if (u == cut) keep = (seen++ < ties_kept);
            if (!keep) continue;
            last_kept = i;
            acc += (double)p[i];
            if (draw <= acc) {
                chosen = i;
                break;
            }
        }
        out[b] = chosen >= 0 ? chosen : (last_kept >= 0 ? last_kept : 0);
    }
    if (who < 0 && threadIdx.x == 0) out[b] = 0;
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

// Bytes of working memory a call with B rows of V entries needs besides `probs`.
static size_t sample_work_layout(int B, int V, char* base, SampleWork* w) {
    const size_t C = (size_t)(V + SCHUNK - 1) / SCHUNK;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char* p = base ? base + off : nullptr;
        off += (bytes + 255) / 256 * 256;
        return p;
    };
    char* hist_n = take((size_t)3 * B * NBINS * sizeof(int));
    char* hist_m = take((size_t)3 * B * NBINS * sizeof(unsigned long long));
    const size_t hist_bytes = off;  // zeroed before a call with a cut
    char* cmax = take((size_t)B * C * sizeof(float));
    char* csum = take((size_t)B * C * sizeof(double));
    char* rows = take((size_t)3 * B * sizeof(SampleRow));
    char* tie_cnt = take((size_t)B * C * sizeof(int));
    char* above_sum = take((size_t)B * C * sizeof(double));
    if (w) {
        w->hist_n = (int*)hist_n;
        w->hist_m = (unsigned long long*)hist_m;
        w->cmax = (float*)cmax;
        w->csum = (double*)csum;
        w->rows = (SampleRow*)rows;
        w->tie_cnt = (int*)tie_cnt;
        w->above_sum = (double*)above_sum;
        // what the caller has to clear is the front of the buffer
        w->pad_hist_bytes = hist_bytes;
    }
    return off;
}

extern "C" long long rfx_sample_work_bytes(int B, int V) {
    if (B <= 0 || V <= 0) return 0;
    return (long long)sample_work_layout(B, V, nullptr, nullptr);
}

// temperature[B] > 0; top_k[B] (<= 0: off) or NULL; top_p[B] (>= 1: off) or
// NULL; uniform[B] in [0, 1); probs: scratch of B * V floats; work: scratch of
// rfx_sample_work_bytes(B, V) bytes, 256-byte aligned.
extern "C" int rfx_sample(const float* logits, long long stride, int B, int V,
                          const float* temperature, const int* top_k, const float* top_p,
                          const float* uniform, float* probs, void* work, int* out, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !probs || !work) return RFX_ERR_BAD_ARG;
    if (B > 65535) return RFX_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(work) & 255) != 0) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    SampleWork w;
    sample_work_layout(B, V, (char*)work, &w);
    // chunks of SCHUNK entries (many small blocks are faster than few large ones: 35 us against
    // 119 us for 64 rows of 151,936); larger chunks only for grids of tens of thousands of blocks
    const long long blocks = (long long)B * ((V + SCHUNK - 1) / SCHUNK);
    const int chunk = SCHUNK * (int)((blocks + 16383) / 16384);
    const int C = (V + chunk - 1) / chunk;
    const int cuts = top_p ? 2 : (top_k ? 1 : 0);
    const dim3 grid(C, B);
    if (cuts) {
        cudaError_t e = cudaMemsetAsync(work, 0, w.pad_hist_bytes, s);
        if (e != cudaSuccess) return (int)e;
    }
    RFX_LAUNCH(sample_max_kernel, grid, STHREADS, 0, s, logits, stride, V, w, chunk);
    RFX_LAUNCH(sample_exp_kernel, grid, STHREADS, 0, s, logits, stride, V, temperature, probs, w, cuts, B, chunk);
    if (cuts) {
        RFX_LAUNCH(sample_select_kernel<1>, grid, STHREADS, 0, s, V, top_k, top_p, (const float*)probs, w, B, chunk);
        RFX_LAUNCH(sample_select_kernel<2>, grid, STHREADS, 0, s, V, top_k, top_p, (const float*)probs, w, B, chunk);
        RFX_LAUNCH(sample_cut_kernel, grid, STHREADS, 0, s, V, top_k, top_p, (const float*)probs, w, B, chunk);
    }
    RFX_LAUNCH(sample_pick_kernel, B, STHREADS, 0, s, V, C, uniform, (const float*)probs, w, cuts, B, chunk, out);
    return 0;
}
