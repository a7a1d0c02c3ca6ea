// Building blocks of the bfloat16 attention kernels: shared-memory tiles with
// padded rows, asynchronous copies, ldmatrix fragment loads and the
// m16n8k16 tensor-core step, plus the online-softmax update of one
// 16-row x (8 * NT)-key score tile.
//
// Tiles are [rows][D + 8] bfloat16: the 16 bytes of padding per row shift
// consecutive rows by four banks, which makes every ldmatrix access pattern used
// here conflict-free for any D that is a multiple of 16.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace attn {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16-byte asynchronous copy; with valid == false the destination is zero-filled.
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int src = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem),
                 "r"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"(smem_u32(p)));
}
// An 8 x 8 matrix of 16-bit elements held one row pair per thread, transposed
// across the warp.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}

// d (16x8 float) += a (16x16 bf16, row) * b (16x8 bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copy `rows_valid` rows of a contiguous [rows][D] global tile into a padded
// shared tile; rows beyond are zero-filled.  All `nthreads` threads take part.
template <int D>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* smem, const __nv_bfloat16* gmem,
                                                int rows, int rows_valid, int tid, int nthreads) {
    constexpr int CPR = D / 8;  // 16-byte chunks per row
    for (int i = tid; i < rows * CPR; i += nthreads) {
        const int r = i / CPR, c = i % CPR;
        cp_async_16(smem + r * (D + 8) + c * 8, gmem + (size_t)r * D + c * 8, r < rows_valid);
    }
}

// One warp: scores of its 16 query rows against NT * 8 keys of a K tile
// (starting at tile row `key0`), masked, then the online-softmax update of
// (m, l, acc) with the same rows of the V tile.
//   qs: [16][D + 8] query rows (already in shared memory)
//   kvalid(j): whether tile key j (0-based in the tile) is visible to row half
//   hrow (0: row lane/4, 1: row lane/4 + 8)
// scale_log2 = scale * log2(e); probabilities are 2^(s * scale_log2 - m).
template <int D, int NT, typename Visible>
__device__ __forceinline__ void attend_tile(const __nv_bfloat16* qs, const __nv_bfloat16* ks,
                                            const __nv_bfloat16* vs, int key0, float scale_log2,
                                            Visible visible, float (&m)[2], float (&l)[2],
                                            float (&acc)[D / 8][4]) {
    static_assert(NT % 2 == 0, "keys come in pairs of 8-key tiles");
    const int lane = threadIdx.x & 31;
    constexpr int LD = D + 8;
    float s[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[t][i] = 0.0f;

#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16) {
        uint32_t a[4];
        ldmatrix_x4(a, qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + k0 + 8 * (lane >> 4));
#pragma unroll
        for (int t = 0; t < NT; t += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, ks + (key0 + t * 8 + (lane & 7) + 8 * (lane >> 4)) * LD + k0 +
                               8 * ((lane >> 3) & 1));
            mma_bf16(s[t], a, b[0], b[1]);
            mma_bf16(s[t + 1], a, b[2], b[3]);
        }
    }

    // mask, scale, row maxima
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = key0 + t * 8 + 2 * (lane & 3) + (i & 1);
            const int h = i >> 1;
            const float v = visible(key, h) ? s[t][i] * scale_log2 : -INFINITY;
            s[t][i] = v;
            mx[h] = fmaxf(mx[h], v);
        }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        // all keys of this tile and all earlier ones masked: keep the state untouched
        corr[h] = (m_new == -INFINITY) ? 1.0f : exp2f(m[h] - m_new);
        m[h] = m_new;
    }
    float rs[2] = {0.0f, 0.0f};
    uint32_t p[NT][2];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = i >> 1;
            e[i] = (m[h] == -INFINITY) ? 0.0f : exp2f(s[t][i] - m[h]);
            rs[h] += e[i];
        }
        p[t][0] = pack_bf16(e[0], e[1]);
        p[t][1] = pack_bf16(e[2], e[3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
        l[h] = l[h] * corr[h] + rs[h];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        acc[n][0] *= corr[0];
        acc[n][1] *= corr[0];
        acc[n][2] *= corr[1];
        acc[n][3] *= corr[1];
    }
    // acc += P V: 16 keys per step; P's score fragments are A fragments as they are
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        const uint32_t a[4] = {p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1]};
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vs + (key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD +
                                     n * 8 + 8 * (lane >> 4));
            mma_bf16(acc[n], a, b[0], b[1]);
            mma_bf16(acc[n + 1], a, b[2], b[3]);
        }
    }
}

// ---- decode: the keys as the rows of the MMA ---------------------------------
// One query position has only its group's few heads for rows, so the tile is
// turned around: S^T [16 keys x 8 heads] = K [16 x D] . Q^T, O^T [D x 8 heads] +=
// V^T [D x 16 keys] . P [16 keys x 8 heads].  Against heads as rows this halves
// the MMAs and fragment loads per key, and all eight columns are heads (four
// of them real at a group of four, against four of sixteen rows).
//
// The query heads are the B operand of every step: their fragments are loaded
// once (qf[k] for the k-th 16 columns of D) from a tile qs [8][D + 8].
template <int D>
__device__ __forceinline__ void load_query_fragments(const __nv_bfloat16* qs, uint32_t (&qf)[D / 16][2]) {
    const int lane = threadIdx.x & 31;
    constexpr int LD = D + 8;
#pragma unroll
    for (int k = 0; k < D / 16; ++k)
        ldmatrix_x2(qf[k], qs + (lane & 7) * LD + k * 16 + 8 * ((lane >> 3) & 1));
}

// One warp, 16 keys of a K/V tile starting at tile row `key0`.  A thread's
// state covers heads 2 (lane % 4) and 2 (lane % 4) + 1: running maxima m[2]
// (the same in the eight lanes that share lane % 4), its own share of their
// sums l[2] (added across those lanes by the caller at the end), and
// acc[i][..]: rows 16 i + lane / 4 (+ 8) of O^T for the two heads.
//   visible(j): whether tile key j (0-based in the tile) is visible
//   SWZ: the tiles' layout.  false: [keys][D + 8], rows padded.  true: as the TMA
//   writes them with the 128-byte swizzle, blocks of 64 columns, [D / 64][keys][64],
//   a row's 16-byte chunk c at chunk c ^ (row & 7) (tile base 1024-byte aligned).
template <int D, bool SWZ>
__device__ __forceinline__ const __nv_bfloat16* tile_at(const __nv_bfloat16* tile, int row, int col) {
    if (SWZ) {
        const int chunk = ((col & 63) >> 3) ^ (row & 7);
        return tile + (col >> 6) * (64 * 64) + row * 64 + chunk * 8 + (col & 7);
    }
    return tile + row * (D + 8) + col;
}

template <int D, bool SWZ = false, typename Visible>
__device__ __forceinline__ void attend_keys16(const uint32_t (&qf)[D / 16][2], const __nv_bfloat16* ks,
                                              const __nv_bfloat16* vs, int key0, float scale_log2,
                                              Visible visible, float (&m)[2], float (&l)[2],
                                              float (&acc)[D / 16][4]) {
    const int lane = threadIdx.x & 31;
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int k = 0; k < D / 16; ++k) {
        uint32_t a[4];
        ldmatrix_x4(a, tile_at<D, SWZ>(ks, key0 + (lane & 7) + 8 * ((lane >> 3) & 1), k * 16 + 8 * (lane >> 4)));
        mma_bf16(s, a, qf[k][0], qf[k][1]);
    }
    // s[0], s[1]: key lane / 4, the two heads; s[2], s[3]: key lane / 4 + 8
    const int ka = key0 + (lane >> 2), kb = ka + 8;
    const bool va = visible(ka), vb = visible(kb);
    float v[4];
    v[0] = va ? s[0] * scale_log2 : -INFINITY;
    v[1] = va ? s[1] * scale_log2 : -INFINITY;
    v[2] = vb ? s[2] * scale_log2 : -INFINITY;
    v[3] = vb ? s[3] * scale_log2 : -INFINITY;
    float corr[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        float mx = fmaxf(v[j], v[j + 2]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m[j], mx);
        // all keys so far masked: keep the state untouched
        corr[j] = (m_new == -INFINITY) ? 1.0f : exp2f(m[j] - m_new);
        m[j] = m_new;
    }
    float e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = (m[i & 1] == -INFINITY) ? 0.0f : exp2f(v[i] - m[i & 1]);
    l[0] = l[0] * corr[0] + (e[0] + e[2]);
    l[1] = l[1] * corr[1] + (e[1] + e[3]);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
        acc[i][0] *= corr[0];
        acc[i][1] *= corr[1];
        acc[i][2] *= corr[0];
        acc[i][3] *= corr[1];
    }
    // P [keys x heads] as the B operand: each 8 x 8 half transposed across the warp
    const uint32_t b0 = movmatrix_trans(pack_bf16(e[0], e[1]));
    const uint32_t b1 = movmatrix_trans(pack_bf16(e[2], e[3]));
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, tile_at<D, SWZ>(vs, key0 + (lane & 7) + 8 * (lane >> 4), i * 16 + 8 * ((lane >> 3) & 1)));
        mma_bf16(acc[i], a, b0, b1);
    }
}

}  // namespace attn
