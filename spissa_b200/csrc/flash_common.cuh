// Pieces shared by the mma.sync attention kernels: cp.async and ldmatrix wrappers, the padded
// shared-memory tile of one cache page, one online-softmax step of a warp over the keys of a tile.
#pragma once
#include "async_copy.cuh"

namespace {

constexpr int KT = 64;                        // keys per tile = page size
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {           // 2^x, flushes denormals, exp2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&p;
}

template <int HD>
struct Tile {
    static constexpr int ROW = HD * 2 + 16;           // bytes per shared-memory row; the pad spreads banks
    static constexpr int BYTES = KT * ROW;
    static constexpr int CHUNKS = HD / 8;             // 16-byte pieces per row
};

// Copy rows [0, n_rows) x HD of a bfloat16 matrix with row stride ``ld`` (elements) into a padded
// shared tile; rows from n_rows to 64 are zeroed. All ``nthreads`` threads take part.
template <int HD>
__device__ __forceinline__ void load_tile_async(uint32_t dst, const __nv_bfloat16* src, size_t ld, int n_rows,
                                                int tid, int nthreads) {
    using T = Tile<HD>;
    for (int c = tid; c < KT * T::CHUNKS; c += nthreads) {
        const int r = c / T::CHUNKS, k = c % T::CHUNKS;
        const uint32_t d = dst + r * T::ROW + k * 16;
        if (r < n_rows) cp_async16(d, src + (size_t)r * ld + k * 8);
        else asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(d), "r"(0u) : "memory");
    }
}

// One warp, 16 query rows (fragments ``qf``), keys [key0, key0 + 8*NT) of the tile in shared memory.
// Row ``g`` of the fragment sees keys lo[0]..hi[0], row g+8 keys lo[1]..hi[1] (absolute positions);
// with MASKED false the caller vouches that every key of the tile is visible to every row.
// m holds the running maximum of the raw scores times scale_log2 (the log2 domain).
template <int HD, int NT, bool MASKED>
__device__ __forceinline__ void flash_step(const uint32_t (&qf)[HD / 16][4], uint32_t k_tile, uint32_t v_tile,
                                           int key0, int tile_pos0, const int (&lo)[2], const int (&hi)[2],
                                           float scale_log2, float (&o)[HD / 8][4], float (&m)[2], float (&l)[2],
                                           int lane) {
    using T = Tile<HD>;
    float s[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    // S = Q · Kᵀ. With few key blocks per warp the products of even and odd steps along head_dim go to
    // accumulators of their own, so that an mma does not have to wait for the one before it.
    constexpr bool SPLIT = NT <= 2 && (HD / 16) % 2 == 0;
    float s2[SPLIT ? NT : 1][4];
    if (SPLIT) {
#pragma unroll
        for (int i = 0; i < NT; ++i) s2[i][0] = s2[i][1] = s2[i][2] = s2[i][3] = 0.0f;
    }
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            const int key = key0 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int d = kk * 16 + (((lane >> 3) & 1) << 3);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_tile + key * T::ROW + d * 2, b0, b1, b2, b3);
            if (SPLIT && (kk & 1)) {
                mma_bf16(s2[2 * np], qf[kk], b0, b1);
                mma_bf16(s2[2 * np + 1], qf[kk], b2, b3);
            } else {
                mma_bf16(s[2 * np], qf[kk], b0, b1);
                mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
            }
        }
    }
    if (SPLIT) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] += s2[i][e];
    }
    // mask, running maximum (of the raw scores; the scale is positive)
    const int t = lane & 3;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            if (MASKED) {
                const int key = tile_pos0 + key0 + nt * 8 + 2 * t + (e & 1);
                if (key > hi[r] || key < lo[r]) s[nt][e] = -INFINITY;
            }
            mx[r] = fmaxf(mx[r], s[nt][e]);
        }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mnew = fmaxf(m[r], mx[r] * scale_log2);
        msafe[r] = (mnew == -INFINITY) ? 0.0f : mnew;
        corr[r] = fast_exp2(m[r] - msafe[r]);         // m = -inf gives 0
        m[r] = mnew;
    }
    float sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = fast_exp2(fmaf(s[nt][e], scale_log2, -msafe[e >> 1]));   // one FFMA, one MUFU
            s[nt][e] = p;
            sum[e >> 1] += p;
        }
    }
    l[0] = l[0] * corr[0] + sum[0];                   // per-lane partial; lanes are summed at the end
    l[1] = l[1] * corr[1] + sum[1];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // O += P · V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            const int key = key0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int d = dp * 16 + ((lane >> 4) << 3);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_tile + key * T::ROW + d * 2, b0, b1, b2, b3);
            mma_bf16(o[2 * dp], a, b0, b1);
            mma_bf16(o[2 * dp + 1], a, b2, b3);
        }
    }
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {   // the 8x8 matrix of 16-bit values a warp holds, transposed
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// Decoding: few query rows (the heads that share a kv head), many keys. Here the KEYS are the M of the
// instruction and the heads its N (8 per tile), so up to 8 heads cost one mma per 16 keys and 16 dims, where
// the form with the heads as M costs two with most of its rows idle.
//   Sᵀ[key, head] = K[key, :] · Qᵀ       A = K tile (ldmatrix), B = fragments of Qᵀ (``qb``)
//   Oᵀ[d, head]  += Vᵀ[d, key] · Pᵀ      A = V tile (ldmatrix.trans), B = Pᵀ = the transposed fragment of Sᵀ
// One warp, keys [key0, key0 + 16) of the tile; a lane holds keys g, g + 8 of heads 2t, 2t + 1 of each head
// tile (g = lane / 4, t = lane % 4). ``m`` is the reference maximum per head in the log2 domain, the same in
// the 8 lanes that share t. It moves only when a score exceeds it by more than 8 (then the lanes agree on the
// new maximum and rescale o and l); otherwise P = 2^(s - m) ≤ 256 and no lane talks to another. The result
// o / l does not depend on the reference. ``l`` is per lane (its own keys); the caller adds the lanes.
template <int HD, int NH, bool MASKED>
__device__ __forceinline__ void decode_step_t(const uint32_t (&qb)[HD / 16][NH][2], uint32_t k_tile, uint32_t v_tile,
                                              int key0, int tile_pos0, int lo, int hi, float scale_log2,
                                              float (&o)[HD / 16][NH][4], float (&m)[NH][2], float (&l)[NH][2],
                                              int lane) {
    using T = Tile<HD>;
    const int g = lane >> 2;
    float s[NH][4], s2[NH][4];                        // two chains of products: an mma need not wait for the one before
#pragma unroll
    for (int i = 0; i < NH; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] = s2[i][e] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(k_tile + (key0 + (lane & 15)) * T::ROW + (kk * 16 + ((lane >> 4) << 3)) * 2, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int i = 0; i < NH; ++i) {
            if (kk & 1) mma_bf16(s2[i], a, qb[kk][i][0], qb[kk][i][1]);
            else mma_bf16(s[i], a, qb[kk][i][0], qb[kk][i][1]);
        }
    }
    bool move = false;
#pragma unroll
    for (int i = 0; i < NH; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = (s[i][e] + s2[i][e]) * scale_log2;
            if (MASKED) {
                const int key = tile_pos0 + key0 + g + ((e >> 1) << 3);
                if (key > hi || key < lo) v = -INFINITY;
            }
            s[i][e] = v;
        }
        move = move || fmaxf(s[i][0], s[i][2]) > m[i][0] + 8.0f || fmaxf(s[i][1], s[i][3]) > m[i][1] + 8.0f;
    }
    if (__any_sync(0xffffffffu, move)) {
#pragma unroll
        for (int i = 0; i < NH; ++i) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float mx = fmaxf(s[i][c], s[i][c + 2]);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float mnew = fmaxf(m[i][c], mx);
                const float corr = fast_exp2(m[i][c] - ((mnew == -INFINITY) ? 0.0f : mnew));     // m = -inf gives 0
                m[i][c] = mnew;
                l[i][c] *= corr;
#pragma unroll
                for (int dt = 0; dt < HD / 16; ++dt) { o[dt][i][c] *= corr; o[dt][i][c + 2] *= corr; }
            }
        }
    }
    uint32_t pb[NH][2];
#pragma unroll
    for (int i = 0; i < NH; ++i) {
        const float m0 = (m[i][0] == -INFINITY) ? 0.0f : m[i][0], m1 = (m[i][1] == -INFINITY) ? 0.0f : m[i][1];
        const float p0 = fast_exp2(s[i][0] - m0), p1 = fast_exp2(s[i][1] - m1);
        const float p2 = fast_exp2(s[i][2] - m0), p3 = fast_exp2(s[i][3] - m1);
        l[i][0] += p0 + p2;
        l[i][1] += p1 + p3;
        pb[i][0] = movmatrix_trans(pack_bf16(p0, p1));            // keys key0 .. +7 of head g
        pb[i][1] = movmatrix_trans(pack_bf16(p2, p3));            // keys key0 + 8 .. +15
    }
#pragma unroll
    for (int dt = 0; dt < HD / 16; ++dt) {
        uint32_t a[4];
        ldmatrix_x4_trans(v_tile + (key0 + (lane & 7) + ((lane >> 4) << 3)) * T::ROW + (dt * 16 + (((lane >> 3) & 1) << 3)) * 2,
                          a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int i = 0; i < NH; ++i) mma_bf16(o[dt][i], a, pb[i][0], pb[i][1]);
    }
}

template <int HD>
__device__ __forceinline__ void load_q_frags(uint32_t q_tile, int row0, int lane, uint32_t (&qf)[HD / 16][4]) {
    using T = Tile<HD>;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = row0 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int d = kk * 16 + ((lane >> 4) << 3);
        ldmatrix_x4(q_tile + row * T::ROW + d * 2, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
}

struct PagedKV {
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    const int* page_table;      // [rows][max_pages]
    const int* seq_row;         // [B] row of each sequence in the table
    int max_pages;
    int nkv;
    SpRange rg;                 // what the debug build checks table entries against
};

}  // namespace
