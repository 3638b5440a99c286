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
};

}  // namespace
