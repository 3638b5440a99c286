// Generic kernels: every op of the forward pass for every storage type and every size.
//
// These are the true 32-bit path of the whole model (plain FFMA, accurate expf /
// sqrtf / division, no tensor cores, no reduced-precision matrix mode) and the
// fallback for sizes that a specialised kernel refuses. Each output element is
// reduced in an order that depends only on its own row, never on what else is in
// the batch, so that cutting the same tokens into other steps changes no bit.
//
// Formulas follow the reference runtime (paths within Erik-cpu-create/spissa):
//   embedding       crates/spissa-runtime/src/ops.rs:6-30
//   rms norm        crates/spissa-runtime/src/ops.rs:159-179
//   linear          crates/spissa-runtime/src/ops.rs:62-105   (y = x·Wᵀ, W [out,in])
//   rotate-half     crates/spissa-runtime/src/rotary.rs:98-123, :454-481
//   attention       crates/spissa-runtime/src/rotary.rs:335-415, :549-569
//   silu            crates/spissa-runtime/src/ops.rs:192-194
//   argmax          crates/spissa-runtime/src/ops.rs:309-324  (first maximum wins)
#include "async_copy.cuh"

SP_API const char* sp_generic_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(generic)

// ============================================================== embedding
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int T, int H, int V, int* status) {
    const int t = blockIdx.x;
    if (t >= T) return;
    const int id = ids[t];
    const bool ok = (id >= 0 && id < V);
    if (!ok && threadIdx.x == 0 && status) atomicCAS(status, 0, 301);     // a token id outside the table
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[(size_t)t * H + c] = ok ? sp_ld(table, (size_t)id * H + c) : 0.0f;
}

SP_API int sp_embed_gather(const void* table, int table_dt, const int* ids, float* out,
                           int T, int H, int V, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dt == SP_DT_F32)
        SP_CHECK_CALL("embed_gather", sp_launch_cluster(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream, 1,
                                                   (const float*)table, ids, out, T, H, V, status));
    else if (table_dt == SP_DT_BF16)
        SP_CHECK_CALL("embed_gather", sp_launch_cluster(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                                                   1, (const __nv_bfloat16*)table, ids, out, T, H, V, status));
    else
        SP_FAIL("embed_gather: unsupported table dtype code %d", table_dt);
    return 0;
}

// ============================================================== rms norm
// One block per output row. ``rows`` (optional) gathers input rows: out row r is the
// norm of x row rows[r]. Statistics and the product are 32-bit; the result is rounded
// once, on the store.
__global__ void rmsnorm_kernel(const float* __restrict__ x, const void* __restrict__ w, int w_dt,
                               void* __restrict__ out, int out_dt, const int* __restrict__ rows,
                               int n_rows, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = x[src + c];
        ss = fmaf(v, v, ss);
    }
    ss = sp_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = x[src + c] * inv * sp_ld_dt(w, w_dt, c);
        sp_st_dt(out, out_dt, (size_t)r * H + c, v);
    }
}

// The same with each row held in registers: one read of x. For H a multiple of 4 up to 4096.
__global__ void __launch_bounds__(256)
rmsnorm_row_kernel(const float* __restrict__ x, const void* __restrict__ w, int w_dt, void* __restrict__ out,
                   int out_dt, const int* __restrict__ rows, int n_rows, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const float4* src = (const float4*)(x + (size_t)(rows ? rows[r] : r) * H);
    const int n4 = H >> 2;
    float4 v[4];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        v[i] = c < n4 ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = sp_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c >= n4) continue;
        float wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = sp_ld_dt(w, w_dt, (size_t)c * 4 + j);
        const float o0 = v[i].x * inv * wv[0], o1 = v[i].y * inv * wv[1];
        const float o2 = v[i].z * inv * wv[2], o3 = v[i].w * inv * wv[3];
        const size_t o = (size_t)r * H + (size_t)c * 4;
        if (out_dt == SP_DT_F32) {
            *(float4*)((float*)out + o) = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
            uint2 pk;
            pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
            *(uint2*)((__nv_bfloat16*)out + o) = pk;
        }
    }
}

// One warp per row, the row in registers (NV float4 per lane), eight rows per block: every lane has all its loads
// in flight at once and the row sum needs no shared memory. For H = 128·NV.
template <int NV, bool WBF16>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* __restrict__ x, const void* __restrict__ w, int w_dt, void* __restrict__ out,
                    int out_dt, const int* __restrict__ rows, int n_rows, int H, float eps) {
    sp_allow_dependents();
    sp_wait_for_predecessor();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    if (r >= n_rows) return;
    const float4* src = (const float4*)(x + (size_t)(rows ? rows[r] : r) * H);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = src[lane + 32 * i];
    // bfloat16 weights are asked for before the row's sum is known: one trip to memory instead of two in a row
    // (float32 weights would not fit the registers next to the row)
    uint2 wb[WBF16 ? NV : 1];
    if (WBF16) {
#pragma unroll
        for (int i = 0; i < NV; ++i) wb[i] = ((const uint2*)w)[lane + 32 * i];
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = sp_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        float wv[4];
        if (WBF16) {
            const __nv_bfloat162 w01 = *(const __nv_bfloat162*)&wb[i].x, w23 = *(const __nv_bfloat162*)&wb[i].y;
            wv[0] = __low2float(w01); wv[1] = __high2float(w01); wv[2] = __low2float(w23); wv[3] = __high2float(w23);
        } else {
            const float4 wf = ((const float4*)w)[c];
            wv[0] = wf.x; wv[1] = wf.y; wv[2] = wf.z; wv[3] = wf.w;
        }
        const float o0 = v[i].x * inv * wv[0], o1 = v[i].y * inv * wv[1];
        const float o2 = v[i].z * inv * wv[2], o3 = v[i].w * inv * wv[3];
        const size_t o = (size_t)r * H + (size_t)c * 4;
        if (out_dt == SP_DT_F32) {
            *(float4*)((float*)out + o) = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
            uint2 pk;
            pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
            *(uint2*)((__nv_bfloat16*)out + o) = pk;
        }
    }
}

SP_API int sp_rmsnorm(const float* x, const void* w, int w_dt, void* out, int out_dt, const int* rows,
                      int n_rows, int H, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((w_dt | out_dt) & ~1) SP_FAIL("rmsnorm: unsupported dtype code");
    // fixed block sizes: the order of the row sum must not depend on the batch
    const bool aligned = ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)w) & 15) == 0);
#define SP_NORM_WARP(NV)                                                                                        \
    if (aligned && H == 128 * NV) {                                                                             \
        if (w_dt == SP_DT_BF16)                                                                                 \
            sp_launch_dependent(rmsnorm_warp_kernel<NV, true>, dim3((n_rows + 7) / 8), dim3(256), 0, stream, x, w, w_dt, out, out_dt, rows, n_rows, H, eps); \
        else                                                                                                    \
            sp_launch_dependent(rmsnorm_warp_kernel<NV, false>, dim3((n_rows + 7) / 8), dim3(256), 0, stream, x, w, w_dt, out, out_dt, rows, n_rows, H, eps); \
        SP_CHECK_LAUNCH("rmsnorm");                                                                             \
        return 0;                                                                                               \
    }
    SP_NORM_WARP(4) SP_NORM_WARP(8) SP_NORM_WARP(16) SP_NORM_WARP(24) SP_NORM_WARP(32)
#undef SP_NORM_WARP
    if ((H & 3) == 0 && H <= 4096 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0)
        SP_CHECK_CALL("rmsnorm", sp_launch_cluster(rmsnorm_row_kernel, dim3(n_rows), dim3(256), 0, stream, 1, x, w, w_dt, out,
                                              out_dt, rows, n_rows, H, eps));
    else
        SP_CHECK_CALL("rmsnorm", sp_launch_cluster(rmsnorm_kernel, dim3(n_rows), dim3(256), 0, stream, 1, x, w, w_dt, out,
                                              out_dt, rows, n_rows, H, eps));
    return 0;
}

// ============================================================== matrix product
// C[M,N] (+)= A[M,K] · W[N,K]ᵀ, FFMA, 64x64 tile, 16-deep slices, 4x4 per thread.
// Each output's sum runs over k = 0..K-1 in order, whatever M is.
#define GG_BM 64
#define GG_BN 64
#define GG_BK 16

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TA* __restrict__ A, const TW* __restrict__ W, void* __restrict__ C, int c_dt,
                    int M, int N, int K, int lda, int ldw, int ldc, int accumulate) {
    __shared__ float As[GG_BK][GG_BM + 4];
    __shared__ float Ws[GG_BK][GG_BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * GG_BM, n0 = blockIdx.x * GG_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread; k runs fastest in memory
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int r = e >> 4, kk = e & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? sp_ld(A, (size_t)gm * lda + gk) : 0.0f;
            Ws[kk][r] = (gn < N && gk < K) ? sp_ld(W, (size_t)gn * ldw + gk) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            const size_t o = (size_t)gm * ldc + gn;
            float v = acc[i][j];
            if (accumulate) v += ((float*)C)[o];
            sp_st_dt(C, c_dt, o, v);
        }
    }
}

// The same product for a few rows of A (a decode step of the 32-bit path): W is streamed once with 16-byte loads,
// a CTA of four warps owns eight rows of W (two per warp), the rows of A pass through shared memory in slices of
// 512 columns. Each lane sums its columns k = 4·lane + 128·i in order, the lanes' sums are added by a shuffle tree:
// the order is fixed and the same for every row of A, whatever M is, but it is another order than the tiled
// kernel's, so a token's result differs between a decode step and a prompt step by 32-bit rounding.
#define GS_KC 512
#define GS_ROWS 2
template <int MT>
__global__ void __launch_bounds__(128)
gemm_stream_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, void* __restrict__ C, int c_dt,
                       int M, int N, int K, int lda, int ldw, int ldc, int accumulate) {
    __shared__ __align__(16) float xs[MT][GS_KC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * 4 + warp) * GS_ROWS;
    float acc[GS_ROWS][MT];
#pragma unroll
    for (int r = 0; r < GS_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;
    const float* wrow[GS_ROWS];
#pragma unroll
    for (int r = 0; r < GS_ROWS; ++r) wrow[r] = W + (size_t)min(n0 + r, N - 1) * ldw;

    for (int k0 = 0; k0 < K; k0 += GS_KC) {
        __syncthreads();                                     // the slice before has been used by every warp
        for (int e = threadIdx.x; e < MT * (GS_KC / 4); e += 128) {
            const int m = e / (GS_KC / 4), c = (e % (GS_KC / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < M && k0 + c < K) v = *(const float4*)(A + (size_t)m * lda + k0 + c);     // K is a multiple of 4
            *(float4*)&xs[m][c] = v;
        }
        __syncthreads();
        float4 w[GS_ROWS][GS_KC / 128];
#pragma unroll
        for (int r = 0; r < GS_ROWS; ++r)
#pragma unroll
            for (int i = 0; i < GS_KC / 128; ++i) {
                const int k = k0 + i * 128 + lane * 4;
                w[r][i] = k < K ? __ldcs((const float4*)(wrow[r] + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
        for (int i = 0; i < GS_KC / 128; ++i)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float4 x = *(const float4*)&xs[m][i * 128 + lane * 4];
#pragma unroll
                for (int r = 0; r < GS_ROWS; ++r) {
                    acc[r][m] = fmaf(w[r][i].x, x.x, acc[r][m]);
                    acc[r][m] = fmaf(w[r][i].y, x.y, acc[r][m]);
                    acc[r][m] = fmaf(w[r][i].z, x.z, acc[r][m]);
                    acc[r][m] = fmaf(w[r][i].w, x.w, acc[r][m]);
                }
            }
    }
#pragma unroll
    for (int r = 0; r < GS_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float v = sp_warp_sum(acc[r][m]);
            if (lane == 0 && m < M && n0 + r < N) {
                const size_t o = (size_t)m * ldc + n0 + r;
                sp_st_dt(C, c_dt, o, accumulate ? v + ((float*)C)[o] : v);
            }
        }
}

SP_API int sp_gemm_generic(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt,
                           int M, int N, int K, int lda, int ldw, int ldc, int accumulate,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) SP_FAIL("gemm: K must be positive, got %d", K);
    if (accumulate && c_dt != SP_DT_F32) SP_FAIL("gemm: accumulation needs a 32-bit output");
    if (M <= 16 && a_dt == SP_DT_F32 && w_dt == SP_DT_F32 && ((K | lda | ldw) & 3) == 0 &&
        ((((uintptr_t)A) | ((uintptr_t)W)) & 15) == 0) {
        const unsigned blocks = (unsigned)((N + 4 * GS_ROWS - 1) / (4 * GS_ROWS));
#define GS_LAUNCH(MT) \
        gemm_stream_f32_kernel<MT><<<blocks, 128, 0, stream>>>((const float*)A, (const float*)W, C, c_dt, M, N, K, lda, ldw, ldc, accumulate)
        if (M <= 1) GS_LAUNCH(1);
        else if (M <= 2) GS_LAUNCH(2);
        else if (M <= 4) GS_LAUNCH(4);
        else if (M <= 8) GS_LAUNCH(8);
        else GS_LAUNCH(16);
#undef GS_LAUNCH
        SP_CHECK_LAUNCH("gemm_stream_f32");
        return 0;
    }
    dim3 grid((N + GG_BN - 1) / GG_BN, (M + GG_BM - 1) / GG_BM);
    if (grid.y > 65535) SP_FAIL("gemm: M=%d is beyond this kernel's grid", M);
#define GG_LAUNCH(TA, TW) \
    gemm_generic_kernel<TA, TW><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, C, c_dt, M, N, K, lda, ldw, ldc, accumulate)
    if (a_dt == SP_DT_F32 && w_dt == SP_DT_F32) GG_LAUNCH(float, float);
    else if (a_dt == SP_DT_F32 && w_dt == SP_DT_BF16) GG_LAUNCH(float, __nv_bfloat16);
    else if (a_dt == SP_DT_BF16 && w_dt == SP_DT_F32) GG_LAUNCH(__nv_bfloat16, float);
    else if (a_dt == SP_DT_BF16 && w_dt == SP_DT_BF16) GG_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else SP_FAIL("gemm: unsupported dtype codes %d/%d", a_dt, w_dt);
#undef GG_LAUNCH
    SP_CHECK_LAUNCH("gemm_generic");
    return 0;
}

#define AG_WARPS 4
#define AG_MAX_HD 256          // largest head size of the generic kernels

// ============================================================== rope + cache write
// qkv row t = [q heads | k heads | v heads]. Rotates q and k (rotate-half over the
// first ``rd`` dims of each head, angle = position · inv_freq[i], all 32-bit), stores
// q to ``q_out`` and k, v to the paged cache at the token's position.
// Cache layout per layer: [page][kv head][page_size][hd].
struct KvPlace {
    const int* token_seq;     // [T] sequence index of each token
    const int* positions;     // [T] absolute position of each token
    const int* seq_slot;      // [B] slot of each sequence
    const int* page_table;    // [slots][max_pages]
    int max_pages;
    int page_size;
    SpRange rg;               // what the debug build checks table entries against
};

// the page that holds position ``pos`` of the sequence of token ``t``; false (debug build) when a table entry is bad
__device__ __forceinline__ bool kv_page_of(const KvPlace& pl, int t, int pos, int& page) {
    const int slot = pl.seq_slot[pl.token_seq[t]];
    if (!sp_index_ok(slot, pl.rg.n_rows, pl.rg, 402) || !sp_index_ok(pos / pl.page_size, pl.max_pages, pl.rg, 403)) return false;
    page = pl.page_table[(size_t)slot * pl.max_pages + pos / pl.page_size];
    return sp_index_ok(page, pl.rg.n_pages, pl.rg, 401);
}

template <typename TIN, typename TQ, typename TC>
__global__ void rope_kv_write_kernel(const TIN* __restrict__ qkv, TQ* __restrict__ q_out,
                                     TC* __restrict__ kpool, TC* __restrict__ vpool, KvPlace pl,
                                     const float* __restrict__ inv_freq, int T, int nh, int nkv, int hd,
                                     int rd, int write_kv) {
    const int t = blockIdx.x;
    if (t >= T) return;
    const int pos = pl.positions[t];
    const int half = rd >> 1;
    const int row = (nh + 2 * nkv) * hd;
    const TIN* src = qkv + (size_t)t * row;
    int page = 0, off = 0;
    if (write_kv) {
        if (!kv_page_of(pl, t, pos, page)) write_kv = 0;          // debug build: a bad entry is reported, nothing is written
        off = pos % pl.page_size;
    }
    const int n_rot_heads = nh + nkv;
    // the token's cosines and sines once, shared by every head
    __shared__ float cs[2][AG_MAX_HD / 2];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[0][i] = cosf(ang);
        cs[1][i] = sinf(ang);
    }
    __syncthreads();
    const size_t qrow = (size_t)t * nh * hd;
    if ((half & 1) == 0 && (hd & 1) == 0) {
        // two neighbouring pairs per thread: 8-byte reads, one rounding and one store per two outputs
        const int hp = half >> 1;                            // pairs of pairs per head
        for (int e = threadIdx.x; e < n_rot_heads * hp; e += blockDim.x) {
            const int h = e / hp, i = (e % hp) * 2;
            const float a0 = sp_ld(src, (size_t)h * hd + i), a1 = sp_ld(src, (size_t)h * hd + i + 1);
            const float b0 = sp_ld(src, (size_t)h * hd + half + i), b1 = sp_ld(src, (size_t)h * hd + half + i + 1);
            const float c0 = cs[0][i], s0 = cs[1][i], c1 = cs[0][i + 1], s1 = cs[1][i + 1];
            const float lo0 = a0 * c0 - b0 * s0, lo1 = a1 * c1 - b1 * s1;
            const float hi0 = b0 * c0 + a0 * s0, hi1 = b1 * c1 + a1 * s1;
            if (h < nh) {
                sp_st2(q_out, qrow + (size_t)h * hd + i, lo0, lo1);
                sp_st2(q_out, qrow + (size_t)h * hd + half + i, hi0, hi1);
            } else if (write_kv) {
                const size_t kb = (((size_t)page * nkv + (h - nh)) * pl.page_size + off) * hd;
                sp_st2(kpool, kb + i, lo0, lo1);
                sp_st2(kpool, kb + half + i, hi0, hi1);
            }
        }
        // dims beyond the rotated ones pass through
        const int tail = hd - rd;
        for (int e = threadIdx.x; e < n_rot_heads * tail; e += blockDim.x) {
            const int h = e / tail, d = rd + e % tail;
            const float v = sp_ld(src, (size_t)h * hd + d);
            if (h < nh) sp_st(q_out, qrow + (size_t)h * hd + d, v);
            else if (write_kv) sp_st(kpool, (((size_t)page * nkv + (h - nh)) * pl.page_size + off) * hd + d, v);
        }
        if (write_kv) {
            for (int e = threadIdx.x; e < nkv * (hd >> 1); e += blockDim.x) {
                const int g = e / (hd >> 1), d = (e % (hd >> 1)) * 2;
                const float v0 = sp_ld(src, (size_t)(nh + nkv) * hd + (size_t)g * hd + d);
                const float v1 = sp_ld(src, (size_t)(nh + nkv) * hd + (size_t)g * hd + d + 1);
                sp_st2(vpool, (((size_t)page * nkv + g) * pl.page_size + off) * hd + d, v0, v1);
            }
        }
        return;
    }
    for (int e = threadIdx.x; e < n_rot_heads * hd; e += blockDim.x) {
        const int h = e / hd, d = e % hd;
        float v;
        if (d < rd) {
            const int i = d < half ? d : d - half;
            const float c = cs[0][i], s = cs[1][i];
            const float a = sp_ld(src, (size_t)h * hd + i);
            const float b = sp_ld(src, (size_t)h * hd + i + half);
            v = d < half ? a * c - b * s : b * c + a * s;
        } else {
            v = sp_ld(src, (size_t)h * hd + d);
        }
        if (h < nh) {
            sp_st(q_out, qrow + (size_t)h * hd + d, v);
        } else if (write_kv) {
            const int g = h - nh;
            sp_st(kpool, (((size_t)page * nkv + g) * pl.page_size + off) * hd + d, v);
        }
    }
    if (write_kv) {
        for (int e = threadIdx.x; e < nkv * hd; e += blockDim.x) {
            const int g = e / hd, d = e % hd;
            const float v = sp_ld(src, (size_t)(nh + nkv) * hd + e);
            sp_st(vpool, (((size_t)page * nkv + g) * pl.page_size + off) * hd + d, v);
        }
    }
}

// The common case in one pass of 16-byte reads: float32 products in, bfloat16 q and cache out, the whole head
// rotated (rd == hd), hd a multiple of 8. One block of 128 threads per token; a thread takes four neighbouring
// pairs (a[i..i+3], b[i..i+3]) of one head, or four values of v.
__global__ void __launch_bounds__(128)
rope_kv_write_bf16_kernel(const float* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                          __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool, KvPlace pl,
                          const float* __restrict__ inv_freq, int T, int nh, int nkv, int hd, int write_kv) {
    sp_allow_dependents();
    sp_wait_for_predecessor();
    const int t = blockIdx.x;
    if (t >= T) return;
    const int pos = pl.positions[t];
    const int half = hd >> 1;
    const float* src = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    int page = 0, off = 0;
    if (write_kv) {
        if (!kv_page_of(pl, t, pos, page)) write_kv = 0;          // debug build: a bad entry is reported, nothing is written
        off = pos % pl.page_size;
    }
    __shared__ float cs[2][AG_MAX_HD / 2];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[0][i] = cosf(ang);
        cs[1][i] = sinf(ang);
    }
    __syncthreads();
    auto pack4 = [](float a, float b, float c, float d) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a, b), p1 = __floats2bfloat162_rn(c, d);
        uint2 pk;
        pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
        return pk;
    };
    const int per_head = half >> 2;                          // groups of four pairs
    const int n_rot = (nh + (write_kv ? nkv : 0)) * per_head;
    for (int e = threadIdx.x; e < n_rot; e += blockDim.x) {
        const int h = e / per_head, i = (e - h * per_head) * 4;
        const float4 a = *(const float4*)(src + (size_t)h * hd + i);
        const float4 b = *(const float4*)(src + (size_t)h * hd + half + i);
        const float4 c = *(const float4*)&cs[0][i], sn = *(const float4*)&cs[1][i];
        const uint2 lo = pack4(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w);
        const uint2 hi = pack4(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y, b.z * c.z + a.z * sn.z, b.w * c.w + a.w * sn.w);
        __nv_bfloat16* dst = h < nh ? q_out + (size_t)t * nh * hd + (size_t)h * hd
                                    : kpool + (((size_t)page * nkv + (h - nh)) * pl.page_size + off) * hd;
        *(uint2*)(dst + i) = lo;
        *(uint2*)(dst + half + i) = hi;
    }
    if (write_kv) {
        const int per_v = hd >> 2;
        for (int e = threadIdx.x; e < nkv * per_v; e += blockDim.x) {
            const int g = e / per_v, d = (e - g * per_v) * 4;
            const float4 v = *(const float4*)(src + (size_t)(nh + nkv) * hd + (size_t)g * hd + d);
            *(uint2*)(vpool + (((size_t)page * nkv + g) * pl.page_size + off) * hd + d) = pack4(v.x, v.y, v.z, v.w);
        }
    }
}

SP_API int sp_rope_kv_write(const void* qkv, int in_dt, void* q_out, int q_dt, void* kpool, void* vpool,
                            int cache_dt, const int* token_seq, const int* positions, const int* seq_slot,
                            const int* page_table, int max_pages, int page_size, const float* inv_freq,
                            int T, int nh, int nkv, int hd, int rd, int write_kv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rd < 0 || rd > hd || (rd & 1)) SP_FAIL("rope: rotary_dim %d must be even and at most head_dim %d", rd, hd);
    if (rd > AG_MAX_HD) SP_FAIL("rope: rotary_dim %d is beyond this kernel's limit %d", rd, AG_MAX_HD);
    if (rd > 0 && !inv_freq) SP_FAIL("rope: a frequency table is needed when rotary_dim > 0");
    KvPlace pl{token_seq, positions, seq_slot, page_table, max_pages, page_size, sp_range_host};
    if (in_dt == SP_DT_F32 && q_dt == SP_DT_BF16 && cache_dt == SP_DT_BF16 && rd == hd && (hd % 8) == 0 &&
        ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)kpool | (uintptr_t)vpool) & 15) == 0)) {
        sp_launch_dependent(rope_kv_write_bf16_kernel, dim3(T), dim3(128), 0, stream, (const float*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kpool,
                                                         (__nv_bfloat16*)vpool, pl, inv_freq, T, nh, nkv, hd, write_kv);
        SP_CHECK_LAUNCH("rope_kv_write");
        return 0;
    }
    const int threads = 256;
#define RK_LAUNCH(TIN, TQ, TC)                                                                                  \
    SP_CHECK_CALL("rope_kv_write", sp_launch_cluster(rope_kv_write_kernel<TIN, TQ, TC>, dim3(T), dim3(threads), 0, stream, 1, \
                                                (const TIN*)qkv, (TQ*)q_out, (TC*)kpool, (TC*)vpool, pl, inv_freq, T, nh, \
                                                nkv, hd, rd, write_kv))
    const int key = in_dt * 4 + q_dt * 2 + cache_dt;
    switch (key) {
        case 0: RK_LAUNCH(float, float, float); break;
        case 1: RK_LAUNCH(float, float, __nv_bfloat16); break;
        case 2: RK_LAUNCH(float, __nv_bfloat16, float); break;
        case 3: RK_LAUNCH(float, __nv_bfloat16, __nv_bfloat16); break;
        case 4: RK_LAUNCH(__nv_bfloat16, float, float); break;
        case 5: RK_LAUNCH(__nv_bfloat16, float, __nv_bfloat16); break;
        case 6: RK_LAUNCH(__nv_bfloat16, __nv_bfloat16, float); break;
        case 7: RK_LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
        default: SP_FAIL("rope: unsupported dtype codes");
    }
#undef RK_LAUNCH
    return 0;
}

// ============================================================== attention over the cache
// One warp per (token, query head). Keys are visited in chunks of 32 from the first
// visible position; lane j scores key j, the softmax runs online in 32-bit, and lane d
// owns output dims d, d+32, ... . A token at position p sees keys lo..p with
// lo = max(0, p-window+1) when window > 0, else 0. All keys, this step's included,
// are read from the cache.

// q · k over hd dims for one key row; 16-byte loads where the row allows them
__device__ __forceinline__ float ag_dot(const float* __restrict__ qv, const float* __restrict__ kr, int hd) {
    float dot = 0.0f;
    if ((hd & 3) == 0 && (((uintptr_t)kr) & 15) == 0) {
        int d = 0;
        for (; d + 16 <= hd; d += 16) {                      // four loads in flight, then their products in order
            float4 k4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) k4[u] = *(const float4*)(kr + d + 4 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 q4 = *(const float4*)(qv + d + 4 * u);
                dot = fmaf(q4.x, k4[u].x, dot); dot = fmaf(q4.y, k4[u].y, dot);
                dot = fmaf(q4.z, k4[u].z, dot); dot = fmaf(q4.w, k4[u].w, dot);
            }
        }
        for (; d < hd; d += 4) {
            const float4 k4 = *(const float4*)(kr + d);
            const float4 q4 = *(const float4*)(qv + d);
            dot = fmaf(q4.x, k4.x, dot); dot = fmaf(q4.y, k4.y, dot);
            dot = fmaf(q4.z, k4.z, dot); dot = fmaf(q4.w, k4.w, dot);
        }
    } else {
        for (int d = 0; d < hd; ++d) dot = fmaf(qv[d], kr[d], dot);
    }
    return dot;
}
__device__ __forceinline__ float ag_dot(const float* __restrict__ qv, const __nv_bfloat16* __restrict__ kr, int hd) {
    float dot = 0.0f;
    for (int d = 0; d < hd; ++d) dot = fmaf(qv[d], __bfloat162float(kr[d]), dot);
    return dot;
}

// SPLIT: the CTA's warps share ONE (token, head) and take the chunks of 32 keys in turn (few pairs, many keys: a
// decode step); their partial results are merged in warp order through shared memory.
template <typename TQ, typename TC, bool SPLIT>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const TQ* __restrict__ q, const TC* __restrict__ kpool, const TC* __restrict__ vpool,
                         TQ* __restrict__ out, KvPlace pl, int T, int nh, int nkv, int hd, int window,
                         float scale) {
    __shared__ __align__(16) float qs[AG_WARPS][AG_MAX_HD];
    __shared__ float part_ml[AG_WARPS][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = SPLIT ? (long long)blockIdx.x : (long long)blockIdx.x * AG_WARPS + warp;
    if (gw >= (long long)T * nh) return;
    const int t = (int)(gw / nh), h = (int)(gw % nh);
    const int g = h / (nh / nkv);
    const int p = pl.positions[t];
    const int slot = sp_checked_row(pl.seq_slot[pl.token_seq[t]], pl.rg);
    const int* pt = pl.page_table + (size_t)slot * pl.max_pages;
    const int ps = pl.page_size;

    for (int d = lane; d < hd; d += 32) qs[warp][d] = sp_ld(q, (size_t)t * nh * hd + (size_t)h * hd + d);
    __syncwarp();

    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[AG_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] = 0.0f;

    for (int j0 = lo + (SPLIT ? 32 * warp : 0); j0 <= p; j0 += SPLIT ? 32 * AG_WARPS : 32) {
        const int j = j0 + lane;
        const bool valid = j <= p;
        float s = -INFINITY;
        int my_page = 0, my_off = 0;
        if (valid) {
            my_page = sp_checked_page(pt[sp_checked_entry(j / ps, pl.max_pages, pl.rg)], pl.rg);
            my_off = j % ps;
            const TC* kr = kpool + (((size_t)my_page * nkv + g) * ps + my_off) * hd;
            s = ag_dot(qs[warp], kr, hd) * scale;
        }
        const float m_new = fmaxf(m, sp_warp_max(s));
        const float e = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);              // first chunk: exp(-inf) = 0
        l = l * corr + sp_warp_sum(e);
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] *= corr;
        const int n_valid = min(32, p - j0 + 1);
        // eight keys at a time: their value rows are asked for together, then added in key order
        for (int jj0 = 0; jj0 < n_valid; jj0 += 8) {
            float pj[8];
            const TC* vr[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                pj[u] = __shfl_sync(0xffffffffu, e, jj0 + u);
                const int pg = __shfl_sync(0xffffffffu, my_page, jj0 + u);
                const int of = __shfl_sync(0xffffffffu, my_off, jj0 + u);
                vr[u] = vpool + (((size_t)pg * nkv + g) * ps + of) * hd;
            }
#pragma unroll
            for (int i = 0; i < AG_MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) {
                    float v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = jj0 + u < n_valid ? sp_ld(vr[u], d) : 0.0f;
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc[i] = fmaf(pj[u], v[u], acc[i]);
                }
            }
        }
        m = m_new;
    }
    if (SPLIT) {
        // every warp leaves (m, l, acc) in shared memory (its query row is no longer needed); warp 0 merges in warp order
        __syncwarp();
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) qs[warp][d] = acc[i];
        }
        if (lane == 0) { part_ml[warp][0] = m; part_ml[warp][1] = l; }
        __syncthreads();
        if (warp != 0) return;
        float mm = -INFINITY;
        for (int w = 0; w < AG_WARPS; ++w) mm = fmaxf(mm, part_ml[w][0]);
        float ll = 0.0f;
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] = 0.0f;
        for (int w = 0; w < AG_WARPS; ++w) {
            if (part_ml[w][1] <= 0.0f) continue;                 // a warp that saw no key
            const float f = expf(part_ml[w][0] - mm);
            ll += part_ml[w][1] * f;
#pragma unroll
            for (int i = 0; i < AG_MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(qs[w][d], f, acc[i]);
            }
        }
        l = ll;
    }
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) sp_st(out, (size_t)t * nh * hd + (size_t)h * hd + d, acc[i] / l);
    }
}

SP_API int sp_attention_generic(const void* q, int q_dt, const void* kpool, const void* vpool, int cache_dt,
                                void* out, const int* token_seq, const int* positions, const int* seq_slot,
                                const int* page_table, int max_pages, int page_size, int T, int nh, int nkv,
                                int hd, int window, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > AG_MAX_HD) SP_FAIL("attention: head_dim %d is beyond this kernel's limit %d", hd, AG_MAX_HD);
    if (nkv <= 0 || nh % nkv) SP_FAIL("attention: %d heads are no multiple of %d kv heads", nh, nkv);
    KvPlace pl{token_seq, positions, seq_slot, page_table, max_pages, page_size, sp_range_host};
    const long long warps = (long long)T * nh;
    // few (token, head) pairs (a decode step): a CTA per pair, its warps share the keys
    const bool split = warps <= 4096;
    const long long blocks = split ? warps : (warps + AG_WARPS - 1) / AG_WARPS;
    if (blocks > 2147483647LL) SP_FAIL("attention: too many (token, head) pairs for one launch");
#define AG_LAUNCH(TQ, TC)                                                                                              \
    do {                                                                                                               \
        if (split)                                                                                                     \
            attention_generic_kernel<TQ, TC, true><<<(unsigned)blocks, AG_WARPS * 32, 0, stream>>>((const TQ*)q, (const TC*)kpool, (const TC*)vpool, (TQ*)out, pl, T, nh, nkv, hd, window, scale); \
        else                                                                                                           \
            attention_generic_kernel<TQ, TC, false><<<(unsigned)blocks, AG_WARPS * 32, 0, stream>>>((const TQ*)q, (const TC*)kpool, (const TC*)vpool, (TQ*)out, pl, T, nh, nkv, hd, window, scale); \
    } while (0)
    if (q_dt == SP_DT_F32 && cache_dt == SP_DT_F32) AG_LAUNCH(float, float);
    else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_BF16) AG_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dt == SP_DT_F32 && cache_dt == SP_DT_BF16) AG_LAUNCH(float, __nv_bfloat16);
    else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_F32) AG_LAUNCH(__nv_bfloat16, float);
    else SP_FAIL("attention: unsupported dtype codes %d/%d", q_dt, cache_dt);
#undef AG_LAUNCH
    SP_CHECK_LAUNCH("attention_generic");
    return 0;
}

// ============================================================== silu(gate) * up
// gu row = [gate(0..I) | up(0..I)]; out row = silu(gate) ⊙ up, silu(z) = z / (1 + e^-z).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t rows, int I) {
    const size_t n = rows * (size_t)I;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / I;
        const int c = (int)(e % I);
        const float g = sp_ld(gu, r * 2 * I + c);
        const float u = sp_ld(gu, r * 2 * I + I + c);
        sp_st(out, e, (g / (1.0f + expf(-g))) * u);
    }
}

SP_API int sp_silu_mul(const void* gu, void* out, int dt, int rows, int I, cudaStream_t stream) {
    if (rows <= 0 || I <= 0) return 0;
    const size_t n = (size_t)rows * I;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    if (dt == SP_DT_F32) silu_mul_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, rows, I);
    else if (dt == SP_DT_BF16) silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, I);
    else SP_FAIL("silu_mul: unsupported dtype code %d", dt);
    SP_CHECK_LAUNCH("silu_mul");
    return 0;
}

// ============================================================== residual add
__global__ void add_inplace_kernel(float* __restrict__ dst, const void* __restrict__ src, int src_dt, size_t n) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x)
        dst[e] += sp_ld_dt(src, src_dt, e);
}

SP_API int sp_add_inplace(float* dst, const void* src, int src_dt, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    add_inplace_kernel<<<blocks, 256, 0, stream>>>(dst, src, src_dt, (size_t)n);
    SP_CHECK_LAUNCH("add_inplace");
    return 0;
}

// ============================================================== gather of int32
// dst[i] = src[idx[i]]: the tokens a step takes from the sampler's output of the step before, on the device
__global__ void gather_i32_kernel(const int* __restrict__ src, const int* __restrict__ idx, int* __restrict__ dst, int n,
                                  int n_src) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int j = idx[i];
    dst[i] = (j >= 0 && j < n_src) ? src[j] : 0;
}

SP_API int sp_gather_i32(const int* src, const int* idx, int* dst, int n, int n_src, cudaStream_t stream) {
    if (n <= 0) return 0;
    gather_i32_kernel<<<(n + 127) / 128, 128, 0, stream>>>(src, idx, dst, n, n_src);
    SP_CHECK_LAUNCH("gather_i32");
    return 0;
}

// ============================================================== argmax
// The lowest index among equal maxima wins, as a serial scan with a strict ``>`` would choose. NaNs never
// win. A row is cut over the CTAs of a thread-block cluster (one CTA for short rows); rank 0 takes the best
// of the CTAs' finds through distributed shared memory.
constexpr int ARGMAX_CLUSTER = 8;

__device__ __forceinline__ void argmax_take(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

template <int CLUSTER>
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, int ld) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float cta_v;
    __shared__ int cta_i;
    unsigned rank = 0;
    if (CLUSTER > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int row_id = blockIdx.x / CLUSTER;
    const float* row = logits + (size_t)row_id * ld;
    const int per = (V + CLUSTER - 1) / CLUSTER;
    const int i0 = min(V, (int)rank * per), i1 = min(V, i0 + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = i0 + threadIdx.x; c < i1; c += blockDim.x) argmax_take(bv, bi, row[c], c);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_take(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            argmax_take(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) { cta_v = bv; cta_i = bi; }
    }
    if (CLUSTER == 1) {
        if (threadIdx.x == 0) out[row_id] = (bi == 0x7fffffff) ? 0 : bi;
        return;
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank == 0 && threadIdx.x == 0) {
        bv = -INFINITY;
        bi = 0x7fffffff;
        for (unsigned r = 0; r < (unsigned)CLUSTER; ++r) {
            unsigned av, ai;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(av) : "r"((unsigned)__cvta_generic_to_shared(&cta_v)), "r"(r));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ai) : "r"((unsigned)__cvta_generic_to_shared(&cta_i)), "r"(r));
            float ov;
            int oi;
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ov) : "r"(av) : "memory");
            asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(oi) : "r"(ai) : "memory");
            argmax_take(bv, bi, ov, oi);
        }
        out[row_id] = (bi == 0x7fffffff) ? 0 : bi;
    }
    // no CTA leaves while rank 0 may still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

SP_API int sp_argmax_rows(const float* logits, int* out, int rows, int V, int ld, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0) SP_FAIL("argmax: empty rows");
    if (V >= 16384)
        SP_CHECK_CALL("argmax_rows", sp_launch_cluster(argmax_rows_kernel<ARGMAX_CLUSTER>, dim3(rows * ARGMAX_CLUSTER), dim3(1024), 0,
                                                  stream, ARGMAX_CLUSTER, logits, out, V, ld));
    else
        SP_CHECK_CALL("argmax_rows", sp_launch_cluster(argmax_rows_kernel<1>, dim3(rows), dim3(V >= 4096 ? 1024 : 256), 0, stream, 1,
                                                  logits, out, V, ld));
    return 0;
}


// ============================================================== per-step tables for fused prompt kernels
// Once per step and cache group, for every token of the step: the cosines and sines of its rotation angles
// (angle = position · inv_freq[i], float32, accurate cosf / sinf: crates/spissa-runtime/src/rotary.rs:454-465) and the
// cache page that holds its position. Every layer's QKV product reads them in its epilogue.
__global__ void rope_table_kernel(const int* __restrict__ positions, const int* __restrict__ token_seq,
                                  const int* __restrict__ seq_row, const int* __restrict__ page_table, int max_pages,
                                  int page_size, const float* __restrict__ inv_freq, int half, int T,
                                  float2* __restrict__ cs, int* __restrict__ tok_page, SpRange rg) {
    const int t = blockIdx.x;
    if (t >= T) return;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[(size_t)t * half + i] = make_float2(cosf(ang), sinf(ang));
    }
    if (threadIdx.x == 0 && tok_page) {
        const int row = sp_checked_row(seq_row[token_seq[t]], rg);
        // a bad page is kept as it is: the kernels that use it check it again before they write
        tok_page[t] = page_table[(size_t)row * max_pages + sp_checked_entry(pos / page_size, max_pages, rg)];
    }
}

SP_API int sp_rope_table(const int* positions, const int* token_seq, const int* seq_row, const int* page_table,
                         int max_pages, int page_size, const float* inv_freq, int half, int T, void* cs, int* tok_page,
                         cudaStream_t stream) {
    if (T <= 0) return 0;
    if (half <= 0 || !inv_freq) SP_FAIL("rope_table: a frequency table of at least one entry is needed");
    if (tok_page && (!page_table || page_size <= 0)) SP_FAIL("rope_table: the tokens' pages need the page table");
    rope_table_kernel<<<T, half >= 64 ? 64 : 32, 0, stream>>>(positions, token_seq, seq_row, page_table, max_pages, page_size,
                                                            inv_freq, half, T, (float2*)cs, tok_page, sp_range_host);
    SP_CHECK_LAUNCH("rope_table");
    return 0;
}

// The first norm of a fused prompt step: xw = x ⊙ w (bfloat16, the next product's input) and the rows' sums of
// squares; the product multiplies its result by 1/rms (crates/spissa-runtime/src/ops.rs:159-179 is the norm).
__global__ void norm_prepare_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                    __nv_bfloat16* __restrict__ xw, float* __restrict__ ssq, int T, int H) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= T) return;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = x[(size_t)r * H + c];
        ss = fmaf(v, v, ss);
        xw[(size_t)r * H + c] = __float2bfloat16_rn(v * __bfloat162float(w[c]));
    }
    ss = sp_block_sum(ss, scratch);
    if (threadIdx.x == 0) ssq[r] = ss;
}

SP_API int sp_norm_prepare(const float* x, const void* w, void* xw, float* ssq, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    norm_prepare_kernel<<<T, 256, 0, stream>>>(x, (const __nv_bfloat16*)w, (__nv_bfloat16*)xw, ssq, T, H);
    SP_CHECK_LAUNCH("norm_prepare");
    return 0;
}

// ============================================================== the best of a row of candidates
// Second stage of the greedy head: the head's product kept, per token, one (value, row) candidate for each of its
// tiles (``cand`` [rows][ld] pairs of float, int32; a tile without a winner has row 0x7fffffff). One CTA per token
// takes the best of them: the largest value, the lowest row among equal values, as a serial scan of the logits with
// a strict ``>`` would (crates/spissa-runtime/src/ops.rs:309-324). With ``header`` the token is also noted in the
// header of the token's sequence (see header_note below), so that a greedy step needs no kernel after this one.
struct Candidate { float value; int index; };

__global__ void argmax_candidates_kernel(const Candidate* __restrict__ cand, int n_cand, int ld, int* __restrict__ out,
                                         int* __restrict__ header, int n_slots, const int* __restrict__ seq_slot,
                                         const int* __restrict__ seq_len) {
    __shared__ float sv[32];
    __shared__ int si[32];
    sp_allow_dependents();
    sp_wait_for_predecessor();                                     // the candidates are the head kernel's
    const int r = blockIdx.x;
    const Candidate* row = cand + (size_t)r * ld;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < n_cand; c += blockDim.x) {
        const Candidate k = row[c];
        if (k.index != 0x7fffffff) argmax_take(bv, bi, k.value, k.index);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_take(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            argmax_take(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) {
            const int tok = (bi == 0x7fffffff) ? 0 : bi;
            out[r] = tok;
            if (header) {
                const int slot = seq_slot[r];
                if (slot >= 0 && slot < n_slots) {
                    int* h = header + (size_t)slot * 4;
                    h[0] = seq_len[r];
                    h[1] += 1;
                    h[2] = tok;
                }
            }
        }
    }
}

SP_API int sp_argmax_candidates(const void* cand, int rows, int n_cand, int ld, int* out, int* header, int n_slots,
                                const int* seq_slot, const int* seq_len, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n_cand <= 0 || ld < n_cand) SP_FAIL("argmax_candidates: %d candidates in rows of %d", n_cand, ld);
    if (header && (!seq_slot || !seq_len)) SP_FAIL("argmax_candidates: noting tokens needs the step's slots and lengths");
    sp_launch_dependent(argmax_candidates_kernel, dim3(rows), dim3(n_cand >= 4096 ? 1024 : 256), 0, stream, (const Candidate*)cand,
                        n_cand, ld, out, header, n_slots, seq_slot, seq_len);
    SP_CHECK_LAUNCH("argmax_candidates");
    return 0;
}

// ============================================================== the per-slot header
// header [slots, 4] int32: position (tokens cached), draws (tokens sampled so far), last sampled token, spare.
// After a step's logits were turned into tokens: sequence b of the step sits in slot seq_slot[b] and is
// seq_len[b] tokens long now. A slot outside the header is skipped.
__global__ void header_note_kernel(int* __restrict__ header, int n_slots, const int* __restrict__ seq_slot,
                                   const int* __restrict__ seq_len, const int* __restrict__ tokens, int n) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n) return;
    const int slot = seq_slot[b];
    if (slot < 0 || slot >= n_slots) return;
    int* h = header + (size_t)slot * 4;
    h[0] = seq_len[b];
    h[1] += 1;
    h[2] = tokens[b];
}

SP_API int sp_header_note(int* header, int n_slots, const int* seq_slot, const int* seq_len, const int* tokens, int n,
                          cudaStream_t stream) {
    if (n <= 0) return 0;
    header_note_kernel<<<(n + 127) / 128, 128, 0, stream>>>(header, n_slots, seq_slot, seq_len, tokens, n);
    SP_CHECK_LAUNCH("header_note");
    return 0;
}

// ============================================================== a wait that runs out (for tests of the fault path)
// One thread waits on a shared-memory barrier on which nobody ever arrives, with the same bounded wait that the
// tensor-core kernels use but a limit the caller gives (at most 10 ms). When the limit is reached the wait gives
// up, records ``code`` in ``status`` and the kernel returns: the way every kernel of this library ends a wait that
// does not complete. Nothing faults, traps or spins beyond the limit.
__global__ void wait_runs_out_kernel(int* status, int code, unsigned long long limit_ns, unsigned long long* waited_ns) {
    __shared__ __align__(8) uint64_t bar;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const unsigned long long t0 = global_ns();
    bool done = false;
    while (!(done = mbar_try_wait(smem_u32(&bar), 0))) {
        if (global_ns() - t0 > limit_ns) {
            if (status) atomicCAS(status, 0, code);
            break;
        }
    }
    if (waited_ns) *waited_ns = done ? 0ull : global_ns() - t0;
}

SP_API int sp_wait_runs_out(int* status, int code, long long limit_us, unsigned long long* waited_ns, cudaStream_t stream) {
    if (limit_us < 1 || limit_us > 10000) SP_FAIL("wait_runs_out: the limit is 1 to 10000 microseconds, got %lld", limit_us);
    if (code <= 0) SP_FAIL("wait_runs_out: the code to record must be positive");
    wait_runs_out_kernel<<<1, 1, 0, stream>>>(status, code, (unsigned long long)limit_us * 1000ull, waited_ns);
    SP_CHECK_LAUNCH("wait_runs_out");
    return 0;
}
