// Skinny bfloat16 products for decoding: out[M,N] = x[M,K] · W[N,K]ᵀ with M ≤ 64 tokens.
//
// The step is bound by streaming W from HBM once (the reference's batch-1 path streams rows
// the same way, crates/spissa-runtime/src/streaming/kernels_raw16.rs:532-692, and fuses
// silu(gate)·up at batch 1, crates/spissa-runtime/src/streaming/linear_multiply.rs:376-497).
//
// A CTA owns RT groups of 8 rows of W and one slice of K; the CTAs of a thread-block cluster
// (1, 2, 4 or 8) own the slices of the same rows, and the warps of a CTA split its slice again.
// Per 32 columns of K each lane loads 16 contiguous bytes of "its" row of every row group straight
// from global memory, and 16 bytes of x per 8-token group (x is small and stays in L1/L2); both
// feed mma.sync m16n8k16 with the tokens as the 16 rows of A and 8 rows of W as the columns of B.
// The K positions inside a 32-block are permuted the same way for both operands, which leaves the
// sum unchanged. Partial sums are added in warp order in shared memory, then in cluster-rank order
// by rank 0, which reads its peers' shared memory; the result does not depend on timing or on M.
// Epilogues: store, add into a float32 tensor, or silu(gate)·up when the weight interleaves gate
// and up rows in blocks of ``pair``.
#include "common.cuh"

SP_API const char* sp_gemv_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(gemv)

namespace {

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SILU_MUL = 2, MODE_ROPE_KV = 3, MODE_ARGMAX = 4 };

// MODE_ARGMAX keeps, per token, only the best (value, row) of the rows a warp owns, as the reference's greedy head
// does while it streams the rows (crates/spissa-runtime/src/streaming/linear_argmax.rs:13,
// crates/spissa-runtime/src/streaming/argmax.rs:30-51, :85-97: a strict ``>`` so that the lowest row wins among equal
// values). ``out`` is then a table of candidates [token][warp tile]; a second, tiny kernel takes the best of a row.
struct Candidate { float value; int index; };
__device__ __forceinline__ void take_better(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }       // a NaN never wins
}
constexpr int MAX_KS = 8;

// Where MODE_ROPE_KV sends its rows: W is [q heads | k heads | v heads] x head_dim rows; q and k are
// rotated (rotate-half over the whole head, angle = position · inv_freq[i], float32), q goes to q_out,
// k and v into the paged cache at the token's position ([page][kv head][page_size][head_dim]).
struct RopeOut {
    __nv_bfloat16* q_out;    // [M, nh * hd]
    __nv_bfloat16* kpool;
    __nv_bfloat16* vpool;
    const int* positions;    // [M]
    const int* token_seq;    // [M]
    const int* seq_row;      // [sequences] row of the page table
    const int* page_table;
    const float* inv_freq;   // [hd / 2]
    int max_pages, page_size, nh, nkv, hd;
    SpRange rg;              // what the debug build checks table entries against
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {          // weights: read once, do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_act(const void* p) {             // activations: reused by every CTA, keep in L1
    uint4 v;
    asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_peer_f4(const void* local, uint32_t rank) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(local);
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra) : "memory");
    return v;
}

// MT: groups of 16 tokens; RT: groups of 8 rows of W per CTA; UNROLL: 32-column blocks requested at once.
// MODE_SILU_MUL: the first RT/2 row groups are gate rows, the others the up rows ``pair`` rows further on.
template <int MT, int RT, int UNROLL>
__global__ void __launch_bounds__(MAX_KS * 32)
gemv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, void* __restrict__ out,
            int out_dt, int M, int N, int K, int ldx, int ldw, int ldo, int mode, int pair, int ks, int cs,
            RopeOut rope) {
    __shared__ __align__(16) float red[MAX_KS][MT][RT][32][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rank = cs > 1 ? (int)cluster_rank() : 0;
    const int tile = blockIdx.x / cs;

    // rows of W this CTA owns
    int row_base[RT];
    if (mode == MODE_SILU_MUL || mode == MODE_ROPE_KV) {
        constexpr int HALF = RT / 2 > 0 ? RT / 2 : 1;
        const int o0 = tile * 8 * HALF;                   // first output of this CTA
#pragma unroll
        for (int r = 0; r < HALF; ++r) {
            const int o = o0 + r * 8;
            row_base[r] = (o / pair) * 2 * pair + (o % pair);
            row_base[HALF + r < RT ? HALF + r : r] = row_base[r] + pair;
        }
    } else {
#pragma unroll
        for (int r = 0; r < RT; ++r) row_base[r] = (tile * RT + r) * 8;
    }

    // this warp's slice of K, in blocks of 32 columns: first by cluster rank, then by warp
    const int kblocks = (K + 31) / 32;
    const int per_cta = (kblocks + cs - 1) / cs;
    const int cta0 = rank * per_cta, cta1 = min(kblocks, cta0 + per_cta);
    const int per = (per_cta + ks - 1) / ks;
    const int kb0 = min(cta1, cta0 + warp * per), kb1 = min(cta1, kb0 + per);

    float acc[MT][RT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int r = 0; r < RT; ++r) acc[i][r][0] = acc[i][r][1] = acc[i][r][2] = acc[i][r][3] = 0.0f;

    const __nv_bfloat16* wrow[RT];
    bool wok[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const int row = row_base[r] + g;
        wok[r] = row < N;
        wrow[r] = W + (size_t)(wok[r] ? row : 0) * ldw;
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);

    for (int kb = kb0; kb < kb1; kb += UNROLL) {
        uint4 wv[UNROLL][RT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (kb + u) * 32 + 8 * t;
            const bool kok = (kb + u) < kb1 && k < K;                 // K is a multiple of 8: whole 16 bytes or none
#pragma unroll
            for (int r = 0; r < RT; ++r) wv[u][r] = (kok && wok[r]) ? ld_stream(wrow[r] + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (kb + u) * 32 + 8 * t;
            const bool kok = (kb + u) < kb1 && k < K;
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int m0 = i * 16 + g, m1 = m0 + 8;
                const uint4 xa = (kok && m0 < M) ? ld_act(x + (size_t)m0 * ldx + k) : zero;
                const uint4 xb = (kok && m1 < M) ? ld_act(x + (size_t)m1 * ldx + k) : zero;
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    mma_bf16(acc[i][r], xa.x, xb.x, xa.y, xb.y, wv[u][r].x, wv[u][r].y);
                    mma_bf16(acc[i][r], xa.z, xb.z, xa.w, xb.w, wv[u][r].z, wv[u][r].w);
                }
            }
        }
    }

    // add the K slices of the warps in warp order ...
    if (ks > 1 || cs > 1) {
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int r = 0; r < RT; ++r)
                *(float4*)red[warp][i][r][lane] = make_float4(acc[i][r][0], acc[i][r][1], acc[i][r][2], acc[i][r][3]);
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    float4 s = *(float4*)red[0][i][r][lane];
                    for (int w = 1; w < ks; ++w) {
                        const float4 v = *(float4*)red[w][i][r][lane];
                        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
                    }
                    acc[i][r][0] = s.x; acc[i][r][1] = s.y; acc[i][r][2] = s.z; acc[i][r][3] = s.w;
                    if (cs > 1) *(float4*)red[0][i][r][lane] = s;      // where the cluster's rank 0 looks
                }
        }
    }
    // ... then the K slices of the cluster in rank order
    if (cs > 1) {
        cluster_sync();                                    // every CTA's sum stands in its red[0]
        if (rank == 0 && warp == 0) {
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int r = 0; r < RT; ++r)
                    for (int c = 1; c < cs; ++c) {
                        const float4 v = ld_peer_f4(red[0][i][r][lane], (uint32_t)c);
                        acc[i][r][0] += v.x; acc[i][r][1] += v.y; acc[i][r][2] += v.z; acc[i][r][3] += v.w;
                    }
        }
        cluster_sync();                                    // peers keep their shared memory until rank 0 has read it
        if (rank != 0) return;
    }
    if (warp != 0) return;
    // lane holds tokens (16i+g, 16i+g+8) x rows (2t, 2t+1) of every row group
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = i * 16 + g + (e >> 1) * 8;
            if (m >= M) continue;
            if (mode == MODE_SILU_MUL) {
                constexpr int HALF = RT / 2 > 0 ? RT / 2 : 1;
#pragma unroll
                for (int r = 0; r < HALF; ++r) {
                    const int col = tile * 8 * HALF + r * 8 + 2 * t + (e & 1);
                    if (col < N / 2) {
                        const float gate = acc[i][r][e], up = acc[i][HALF + r < RT ? HALF + r : r][e];
                        sp_st_dt(out, out_dt, (size_t)m * ldo + col, (gate / (1.0f + expf(-gate))) * up);
                    }
                }
            } else if (mode == MODE_ROPE_KV) {
                constexpr int HALF = RT / 2 > 0 ? RT / 2 : 1;
                const int half = rope.hd >> 1;
                const int pos = rope.positions[m];
#pragma unroll
                for (int r = 0; r < HALF; ++r) {
                    const int row = row_base[r] + 2 * t + (e & 1);       // row of the first half; its partner is half on
                    if (row >= N) continue;
                    const int blk = row / rope.hd, d = row % rope.hd;    // head-sized block and dim < half
                    const float a = acc[i][r][e], b = acc[i][HALF + r < RT ? HALF + r : r][e];
                    float lo = a, hi = b;
                    if (blk < rope.nh + rope.nkv) {
                        const float ang = (float)pos * rope.inv_freq[d];
                        const float c = cosf(ang), sn = sinf(ang);
                        lo = a * c - b * sn;
                        hi = b * c + a * sn;
                    }
                    if (blk < rope.nh) {
                        __nv_bfloat16* q = rope.q_out + (size_t)m * rope.nh * rope.hd + (size_t)blk * rope.hd;
                        q[d] = __float2bfloat16_rn(lo);
                        q[d + half] = __float2bfloat16_rn(hi);
                    } else {
                        const bool is_k = blk < rope.nh + rope.nkv;
                        const int kvh = is_k ? blk - rope.nh : blk - rope.nh - rope.nkv;
                        const int prow = rope.seq_row[rope.token_seq[m]];
                        if (!sp_index_ok(prow, rope.rg.n_rows, rope.rg, 402) || !sp_index_ok(pos / rope.page_size, rope.max_pages, rope.rg, 403)) continue;
                        const int page = rope.page_table[(size_t)prow * rope.max_pages + pos / rope.page_size];
                        if (!sp_index_ok(page, rope.rg.n_pages, rope.rg, 401)) continue;      // debug build: reported, not written
                        __nv_bfloat16* dst = (is_k ? rope.kpool : rope.vpool) +
                            (((size_t)page * rope.nkv + kvh) * rope.page_size + pos % rope.page_size) * rope.hd;
                        dst[d] = __float2bfloat16_rn(lo);
                        dst[d + half] = __float2bfloat16_rn(hi);
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    const int col = row_base[r] + 2 * t + (e & 1);
                    if (col >= N) continue;
                    const size_t o = (size_t)m * ldo + col;
                    float v = acc[i][r][e];
                    if (mode == MODE_ACCUMULATE) v += ((float*)out)[o];
                    sp_st_dt(out, out_dt, o, v);
                }
            }
        }
    }
}

// Many rows, few tokens (N ≥ 8192, M ≤ 16): no split of K. Every warp owns RT groups of 8 rows over all of
// K and streams them through two register buffers, so that the next U blocks of W are always on their way
// while the current ones are multiplied; there is no shared memory and no barrier. The sum over K runs in
// order of K within a warp: it depends on neither timing nor M.
template <int RT, int U>
__global__ void __launch_bounds__(128)
gemv_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, void* __restrict__ out,
                   int out_dt, int M, int N, int K, int ldx, int ldw, int ldo, int mode, int pair, int tiles) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x * 4 + warp;
    // launched as a programmatic dependent: x is what the kernel before wrote
    sp_allow_dependents();
    sp_wait_for_predecessor();
    if (tile >= tiles) return;
    constexpr int HALF = RT / 2 > 0 ? RT / 2 : 1;
    int row_base[RT];
    if (mode == MODE_SILU_MUL) {
#pragma unroll
        for (int r = 0; r < HALF; ++r) {
            const int o = tile * 8 * HALF + r * 8;
            row_base[r] = (o / pair) * 2 * pair + (o % pair);
            row_base[HALF + r < RT ? HALF + r : r] = row_base[r] + pair;
        }
    } else {
#pragma unroll
        for (int r = 0; r < RT; ++r) row_base[r] = (tile * RT + r) * 8;
    }
    const __nv_bfloat16* wrow[RT];
    bool wok[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const int row = row_base[r] + g;
        wok[r] = row < N;
        wrow[r] = W + (size_t)(wok[r] ? row : 0) * ldw;
    }
    const int kblocks = (K + 31) / 32;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    float acc[RT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;

    auto load = [&](uint4 (&b)[U][RT], int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb + u) * 32 + 8 * t;
            const bool kok = (kb + u) < kblocks && k < K;
#pragma unroll
            for (int r = 0; r < RT; ++r) b[u][r] = (kok && wok[r]) ? ld_stream(wrow[r] + k) : zero;
        }
    };
    auto compute = [&](const uint4 (&b)[U][RT], int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb + u) * 32 + 8 * t;
            const bool kok = (kb + u) < kblocks && k < K;
            const uint4 xa = (kok && g < M) ? ld_act(x + (size_t)g * ldx + k) : zero;
            const uint4 xb = (kok && g + 8 < M) ? ld_act(x + (size_t)(g + 8) * ldx + k) : zero;
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                mma_bf16(acc[r], xa.x, xb.x, xa.y, xb.y, b[u][r].x, b[u][r].y);
                mma_bf16(acc[r], xa.z, xb.z, xa.w, xb.w, b[u][r].z, b[u][r].w);
            }
        }
    };
    uint4 buf0[U][RT], buf1[U][RT];
    load(buf0, 0);
    for (int kb = 0; kb < kblocks; kb += 2 * U) {
        load(buf1, kb + U);
        compute(buf0, kb);
        load(buf0, kb + 2 * U);
        compute(buf1, kb + U);
    }
    if (mode == MODE_ARGMAX) {
        // lane (g, t) holds tokens g and g + 8 of rows 2t and 2t + 1 of every row group: the best of the warp's
        // rows per token, first among the lane's own, then over the four lanes that share g
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int row = row_base[r] + 2 * t + c;
                    if (row < N) take_better(bv, bi, acc[r][2 * h + c], row);
                }
#pragma unroll
            for (int o = 1; o <= 2; o <<= 1)
                take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
            const int m = g + 8 * h;
            if (t == 0 && m < M) ((Candidate*)out)[(size_t)m * ldo + tile] = Candidate{bv, bi};
        }
        return;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int m = g + (e >> 1) * 8;
        if (m >= M) continue;
        if (mode == MODE_SILU_MUL) {
#pragma unroll
            for (int r = 0; r < HALF; ++r) {
                const int col = tile * 8 * HALF + r * 8 + 2 * t + (e & 1);
                if (col < N / 2) {
                    const float gate = acc[r][e], up = acc[HALF + r < RT ? HALF + r : r][e];
                    sp_st_dt(out, out_dt, (size_t)m * ldo + col, (gate / (1.0f + expf(-gate))) * up);
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                const int col = row_base[r] + 2 * t + (e & 1);
                if (col >= N) continue;
                const size_t o = (size_t)m * ldo + col;
                float v = acc[r][e];
                if (mode == MODE_ACCUMULATE) v += ((float*)out)[o];
                sp_st_dt(out, out_dt, o, v);
            }
        }
    }
}

// How the work of one product is cut: row groups per CTA, CTAs per cluster along K, warps per CTA.
struct Plan { int rt, cs, ks, tiles; };

Plan make_plan(int M, int N, int K, int mode) {
    Plan p;
    const int outputs = (mode == MODE_SILU_MUL || mode == MODE_ROPE_KV) ? N / 2 : N;
    // few tokens: one row group per CTA (a gate/up pair for the fused epilogue) keeps the most CTAs in flight;
    // more tokens: several row groups share the x fragments
    const int wide = M <= 16 ? 1 : (M <= 32 ? 4 : 2);
    const bool paired = mode == MODE_SILU_MUL || mode == MODE_ROPE_KV;
    p.rt = paired ? (wide < 2 ? 2 : wide) : wide;
    const int per_tile = paired ? 8 * (p.rt / 2) : 8 * p.rt;
    p.tiles = (outputs + per_tile - 1) / per_tile;
    // a cluster splits K when one CTA's warps would need more than one round of loads for their slice
    const int kblocks = (K + 31) / 32;
    p.cs = 1;
    while (p.cs < 8 && kblocks > p.cs * MAX_KS * 16) p.cs *= 2;       // measured: two rounds per warp beat a wider cluster
    const int per_cta = (kblocks + p.cs - 1) / p.cs;
    const int max_ks = mode == MODE_SILU_MUL ? MAX_KS / 2 : MAX_KS;     // measured: the gate/up product runs best with four warps
    p.ks = per_cta < max_ks ? (per_cta < 1 ? 1 : per_cta) : max_ks;
    return p;
}

}  // namespace

SP_API int sp_gemv_supported(const void* x, const void* W, int M, int K, int ldx, int ldw) {
    if (M <= 0 || M > 64) SP_FAIL("gemv: built for 1 to 64 tokens, got %d", M);
    if (K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8)) SP_FAIL("gemv: K and the leading dimensions must be multiples of 8");
    if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) SP_FAIL("gemv: operands must start on a 16-byte boundary");
    return 0;
}

namespace {

int launch_gemv(const void* x, const void* W, void* out, int out_dt, int M, int N, int K, int ldx, int ldw, int ldo,
                int mode, int pair, const RopeOut& rope, cudaStream_t stream) {
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)W;
    const int stream_tiles = mode == MODE_SILU_MUL ? (N / 2 + 7) / 8 : (N + 7) / 8;
    if (M <= 16 && stream_tiles >= 148 * 16 && mode != MODE_ROPE_KV) {
        // enough rows (the output head) to give every warp rows of its own and still fill every SM sixteen warps deep
        if (mode == MODE_SILU_MUL)
            sp_launch_dependent(gemv_stream_kernel<2, 4>, dim3((stream_tiles + 3) / 4), dim3(128), 0, stream, xp, wp, out, out_dt, M,
                                N, K, ldx, ldw, ldo, mode, pair, stream_tiles);
        else
            sp_launch_dependent(gemv_stream_kernel<1, 8>, dim3((stream_tiles + 3) / 4), dim3(128), 0, stream, xp, wp, out, out_dt, M,
                                N, K, ldx, ldw, ldo, mode, pair, stream_tiles);
        SP_CHECK_LAUNCH("gemv_stream");
        return 0;
    }
    const Plan p = make_plan(M, N, K, mode);
    const dim3 grid(p.tiles * p.cs), block(p.ks * 32);
#define GV_LAUNCH(MT, RT, UN)                                                                              \
    SP_CHECK_CALL("gemv", sp_launch_cluster(gemv_kernel<MT, RT, UN>, grid, block, 0, stream, p.cs, xp, wp, out, out_dt,  \
                                            M, N, K, ldx, ldw, ldo, mode, pair, p.ks, p.cs, rope))
    if (p.rt == 4) GV_LAUNCH(2, 4, 2);
    else if (p.rt == 2 && M <= 16) GV_LAUNCH(1, 2, 4);
    else if (p.rt == 2) GV_LAUNCH(4, 2, 2);
    else GV_LAUNCH(1, 1, 8);
#undef GV_LAUNCH
    return 0;
}

int check_gemv(const void* x, const void* W, int M, int N, int K, int ldx, int ldw, int out_dt, int mode, int pair) {
    if (sp_gemv_supported(x, W, M, K, ldx, ldw)) return 1;
    if (mode == MODE_ACCUMULATE && out_dt != SP_DT_F32) SP_FAIL("gemv: accumulation needs a float32 output");
    if (mode < 0 || mode > 3) SP_FAIL("gemv: unknown mode %d", mode);
    if ((mode == MODE_SILU_MUL || mode == MODE_ROPE_KV) && (pair <= 0 || (pair % 8) || N % (2 * pair)))
        SP_FAIL("gemv: paired rows need blocks of a multiple of 8 rows that divide N/2 (N=%d, block %d)", N, pair);
    return 0;
}

}  // namespace

// mode 0: out = x·Wᵀ (bfloat16 or float32); 1: out (float32) += x·Wᵀ;
// 2: W interleaves ``pair`` gate rows and ``pair`` up rows; out [M, N/2] = silu(gate)·up.
SP_API int sp_gemv(const void* x, const void* W, void* out, int out_dt, int M, int N, int K, int ldx, int ldw,
                   int ldo, int mode, int pair, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (mode == MODE_ROPE_KV) SP_FAIL("gemv: the rotate-and-store epilogue has an entry point of its own");
    if (check_gemv(x, W, M, N, K, ldx, ldw, out_dt, mode, pair)) return 1;
    return launch_gemv(x, W, out, out_dt, M, N, K, ldx, ldw, ldo, mode, pair, RopeOut{}, stream);
}

// QKV for decoding in one kernel: W = [Wq; Wk; Wv], rotate-half on q and k in the epilogue, q to ``q_out``
// (bfloat16), k and v into the paged bfloat16 cache at each token's position. x [M, K] bfloat16.
SP_API int sp_gemv_qkv_rope(const void* x, int ldx, const void* W, int ldw, int M, int K, int nh, int nkv, int hd,
                            void* q_out, void* kpool, void* vpool, const int* positions, const int* token_seq,
                            const int* seq_row, const int* page_table, int max_pages, int page_size,
                            const float* inv_freq, cudaStream_t stream) {
    const int N = (nh + 2 * nkv) * hd;
    if (hd % 16) SP_FAIL("gemv (qkv): head_dim %d must be a multiple of 16 for the fused rotation", hd);
    if (check_gemv(x, W, M, N, K, ldx, ldw, SP_DT_BF16, MODE_ROPE_KV, hd / 2)) return 1;
    RopeOut rope{(__nv_bfloat16*)q_out, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, positions, token_seq, seq_row,
                 page_table, inv_freq, max_pages, page_size, nh, nkv, hd, sp_range_host};
    return launch_gemv(x, W, nullptr, SP_DT_BF16, M, N, K, ldx, ldw, 0, MODE_ROPE_KV, hd / 2, rope, stream);
}


// The greedy head for up to 16 tokens: the product with W [N, K] (the vocabulary's rows) of which only each warp's
// best (value, row) per token is kept. ``cand`` holds [M][sp_gemv_argmax_candidates(N)] pairs of (float, int32);
// the lowest row wins among equal values, rows beyond N and NaNs never win (a tile without a winner has row
// 0x7fffffff). A second kernel (argmax_candidates of the generic library) takes the best of each token's row.
SP_API int sp_gemv_argmax_candidates(int N) { return (N + 7) / 8; }

SP_API int sp_gemv_argmax(const void* x, const void* W, void* cand, int M, int N, int K, int ldx, int ldw, int ld_cand,
                          cudaStream_t stream) {
    if (N <= 0 || M <= 0) return 0;
    if (M > 16) SP_FAIL("gemv (argmax): built for 1 to 16 tokens, got %d", M);
    if (sp_gemv_supported(x, W, M, K, ldx, ldw)) return 1;
    const int tiles = sp_gemv_argmax_candidates(N);
    if (ld_cand < tiles) SP_FAIL("gemv (argmax): the candidate table has %d columns, %d are needed", ld_cand, tiles);
    sp_launch_dependent(gemv_stream_kernel<1, 8>, dim3((tiles + 3) / 4), dim3(128), 0, stream, (const __nv_bfloat16*)x,
                        (const __nv_bfloat16*)W, cand, (int)SP_DT_F32, M, N, K, ldx, ldw, ld_cand, (int)MODE_ARGMAX, 0, tiles);
    SP_CHECK_LAUNCH("gemv_argmax");
    return 0;
}
