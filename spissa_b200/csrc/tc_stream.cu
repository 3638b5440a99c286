// bfloat16 product for a few dozen tokens on the 5th-generation tensor cores: C[M,N] = A[M,K] · W[N,K]ᵀ with
// M ≤ 128, built to stream W (crates/spissa-runtime/src/ops.rs:62-105 states the layout and the product).
//
// With so few tokens the product is a stream of weights; what matters is that every SM pulls its share of W all
// the time. The tile kernel of tc_gemm.cu has one row of 128-token tiles here, so only N / 256 CTAs exist, each
// computing on 128 rows of which most are padding. This kernel turns the product round: 128 rows of W are the
// M of the tensor-core instruction and the tokens its N (16 to 128 columns), so an instruction does no more
// work than there are tokens, and K is cut into pieces so that about two CTAs per SM exist:
//   grid (W tiles of 128 rows, pieces of K); a CTA computes its piece of Wtile · Aᵀ into tensor memory:
//   warp 0   one thread fetches, per stage, a 128 x 64 box of W and a tokens x 64 box of A with TMA (128-byte swizzle);
//   warp 1   one thread issues tcgen05.mma (M 128 = rows of W, N = tokens, K 16, four per stage);
//   warps 2-5 read the accumulator (one row of W per thread, the tokens along its columns).
// The CTAs of one W tile form a thread-block cluster. Each leaves its piece of the sum in its own shared memory;
// then every CTA takes a share of the tokens, adds the pieces of all CTAs for them through distributed shared
// memory, in order of K, and runs the epilogue for them: store / add into a float32 C / silu(gate)·up (the CTA
// then computes the gate tile and the up tile of the same outputs into two accumulators). A row of W is a column of C: the 32 lanes of a warp write 32 neighbouring elements of one
// token's row. Every mbarrier wait is bounded and records a code in ``status``; no load uses cluster multicast.
#include "tcgen05.cuh"
#include <string.h>

SP_API const char* sp_tc_stream_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(tc_stream)

namespace {

constexpr int BW = 128;                     // rows of W per CTA
constexpr int BK = 64;                      // 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int MAX_SPLITS = 8;

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SILU_MUL = 2, MODE_ARGMAX = 3, MODE_QKV_ROPE = 4 };

// What the fused epilogues need beyond C; all zero for the plain ones. The layout is the one the tile kernel
// (tc_gemm.cu) takes, so that the host packs one structure for both. They fold a layer's RMS norms, the rotation and
// the cache write into the products of a step of 17 to 128 tokens (crates/spissa-runtime/src/models/llama/
// generate.rs:193-199 norm, :373-390 rotation, :410-416 cache append, :459-471 residual and second norm).
struct EpiArgs {
    // the rows of A are x ⊙ w of an RMS norm without its 1/rms: the result is multiplied by it here
    const float* row_ssq;          // [M][n_ssq] partial sums of squares of the residual rows (null: no scaling)
    int n_ssq, norm_width;         // norm_width: the residual's width H (1/rms = 1/sqrt(sum/H + eps))
    float eps;
    int pad0;
    // MODE_ACCUMULATE: also prepare the next norm's input
    __nv_bfloat16* xw;             // [M][N] new C ⊙ next_w (null: plain accumulation)
    const __nv_bfloat16* next_w;   // [N]
    float* ssq_out;                // [M][tiles of 128 columns] sums of squares of the new C over each tile's columns
    // MODE_QKV_ROPE: W = [q heads | k heads | v heads] x head_dim rows
    const float2* cs;              // [M][hd / 2] (cos, sin) of each token's angles
    const int* tok_page;           // [M] the cache page that holds the token's position
    const int* positions;          // [M]
    __nv_bfloat16* q_out;          // [M][nh * hd]
    __nv_bfloat16* kpool;          // [pages][nkv][page_size][hd]
    __nv_bfloat16* vpool;
    int nh, nkv, hd, page_size;
};
static_assert(sizeof(EpiArgs) == 112, "the host packs this layout");

// MODE_ARGMAX (the greedy head): of a tile's 128 rows of W only the best (value, row) per token is kept, the lowest
// row among equal values (crates/spissa-runtime/src/streaming/argmax.rs:30-51, :85-97); C is then a table of
// candidates [token][tile] and a second, tiny kernel takes the best of each token's row.
struct Candidate { float value; int index; };
// a float as an unsigned key of the same order; NaN -> 1 and "no row" -> 0 lie below every number
__device__ __forceinline__ uint32_t order_key(float v, bool valid) {
    if (!valid) return 0u;
    if (v != v) return 1u;
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

// NT: tokens padded to a multiple of 16 (the N of the instruction); GATED: two W tiles per CTA
template <int NT, bool GATED>
struct Layout {
    static constexpr int W_BYTES = BW * BK * 2;
    static constexpr int A_BYTES = NT * BK * 2;
    static constexpr int STAGE_BYTES = (GATED ? 2 : 1) * W_BYTES + A_BYTES;
    static constexpr int STAGES = GATED ? 2 : 4;                 // two CTAs per SM either way: one computes while the other adds up
    // after the products the same memory holds this CTA's piece of the sum: [part][token][128 rows] float32
    static constexpr int PIECE_BYTES = (GATED ? 2 : 1) * NT * BW * 4;
    static constexpr int TOTAL = (STAGES * STAGE_BYTES > PIECE_BYTES ? STAGES * STAGE_BYTES : PIECE_BYTES) + 1024;
    static constexpr uint32_t TMEM_COLS = (GATED ? 2 : 1) * NT <= 32 ? 32 : (GATED ? 2 : 1) * NT <= 64 ? 64
                                          : (GATED ? 2 : 1) * NT <= 128 ? 128 : 256;
};

struct Args {
    void* C;                // [M, ldc]: float32 or bfloat16
    int* status;
    int c_dt, M, N, K, ldc, mode, pair, pieces;
    EpiArgs ep;
    SpRange rg;
};

template <int NT, bool GATED>
__global__ void __launch_bounds__(192)
tc_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const Args a) {
    using L = Layout<NT, GATED>;
    constexpr int STAGES = L::STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t best_key[4][NT];                          // MODE_ARGMAX: each epilogue warp's best per token
    __shared__ int best_row[4][NT];
    __shared__ float rstd_s[NT];                                  // each token's 1/rms (1 without row statistics)
    __shared__ float ssq_w[4][NT];                                // preparing the next norm: each warp's sum of squares per token
    __shared__ float xch[2][4][BW];                               // MODE_QKV_ROPE: four tokens' 128 columns, for the rotation partners
    __shared__ int unhealthy;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.pieces, piece = blockIdx.x % a.pieces;     // the cluster's rank is the piece of K
    const int num_kb = (a.K + BK - 1) / BK;
    const int per = (num_kb + a.pieces - 1) / a.pieces;
    const int kb0 = piece * per, kb1 = min(num_kb, kb0 + per);        // the host makes every piece non-empty
    // rows of W: plain tiles, or the gate rows of block ``tile`` and the up rows ``pair`` further on
    const int row_g = GATED ? tile * 2 * a.pair : tile * BW;
    const int row_u = row_g + a.pair;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        unhealthy = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // set up; from here on the kernel reads what its predecessor in the stream wrote
    sp_allow_dependents();
    sp_wait_for_predecessor();

    constexpr int PARTS = GATED ? 2 : 1;
    const int q = warp & 3;                                       // epilogue warps: tensor-memory lanes 32q .. 32q+31
    const int row = q * 32 + lane;                                 // row of the W tile = column of C within the tile
    // where this thread's row of the tile goes in C
    const int col = GATED ? tile * a.pair + row : tile * BW + row;
    const bool col_ok = GATED ? (row < a.pair && col < a.N / 2) : col < a.N;
    const EpiArgs& ep = a.ep;
    const bool prepares_norm = !GATED && a.mode == MODE_ACCUMULATE && ep.xw != nullptr;
    const bool rope_mode = !GATED && a.mode == MODE_QKV_ROPE;
    float next_w = 0.0f;
    int rope_turn = 0;
    // MODE_QKV_ROPE: where this thread's column lies. A tile holds whole heads; dims d and d + hd/2 of a head are
    // rotation partners, 32 or 64 threads apart.
    int r_head = 0, r_d = 0, r_half = 1, r_kvh = 0;
    bool r_rot = false, r_q = false, r_k = false;
    if (rope_mode) {
        r_half = ep.hd >> 1;
        r_head = col / ep.hd;
        r_d = col - r_head * ep.hd;
        r_q = r_head < ep.nh;
        r_k = !r_q && r_head < ep.nh + ep.nkv;
        r_rot = r_q || r_k;
        r_kvh = r_k ? r_head - ep.nh : r_head - ep.nh - ep.nkv;
    }
    // What the epilogue of four tokens reads from global memory. A warp issues in order and such a load takes a
    // microsecond under load, so the loads of four tokens are issued together, before the first of them is used.
    struct Pre {
        float oldc[4];
        float2 cs[4];
        int page[4], pos[4];
    };
    auto prefetch4 = [&](int jb, int j_end, Pre& pre) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int j = jb + t;
            pre.oldc[t] = 0.0f;
            pre.cs[t] = make_float2(1.0f, 0.0f);
            pre.page[t] = pre.pos[t] = 0;
            if (j >= j_end || !col_ok || GATED) continue;
            if (a.mode == MODE_ACCUMULATE) pre.oldc[t] = ((const float*)a.C)[(size_t)j * a.ldc + col];
            if (rope_mode) {
                if (r_rot) pre.cs[t] = __ldg(ep.cs + (size_t)j * r_half + (r_d < r_half ? r_d : r_d - r_half));
                if (!r_q) {
                    pre.page[t] = __ldg(ep.tok_page + j);
                    pre.pos[t] = __ldg(ep.positions + j);
                }
            }
        }
    };
    // Tokens jb .. jb+3 (those below j_end) of this thread's column. The 128 epilogue threads call it together (the
    // fused epilogues add up or exchange across the threads): nothing here depends on the thread but the data.
    auto emit4 = [&](int jb, int j_end, const float (&g)[4], const float (&u)[4], const Pre& pre) {
        if (rope_mode) {
            float v[4];
            float* mine = xch[rope_turn & 1][0] + row;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                v[t] = jb + t < j_end ? g[t] * rstd_s[jb + t] : 0.0f;
                mine[t * BW] = v[t];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");         // two buffers: the next four tokens go to the other one
            const float* theirs = xch[rope_turn & 1][0] + (r_d < r_half ? row + r_half : row - r_half);
            ++rope_turn;
            if (!col_ok) return;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int j = jb + t;
                if (j >= j_end) continue;
                float outv = v[t];
                if (r_rot) {
                    const float other = theirs[t * BW];
                    outv = r_d < r_half ? v[t] * pre.cs[t].x - other * pre.cs[t].y : v[t] * pre.cs[t].x + other * pre.cs[t].y;
                }
                if (r_q) {
                    ep.q_out[((size_t)j * ep.nh + r_head) * ep.hd + r_d] = __float2bfloat16(outv);
                } else if (sp_index_ok(pre.page[t], a.rg.n_pages, a.rg, 401)) {      // debug build: reported, not written
                    (r_k ? ep.kpool : ep.vpool)[(((size_t)pre.page[t] * ep.nkv + r_kvh) * ep.page_size + pre.pos[t] % ep.page_size) * ep.hd + r_d] =
                        __float2bfloat16(outv);
                }
            }
            return;
        }
        float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (col_ok) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int j = jb + t;
                if (j >= j_end) continue;
                const size_t o = (size_t)j * a.ldc + col;
                const float rs = rstd_s[j];
                if (GATED) {
                    const float gg = g[t] * rs, uu = u[t] * rs;
                    sp_st_dt(a.C, a.c_dt, o, (gg / (1.0f + expf(-gg))) * uu);
                } else if (a.mode == MODE_ACCUMULATE) {
                    const float hn = pre.oldc[t] + g[t];
                    ((float*)a.C)[o] = hn;
                    if (prepares_norm) {
                        ep.xw[(size_t)j * a.N + col] = __float2bfloat16(hn * next_w);
                        sq[t] = hn * hn;
                    }
                } else {
                    sp_st_dt(a.C, a.c_dt, o, g[t] * rs);
                }
            }
        }
        if (prepares_norm) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float sum = sp_warp_sum(sq[t]);
                if (lane == 0 && jb + t < j_end) ssq_w[q][jb + t] = sum;
            }
        }
    };
    // after the tokens [j_lo, j_hi) of this CTA: the four warps' sums in warp order, one token per thread
    auto emit_ssq = [&](int j_lo, int j_hi) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int j = (warp - 2) * 32 + lane;
        if (j >= j_lo && j < j_hi && j < NT)
            ep.ssq_out[(size_t)j * ((a.N + BW - 1) / BW) + tile] = ssq_w[0][j] + ssq_w[1][j] + ssq_w[2][j] + ssq_w[3][j];
    };
    bool healthy = false;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = kb0, i = 0; kb < kb1; ++kb, ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(smem_u32(&bar_empty[s]), (((uint32_t)i / STAGES) & 1u) ^ 1u, a.status, 121)) break;
                const uint32_t w_dst = smem_base + s * L::STAGE_BYTES;
                mbar_expect_tx(smem_u32(&bar_full[s]), L::STAGE_BYTES);
                tma_load_2d(w_dst, &map_w, kb * BK, row_g, smem_u32(&bar_full[s]));
                if (GATED) tma_load_2d(w_dst + L::W_BYTES, &map_w, kb * BK, row_u, smem_u32(&bar_full[s]));
                tma_load_2d(w_dst + (GATED ? 2 : 1) * L::W_BYTES, &map_a, kb * BK, 0, smem_u32(&bar_full[s]));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BW, NT);
            for (int kb = kb0, i = 0; kb < kb1; ++kb, ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(smem_u32(&bar_full[s]), ((uint32_t)i / STAGES) & 1u, a.status, 122)) break;
                tc_fence_after();
                const uint32_t w_src = smem_base + s * L::STAGE_BYTES;
                const uint64_t dw = umma_desc_sw128(w_src);
                const uint64_t du = umma_desc_sw128(w_src + L::W_BYTES);
                const uint64_t da = umma_desc_sw128(w_src + (GATED ? 2 : 1) * L::W_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    tc_mma_bf16(tmem_base, dw + 2 * k, da + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
                    if (GATED) tc_mma_bf16(tmem_base + NT, du + 2 * k, da + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&bar_empty[s]));
            }
            tc_commit(smem_u32(&bar_acc));                         // also after a failed wait: the epilogue must not hang
        }
    } else {
        {
            // before the accumulator is waited for: each token's 1/rms from the partial sums, in their order
            const int e = (warp - 2) * 32 + lane;
            if (e < NT) {
                float r = 1.0f;
                if (ep.row_ssq && e < a.M) {
                    float sum = 0.0f;
                    for (int i = 0; i < ep.n_ssq; ++i) sum += __ldg(ep.row_ssq + (size_t)e * ep.n_ssq + i);
                    r = 1.0f / sqrtf(sum / (float)ep.norm_width + ep.eps);
                }
                rstd_s[e] = r;
            }
            if (prepares_norm && col_ok) next_w = __bfloat162float(__ldg(ep.next_w + col));
        }
        const bool ok = mbar_wait(smem_u32(&bar_acc), 0, a.status, 123);
        tc_fence_after();
        // the epilogue threads act together from here on: one verdict for all of them
        if (!(ok && !(a.status && *(volatile int*)a.status != 0))) unhealthy = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        healthy = unhealthy == 0;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        if (a.pieces == 1) {
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t rg[32], ru[32];
                tc_ld_32x32(lane_base + (uint32_t)c0, rg);
                if (GATED) tc_ld_32x32(lane_base + (uint32_t)(NT + c0), ru);
                tc_ld_wait();
                if (!GATED && a.mode == MODE_ARGMAX) {
                    // lanes are rows of W in rising order: the warp's largest key, and the lowest lane that holds it
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t key = order_key(__uint_as_float(rg[j]), col_ok);
                        const uint32_t top = __reduce_max_sync(0xffffffffu, key);
                        const uint32_t who = __ballot_sync(0xffffffffu, key == top);
                        if (lane == 0) {
                            best_key[q][c0 + j] = top;
                            best_row[q][c0 + j] = top > 1u ? tile * BW + q * 32 + (__ffs(who) - 1) : 0x7fffffff;
                        }
                    }
                } else if (healthy) {
#pragma unroll
                    for (int jb = 0; jb < 32; jb += 4) {
                        Pre pre;
                        prefetch4(c0 + jb, a.M, pre);
                        float g4[4], u4[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            g4[t] = __uint_as_float(rg[jb + t]);
                            u4[t] = GATED ? __uint_as_float(ru[jb + t]) : 0.0f;
                        }
                        emit4(c0 + jb, a.M, g4, u4, pre);
                    }
                }
            }
            if (prepares_norm && healthy) emit_ssq(0, a.M);
            if (!GATED && a.mode == MODE_ARGMAX) {
                asm volatile("bar.sync 1, 128;" ::: "memory");     // the four epilogue warps
                const int j = (warp - 2) * 32 + lane;              // one token per thread
                if (healthy && j < a.M && j < NT) {
                    uint32_t top = 0u;
                    int row_of = 0x7fffffff;
#pragma unroll
                    for (int w = 0; w < 4; ++w)                     // warps hold rising rows: a strict > keeps the lowest
                        if (best_key[w][j] > top) { top = best_key[w][j]; row_of = best_row[w][j]; }
                    ((Candidate*)a.C)[(size_t)j * a.ldc + tile] = Candidate{top > 1u ? key_value(top) : -INFINITY, row_of};
                }
            }
        } else {
            // this piece into this CTA's shared memory (the pipeline's stages are free by now), [part][token][row]
#pragma unroll 1
            for (int c0 = 0; c0 < PARTS * NT; c0 += 32) {
                uint32_t r[32];
                tc_ld_32x32(lane_base + (uint32_t)c0, r);
                tc_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(smem_base + (uint32_t)(((c0 + j) * BW + row) * 4)), "r"(r[j]) : "memory");
            }
        }
    }
    if (a.pieces > 1) {
        // every CTA of the cluster has left its piece in its shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2 && healthy) {
            // this CTA's share of the tokens: the pieces in order of K through distributed shared memory
            const int per_t = (a.M + a.pieces - 1) / a.pieces;
            const int j0 = piece * per_t, j1 = min(a.M, j0 + per_t);
            uint32_t peer[MAX_SPLITS];
#pragma unroll
            for (int sp = 0; sp < MAX_SPLITS; ++sp)
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[sp]) : "r"(smem_base), "r"(sp < a.pieces ? sp : 0));
            // four tokens at a time: a load from another CTA's shared memory takes long, so many are asked for at once
            for (int jb = j0; jb < j1; jb += 4) {
                float pg[4][MAX_SPLITS], pu[4][MAX_SPLITS];
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int sp = 0; sp < MAX_SPLITS; ++sp) {
                        pg[t][sp] = pu[t][sp] = 0.0f;
                        if (sp < a.pieces && jb + t < j1) {
                            const uint32_t at = peer[sp] + (uint32_t)(((jb + t) * BW + row) * 4);
                            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pg[t][sp]) : "r"(at));
                            if (GATED) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pu[t][sp]) : "r"(at + (uint32_t)(NT * BW * 4)));
                        }
                    }
                Pre pre;
                prefetch4(jb, j1, pre);
                float g4[4], u4[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    float g = pg[t][0], u = pu[t][0];
#pragma unroll
                    for (int sp = 1; sp < MAX_SPLITS; ++sp) { g += pg[t][sp]; u += pu[t][sp]; }
                    g4[t] = g;
                    u4[t] = u;
                }
                emit4(jb, j1, g4, u4, pre);
            }
            if (prepares_norm) emit_ssq(j0, j1);
        }
        // nobody leaves (and frees its shared memory) before every CTA has read what it needs
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with leading dimension ld, fetched in boxes of box_rows x 64
int encode_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) SP_FAIL("tc_stream: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) SP_FAIL("tc_stream: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

// Encoded maps are kept: a map depends on the matrix's address, shape, leading dimension and box only, the weights
// never move and the activations come back at the same addresses step after step. Encoding takes the driver a
// microsecond or two, which is most of what a short step's launch costs the host. A small direct-mapped table; the
// callers are one host thread per library (two threads would at worst encode the same map twice).
struct MapKey {
    const void* ptr;
    int rows, K, ld, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows; }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int MAP_SLOTS = 1024;
MapSlot map_cache[MAP_SLOTS];

int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
    const MapKey key{ptr, rows, K, ld, box_rows};
    size_t h = (size_t)((uintptr_t)ptr >> 4) * 1000003u + (size_t)rows * 8191u + (size_t)K * 131u + (size_t)ld * 31u + (size_t)box_rows;
    MapSlot& slot = map_cache[h % MAP_SLOTS];
    if (slot.used && slot.key == key) {
        *map = slot.map;
        return 0;
    }
    if (encode_map(map, ptr, rows, K, ld, box_rows)) return 1;
    slot.key = key;
    slot.map = *map;
    slot.used = true;
    return 0;
}

int sm_count() {
    const int n = sp_sm_count();
    return n > 0 ? n : 1;
}

template <int NT, bool GATED>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const Args& args, int tiles, cudaStream_t stream) {
    using L = Layout<NT, GATED>;
    static SpPerDevice configured;
    if (!configured.done()) {
        cudaError_t e = cudaFuncSetAttribute(tc_stream_kernel<NT, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) SP_FAIL("tc_stream: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
        configured.mark();
    }
    SP_CHECK_CALL("tc_stream", sp_launch_cluster(tc_stream_kernel<NT, GATED>, dim3(tiles * args.pieces), dim3(192),
                                                 (size_t)L::TOTAL, stream, -args.pieces, mw, ma, args));
    return 0;
}

int tiles_of(int N, int mode, int pair) { return mode == MODE_SILU_MUL ? N / (2 * pair) : (N + BW - 1) / BW; }

// Pieces of K = CTAs of a cluster: a power of two (clusters of other sizes pack badly into a GPC), as many as give
// about two CTAs per SM in one wave, each with at least one block of K.
int pieces_of(int tiles, int K) {
    const int num_kb = (K + BK - 1) / BK;
    int pieces = 1;
    while (pieces * 2 <= MAX_SPLITS && pieces * 2 <= num_kb && tiles * pieces * 2 <= 2 * sm_count()) pieces *= 2;
    while (pieces > 1 && (pieces - 1) * ((num_kb + pieces - 1) / pieces) >= num_kb) pieces /= 2;      // no empty piece
    return pieces;
}

}  // namespace

SP_API int sp_tc_stream_max_tokens() { return 128; }
// Candidates per token that MODE_ARGMAX writes for a weight of N rows (C is then [M][this] pairs of float, int32).
SP_API int sp_tc_stream_argmax_candidates(int N) { return (N + BW - 1) / BW; }

// Whether this kernel takes the product (0) or another has to (1, the reason as the last error).
SP_API int sp_tc_stream_supported(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int mode, int pair) {
    if (M <= 0 || M > 128) SP_FAIL("tc_stream: built for 1 to 128 tokens, got %d", M);
    if (K <= 0 || (K % 8) || (lda % 8) || (ldw % 8)) SP_FAIL("tc_stream: K and the leading dimensions must be multiples of 8 (16-byte rows for TMA)");
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) SP_FAIL("tc_stream: operands must start on a 16-byte boundary");
    if (mode == MODE_SILU_MUL && (pair <= 0 || pair > BW || (pair % 8) || (N % (2 * pair))))
        SP_FAIL("tc_stream: gate and up rows in blocks of %d do not fit tiles of %d rows", pair, BW);
    return 0;
}

static int tc_stream_any(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                         int mode, int pair, const EpiArgs* epp, int* status, cudaStream_t stream);

// mode 0: C = A·Wᵀ (bfloat16 or float32); 1: C (float32) += A·Wᵀ; 2: W interleaves ``pair`` gate rows and ``pair``
// up rows, C [M, N/2] = silu(gate)·up; 3: the greedy head's candidates.
SP_API int sp_tc_stream(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                        int mode, int pair, int* status, cudaStream_t stream) {
    if (mode == MODE_QKV_ROPE) SP_FAIL("tc_stream: the rotate-and-store epilogue needs sp_tc_stream_fused");
    return tc_stream_any(A, W, C, c_dt, M, N, K, lda, ldw, ldc, mode, pair, nullptr, status, stream);
}

// Floats per token that the accumulating epilogue writes into ssq_out when it prepares the next norm.
SP_API int sp_tc_stream_n_tiles(int N) { return (N + BW - 1) / BW; }

// The product with a fused epilogue (see EpiArgs; ``ep`` null or all zero: the plain epilogues of sp_tc_stream).
//   ep->row_ssq: the result is multiplied by each token's 1/rms (modes 0, 2 and 4);
//   mode 1 with ep->xw: C += A·Wᵀ, and xw = new C ⊙ next_w (bfloat16) and ssq_out[token][tile of 128 columns] are written;
//   mode 4: W = [q | k | v] heads x head_dim rows (head size 64 or 128); q and k are rotated with the per-token
//     (cos, sin) table, q goes to q_out and k, v into the paged cache; C is not used.
SP_API int sp_tc_stream_fused(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw,
                              int ldc, int mode, int pair, const void* ep, int* status, cudaStream_t stream) {
    return tc_stream_any(A, W, C, c_dt, M, N, K, lda, ldw, ldc, mode, pair, (const EpiArgs*)ep, status, stream);
}

static int tc_stream_any(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                         int mode, int pair, const EpiArgs* epp, int* status, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (mode < 0 || mode > 4) SP_FAIL("tc_stream: unknown mode %d", mode);
    if (mode == MODE_ACCUMULATE && c_dt != SP_DT_F32) SP_FAIL("tc_stream: accumulation needs a float32 C");
    if (sp_tc_stream_supported(A, W, M, N, K, lda, ldw, mode, pair)) return 1;
    EpiArgs ep;
    memset(&ep, 0, sizeof(ep));
    if (epp) ep = *epp;
    if (ep.row_ssq && (ep.n_ssq <= 0 || ep.norm_width <= 0)) SP_FAIL("tc_stream: the row statistics need their count and the norm's width");
    if (ep.row_ssq && (mode == MODE_ACCUMULATE || mode == MODE_ARGMAX)) SP_FAIL("tc_stream: row statistics do not go with mode %d", mode);
    if (ep.xw && (mode != MODE_ACCUMULATE || !ep.next_w || !ep.ssq_out))
        SP_FAIL("tc_stream: preparing the next norm's input belongs to the accumulating epilogue and needs its weight and a place for the sums");
    if (mode == MODE_QKV_ROPE) {
        if (ep.hd != 64 && ep.hd != 128) SP_FAIL("tc_stream: the rotate-and-store epilogue is built for head sizes 64 and 128, got %d", ep.hd);
        if (ep.nh <= 0 || ep.nkv <= 0 || N != (ep.nh + 2 * ep.nkv) * ep.hd) SP_FAIL("tc_stream: W has %d rows, %d q and %d kv heads of %d need %d", N, ep.nh, ep.nkv, ep.hd, (ep.nh + 2 * ep.nkv) * ep.hd);
        if (!ep.cs || !ep.tok_page || !ep.positions || !ep.q_out || !ep.kpool || !ep.vpool || ep.page_size <= 0)
            SP_FAIL("tc_stream: the rotate-and-store epilogue needs the angle table, the tokens' pages and positions, q and the cache");
    }
    const int tiles = tiles_of(N, mode, pair);
    Args args;
    args.ep = ep;
    args.rg = sp_range_host;
    args.C = C; args.status = status;
    args.c_dt = c_dt; args.M = M; args.N = N; args.K = K; args.ldc = ldc; args.mode = mode; args.pair = pair;
    // the greedy head keeps candidates per tile: one CTA computes a tile over all of K
    args.pieces = mode == MODE_ARGMAX ? 1 : pieces_of(tiles, K);
    const int nt = M <= 32 ? 32 : M <= 64 ? 64 : 128;
    CUtensorMap mw, ma;
    // gate/up tiles are ``pair`` rows each (the box still has 128 rows: those beyond belong to the next block and are ignored)
    if (make_map(&mw, W, N, K, ldw, BW)) return 1;
    if (make_map(&ma, A, M, K, lda, nt)) return 1;
    const bool gated = mode == MODE_SILU_MUL;
    if (nt == 32) return gated ? launch<32, true>(mw, ma, args, tiles, stream) : launch<32, false>(mw, ma, args, tiles, stream);
    if (nt == 64) return gated ? launch<64, true>(mw, ma, args, tiles, stream) : launch<64, false>(mw, ma, args, tiles, stream);
    return gated ? launch<128, true>(mw, ma, args, tiles, stream) : launch<128, false>(mw, ma, args, tiles, stream);
}
