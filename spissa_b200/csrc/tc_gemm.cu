// bfloat16 matrix product on the 5th-generation tensor cores: C[M,N] = A[M,K] · W[N,K]ᵀ.
//
// Both operands are K-major (a row of A or W is contiguous in K), as activations and the
// checkpoint's [out, in] weights are (crates/spissa-runtime/src/ops.rs:62-105 states the
// layout; the reference computes it with scalar/NEON dot products,
// crates/spissa-runtime/src/streaming/kernels_raw16.rs:442-530).
//
// A CTA computes 128 x BN tiles of C, one after another (a persistent grid of one CTA per SM):
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a
//            128x64 tile of A and a BNx64 tile of W per pipeline stage;
//   warp 1   allocates tensor memory and one thread issues tcgen05.mma (M=128, N=BN, K=16,
//            four per stage) with the accumulator in tensor memory; tcgen05.commit hands
//            each stage back to the loader and, at the end, the accumulator to
//   warps 2-5 which read it with tcgen05.ld (each warp its own 32 lanes) and store it:
//            plain, added into a float32 C, or as silu(gate)·up of an interleaved gate/up weight.
// Tensor memory holds two accumulators: while warps 2-5 store tile i, warp 1 already issues tile i+1.
// Every wait on an mbarrier is bounded by a wall-clock limit; when it runs out the kernel
// records a code in ``status``, every role falls through to the common exit, and tensor
// memory is freed. No load uses cluster multicast.
//
// Epilogues that save a pass over the activations of a prompt (the reference's block does norm, projections,
// rotation and cache append phase by phase, crates/spissa-runtime/src/models/llama/generate.rs:193-199, :373-390,
// :410-416, :459-471):
//   * an RMS norm costs no kernel: whoever adds into the 32-bit residual (the output and down projections) also
//     stores the new residual times the NEXT norm's weight in bfloat16 (the next product's A) and the row's sum of
//     squares over its tile's columns; the next product adds those partial sums in tile order and multiplies its
//     RESULT by 1/rms: y = rstd · (x ⊙ w)·Wᵀ;
//   * the QKV product rotates q and k (rotate-half, cosines and sines from a per-token table made once per step),
//     stores q and writes k and v into the paged cache at each token's position.
#include "tcgen05.cuh"

SP_API const char* sp_tc_gemm_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(tc_gemm)

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                      // 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SILU_MUL = 2, MODE_QKV_ROPE = 3 };

// What the fused epilogues need beyond C; all zero for the plain ones. The host mirrors this layout.
struct EpiArgs {
    // the rows of A are x ⊙ w of an RMS norm without its 1/rms: the result is multiplied by it here
    const float* row_ssq;          // [M][n_ssq] partial sums of squares of the residual rows (null: no scaling)
    int n_ssq, norm_width;         // norm_width: the residual's width H (1/rms = 1/sqrt(sum/H + eps))
    float eps;
    int pad0;
    // MODE_ACCUMULATE: also prepare the next norm's input
    __nv_bfloat16* xw;             // [M][N] new C ⊙ next_w (null: plain accumulation)
    const __nv_bfloat16* next_w;   // [N]
    float* ssq_out;                // [M][tiles along N] sums of squares of the new C over each tile's columns
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

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
    uint4 w;
    w.x = *(uint32_t*)&p0; w.y = *(uint32_t*)&p1; w.z = *(uint32_t*)&p2; w.w = *(uint32_t*)&p3;
    return w;
}

template <int BN, int STAGES, int CG = 1>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = (BN / CG) * BK * 2;            // a CTA of a pair holds its half of the W tile
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TRANSPOSE_BYTES = 4 * 32 * 36 * 4;        // a 32 x 32 float tile (rows padded to 36) per epilogue warp
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + TRANSPOSE_BYTES;      // + slack to align to 1024
};

// Stores 32 consecutive columns of one row, held as float32 in ``v``, the way ``mode`` asks.
__device__ __forceinline__ void store_row32(void* C, int c_dt, size_t base, int col0, int n_cols, const float* v,
                                            bool accumulate) {
    const bool full = col0 + 32 <= n_cols;
    if (c_dt == SP_DT_F32) {
        float* out = (float*)C + base;
        if (full && ((base & 3) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                if (accumulate) {
                    // this CTA is the only one that adds to these elements, so the sum is the same as read-add-write;
                    // the reduction needs no answer and hides the memory's latency
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                 ::"l"(out + j), "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3]) : "memory");
                } else {
                    *(float4*)(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < n_cols) out[j] = accumulate ? v[j] + out[j] : v[j];
        }
    } else {
        __nv_bfloat16* out = (__nv_bfloat16*)C + base;
        if (full && ((base & 7) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 w;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                __nv_bfloat162 p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                __nv_bfloat162 p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                w.x = *(uint32_t*)&p0; w.y = *(uint32_t*)&p1; w.z = *(uint32_t*)&p2; w.w = *(uint32_t*)&p3;
                *(uint4*)(out + j) = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < n_cols) out[j] = __float2bfloat16_rn(v[j]);
        }
    }
}

// Persistent: CTA b computes tiles b, b + gridDim.x, ... (M runs fastest over the tile index, so the
// CTAs that run together share few tiles of W). Two accumulators in tensor memory let the epilogue
// of one tile run while the next tile's products are issued.
//
// CG = 2: the CTAs of a cluster of two (on two SMs) work on ONE tile of 256 rows x BN columns with
// tcgen05.mma.cta_group::2. Each CTA fetches its 128 rows of A and its HALF of the W tile (BN/2 rows) into its own
// shared memory and keeps its 128 rows of the result in its own tensor memory; the tensor cores of both SMs read
// both halves of W. A stage then costs a CTA 32 KB instead of 48 KB for the same products: a third less traffic
// from L2 into each SM. The pair's first CTA issues the products; both CTAs' copies complete on its barrier
// (cp.async.bulk.tensor with .cta_group::2, no multicast), its commits arrive on both CTAs' barriers, and the second
// CTA's epilogue warps arrive on the first's "accumulator free" barrier through the cluster's shared window.
__device__ __forceinline__ uint32_t pair_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t in_first_cta(uint32_t local_addr) {          // the same variable in the pair's first CTA
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(0u));
    return a;
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a tile of this CTA's own shared memory; the bytes count on the barrier ``bar_first`` of the pair's first CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_first) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_first) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrives, once the products issued so far are done, on the barrier at this address in BOTH CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_first_cta(uint32_t local_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(in_first_cta(local_bar)) : "memory");
}

template <int BN, int STAGES, int CG = 1>
__global__ void __launch_bounds__(192, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ C, int c_dt, int M, int N, int K, int ldc, int mode, int* status,
               const __grid_constant__ EpiArgs ep, const SpRange rg) {
    using L = SmemLayout<BN, STAGES, CG>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_slot;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    constexpr int TM = BM * CG;                                  // rows of a tile
    const int m_tiles = (M + TM - 1) / TM, n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int rank = CG == 2 ? (int)pair_rank() : 0;
    const int walker = CG == 2 ? (int)blockIdx.x / 2 : (int)blockIdx.x;          // which of the tile walkers this CTA belongs to
    const int walkers = CG == 2 ? (int)gridDim.x / 2 : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 4 * CG);     // one arrival per epilogue warp (of both CTAs of a pair)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // two accumulators, each at a power-of-two column (tensor memory is handed out in powers of two)
    constexpr uint32_t ACC_STRIDE = BN <= 128 ? 128u : 256u, TMEM_COLS = 2u * ACC_STRIDE;
    if (warp == 1) {
        if (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CG == 2) pair_sync();                                   // the other CTA's barriers exist before anything arrives there
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // Set up. From here on the kernel reads what its predecessor in the stream wrote (A, C, the rows' statistics).
    // (Asking for the first W tiles before this wait, since the weights are nobody's output, changed nothing: a CTA of
    // this kernel becomes resident only when the predecessor's CTA has left its SM.)
    sp_allow_dependents();
    sp_wait_for_predecessor();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t kbc = 0;                                   // pipeline slots used so far, over all tiles
            bool ok = true;
            for (int tile = walker; tile < total_tiles && ok; tile += walkers) {
                const int m0 = (tile % m_tiles) * TM + rank * BM, n0 = (tile / m_tiles) * BN + rank * (BN / CG);
                for (int kb = 0; kb < num_kb; ++kb, ++kbc) {
                    const int s = kbc % STAGES;
                    const uint32_t phase = (kbc / STAGES) & 1u;
                    const uint32_t a_dst = smem_base + s * L::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + L::A_BYTES;
                    ok = mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1u, status, 101);
                    if (!ok) break;
                    if (CG == 2) {
                        // both CTAs' bytes count on the first CTA's barrier, which expects them all
                        const uint32_t full_first = in_first_cta(smem_u32(&bar_full[s]));
                        if (rank == 0) mbar_expect_tx(smem_u32(&bar_full[s]), 2 * L::STAGE_BYTES);
                        tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, full_first);
                        tma_load_2d_pair(b_dst, &map_w, kb * BK, n0, full_first);
                    } else {
                        mbar_expect_tx(smem_u32(&bar_full[s]), L::STAGE_BYTES);
                        tma_load_2d(a_dst, &map_a, kb * BK, m0, smem_u32(&bar_full[s]));
                        tma_load_2d(b_dst, &map_w, kb * BK, n0, smem_u32(&bar_full[s]));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                           // of a pair, the first CTA issues the products of both
            constexpr uint32_t idesc = umma_idesc_bf16(TM, BN);
            uint32_t kbc = 0, it = 0;
            bool ok = true;
            for (int tile = walker; tile < total_tiles && ok; tile += walkers, ++it) {
                const uint32_t buf = it & 1u, use = it >> 1;
                ok = mbar_wait(smem_u32(&bar_acc_empty[buf]), (use & 1u) ^ 1u, status, 104);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * ACC_STRIDE;
                for (int kb = 0; kb < num_kb; ++kb, ++kbc) {
                    const int s = kbc % STAGES;
                    const uint32_t phase = (kbc / STAGES) & 1u;
                    ok = mbar_wait(smem_u32(&bar_full[s]), phase, status, 102);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_src = smem_base + s * L::STAGE_BYTES;
                    const uint64_t da = umma_desc_sw128(a_src);
                    const uint64_t db = umma_desc_sw128(a_src + L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 bf16 = 32 bytes further along K inside the swizzle span: +2 in 16-byte units
                        if (CG == 2) tc_mma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else tc_mma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    if (CG == 2) tc_commit_pair(smem_u32(&bar_empty[s]));
                    else tc_commit(smem_u32(&bar_empty[s]));
                }
                // also after a failed wait: the epilogue must not hang
                if (CG == 2) tc_commit_pair(smem_u32(&bar_acc_full[buf]));
                else tc_commit(smem_u32(&bar_acc_full[buf]));
            }
        }
    } else {
        const int q = warp & 3;                      // this warp may touch tensor-memory lanes 32q .. 32q+31
        uint32_t it = 0;
        auto acc_free = [&](uint32_t buf) {          // the accumulator may be overwritten: the issuing CTA keeps count
            if (CG == 2 && rank != 0) mbar_arrive_first_cta(smem_u32(&bar_acc_empty[buf]));
            else mbar_arrive(smem_u32(&bar_acc_empty[buf]));
        };
        for (int tile = walker; tile < total_tiles; tile += walkers, ++it) {
            const int m0 = (tile % m_tiles) * TM + rank * BM, n0 = (tile / m_tiles) * BN;
            const uint32_t buf = it & 1u, use = it >> 1;
            const int row = m0 + q * 32 + lane;
            constexpr int SPAN = 32;
            // What the epilogue reads from global memory does not depend on the accumulator: it is asked for now,
            // while the tile's products still run, and costs no waiting afterwards. (A load's round trip is a
            // microsecond under load; a tile has up to eight chunks.)
            float ssq_sum = 0.0f;                                   // the row's partial sums of squares, in tile order
            if (ep.row_ssq && row < M)
                for (int i = 0; i < ep.n_ssq; ++i) ssq_sum += __ldg(ep.row_ssq + (size_t)row * ep.n_ssq + i);
            // The accumulating epilogue that also prepares the next norm regroups each 32 x 32 chunk so that eight
            // lanes cover the 128 bytes of one row (a lane: 4 columns of rows sub, sub + 4, ... sub + 28): a warp's
            // load or store of the residual then touches 4 whole lines instead of a piece of 32 lines.
            const bool emit = mode == MODE_ACCUMULATE && ep.xw != nullptr;
            const int sub = lane >> 3, c4 = (lane & 7) * 4;
            const int rows_here = min(32, M - (m0 + q * 32));                       // rows of this warp that exist (may be <= 0)
            const bool wide_ok = ((ldc & 3) == 0) && ((N & 3) == 0) && ((((uintptr_t)C | (uintptr_t)ep.xw) & 15) == 0);
            float* cbase = (float*)C + (size_t)(m0 + q * 32 + sub) * ldc + n0 + c4;
            constexpr int AHEAD = 2;                                // chunks of the old residual in flight
            float4 old[AHEAD][8];
            auto fetch_old = [&](int c0, float4 (&o)[8]) {
                if (c0 < BN && n0 + c0 + c4 + 4 <= N) {
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (sub + 4 * k < rows_here) o[k] = *(const float4*)(cbase + (size_t)(4 * k) * ldc + c0);
                }
            };
            if (emit && wide_ok) {
#pragma unroll
                for (int u = 0; u < AHEAD; ++u) fetch_old(u * SPAN, old[u]);
            }
            float4 cs_reg[16];                                      // (cos, sin) of 32 dims of this thread's token
            int pos = 0, page = 0;
            if (mode == MODE_QKV_ROPE && row < M) {
                pos = __ldg(ep.positions + row);
                page = __ldg(ep.tok_page + row);
                const float4* t4 = (const float4*)(ep.cs + (size_t)row * (ep.hd >> 1));
#pragma unroll
                for (int j = 0; j < 16; ++j) cs_reg[j] = __ldg(t4 + j);
            }
            const bool ok = mbar_wait(smem_u32(&bar_acc_full[buf]), use & 1u, status, 103);
            tc_fence_after();
            if (!ok || (status && *(volatile int*)status != 0)) break;
            const uint32_t taddr = tmem_base + buf * ACC_STRIDE + ((uint32_t)(q * 32) << 16);
            const int c_end = (mode == MODE_SILU_MUL) ? BN / 2 : BN;
            // 1/rms of this thread's row
            const float rstd = ep.row_ssq ? 1.0f / sqrtf(ssq_sum / (float)ep.norm_width + ep.eps) : 1.0f;
            if (mode == MODE_QKV_ROPE) {
                // the tile holds whole heads; dims d and d + hd/2 of a head are rotation partners
                const int hd = ep.hd, half = hd >> 1, heads_here = BN / hd;
#pragma unroll 1
                for (int hh = 0; hh < heads_here; ++hh) {
                    const int col0 = n0 + hh * hd;
                    const int blk = col0 / hd;                          // q heads, then k heads, then v heads
                    bool live = row < M && col0 < N;
                    __nv_bfloat16* dst = nullptr;
                    if (live) {
                        if (blk < ep.nh) dst = ep.q_out + ((size_t)row * ep.nh + blk) * hd;
                        else if (!sp_index_ok(page, rg.n_pages, rg, 401)) live = false;      // debug build: reported, not written
                        else {
                            const bool is_k = blk < ep.nh + ep.nkv;
                            const int kvh = is_k ? blk - ep.nh : blk - ep.nh - ep.nkv;
                            dst = (is_k ? ep.kpool : ep.vpool) +
                                  (((size_t)page * ep.nkv + kvh) * ep.page_size + pos % ep.page_size) * hd;
                        }
                    }
                    const bool rotate = blk < ep.nh + ep.nkv;
#pragma unroll 1
                    for (int c = 0; c < half; c += SPAN) {
                        uint32_t ra[32], rb[32];
                        if (half > SPAN && live && rotate && !(hh == 0 && c == 0)) {
                            // head size 128: the table's other half (one half per head otherwise: loaded once per tile)
                            const float4* t4 = (const float4*)(ep.cs + (size_t)row * half + c);
#pragma unroll
                            for (int j = 0; j < 16; ++j) cs_reg[j] = __ldg(t4 + j);
                        }
                        tc_ld_32x32(taddr + (uint32_t)(hh * hd + c), ra);
                        tc_ld_32x32(taddr + (uint32_t)(hh * hd + half + c), rb);
                        tc_ld_wait();
                        if (hh == heads_here - 1 && c + SPAN >= half) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) acc_free(buf);
                        }
                        if (!live) continue;
                        float lo[32], hi[32];
                        if (rotate) {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                const float4 cc = cs_reg[j >> 1];                       // cos, sin of two dims
                                const float a0 = __uint_as_float(ra[j]) * rstd, b0 = __uint_as_float(rb[j]) * rstd;
                                const float a1 = __uint_as_float(ra[j + 1]) * rstd, b1 = __uint_as_float(rb[j + 1]) * rstd;
                                lo[j] = a0 * cc.x - b0 * cc.y;
                                hi[j] = b0 * cc.x + a0 * cc.y;
                                lo[j + 1] = a1 * cc.z - b1 * cc.w;
                                hi[j + 1] = b1 * cc.z + a1 * cc.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                lo[j] = __uint_as_float(ra[j]) * rstd;
                                hi[j] = __uint_as_float(rb[j]) * rstd;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            *(uint4*)(dst + c + j) = pack8_bf16(lo + j);
                            *(uint4*)(dst + half + c + j) = pack8_bf16(hi + j);
                        }
                    }
                }
                continue;
            }
            if (emit) {
                // new residual = C + product; its product with the next norm's weight; its sum of squares
                float* tr = (float*)(smem_raw + (smem_base - smem_u32(smem_raw)) + STAGES * L::STAGE_BYTES) + q * (32 * 36);
                __nv_bfloat16* xbase = ep.xw + (size_t)(m0 + q * 32 + sub) * N + n0 + c4;
                float part[8];                                        // this lane's share of the sums of squares of its 8 rows
#pragma unroll
                for (int k = 0; k < 8; ++k) part[k] = 0.0f;
#pragma unroll
                for (int ci = 0; ci < BN / SPAN; ++ci) {
                    const int c0 = ci * SPAN;
                    uint32_t r[32];
                    tc_ld_32x32(taddr + (uint32_t)c0, r);
                    tc_ld_wait();
                    if (c0 + SPAN >= BN) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) acc_free(buf);
                    }
                    // lane = row becomes (lane / 8 = row mod 4, lane % 8 = four columns): through this warp's own tile
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *(float4*)(tr + lane * 36 + 4 * j) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    __syncwarp();
                    float4 acc[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] = *(const float4*)(tr + (sub + 4 * k) * 36 + c4);
                    __syncwarp();
                    const int col = n0 + c0 + c4;
                    if (wide_ok && col + 4 <= N) {
                        const uint2 wq = __ldg((const uint2*)(ep.next_w + col));
                        const float2 w01 = __bfloat1622float2(*(const __nv_bfloat162*)&wq.x);
                        const float2 w23 = __bfloat1622float2(*(const __nv_bfloat162*)&wq.y);
                        float4 (&o)[8] = old[ci % AHEAD];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            if (sub + 4 * k < rows_here) {
                                const float4 v = make_float4(o[k].x + acc[k].x, o[k].y + acc[k].y, o[k].z + acc[k].z, o[k].w + acc[k].w);
                                *(float4*)(cbase + (size_t)(4 * k) * ldc + c0) = v;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(v.x * w01.x, v.y * w01.y);
                                __nv_bfloat162 p1 = __floats2bfloat162_rn(v.z * w23.x, v.w * w23.y);
                                uint2 pk;
                                pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
                                *(uint2*)(xbase + (size_t)(4 * k) * N + c0) = pk;
                                part[k] = fmaf(v.x, v.x, part[k]); part[k] = fmaf(v.y, v.y, part[k]);
                                part[k] = fmaf(v.z, v.z, part[k]); part[k] = fmaf(v.w, v.w, part[k]);
                            }
                        }
                    } else {
                        // ragged or unaligned edges: element by element
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const float a4[4] = {acc[k].x, acc[k].y, acc[k].z, acc[k].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                if (sub + 4 * k < rows_here && col + e < N) {
                                    float* cp = cbase + (size_t)(4 * k) * ldc + c0 + e;
                                    const float v = *cp + a4[e];
                                    *cp = v;
                                    xbase[(size_t)(4 * k) * N + c0 + e] = __float2bfloat16_rn(v * __bfloat162float(ep.next_w[col + e]));
                                    part[k] = fmaf(v, v, part[k]);
                                }
                            }
                        }
                    }
                    // the buffer this chunk used takes the chunk AHEAD further on
                    if (wide_ok) fetch_old(c0 + AHEAD * SPAN, old[ci % AHEAD]);
                }
                // the rows' sums over this tile's columns: the eight lanes of a row added in a fixed (butterfly) order
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    float s_row = part[k];
                    s_row += __shfl_xor_sync(0xffffffffu, s_row, 1);
                    s_row += __shfl_xor_sync(0xffffffffu, s_row, 2);
                    s_row += __shfl_xor_sync(0xffffffffu, s_row, 4);
                    if ((lane & 7) == 0 && sub + 4 * k < rows_here)
                        ep.ssq_out[(size_t)(m0 + q * 32 + sub + 4 * k) * n_tiles + (tile / m_tiles)] = s_row;
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < c_end; c0 += SPAN) {
                uint32_t r[32];
                float v[32];
                tc_ld_32x32(taddr + (uint32_t)c0, r);
                if (mode == MODE_SILU_MUL) {
                    // tile columns [0, BN/2) are gate rows, [BN/2, BN) the up rows of the same outputs
                    uint32_t u[32];
                    tc_ld_32x32(taddr + (uint32_t)(c0 + BN / 2), u);
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g = __uint_as_float(r[j]) * rstd;
                        v[j] = (g / (1.0f + expf(-g))) * (__uint_as_float(u[j]) * rstd);
                    }
                } else {
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * rstd;
                }
                if (c0 + SPAN >= c_end) {            // all of this tile has left tensor memory: hand the buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) acc_free(buf);
                }
                if (row < M) {
                    if (mode == MODE_SILU_MUL)
                        store_row32(C, c_dt, (size_t)row * ldc + n0 / 2 + c0, n0 / 2 + c0, N / 2, v, false);
                    else
                        store_row32(C, c_dt, (size_t)row * ldc + n0 + c0, n0 + c0, N, v, mode == MODE_ACCUMULATE);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CG == 2) pair_sync();           // neither CTA leaves while the other's products read its shared memory or arrive on its barriers
    if (warp == 1) {
        tc_fence_after();
        if (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- few tiles: K split over a cluster
// With a few hundred tokens at most there are few tiles, too few CTAs to pull W from memory at full speed, and each
// walks all of K alone (the down projection of 256 tokens: 32 tiles of 128 blocks of K). Here
// the CTAs of a thread-block cluster share one 128 x BN tile: each takes a slice of K, leaves its partial
// tile in its own shared memory (over the pipeline stages, which are spent by then), and rank 0 adds the
// partial tiles in rank order through distributed shared memory before the usual epilogue. The order of
// the sum is fixed, so results do not depend on timing.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// four neighbouring columns of one row of a peer's partial tile ([column / 4][row][4] float32)
__device__ __forceinline__ float4 ld_peer_f4(uint32_t local_addr, uint32_t rank) {
    uint32_t ra;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
    float4 v;
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra));
    return v;
}
__device__ __forceinline__ uint32_t part_addr(uint32_t part, int col, int row) {
    return part + (uint32_t)((((col >> 2) * BM + row) << 4));
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
tc_gemm_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      void* __restrict__ C, int c_dt, int M, int N, int K, int ldc, int mode, int splits, int* status) {
    using L = SmemLayout<BN, STAGES>;
    static_assert(STAGES * L::STAGE_BYTES >= BM * BN * 4, "the partial tile must fit over the pipeline stages");
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc;
    __shared__ uint32_t tmem_slot;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();
    const int m_tiles = (M + BM - 1) / BM;
    const int tile = blockIdx.x / splits;                     // rows run fastest: clusters that run together share few tiles of W
    const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
    const int num_kb = (K + BK - 1) / BK;
    const int per = (num_kb + splits - 1) / splits;
    const int kb0 = min(num_kb, rank * per), kb1 = min(num_kb, kb0 + per);
    const int my_kb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < my_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1u, status, 101)) break;
                const uint32_t a_dst = smem_base + s * L::STAGE_BYTES;
                mbar_expect_tx(smem_u32(&bar_full[s]), L::STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, m0, smem_u32(&bar_full[s]));
                tma_load_2d(a_dst + L::A_BYTES, &map_w, (kb0 + i) * BK, n0, smem_u32(&bar_full[s]));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
            for (int i = 0; i < my_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(smem_u32(&bar_full[s]), phase, status, 102)) break;
                tc_fence_after();
                const uint32_t a_src = smem_base + s * L::STAGE_BYTES;
                const uint64_t da = umma_desc_sw128(a_src);
                const uint64_t db = umma_desc_sw128(a_src + L::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
                tc_commit(smem_u32(&bar_empty[s]));
            }
            tc_commit(smem_u32(&bar_acc));
        }
    }
    const int q = warp & 3;
    const int row = q * 32 + lane;                            // within the tile
    const int grow = m0 + row;                                // of C
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t part = smem_base;                          // [BN / 4][128 rows][4] float32
    bool ok = true;
    if (warp >= 2) {
        ok = mbar_wait(smem_u32(&bar_acc), 0, status, 103);
        tc_fence_after();
        if (rank != 0) {
            // leave this CTA's partial tile where rank 0 can read it
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                if (my_kb > 0) { tc_ld_32x32(taddr + (uint32_t)c0, r); tc_ld_wait(); }
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const uint32_t z = 0u;
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(part_addr(part, c0 + j, row)),
                                 "r"(my_kb > 0 ? r[j] : z), "r"(my_kb > 0 ? r[j + 1] : z), "r"(my_kb > 0 ? r[j + 2] : z),
                                 "r"(my_kb > 0 ? r[j + 3] : z) : "memory");
                }
            }
        }
    }
    __syncwarp();
    cluster_sync_all();                                       // every partial tile is written
    if (warp >= 2 && rank == 0 && ok && !(status && *(volatile int*)status != 0)) {
        const int c_end = (mode == MODE_SILU_MUL) ? BN / 2 : BN;
#pragma unroll 1
        for (int c0 = 0; c0 < c_end; c0 += 32) {
            uint32_t r[32];
            float v[32];
            if (my_kb > 0) { tc_ld_32x32(taddr + (uint32_t)c0, r); tc_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = my_kb > 0 ? __uint_as_float(r[j]) : 0.0f;
            for (int c = 1; c < splits; ++c) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 pv = ld_peer_f4(part_addr(part, c0 + j, row), (uint32_t)c);
                    v[j] += pv.x; v[j + 1] += pv.y; v[j + 2] += pv.z; v[j + 3] += pv.w;
                }
            }
            if (mode == MODE_SILU_MUL) {
                uint32_t u[32];
                if (my_kb > 0) { tc_ld_32x32(taddr + (uint32_t)(c0 + BN / 2), u); tc_ld_wait(); }
                float b[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) b[j] = my_kb > 0 ? __uint_as_float(u[j]) : 0.0f;
                for (int c = 1; c < splits; ++c) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 pv = ld_peer_f4(part_addr(part, c0 + BN / 2 + j, row), (uint32_t)c);
                        b[j] += pv.x; b[j + 1] += pv.y; b[j + 2] += pv.z; b[j + 3] += pv.w;
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float g = v[j];
                    v[j] = (g / (1.0f + expf(-g))) * b[j];
                }
                if (grow < M) store_row32(C, c_dt, (size_t)grow * ldc + n0 / 2 + c0, n0 / 2 + c0, N / 2, v, false);
            } else if (grow < M) {
                store_row32(C, c_dt, (size_t)grow * ldc + n0 + c0, n0 + c0, N, v, mode == MODE_ACCUMULATE);
            }
        }
    }
    __syncwarp();
    cluster_sync_all();                                       // peers keep their tiles until rank 0 has read them
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// ---------------------------------------------------------------- host side
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
    if (!fn) SP_FAIL("tc_gemm: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) SP_FAIL("tc_gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
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

template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int c_dt, int M, int N, int K, int ldc, int mode,
           int* status, cudaStream_t stream, const EpiArgs& ep) {
    using L = SmemLayout<BN, STAGES>;
    static SpPerDevice configured;
    if (!configured.done()) {
        cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) SP_FAIL("tc_gemm: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
        configured.mark();
    }
    const int sm_count = sp_sm_count();
    if (sm_count <= 0) SP_FAIL("tc_gemm: cannot read the number of SMs");
    const long long tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    SP_CHECK_CALL("tc_gemm", sp_launch_dependent(tc_gemm_kernel<BN, STAGES>, dim3(grid), dim3(192), (size_t)L::TOTAL, stream, ma, mw,
                                                 C, c_dt, M, N, K, ldc, mode, status, ep, sp_range_host));
    return 0;
}

// The same tiles by pairs of CTAs (tcgen05 cta_group::2): tiles of 256 rows, one pair per two SMs.
template <int BN, int STAGES>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw_half, void* C, int c_dt, int M, int N, int K, int ldc, int mode,
                int* status, cudaStream_t stream, const EpiArgs& ep) {
    using L = SmemLayout<BN, STAGES, 2>;
    static_assert(L::TOTAL <= 232448, "a CTA's shared memory");
    static SpPerDevice configured;
    if (!configured.done()) {
        cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<BN, STAGES, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) SP_FAIL("tc_gemm: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
        configured.mark();
    }
    const int sm_count = sp_sm_count();
    if (sm_count < 2) SP_FAIL("tc_gemm: cannot read the number of SMs");
    const long long tiles = (long long)((N + BN - 1) / BN) * ((M + 2 * BM - 1) / (2 * BM));
    const int pairs = (int)(tiles < sm_count / 2 ? tiles : sm_count / 2);
    SP_CHECK_CALL("tc_gemm", sp_launch_cluster(tc_gemm_kernel<BN, STAGES, 2>, dim3(2 * pairs), dim3(192), (size_t)L::TOTAL, stream,
                                               -2, ma, mw_half, C, c_dt, M, N, K, ldc, mode, status, ep, sp_range_host));
    return 0;
}

template <int BN, int STAGES>
int launch_splitk(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int c_dt, int M, int N, int K, int ldc,
                  int mode, int splits, int* status, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    static SpPerDevice configured;
    if (!configured.done()) {
        cudaError_t e = cudaFuncSetAttribute(tc_gemm_splitk_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) SP_FAIL("tc_gemm: cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
        configured.mark();
    }
    const int n_tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    SP_CHECK_CALL("tc_gemm_splitk", sp_launch_cluster(tc_gemm_splitk_kernel<BN, STAGES>, dim3(n_tiles * splits), dim3(192),
                                                     (size_t)L::TOTAL, stream, splits, ma, mw, C, c_dt, M, N, K, ldc,
                                                     mode, splits, status));
    return 0;
}

// How many CTAs share one tile along K: only for few tiles. Measured at 64 tokens on B200: two CTAs help a little
// for K = 2048 (15.6 -> 13.6 us for 24 tiles), four halve the time for K = 8192 (41.6 -> 20.1 us for 16 tiles),
// eight are slower than one, and with 64 tiles or more splitting only hurts. Beyond one row of tiles (more than 128
// tokens) only the long loops over K are split: the down projection of 129 to 1,023 tokens.
int pick_splits(int M, int N, int K, int bn) {
    const int tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM);
    const int num_kb = (K + BK - 1) / BK;
    if (M > BM) return num_kb < 64 ? 1 : tiles <= 36 ? 4 : tiles <= 72 ? 2 : 1;         // one wave of CTAs at most
    if (tiles > 32) return 1;
    if (num_kb >= 64) return 4;
    if (num_kb >= 16) return 2;
    return 1;
}

}  // namespace

// Whether the tensor-core kernel takes these operands; the reason goes to the error text.
SP_API int sp_tc_gemm_supported(const void* A, const void* W, int K, int lda, int ldw) {
    if (K <= 0 || (K % 8) || (lda % 8) || (ldw % 8)) SP_FAIL("tc_gemm: K and the leading dimensions must be multiples of 8 (16-byte rows for TMA)");
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) SP_FAIL("tc_gemm: operands must start on a 16-byte boundary");
    return 0;
}

// The product with a fused epilogue (see EpiArgs; ``ep`` null or all zero: the plain epilogues of sp_tc_gemm).
//   ep->row_ssq: the result is multiplied by each row's 1/rms (modes 0, 2 and 3);
//   mode 1 with ep->xw: C += A·Wᵀ, and xw = new C ⊙ next_w (bfloat16) and ssq_out[row][tile along N] are written;
//     ssq_out holds sp_tc_gemm_n_tiles(N, bn) floats per row;
//   mode 3: W = [q | k | v] heads x head_dim rows; q and k are rotated with the per-token (cos, sin) table, q goes
//     to q_out and k, v into the paged cache; C is not used. bn must be a multiple of head_dim (64 or 128).
// These epilogues belong to the tile kernel: K is never split over a cluster here.
SP_API int sp_tc_gemm_n_tiles(int N, int bn) { return bn > 0 ? (N + bn - 1) / bn : 0; }

static int tc_gemm_any(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                       int mode, int bn, const EpiArgs* epp, int* status, cudaStream_t stream);

// CTAs that would share a tile along K in sp_tc_gemm for these sizes (1: none): the host asks before it chooses
// between a fused epilogue (never split) and the plain one followed by a small kernel.
SP_API int sp_tc_gemm_splits(int M, int N, int K, int bn) { return pick_splits(M, N, K, bn == 192 ? 256 : bn); }

// From this many rows of A on, tiles are computed by pairs of CTAs (cta_group::2); 0: never.
static int pairs_from = 1024;
SP_API void sp_tc_gemm_set_pairs_from(int rows) { pairs_from = rows; }

SP_API int sp_tc_gemm_fused(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw,
                            int ldc, int mode, int bn, const void* ep, int* status, cudaStream_t stream) {
    return tc_gemm_any(A, W, C, c_dt, M, N, K, lda, ldw, ldc, mode, bn, (const EpiArgs*)ep, status, stream);
}

// mode 0: C = A·Wᵀ (C bfloat16 or float32); 1: C (float32) += A·Wᵀ;
// mode 2: W holds gate and up rows interleaved in blocks of bn/2 and C [M, N/2] = silu(gate)·up.
SP_API int sp_tc_gemm(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                      int mode, int bn, int* status, cudaStream_t stream) {
    if (mode == MODE_QKV_ROPE) SP_FAIL("tc_gemm: the rotate-and-store epilogue needs sp_tc_gemm_fused");
    return tc_gemm_any(A, W, C, c_dt, M, N, K, lda, ldw, ldc, mode, bn, nullptr, status, stream);
}

static int tc_gemm_any(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                       int mode, int bn, const EpiArgs* epp, int* status, cudaStream_t stream) {
    EpiArgs ep;
    memset(&ep, 0, sizeof(ep));
    if (epp) ep = *epp;
    const bool fused = ep.row_ssq || ep.xw || mode == MODE_QKV_ROPE;
    if (M <= 0 || N <= 0) return 0;
    if (sp_tc_gemm_supported(A, W, K, lda, ldw)) return 1;
    if (mode == MODE_ACCUMULATE && c_dt != SP_DT_F32) SP_FAIL("tc_gemm: accumulation needs a float32 C");
    if (mode < 0 || mode > 3) SP_FAIL("tc_gemm: unknown mode %d", mode);
    if (bn != 128 && bn != 192 && bn != 256) SP_FAIL("tc_gemm: tile width %d is not built (128, 192 or 256)", bn);
    if (!fused && bn == 192 && pick_splits(M, N, K, bn) > 1) bn = 256;      // the kernel that splits K is built for 128 and 256
    if (ep.row_ssq && (ep.n_ssq <= 0 || ep.norm_width <= 0)) SP_FAIL("tc_gemm: the row statistics need their count and the norm's width");
    if (ep.xw && (mode != MODE_ACCUMULATE || !ep.next_w || !ep.ssq_out))
        SP_FAIL("tc_gemm: preparing the next norm's input belongs to the accumulating epilogue and needs its weight and a place for the sums");
    if (mode == MODE_QKV_ROPE) {
        if ((ep.hd != 64 && ep.hd != 128) || (bn % ep.hd)) SP_FAIL("tc_gemm: the rotate-and-store epilogue is built for head sizes 64 and 128 in tiles of whole heads (head %d, tile %d)", ep.hd, bn);
        if (ep.nh <= 0 || ep.nkv <= 0 || N != (ep.nh + 2 * ep.nkv) * ep.hd) SP_FAIL("tc_gemm: W has %d rows, %d q and %d kv heads of %d need %d", N, ep.nh, ep.nkv, ep.hd, (ep.nh + 2 * ep.nkv) * ep.hd);
        if (!ep.cs || !ep.tok_page || !ep.positions || !ep.q_out || !ep.kpool || !ep.vpool || ep.page_size <= 0)
            SP_FAIL("tc_gemm: the rotate-and-store epilogue needs the angle table, the tokens' pages and positions, q and the cache");
        if (((uintptr_t)ep.q_out | (uintptr_t)ep.kpool | (uintptr_t)ep.vpool | (uintptr_t)ep.cs) & 15)
            SP_FAIL("tc_gemm: q, the cache and the angle table must start on a 16-byte boundary");
    }
    if (mode == MODE_SILU_MUL && (N % bn)) SP_FAIL("tc_gemm: the fused silu epilogue needs N (%d) to be a multiple of the tile width %d", N, bn);
    CUtensorMap ma, mw;
    if (make_map(&ma, A, M, K, lda, BM)) return 1;
    // a prompt's worth of rows: pairs of CTAs on tiles of 256 rows, each fetching half of the W tile
    if (pairs_from > 0 && M >= pairs_from) {
        if (make_map(&mw, W, N, K, ldw, bn / 2)) return 1;
        if (bn == 128) return launch_pair<128, 8>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream, ep);
        if (bn == 192) return launch_pair<192, 7>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream, ep);
        return launch_pair<256, 6>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream, ep);
    }
    if (make_map(&mw, W, N, K, ldw, bn)) return 1;
    const int splits = fused ? 1 : pick_splits(M, N, K, bn);
    if (splits > 1) {
        if (bn == 128) return launch_splitk<128, 6>(ma, mw, C, c_dt, M, N, K, ldc, mode, splits, status, stream);
        return launch_splitk<256, 4>(ma, mw, C, c_dt, M, N, K, ldc, mode, splits, status, stream);
    }
    if (bn == 128) return launch<128, 6>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream, ep);
    if (bn == 192) return launch<192, 5>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream, ep);
    return launch<256, 4>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream, ep);
}
