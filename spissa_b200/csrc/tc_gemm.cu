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
#include "tcgen05.cuh"

SP_API const char* sp_tc_gemm_last_error() { return sp_error_text; }

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                      // 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SILU_MUL = 2 };

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024;      // + slack to align to 1024
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
template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ C, int c_dt, int M, int N, int K, int ldc, int mode, int* status) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_slot;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 4);          // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // two accumulators, each at a power-of-two column (tensor memory is handed out in powers of two)
    constexpr uint32_t ACC_STRIDE = BN <= 128 ? 128u : 256u, TMEM_COLS = 2u * ACC_STRIDE;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t kbc = 0;                                   // pipeline slots used so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++kbc) {
                    const int s = kbc % STAGES;
                    const uint32_t phase = (kbc / STAGES) & 1u;
                    ok = mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1u, status, 101);
                    if (!ok) break;
                    const uint32_t a_dst = smem_base + s * L::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + L::A_BYTES;
                    mbar_expect_tx(smem_u32(&bar_full[s]), L::STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * BK, m0, smem_u32(&bar_full[s]));
                    tma_load_2d(b_dst, &map_w, kb * BK, n0, smem_u32(&bar_full[s]));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
            uint32_t kbc = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
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
                        tc_mma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&bar_empty[s]));
                }
                tc_commit(smem_u32(&bar_acc_full[buf]));        // also after a failed wait: the epilogue must not hang
            }
        }
    } else {
        const int q = warp & 3;                      // this warp may touch tensor-memory lanes 32q .. 32q+31
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const uint32_t buf = it & 1u, use = it >> 1;
            const bool ok = mbar_wait(smem_u32(&bar_acc_full[buf]), use & 1u, status, 103);
            tc_fence_after();
            if (!ok || (status && *(volatile int*)status != 0)) break;
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + buf * ACC_STRIDE + ((uint32_t)(q * 32) << 16);
            constexpr int SPAN = 32;
            const int c_end = (mode == MODE_SILU_MUL) ? BN / 2 : BN;
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
                        const float g = __uint_as_float(r[j]);
                        v[j] = (g / (1.0f + expf(-g))) * __uint_as_float(u[j]);
                    }
                } else {
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                }
                if (c0 + SPAN >= c_end) {            // all of this tile has left tensor memory: hand the buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
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
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- few tokens: K split over a cluster
// With at most 128 tokens there is one row of tiles, too few CTAs to pull W from memory at full speed. Here
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
    const int n0 = (blockIdx.x / splits) * BN;
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
                tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, 0, smem_u32(&bar_full[s]));
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
    const int row = q * 32 + lane;
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
                if (row < M) store_row32(C, c_dt, (size_t)row * ldc + n0 / 2 + c0, n0 / 2 + c0, N / 2, v, false);
            } else if (row < M) {
                store_row32(C, c_dt, (size_t)row * ldc + n0 + c0, n0 + c0, N, v, mode == MODE_ACCUMULATE);
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
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
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

template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int c_dt, int M, int N, int K, int ldc, int mode,
           int* status, cudaStream_t stream) {
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
    tc_gemm_kernel<BN, STAGES><<<grid, 192, L::TOTAL, stream>>>(ma, mw, C, c_dt, M, N, K, ldc, mode, status);
    SP_CHECK_LAUNCH("tc_gemm");
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
    const int n_tiles = (N + BN - 1) / BN;
    SP_CHECK_CALL("tc_gemm_splitk", sp_launch_cluster(tc_gemm_splitk_kernel<BN, STAGES>, dim3(n_tiles * splits), dim3(192),
                                                     (size_t)L::TOTAL, stream, splits, ma, mw, C, c_dt, M, N, K, ldc,
                                                     mode, splits, status));
    return 0;
}

// How many CTAs share one tile along K: only for a single row of few tiles. Measured at 64 tokens on B200:
// two CTAs help a little for K = 2048 (15.6 -> 13.6 us for 24 tiles), four halve the time for K = 8192
// (41.6 -> 20.1 us for 16 tiles), eight are slower than one, and with 64 tiles or more splitting only hurts.
int pick_splits(int M, int N, int K, int bn) {
    if (M > BM) return 1;
    const int n_tiles = (N + bn - 1) / bn;
    const int num_kb = (K + BK - 1) / BK;
    if (n_tiles > 32) return 1;
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

// mode 0: C = A·Wᵀ (C bfloat16 or float32); 1: C (float32) += A·Wᵀ;
// mode 2: W holds gate and up rows interleaved in blocks of bn/2 and C [M, N/2] = silu(gate)·up.
SP_API int sp_tc_gemm(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda, int ldw, int ldc,
                      int mode, int bn, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (sp_tc_gemm_supported(A, W, K, lda, ldw)) return 1;
    if (mode == MODE_ACCUMULATE && c_dt != SP_DT_F32) SP_FAIL("tc_gemm: accumulation needs a float32 C");
    if (mode < 0 || mode > 2) SP_FAIL("tc_gemm: unknown mode %d", mode);
    if (bn != 128 && bn != 192 && bn != 256) SP_FAIL("tc_gemm: tile width %d is not built (128, 192 or 256)", bn);
    if (bn == 192 && pick_splits(M, N, K, bn) > 1) bn = 256;      // the kernel that splits K is built for 128 and 256
    if (mode == MODE_SILU_MUL && (N % bn)) SP_FAIL("tc_gemm: the fused silu epilogue needs N (%d) to be a multiple of the tile width %d", N, bn);
    CUtensorMap ma, mw;
    if (make_map(&ma, A, M, K, lda, BM)) return 1;
    if (make_map(&mw, W, N, K, ldw, bn)) return 1;
    const int splits = pick_splits(M, N, K, bn);
    if (splits > 1) {
        if (bn == 128) return launch_splitk<128, 6>(ma, mw, C, c_dt, M, N, K, ldc, mode, splits, status, stream);
        return launch_splitk<256, 4>(ma, mw, C, c_dt, M, N, K, ldc, mode, splits, status, stream);
    }
    if (bn == 128) return launch<128, 6>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream);
    if (bn == 192) return launch<192, 5>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream);
    return launch<256, 4>(ma, mw, C, c_dt, M, N, K, ldc, mode, status, stream);
}
