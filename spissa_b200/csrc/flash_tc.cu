// Causal prefill attention on the 5th-generation tensor cores, over the paged bfloat16 cache.
//
// Meaning as in the reference (crates/spissa-runtime/src/rotary.rs:335-415, softmax :549-569):
// score = q·k / sqrt(head_dim), keys after the query are not seen, softmax in 32-bit with the maximum
// subtracted, output = sum p·v, query head h reads kv head h / (heads / kv_heads).
//
// One CTA owns 128 consecutive query tokens of one head and walks the keys page by page (64 keys):
//   warp 0   one thread fetches the query tile once and a K page and a V page per block with TMA (128-byte
//            swizzle) into a four-stage ring;
//   warp 1   one thread issues S = Q·Kᵀ (tcgen05.mma, M 128, N 64, A and B from shared memory) into one of TWO
//            score buffers in tensor memory, one block ahead of the softmax, and, once a block's probabilities
//            stand in tensor memory, O += P·V (A = P from tensor memory, B = V as an MN-major operand);
//   warps 2-5 one thread per query row: the row's 64 scores into registers (tcgen05.ld), maximum and sum in the
//            log2 domain, P as bfloat16 pairs over the first half of the score buffer it came from
//            (tcgen05.st). The reference maximum of a row only moves when the block's maximum exceeds it by
//            more than 2^8 (then O's row and the sum are rescaled, after the product before it has finished);
//            until then probabilities may be as large as 256, which bfloat16 and the 32-bit sum hold, and the
//            final division by the sum is exact about it. Keys are masked only in blocks that reach beyond
//            the tile's first query.
// Tensor memory: S0 64 columns, S1 64, O 64 of 256 allocated: two CTAs per SM, so that one CTA's softmax runs
// under the other's products. Heavy tiles (late queries, many keys) are launched first. Every mbarrier wait is
// bounded; a wait that runs out records a code in ``status`` and every role falls through to the common exit,
// where tensor memory is freed. No load uses cluster multicast. Built for head size 64 without a window; the
// host refuses anything else (the mma.sync kernel serves those).
#include "tcgen05.cuh"

SP_API const char* sp_flash_tc_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(flash_tc)

namespace {

constexpr int QT = 128;            // query rows per CTA
constexpr int KB = 64;             // keys per block = one page
constexpr int PAGE = 64;
// key/value stages: with the query tile 81 KB (head 64) or 97 KB (head 128) per CTA, so that two CTAs share an SM
template <int HD> __host__ __device__ constexpr int kv_stages() { return HD == 64 ? 4 : 2; }
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;   // the reference maximum follows the true one in steps of at least this (log2 units)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Operands lie in shared memory as boxes of 64 columns (one 128-byte swizzle span): a query tile is HD / 64 boxes of
// 128 rows, a K or V page HD / 64 boxes of 64 rows.
template <int HD>
struct Smem {
    static constexpr int BOXES = HD / 64;
    static constexpr int Q_BOX = QT * 128, KV_BOX = KB * 128;    // bytes
    static constexpr int Q_BYTES = BOXES * Q_BOX;
    static constexpr int K_BYTES = BOXES * KV_BOX;
    static constexpr int STAGE_BYTES = 2 * K_BYTES;              // K page then V page
    static constexpr int TOTAL = Q_BYTES + kv_stages<HD>() * STAGE_BYTES + 1024;
};

template <int HD>
__global__ void __launch_bounds__(192)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ seq_start, const int* __restrict__ positions,
                        const int* __restrict__ seq_row, const int* __restrict__ page_table, int max_pages,
                        int n_seqs, int nh, int nkv, float scale_log2, int* status, SpRange rg) {
    static_assert(HD == 64 || HD == 128, "scores 2 x 64 columns and the output HD columns of 256 in tensor memory");
    using L = Smem<HD>;
    constexpr int KV_STAGES = kv_stages<HD>();
    constexpr uint32_t TMEM_COLS = 256;                           // S0 64 | S1 64 | O HD
    constexpr uint32_t COL_S = 0, COL_O = 128;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_q, bar_kv_full[KV_STAGES], bar_kv_empty[KV_STAGES], bar_s[2], bar_p[2], bar_o, bar_done;
    __shared__ uint32_t tmem_slot;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;
    const uint32_t kv_smem = smem_base + L::Q_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which sequence and which 128-token tile of it. Heads run fastest over the grid and tiles from the last to the
    // first, so that the tiles with the most keys start first in every head and the short ones fill the end.
    int x = (int)gridDim.y - 1 - (int)blockIdx.y, b = 0, first = 0, n_new = 0;
    for (; b < n_seqs; ++b) {
        first = seq_start[b];
        n_new = seq_start[b + 1] - first;
        const int nt = (n_new + QT - 1) / QT;
        if (x < nt) break;
        x -= nt;
    }
    const bool live = b < n_seqs;
    const int t0 = live ? first + x * QT : 0;
    const int n_rows = live ? min(QT, n_new - x * QT) : 0;
    const int pos0 = live ? positions[t0] : 0;
    const int h = blockIdx.x;
    const int g = h / (nh / nkv);
    const int n_blocks = live ? (pos0 + n_rows - 1) / KB + 1 : 0;
    const int* pt = page_table + (size_t)(live ? sp_checked_row(seq_row[b], rg) : 0) * max_pages;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar_q), 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(smem_u32(&bar_kv_full[s]), 1);
            mbar_init(smem_u32(&bar_kv_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_s[0]), 1);
        mbar_init(smem_u32(&bar_s[1]), 1);
        // one arrival per softmax warp. Two of them, by block parity: a row warp may be one block ahead of the others
        // (the next block's scores are there early), and its arrival must not count for the block they are still on.
        mbar_init(smem_u32(&bar_p[0]), 4);
        mbar_init(smem_u32(&bar_p[1]), 4);
        mbar_init(smem_u32(&bar_o), 1);
        mbar_init(smem_u32(&bar_done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    // set up; from here on the kernel reads what its predecessor in the stream wrote (q, the cache)
    sp_allow_dependents();
    sp_wait_for_predecessor();

    if (warp == 0) {
        if (lane == 0 && live) {
            mbar_expect_tx(smem_u32(&bar_q), L::Q_BYTES);
#pragma unroll
            for (int c = 0; c < L::BOXES; ++c) tma_load_2d(q_smem + c * L::Q_BOX, &map_q, h * HD + c * 64, t0, smem_u32(&bar_q));
            for (int j = 0; j < n_blocks; ++j) {
                const int s = j % KV_STAGES;
                const uint32_t phase = (uint32_t)(j / KV_STAGES) & 1u;
                if (!mbar_wait(smem_u32(&bar_kv_empty[s]), phase ^ 1u, status, 111)) break;
                const uint32_t k_dst = kv_smem + s * L::STAGE_BYTES, v_dst = k_dst + L::K_BYTES;
                mbar_expect_tx(smem_u32(&bar_kv_full[s]), L::STAGE_BYTES);
                const int r0 = (sp_checked_page(pt[sp_checked_entry(j, max_pages, rg)], rg) * nkv + g) * PAGE;
#pragma unroll
                for (int c = 0; c < L::BOXES; ++c) {
                    tma_load_2d(k_dst + c * L::KV_BOX, &map_k, c * 64, r0, smem_u32(&bar_kv_full[s]));
                    tma_load_2d(v_dst + c * L::KV_BOX, &map_v, c * 64, r0, smem_u32(&bar_kv_full[s]));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && live) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(QT, KB);            // S[128,64] = Q·Kᵀ, both K-major
            constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(QT, HD);        // O[128,HD] += P·V, V MN-major
            bool ok = mbar_wait(smem_u32(&bar_q), 0, status, 112);
            auto issue_s = [&](int j) -> bool {
                const int s = j % KV_STAGES;
                if (!mbar_wait(smem_u32(&bar_kv_full[s]), (uint32_t)(j / KV_STAGES) & 1u, status, 113)) return false;
                tc_fence_after();
                const uint32_t d = tmem + COL_S + (uint32_t)(j & 1) * KB;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    // 16 of head_dim further: +2 (16-byte units) inside a box, the next box after four steps
                    const uint64_t dq = umma_desc_sw128(q_smem + (k / 4) * L::Q_BOX) + 2 * (k % 4);
                    const uint64_t dk = umma_desc_sw128(kv_smem + s * L::STAGE_BYTES + (k / 4) * L::KV_BOX) + 2 * (k % 4);
                    tc_mma_bf16(d, dq, dk, idesc_s, k != 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&bar_s[j & 1]));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                // The next block's scores go to the other buffer while the softmax works on this one. That buffer
                // still holds the probabilities of block j-1 for the product issued before: the pipe runs in order.
                if (j + 1 < n_blocks) ok = issue_s(j + 1);
                if (!ok) break;
                ok = mbar_wait(smem_u32(&bar_p[j & 1]), (uint32_t)(j >> 1) & 1u, status, 114);
                if (!ok) break;
                tc_fence_after();
                const int s = j % KV_STAGES;
                const uint32_t v_src = kv_smem + s * L::STAGE_BYTES + L::K_BYTES;
                const uint32_t p_src = tmem + COL_S + (uint32_t)(j & 1) * KB;
#pragma unroll
                for (int k = 0; k < KB / 16; ++k) {
                    // 16 keys further along K: two groups of 8 rows of 128 bytes = 2048 bytes; P: 8 columns; the next 64
                    // of head_dim lie one box further
                    tc_mma_bf16_ts(tmem + COL_O, p_src + 8 * k, umma_desc_mn_sw128(v_src + k * 2048, L::KV_BOX),
                                   idesc_o, (j | k) != 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&bar_kv_empty[s]));
                tc_commit(smem_u32(&bar_o));
                if (j == n_blocks - 1) tc_commit(smem_u32(&bar_done));      // the last product: a barrier of its own
            }
        }
    } else if (live) {
        const int q = warp & 3;                                   // tensor-memory lanes 32q .. 32q+31
        const int row = q * 32 + lane;
        const int qpos = pos0 + row;
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        float m = -INFINITY, l = 0.0f;                            // reference maximum (log2 units) and sum
        bool ok = true;
        for (int j = 0; j < n_blocks; ++j) {
            ok = mbar_wait(smem_u32(&bar_s[j & 1]), (uint32_t)(j >> 1) & 1u, status, 115);
            if (!ok) break;
            tc_fence_after();
            const uint32_t s_addr = lane_base + COL_S + (uint32_t)(j & 1) * KB;
            uint32_t r[KB];
            tc_ld_32x32(s_addr, r);
            tc_ld_32x32(s_addr + 32, r + 32);
            tc_ld_wait();
            const int key0 = j * KB;
            if (key0 + KB - 1 > pos0) {                           // some row of the tile cannot see some key of the block
#pragma unroll
                for (int i = 0; i < KB; ++i)
                    if (key0 + i > qpos) r[i] = 0xff800000u;      // -inf
            }
            // four chains each for the maximum and the sum: one chain of 64 dependent operations would cost more
            // than the exponentials
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < KB; i += 4) {
                mx4[0] = fmaxf(mx4[0], __uint_as_float(r[i]));
                mx4[1] = fmaxf(mx4[1], __uint_as_float(r[i + 1]));
                mx4[2] = fmaxf(mx4[2], __uint_as_float(r[i + 2]));
                mx4[3] = fmaxf(mx4[3], __uint_as_float(r[i + 3]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // move the reference only when it is far behind (or not set yet)
            const bool move = mx > m + RESCALE_STEP || (m == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, move)) {
                const float m_new = move ? mx : m;
                const float corr = (m == -INFINITY) ? 0.0f : ex2(m - m_new);      // 1 for rows that stay
                if (j > 0) {
                    // O's row may only be touched once the product before has finished with it
                    ok = mbar_wait(smem_u32(&bar_o), (uint32_t)(j - 1) & 1u, status, 116);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t o[32];
                        tc_ld_32x32(lane_base + COL_O + c0, o);
                        tc_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tc_st_32x32(lane_base + COL_O + c0, o);
                    }
                }
                l *= corr;
                m = m_new;
            }
            const float m_safe = (m == -INFINITY) ? 0.0f : m;
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t pk[KB / 2];
#pragma unroll
            for (int i = 0; i < KB; i += 2) {
                const float p0 = ex2(fmaf(__uint_as_float(r[i]), scale_log2, -m_safe));
                const float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), scale_log2, -m_safe));
                sum4[(i >> 1) & 3] += p0 + p1;
                __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
                pk[i >> 1] = *(uint32_t*)&pr;
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            tc_st_32x32(s_addr, pk);                              // P over the first half of the scores it came from
            tc_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_p[j & 1]));
        }
        // The last product has a barrier of its own, with this one phase. On bar_o a wait by parity cannot tell the
        // product before the last (a row warp may be a block ahead of the others, so that one may not even be issued)
        // from the last (which may be complete before a slow warp, say one that misses the instruction cache on
        // its way out of the loop, gets to wait: its parity has then come round and the wait never ends).
        if (ok && n_blocks > 0) ok = mbar_wait(smem_u32(&bar_done), 0, status, 117);
        tc_fence_after();
        if (ok && !(status && *(volatile int*)status != 0)) {
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = out + (size_t)(t0 + row) * nh * HD + (size_t)h * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t r[32];
                tc_ld_32x32(lane_base + COL_O + c0, r);
                tc_ld_wait();
                if (row < n_rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        w.x = *(uint32_t*)&a0; w.y = *(uint32_t*)&a1; w.z = *(uint32_t*)&a2; w.w = *(uint32_t*)&a3;
                        *(uint4*)(dst + c0 + i) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
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

// rows x cols bfloat16 with leading dimension ld, fetched in boxes of box_rows x 64 columns
int make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) SP_FAIL("flash_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) SP_FAIL("flash_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

}  // namespace

// Whether this kernel takes the shape (1) or another attention kernel has to run (0).
// Query rows per CTA: the host counts tiles (the grid) with it.
SP_API int sp_flash_tc_query_tile() { return QT; }

SP_API int sp_flash_tc_supported(int hd, int nh, int nkv, int page_size, int window) {
    return (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && page_size == PAGE && window <= 0;
}

// q, out: [T, nh*hd] bfloat16; pools: [n_pages, nkv, 64, hd] bfloat16; n_q_tiles = sum over sequences of
// ceil(new tokens / 128).
SP_API int sp_flash_prefill_tc(const void* q, void* out, const void* kpool, const void* vpool, long long n_pages,
                               int T, const int* seq_start, const int* positions, const int* seq_row,
                               const int* page_table, int max_pages, int page_size, int n_seqs, int n_q_tiles, int nh,
                               int nkv, int hd, int window, float scale, int* status, cudaStream_t stream) {
    if (n_q_tiles <= 0) return 0;
    if (!sp_flash_tc_supported(hd, nh, nkv, page_size, window))
        SP_FAIL("flash_tc: built for head sizes 64 and 128, pages of 64 and no window (got head %d, page %d, window %d)", hd, page_size, window);
    if (((uintptr_t)q & 15) || ((uintptr_t)kpool & 15) || ((uintptr_t)vpool & 15) || ((uintptr_t)out & 15))
        SP_FAIL("flash_tc: operands must start on a 16-byte boundary");
    CUtensorMap mq, mk, mv;
    if (make_map(&mq, q, T, nh * hd, (long long)nh * hd, QT)) return 1;
    if (make_map(&mk, kpool, n_pages * nkv * PAGE, hd, hd, PAGE)) return 1;
    if (make_map(&mv, vpool, n_pages * nkv * PAGE, hd, hd, PAGE)) return 1;
    if (n_q_tiles > 65535) SP_FAIL("flash_tc: %d query tiles are beyond this kernel's grid", n_q_tiles);
    dim3 grid(nh, n_q_tiles);
    static SpPerDevice configured[2];
    if (hd == 64) {
        if (!configured[0].done()) {
            cudaError_t e = cudaFuncSetAttribute(flash_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<64>::TOTAL);
            if (e != cudaSuccess) SP_FAIL("flash_tc: cannot reserve %d bytes of shared memory: %s", Smem<64>::TOTAL, cudaGetErrorString(e));
            configured[0].mark();
        }
        SP_CHECK_CALL("flash_prefill_tc", sp_launch_dependent(flash_prefill_tc_kernel<64>, grid, dim3(192), (size_t)Smem<64>::TOTAL, stream,
            mq, mk, mv, (__nv_bfloat16*)out, seq_start, positions, seq_row, page_table, max_pages, n_seqs, nh, nkv,
            scale * LOG2E, status, sp_range_host));
    } else {
        if (!configured[1].done()) {
            cudaError_t e = cudaFuncSetAttribute(flash_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<128>::TOTAL);
            if (e != cudaSuccess) SP_FAIL("flash_tc: cannot reserve %d bytes of shared memory: %s", Smem<128>::TOTAL, cudaGetErrorString(e));
            configured[1].mark();
        }
        SP_CHECK_CALL("flash_prefill_tc", sp_launch_dependent(flash_prefill_tc_kernel<128>, grid, dim3(192), (size_t)Smem<128>::TOTAL, stream,
            mq, mk, mv, (__nv_bfloat16*)out, seq_start, positions, seq_row, page_table, max_pages, n_seqs, nh, nkv,
            scale * LOG2E, status, sp_range_host));
    }
    SP_CHECK_LAUNCH("flash_prefill_tc");
    return 0;
}
