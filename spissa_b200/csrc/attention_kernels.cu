// Causal grouped-query attention over the paged cache for bfloat16 storage: a prefill kernel
// (many query tokens per sequence) and a decode kernel (one query token per sequence, keys
// split over CTAs, then combined).
//
// Meaning as in the reference (crates/spissa-runtime/src/rotary.rs:335-415, softmax :549-569):
// score = q·k / sqrt(head_dim); keys after the query are not seen (nor keys before
// pos-window+1 when a window is set); softmax in 32-bit with the maximum subtracted;
// output = sum p·v; query head h reads kv head h / (heads / kv_heads).
//
// Both kernels walk the keys in tiles of 64 = one cache page ([page][kv head][64][head_dim],
// so a tile is one contiguous block), staged in shared memory with cp.async, double
// buffered. Products run on mma.sync m16n8k16 (bfloat16 in, float32 out); the running
// maximum, sum and output stay in float32 registers (online softmax in the log2 domain).
// Prefill: a CTA owns 64 consecutive query tokens of one head; each of its 4 warps owns 16.
// Decode: a CTA owns the query heads of one kv head of one sequence (as the 16 rows of one
// tile, unused rows zero) for one chunk of key tiles; each warp takes 16 keys of every tile.
// Keys that no query may see are masked whatever the cache holds there; the cache is
// zero-initialised so that a masked weight of zero never meets a NaN value.
#include "flash_common.cuh"

SP_API const char* sp_attention_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(attention)

namespace {

constexpr int DEC_STAGES = 3;                 // tiles in flight per warp of the decode kernel

// ------------------------------------------------------------------ prefill
template <int HD>
__global__ void __launch_bounds__(128)
flash_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, PagedKV kv,
                     const int* __restrict__ seq_start, const int* __restrict__ positions, int n_seqs, int nh,
                     int window, float scale_log2) {
    using T = Tile<HD>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_tile = smem_u32(smem);
    const uint32_t k_tiles = q_tile + T::BYTES;          // two stages of K, then two of V
    const uint32_t v_tiles = k_tiles + 2 * T::BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    sp_allow_dependents();
    sp_wait_for_predecessor();

    // which sequence and which 64-token tile of it. Heads run fastest over the grid and tiles from the last to the
    // first: the tiles with the most keys start first in every head, the short ones fill the end.
    int x = (int)gridDim.y - 1 - (int)blockIdx.y, b = 0, first = 0, n_new = 0;
    for (; b < n_seqs; ++b) {
        first = seq_start[b];
        n_new = seq_start[b + 1] - first;
        const int nt = (n_new + KT - 1) / KT;
        if (x < nt) break;
        x -= nt;
    }
    if (b >= n_seqs) return;
    const int t0 = first + x * KT;
    const int n_rows = min(KT, n_new - x * KT);
    const int pos0 = positions[t0];
    const int h = blockIdx.x;
    const int g = h / (nh / kv.nkv);
    const int* pt = kv.page_table + (size_t)sp_checked_row(kv.seq_row[b], kv.rg) * kv.max_pages;

    const int last_pos = pos0 + n_rows - 1;
    const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int j_lo = first_key / KT, j_hi = last_pos / KT;

    load_tile_async<HD>(q_tile, q + (size_t)t0 * nh * HD + (size_t)h * HD, (size_t)nh * HD, n_rows, tid, 128);
    {
        const size_t off = ((size_t)sp_checked_page(pt[sp_checked_entry(j_lo, kv.max_pages, kv.rg)], kv.rg) * kv.nkv + g) * KT * HD;
        load_tile_async<HD>(k_tiles, kv.k + off, HD, KT, tid, 128);
        load_tile_async<HD>(v_tiles, kv.v + off, HD, KT, tid, 128);
    }
    cp_async_commit();

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const int r0 = warp * 16 + (lane >> 2);
    const int hi[2] = {pos0 + r0, pos0 + r0 + 8};
    const int lo[2] = {window > 0 ? hi[0] - window + 1 : 0, window > 0 ? hi[1] - window + 1 : 0};
    const int warp_hi = pos0 + warp * 16 + 15;                     // last key any row of this warp may see
    const int warp_lo = window > 0 ? pos0 + warp * 16 - window + 1 : 0;
    const bool warp_active = warp * 16 < n_rows;

    for (int j = j_lo; j <= j_hi; ++j) {
        const int stage = (j - j_lo) & 1;
        if (j < j_hi) {
            const size_t off = ((size_t)sp_checked_page(pt[sp_checked_entry(j + 1, kv.max_pages, kv.rg)], kv.rg) * kv.nkv + g) * KT * HD;
            load_tile_async<HD>(k_tiles + (stage ^ 1) * T::BYTES, kv.k + off, HD, KT, tid, 128);
            load_tile_async<HD>(v_tiles + (stage ^ 1) * T::BYTES, kv.v + off, HD, KT, tid, 128);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (j == j_lo) load_q_frags<HD>(q_tile, warp * 16, lane, qf);
        const int tile_pos0 = j * KT;
        if (warp_active && tile_pos0 <= warp_hi && tile_pos0 + KT - 1 >= warp_lo) {
            // every key of the tile is at or before the warp's first row and inside its last row's window
            const bool all_seen = tile_pos0 + KT - 1 <= pos0 + warp * 16 && (window <= 0 || tile_pos0 >= warp_hi - window + 1);
            if (all_seen)
                flash_step<HD, 8, false>(qf, k_tiles + stage * T::BYTES, v_tiles + stage * T::BYTES, 0, tile_pos0, lo, hi,
                                         scale_log2, o, m, l, lane);
            else
                flash_step<HD, 8, true>(qf, k_tiles + stage * T::BYTES, v_tiles + stage * T::BYTES, 0, tile_pos0, lo, hi,
                                        scale_log2, o, m, l, lane);
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    const int t = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row >= n_rows) continue;
        const float inv = 1.0f / l[r];
        __nv_bfloat16* dst = out + (size_t)(t0 + row) * nh * HD + (size_t)h * HD;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i)
            *(uint32_t*)(dst + i * 8 + 2 * t) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

// The CTA that finishes last for a (sequence, kv head) combines all chunks of its G heads, in chunk
// order whatever the order of arrival, and hands the counter back at zero for the next launch.
template <int HD>
__device__ __forceinline__ void combine_if_last(const float* part_o, const float* part_ml, int* counters, void* out,
                                                int out_dt, int b, int g, int G, int nh, int nkv, int n_chunks,
                                                int* is_last) {
    __threadfence();                                    // this CTA's partials are visible before it is counted
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(&counters[b * nkv + g], 1);
        *is_last = (prev == n_chunks - 1);
        if (*is_last) counters[b * nkv + g] = 0;
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();
    for (int e = threadIdx.x; e < G * HD; e += blockDim.x) {
        const int row = e / HD, d = e % HD;
        const size_t bh = (size_t)b * nh + (size_t)g * G + row;
        float mm = -INFINITY;
        for (int c = 0; c < n_chunks; ++c) mm = fmaxf(mm, __ldcg(&part_ml[(bh * n_chunks + c) * 2]));
        const float msafe = (mm == -INFINITY) ? 0.0f : mm;
        float ll = 0.0f, acc = 0.0f;
        for (int c = 0; c < n_chunks; ++c) {
            const float lc = __ldcg(&part_ml[(bh * n_chunks + c) * 2 + 1]);
            if (lc > 0.0f) {
                const float f = exp2f(__ldcg(&part_ml[(bh * n_chunks + c) * 2]) - msafe);
                ll += lc * f;
                acc += __ldcg(&part_o[(bh * n_chunks + c) * HD + d]) * f;
            }
        }
        sp_st_dt(out, out_dt, bh * HD + d, acc / ll);
    }
}

// ------------------------------------------------------------------ decode
// grid (chunks, kv heads, sequences). part_o [B][nh][chunks][HD], part_ml [B][nh][chunks][2] (m in log2 units).
template <int HD, int NH>
__global__ void __launch_bounds__(128)
flash_decode_kernel(const __nv_bfloat16* __restrict__ q, PagedKV kv, const int* __restrict__ seq_len, int nh,
                    int window, float scale_log2, int chunk_tiles, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int* __restrict__ counters, void* __restrict__ out, int out_dt) {
    using T = Tile<HD>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_tile = smem_u32(smem);                       // 16 rows used
    const uint32_t k_tiles = q_tile + 16 * T::ROW;
    const uint32_t v_tiles = k_tiles + DEC_STAGES * T::BYTES;
    float* merge = (float*)(smem + 16 * T::ROW + 2 * DEC_STAGES * T::BYTES);    // [4 warps][16 rows][HD + 2]
    sp_allow_dependents();
    sp_wait_for_predecessor();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x, n_chunks = gridDim.x, g = blockIdx.y, b = blockIdx.z;
    const int G = nh / kv.nkv;
    const int p = seq_len[b] - 1;                                  // the query's position
    const int first_key = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int j_first = first_key / KT + chunk * chunk_tiles;
    const int j_last = min(p / KT, j_first + chunk_tiles - 1);
    const size_t part_base = ((size_t)b * nh + (size_t)g * G) * n_chunks + chunk;   // + head_in_group * n_chunks

    __shared__ int is_last;
    if (j_first > j_last) {                                        // nothing for this chunk
        for (int i = tid; i < G; i += 128) {
            part_ml[(part_base + (size_t)i * n_chunks) * 2] = -INFINITY;
            part_ml[(part_base + (size_t)i * n_chunks) * 2 + 1] = 0.0f;
        }
        if (counters) combine_if_last<HD>(part_o, part_ml, counters, out, out_dt, b, g, G, nh, kv.nkv, n_chunks, &is_last);
        return;
    }
    const int* pt = kv.page_table + (size_t)sp_checked_row(kv.seq_row[b], kv.rg) * kv.max_pages;

    // the G heads of this kv head as rows 0..G-1 of a 16-row tile
    for (int c = tid; c < 16 * T::CHUNKS; c += 128) {
        const int r = c / T::CHUNKS, k = c % T::CHUNKS;
        const uint32_t d = q_tile + r * T::ROW + k * 16;
        if (r < G) cp_async16(d, q + (size_t)b * nh * HD + (size_t)(g * G + r) * HD + k * 8);
        else asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(d), "r"(0u) : "memory");
    }
    cp_async_commit();                                             // group 0: the queries

    // keys are the M of the products, the group's heads their N, in NH tiles of 8 (decode_step_t)
    uint32_t qb[HD / 16][NH][2];
    float o[HD / 16][NH][4], m[NH][2], l[NH][2];
#pragma unroll
    for (int i = 0; i < NH; ++i) {
        m[i][0] = m[i][1] = -INFINITY;
        l[i][0] = l[i][1] = 0.0f;
#pragma unroll
        for (int dt = 0; dt < HD / 16; ++dt) o[dt][i][0] = o[dt][i][1] = o[dt][i][2] = o[dt][i][3] = 0.0f;
    }

    // Each warp fetches and uses only its own 16 keys of every tile, so inside the loop the warps
    // need no barrier among themselves: a warp waits for its own copies and goes on.
    auto fetch = [&](int j, int stage) {
        const size_t off = ((size_t)sp_checked_page(pt[sp_checked_entry(j, kv.max_pages, kv.rg)], kv.rg) * kv.nkv + g) * KT * HD + (size_t)warp * 16 * HD;
        const uint32_t kd = k_tiles + stage * T::BYTES + warp * 16 * T::ROW;
        const uint32_t vd = v_tiles + stage * T::BYTES + warp * 16 * T::ROW;
        for (int c = lane; c < 16 * T::CHUNKS; c += 32) {
            const int r = c / T::CHUNKS, k = c % T::CHUNKS;
            cp_async16(kd + r * T::ROW + k * 16, kv.k + off + (size_t)r * HD + k * 8);
            cp_async16(vd + r * T::ROW + k * 16, kv.v + off + (size_t)r * HD + k * 8);
        }
    };
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
        if (j_first + s <= j_last) fetch(j_first + s, s);
        cp_async_commit();
    }
    cp_async_wait<DEC_STAGES - 1>();                               // the queries have landed (all later groups may fly)
    __syncthreads();
    // Qᵀ as the B operand: lane (g, t) holds dims 2t, 2t+1 and 2t+8, 2t+9 of head g of each head tile
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
        for (int i = 0; i < NH; ++i) {
            const uint32_t a = q_tile + (i * 8 + (lane >> 2)) * T::ROW + (kk * 16 + 2 * (lane & 3)) * 2;
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(qb[kk][i][0]) : "r"(a));
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(qb[kk][i][1]) : "r"(a + 16));
        }

    for (int j = j_first; j <= j_last; ++j) {
        const int it = j - j_first;
        const int stage = it % DEC_STAGES;
        if (j + DEC_STAGES - 1 <= j_last) fetch(j + DEC_STAGES - 1, (it + DEC_STAGES - 1) % DEC_STAGES);
        cp_async_commit();
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        if (j * KT + KT - 1 <= p && j * KT >= first_key)
            decode_step_t<HD, NH, false>(qb, k_tiles + stage * T::BYTES, v_tiles + stage * T::BYTES, warp * 16, j * KT,
                                         first_key, p, scale_log2, o, m, l, lane);
        else
            decode_step_t<HD, NH, true>(qb, k_tiles + stage * T::BYTES, v_tiles + stage * T::BYTES, warp * 16, j * KT,
                                        first_key, p, scale_log2, o, m, l, lane);
        __syncwarp();                                              // the stage is free for this warp's next fetch
    }
    cp_async_wait<0>();

    // merge the four warps' (m, l, o): each covered other keys of the same rows
    constexpr int MS = HD + 2;
    const int lg = lane >> 2, lt = lane & 3;
#pragma unroll
    for (int i = 0; i < NH; ++i)
#pragma unroll
        for (int c = 0; c < 2; ++c) {                              // head 8i + 2·lt + c: dims lg and lg + 8 of every 16
            l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], 4);   // the lanes that share lt hold the head's other keys
            l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], 8);
            l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], 16);
            float* dst = merge + ((size_t)warp * 16 + i * 8 + 2 * lt + c) * MS;
#pragma unroll
            for (int dt = 0; dt < HD / 16; ++dt) {
                dst[dt * 16 + lg] = o[dt][i][c];
                dst[dt * 16 + lg + 8] = o[dt][i][c + 2];
            }
            if (lg == 0) { dst[HD] = m[i][c]; dst[HD + 1] = l[i][c]; }
        }
    __syncthreads();
    for (int e = tid; e < G * HD; e += 128) {
        const int row = e / HD, d = e % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[((size_t)w * 16 + row) * MS + HD]);
        const float msafe = (mm == -INFINITY) ? 0.0f : mm;
        float acc = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = merge + ((size_t)w * 16 + row) * MS;
            const float f = exp2f(src[HD] - msafe);
            acc += src[d] * f;
            ll += src[HD + 1] * f;
        }
        const size_t pi = part_base + (size_t)row * n_chunks;
        part_o[pi * HD + d] = acc;
        if (d == 0) { part_ml[pi * 2] = mm; part_ml[pi * 2 + 1] = ll; }
    }
    if (counters) combine_if_last<HD>(part_o, part_ml, counters, out, out_dt, b, g, G, nh, kv.nkv, n_chunks, &is_last);
}

// out[b, head, :] = sum_c o_c·2^(m_c - M) / sum_c l_c·2^(m_c - M), chunks in order
template <typename TO>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      TO* __restrict__ out, int n_chunks, int HD) {
    const size_t bh = blockIdx.x;
    float mm = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) mm = fmaxf(mm, part_ml[(bh * n_chunks + c) * 2]);
    const float msafe = (mm == -INFINITY) ? 0.0f : mm;
    float ll = 0.0f;
    for (int c = 0; c < n_chunks; ++c)
        ll += part_ml[(bh * n_chunks + c) * 2 + 1] * exp2f(part_ml[(bh * n_chunks + c) * 2] - msafe);
    const float inv = 1.0f / ll;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.0f;
        for (int c = 0; c < n_chunks; ++c) {
            const float lc = part_ml[(bh * n_chunks + c) * 2 + 1];
            if (lc > 0.0f) acc += part_o[(bh * n_chunks + c) * HD + d] * exp2f(part_ml[(bh * n_chunks + c) * 2] - msafe);
        }
        sp_st(out, bh * HD + d, acc * inv);
    }
}

template <int HD>
constexpr int prefill_smem() { return 5 * Tile<HD>::BYTES; }
template <int HD>
constexpr int decode_smem() { return 16 * Tile<HD>::ROW + 2 * DEC_STAGES * Tile<HD>::BYTES + 4 * 16 * (HD + 2) * 4; }

template <typename Kern>
int opt_in_smem(Kern kern, int bytes, const char* name) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) SP_FAIL("%s: cannot reserve %d bytes of shared memory: %s", name, bytes, cudaGetErrorString(e));
    return 0;
}

// Head sizes the kernels are instantiated for: every multiple of 16 up to 128 (the fragments of mma.sync are 16 wide;
// beyond 128 a thread's output row no longer fits its registers and the generic kernel runs).
#define SP_FLASH_HEAD_SIZES(X) X(16) X(32) X(48) X(64) X(80) X(96) X(112) X(128)

bool head_size_built(int hd) { return hd >= 16 && hd <= 128 && hd % 16 == 0; }

int check_common(int hd, int nh, int nkv, int page_size) {
    if (!head_size_built(hd)) SP_FAIL("flash attention: head_dim %d is not built (multiples of 16 up to 128 are)", hd);
    if (nkv <= 0 || nh % nkv) SP_FAIL("flash attention: %d heads are no multiple of %d kv heads", nh, nkv);
    if (page_size != KT) SP_FAIL("flash attention: pages of %d tokens, this kernel walks pages of %d", page_size, KT);
    return 0;
}

}  // namespace

// Whether the flash kernels are built for this shape (1) or the generic kernel has to run (0).
// Query rows per CTA of the prefill kernel (= the page size its key tiles have): the host counts tiles with it.
SP_API int sp_flash_query_tile() { return KT; }

SP_API int sp_flash_supported(int hd, int nh, int nkv, int page_size) {
    return head_size_built(hd) && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16 && page_size == KT;
}

namespace {
template <int HD>
int launch_flash_prefill_as(dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, __nv_bfloat16* out, const PagedKV& kv,
                            const int* seq_start, const int* positions, int n_seqs, int nh, int window, float sl) {
    static SpPerDevice ok;            // the opt-in holds for one device: asked for on each device's first launch
    if (!ok.done()) { if (opt_in_smem(flash_prefill_kernel<HD>, prefill_smem<HD>(), "flash_prefill")) return 1; ok.mark(); }
    sp_launch_dependent(flash_prefill_kernel<HD>, grid, dim3(128), (size_t)prefill_smem<HD>(), stream, q, out, kv, seq_start,
                        positions, n_seqs, nh, window, sl);
    return 0;
}
}  // namespace

SP_API int sp_flash_prefill(const void* q, void* out, const void* kpool, const void* vpool, const int* seq_start,
                            const int* positions, const int* seq_row, const int* page_table, int max_pages,
                            int page_size, int n_seqs, int n_q_tiles, int nh, int nkv, int hd, int window,
                            float scale, cudaStream_t stream) {
    if (n_q_tiles <= 0) return 0;
    if (check_common(hd, nh, nkv, page_size)) return 1;
    PagedKV kv{(const __nv_bfloat16*)kpool, (const __nv_bfloat16*)vpool, page_table, seq_row, max_pages, nkv, sp_range_host};
    if (n_q_tiles > 65535) SP_FAIL("flash_prefill: %d query tiles are beyond this kernel's grid", n_q_tiles);
    dim3 grid(nh, n_q_tiles);
    const float sl = scale * LOG2E;
    switch (hd) {
#define X(n)                                                                                                        \
    case n:                                                                                                         \
        if (launch_flash_prefill_as<n>(grid, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, kv, seq_start,   \
                                       positions, n_seqs, nh, window, sl)) return 1;                                \
        break;
        SP_FLASH_HEAD_SIZES(X)
#undef X
    }
    SP_CHECK_LAUNCH("flash_prefill");
    return 0;
}

namespace {
// One instantiation per head size and number of head tiles (query heads per kv head: up to 8, up to 16).
template <int HD, int NH>
int launch_flash_decode_as(dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, const PagedKV& kv, const int* seq_len,
                           int nh, int window, float sl, int chunk_tiles, float* part_o, float* part_ml, int* counters,
                           void* out, int out_dt) {
    static SpPerDevice ok;            // the opt-in holds for one device: asked for on each device's first launch
    if (!ok.done()) { if (opt_in_smem(flash_decode_kernel<HD, NH>, decode_smem<HD>(), "flash_decode")) return 1; ok.mark(); }
    sp_launch_dependent(flash_decode_kernel<HD, NH>, grid, dim3(128), (size_t)decode_smem<HD>(), stream, q, kv, seq_len, nh, window, sl,
                        chunk_tiles, part_o, part_ml, counters, out, out_dt);
    return 0;
}
int launch_flash_decode(int hd, dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, const PagedKV& kv,
                        const int* seq_len, int nh, int window, float sl, int chunk_tiles, float* part_o, float* part_ml,
                        int* counters, void* out, int out_dt) {
    const bool one = nh <= 8 * kv.nkv;
    switch (hd) {
#define X(n)                                                                                                              \
    case n:                                                                                                               \
        return one ? launch_flash_decode_as<n, 1>(grid, stream, q, kv, seq_len, nh, window, sl, chunk_tiles, part_o, part_ml, counters, out, out_dt) \
                   : launch_flash_decode_as<n, 2>(grid, stream, q, kv, seq_len, nh, window, sl, chunk_tiles, part_o, part_ml, counters, out, out_dt);
        SP_FLASH_HEAD_SIZES(X)
#undef X
    }
    SP_FAIL("flash decode: head_dim %d is not built", hd);
}

}  // namespace

// Floats of scratch the decode kernels need: part_o then part_ml. ``counters`` (optional, n_seqs·nkv ints,
// zero before the first launch; the kernel returns them to zero) lets the last CTA combine the chunks;
// without it a second kernel does.
SP_API long long sp_flash_decode_scratch_floats(int n_seqs, int nh, int hd, int n_chunks) {
    return (long long)n_seqs * nh * n_chunks * (hd + 2);
}

SP_API int sp_flash_decode(const void* q, void* out, int out_dt, const void* kpool, const void* vpool,
                           const int* seq_len, const int* seq_row, const int* page_table, int max_pages,
                           int page_size, int n_seqs, int nh, int nkv, int hd, int window, float scale,
                           int chunk_tiles, int n_chunks, float* scratch, long long scratch_floats, int* counters,
                           cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (check_common(hd, nh, nkv, page_size)) return 1;
    if (nh / nkv > 16) SP_FAIL("flash decode: %d query heads per kv head, at most 16 fit one tile", nh / nkv);
    if (chunk_tiles <= 0 || n_chunks <= 0 || n_chunks > 65535) SP_FAIL("flash decode: bad chunking %d x %d", n_chunks, chunk_tiles);
    if (n_seqs > 65535) SP_FAIL("flash decode: %d sequences are beyond this kernel's grid", n_seqs);
    const long long need = sp_flash_decode_scratch_floats(n_seqs, nh, hd, n_chunks);
    if (scratch_floats < need) SP_FAIL("flash decode: scratch holds %lld floats, %lld are needed", scratch_floats, need);
    PagedKV kv{(const __nv_bfloat16*)kpool, (const __nv_bfloat16*)vpool, page_table, seq_row, max_pages, nkv, sp_range_host};
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)n_seqs * nh * n_chunks * hd;
    dim3 grid(n_chunks, nkv, n_seqs);
    const float sl = scale * LOG2E;
    if (launch_flash_decode(hd, grid, stream, (const __nv_bfloat16*)q, kv, seq_len, nh, window, sl, chunk_tiles, part_o,
                            part_ml, counters, out, out_dt)) return 1;
    SP_CHECK_LAUNCH("flash_decode");
    if (counters) return 0;                  // the last CTA of every (sequence, kv head) has combined
    if (out_dt == SP_DT_BF16)
        decode_combine_kernel<__nv_bfloat16><<<n_seqs * nh, hd <= 64 ? 64 : 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, n_chunks, hd);
    else
        decode_combine_kernel<float><<<n_seqs * nh, hd <= 64 ? 64 : 128, 0, stream>>>(part_o, part_ml, (float*)out, n_chunks, hd);
    SP_CHECK_LAUNCH("decode_combine");
    return 0;
}

// ------------------------------------------------------------------ decode without a caller's scratch
// See attention_noalloc.h. The scratch of the split-key decode kernel lives here, in the library.
#include "attention_noalloc.h"

static __device__ __align__(256) float sp_static_partials[SP_FLASH_DECODE_STATIC_MAX_FLOATS];
static __device__ __align__(256) int sp_static_counters[SP_FLASH_DECODE_STATIC_MAX_COUNTERS];

namespace {
constexpr int STATIC_MAX_DEVICES = 64;
float* static_partials_ptr[STATIC_MAX_DEVICES];      // device addresses, looked up once per device
int* static_counters_ptr[STATIC_MAX_DEVICES];
}  // namespace

SP_API int sp_flash_decode_static(const void* q, void* out, int out_dt, const void* kpool, const void* vpool,
                                  const int* seq_len, const int* seq_row, const int* page_table, int max_pages,
                                  int page_size, int n_seqs, int nh, int nkv, int hd, int window, float scale,
                                  int chunk_tiles, int n_chunks, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (check_common(hd, nh, nkv, page_size)) return 1;
    if (nh / nkv > 16) SP_FAIL("flash decode: %d query heads per kv head, at most 16 fit one tile", nh / nkv);
    if (chunk_tiles <= 0 || n_chunks <= 0 || n_chunks > 65535) SP_FAIL("flash decode: bad chunking %d x %d", n_chunks, chunk_tiles);
    if (n_seqs > 65535) SP_FAIL("flash decode: %d sequences are beyond this kernel's grid", n_seqs);
    if (out_dt != SP_DT_F32 && out_dt != SP_DT_BF16) SP_FAIL("flash decode: unsupported output dtype code %d", out_dt);
    const long long need = sp_flash_decode_scratch_floats(n_seqs, nh, hd, n_chunks);
    if (need > (long long)SP_FLASH_DECODE_STATIC_MAX_FLOATS)
        SP_FAIL("flash decode (static scratch): %lld floats of partial results are needed, the built-in array holds %d; "
                "use fewer chunks or the entry point that takes a scratch buffer", need, SP_FLASH_DECODE_STATIC_MAX_FLOATS);
    if ((long long)n_seqs * nkv > (long long)SP_FLASH_DECODE_STATIC_MAX_COUNTERS)
        SP_FAIL("flash decode (static scratch): %lld arrival counters are needed, the built-in array holds %d",
                (long long)n_seqs * nkv, SP_FLASH_DECODE_STATIC_MAX_COUNTERS);

    // the arrays' names are host-side handles; kernels need their device addresses, per device
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) SP_FAIL("flash decode (static scratch): cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) SP_FAIL("flash decode (static scratch): device %d is beyond the %d this build tracks", dev, STATIC_MAX_DEVICES);
    if (!static_partials_ptr[dev]) {
        float* pp = nullptr;
        int* cp = nullptr;
        e = cudaGetSymbolAddress((void**)&pp, sp_static_partials);
        if (e != cudaSuccess || !pp) SP_FAIL("flash decode (static scratch): no address for the partial-result array: %s", cudaGetErrorString(e));
        e = cudaGetSymbolAddress((void**)&cp, sp_static_counters);
        if (e != cudaSuccess || !cp) SP_FAIL("flash decode (static scratch): no address for the counter array: %s", cudaGetErrorString(e));
        static_counters_ptr[dev] = cp;
        static_partials_ptr[dev] = pp;
    }
    float* part_o = static_partials_ptr[dev];
    float* part_ml = part_o + (size_t)n_seqs * nh * n_chunks * hd;
    int* counters = static_counters_ptr[dev];
    // the counters must start at zero whatever an earlier, perhaps interrupted, call left there
    e = cudaMemsetAsync(counters, 0, (size_t)n_seqs * nkv * sizeof(int), stream);
    if (e != cudaSuccess) SP_FAIL("flash decode (static scratch): clearing the counters failed: %s", cudaGetErrorString(e));

    PagedKV kv{(const __nv_bfloat16*)kpool, (const __nv_bfloat16*)vpool, page_table, seq_row, max_pages, nkv, sp_range_host};
    dim3 grid(n_chunks, nkv, n_seqs);
    const float sl = scale * LOG2E;
    if (launch_flash_decode(hd, grid, stream, (const __nv_bfloat16*)q, kv, seq_len, nh, window, sl, chunk_tiles, part_o,
                            part_ml, counters, out, out_dt)) return 1;
    SP_CHECK_LAUNCH("flash_decode (static scratch)");
    return 0;
}
