// All layers of a decode step (one new token per sequence, up to 16 sequences) in ONE persistent kernel.
//
// A layer here is the pre-norm block of the reference (crates/spissa-runtime/src/models/llama/generate.rs:190-778: norm → attention
// → residual, norm → feed-forward → residual; kernels in rotary.rs and ops.rs): RMSNorm, stacked QKV projection,
// rotate-half position encoding, grouped-query attention over the paged cache, output projection, RMSNorm,
// gate/up projections with silu(gate)·up, down projection. Which tensors, sizes and constants a layer has
// comes from a table of descriptors that the host builds from the parts of the model; the kernel knows no
// model.
//
// Why one kernel: at a few tokens per step every product is a stream of weights through the SM, and as
// separate kernels each stream starts from an empty pipe. Here one CTA per SM lives through the whole step:
//   * a copy warp walks, for its CTA, the weight tiles of every product of every layer in the order the CTA
//     will use them (blocks of 16 rows of W are dealt to the CTAs round robin, the deal going on from product
//     to product) and fetches them as TMA boxes (8 + 8 rows x 256 columns, 8 KB a request) into a ring of
//     shared-memory stages. The ring does not care about phases: while the CTA waits at a grid barrier or
//     works on attention, the weights of the products to come are already on their way, so HBM stays busy
//     across phase boundaries;
//   * eight consumer warps take the tiles (mma.sync m16n8k16: the block's 16 rows of W are M, eight tokens N,
//     each warp a slice of the tile's columns, K permuted alike in both operands so that fragments are plain
//     16-byte loads), add their slices in warp order through shared memory and run the epilogue: rotate and
//     store q / write k and v into the cache; add into the 32-bit residual; silu(gate)·up;
//   * attention runs inside: the keys of every (sequence, kv head) in chunks over the CTAs (the split comes as
//     launch arguments or, for a launch replayed from a CUDA graph, as two words on the device), two groups of
//     four warps per CTA with cp.async double buffering, the keys as the M of mma.sync and the query heads of
//     the kv head as its N (flash_common.cuh: decode_step_t), then one warp per (token, head) combines the chunks.
//     Where the split is into 1, 2 or 4 chunks (about as many items as warp groups: eight sequences of eight kv
//     heads, for instance) the CTAs are launched as pairs (a thread-block cluster of two) and all chunks of a
//     (sequence, kv head) sit in one pair: the groups leave their partial results in shared memory, the pair's first
//     CTA reads its partner's through distributed shared memory behind a cluster-scope mbarrier and writes the
//     heads' outputs itself, so the combination costs neither a phase of its own nor its grid barrier;
//   * phases that need every CTA's result are separated by a grid barrier (cooperative launch; an atomic
//     counter; bounded spin).
//   * the output head can be the kernel's last product (crates/spissa-runtime/src/streaming/linear_argmax.rs:13: the
//     reference's greedy head streams the rows and keeps the best): the final norm is folded in like the others,
//     the vocabulary's rows stream through the same ring, and the result is the logits or, for a greedy step, one
//     (value, row) candidate per token and CTA, of which the last CTA to finish takes the best.
// RMSNorm costs no pass of its own: whoever adds into the residual also stores it multiplied by the next norm's
// weight (bfloat16, the next product's input) and sums the squares of what it wrote, per CTA and token; the
// next product adds the CTAs' sums in CTA order and multiplies its RESULT by 1/rms: y = rstd·(x ⊙ w)·Wᵀ.
// Statistics, rotation angles, softmax and the residual are 32-bit. Every sum has a fixed order: a token's
// result depends neither on timing nor on the other tokens of the step.
//
// A warp issues in order and a load from L2 takes a microsecond or two while the weights stream, so wherever
// a phase needs data from global memory all loads are issued before the first use, the token positions and
// page-table entries stay in shared memory across layers, and an epilogue's reads are asked for before its
// tiles.
//
// Every wait (mbarrier, grid barrier) is bounded. A wait that runs out records a code in ``status`` and sets
// an abort flag; from then on waits are skipped but the control flow stays the same, so that no warp is left
// behind at a barrier: the kernel ends with a meaningless result and the host sees the code. No load uses
// cluster multicast.
#include "flash_common.cuh"
#include <cuda.h>

SP_API const char* sp_decode_layers_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(decode_layers)

namespace {

constexpr int CWARPS = 8;                       // consumer warps
constexpr int CTHREADS = CWARPS * 32;
constexpr int THREADS = CTHREADS + 32;          // and the copy warp
constexpr int KC = 1024;                        // columns of W per stage
constexpr int BOXC = 256;                       // columns per TMA box (the most a box may have)
constexpr int WSL = KC / CWARPS;                // columns of a tile per consumer warp
constexpr int SS = WSL / 32;                    // steps of 32 columns per warp and tile
constexpr int BOX_BYTES = 16 * BOXC * 2;        // one box: 2 halves x 8 rows x 256 columns
constexpr int STAGE_BYTES = (KC / BOXC) * BOX_BYTES;
constexpr int MAX_STAGES = 12;
constexpr int MAXT = 16;                        // tokens per step
constexpr int RED_FLOATS = CWARPS * 2 * 32 * 4; // one buffer of the K-slice sums
constexpr int MAX_CHUNKS = 32;                  // key chunks per sequence (a single long sequence still gives most warp groups an item)
constexpr int MAX_CHUNK_PAGES = 512;            // pages per chunk (their table entries wait in shared memory)
constexpr int SMEM_LIMIT = 232448;              // per CTA on sm_100
constexpr int STATIC_SMEM = 1536;               // barriers and small arrays below, rounded up

struct LayerDesc {
    const __nv_bfloat16* w_qkv;     // [(nh + 2 nkv) hd, H]  q heads, k heads, v heads
    const __nv_bfloat16* w_o;       // [H, nh hd]
    const __nv_bfloat16* w_gu;      // [2 I, H]  gu_pair gate rows, their gu_pair up rows, and so on
    const __nv_bfloat16* w_down;    // [H, I]
    const __nv_bfloat16* norm1;     // [H]
    const __nv_bfloat16* norm2;     // [H]
    __nv_bfloat16* k_pool;          // [pages, nkv, 64, hd]
    __nv_bfloat16* v_pool;
    const float* inv_freq;          // [hd / 2]
    int nh, nkv, I, gu_pair;
    float eps1, eps2, scale_log2;
    int pad;
};
static_assert(sizeof(LayerDesc) == 104, "the host packs this layout");

struct Params {
    const LayerDesc* layers;
    float* x;                       // [T, H] residual, in and out
    __nv_bfloat16* q;               // [T, nh hd]
    __nv_bfloat16* attn;            // [T, nh hd]
    __nv_bfloat16* act;             // [T, I]
    __nv_bfloat16* xw;              // [T, H] residual times the weight of the norm that reads it next
    float* ssq;                     // [2][16][CTAs rounded up to 4] sums of squares of the residual, per token and CTA
    float* part_o;                  // [T][nh][chunks][hd]
    float* part_ml;                 // [T][nh][chunks][2]
    const int* positions;           // [T] position of each new token = keys before it
    const int* seq_row;             // [T] row of the page table
    const int* page_table;
    unsigned* sync;                 // [0] barrier arrivals (and the abort bit), [1] CTAs finished
    int* status;
    const CUtensorMap* maps;        // [layers][4]: QKV, output, gate/up, down; see sp_decode_layers_encode_map
    unsigned long long* trace;      // optional: the global timer at each grid barrier, see sp_decode_layers_set_trace
    int n_layers, T, H, n_stages, max_pages, chunk_pages, n_chunks, xn_row;
    const int* plan;                // optional, on the device: {chunk_pages, n_chunks} instead of the two above
    int pairs;                      // 1: launched as clusters of two CTAs (the pair-wise combination is possible)
    // the output head as one more product behind the last layer (head_mode 0: none): the final RMS norm is folded in
    // like the layers' norms; its tensor map is maps[n_layers * 4]
    int head_mode;                  // 1: logits [T, head_ld] float32; 2: one (value, row) candidate per token and CTA, [T, head_ld]
    const __nv_bfloat16* head_w;    // [head_rows, H]
    const __nv_bfloat16* final_norm;   // [H]
    void* head_out;
    float final_eps;
    int head_rows, head_ld, n_slots;
    // head_mode 2 with ``tokens``: the last CTA to finish takes the best of each token's candidates, writes the token
    // and (with ``header``) notes it in the sequence's header [slots, 4]: position, draws, last token, spare
    int* tokens;                    // [T]
    int* header;
    // the embedding as the kernel's first phase (null: ``x`` holds the rows already): x[m] = table[ids[m]], a zero row
    // and code 301 for an id outside the table (crates/spissa-runtime/src/ops.rs:6-30: no scale)
    const __nv_bfloat16* embed_w;   // [embed_rows, H]
    const int* embed_ids;           // [T]
    int embed_rows, pad4;
    const int* seq_slot;            // [T]
    const int* seq_len;             // [T] the sequences' lengths after this step
    SpRange rg;                     // what the debug build checks table entries against
};

// MODE 2 of the head: the best (value, row) of a token among the rows a CTA computed; a second, tiny kernel takes the
// best of each token's row of candidates (the lowest row wins among equal values, NaN never wins:
// crates/spissa-runtime/src/streaming/argmax.rs:30-51, :85-97).
struct Candidate { float value; int index; };
__device__ __forceinline__ void candidate_take(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
// Predicated loads that leave zeros when ``pred`` is false (what other CTAs produced inside this kernel is read at L2,
// never from this SM's L1). The zero is set BEFORE the load and nothing reads
// the registers until their use: the warp goes on while the load is in flight.
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t a, bool pred) {
    v = make_uint4(0, 0, 0, 0);
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t@q ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n\t}"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) : "r"(a), "r"((int)pred));
}
__device__ __forceinline__ void ld_cg_u4_if(uint4& v, const void* p, bool pred) {
    v = make_uint4(0, 0, 0, 0);
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t@q ld.global.cg.v4.b32 {%0,%1,%2,%3}, [%4];\n\t}"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) : "l"(p), "r"((int)pred));
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- the products of a layer
struct Job {
    const __nv_bfloat16* W;
    int N, K;          // rows and columns of W
    int pair;          // > 0: rows come in pairs ``pair`` apart (rotation halves, gate and up); 0: plain rows
    int n_blocks;      // blocks of 16 rows of W
};

template <int HD>
__device__ __forceinline__ Job job_of(const LayerDesc& L, int which, int H) {
    Job j;
    if (which == 0) { j.W = L.w_qkv; j.N = (L.nh + 2 * L.nkv) * HD; j.K = H; j.pair = HD / 2; }
    else if (which == 1) { j.W = L.w_o; j.N = H; j.K = L.nh * HD; j.pair = 0; }
    else if (which == 2) { j.W = L.w_gu; j.N = 2 * L.I; j.K = H; j.pair = L.gu_pair; }
    else { j.W = L.w_down; j.N = H; j.K = L.I; j.pair = 0; }
    j.n_blocks = j.pair ? (j.N / 2 + 7) / 8 : (j.N + 15) / 16;
    return j;
}

// rows of W in the two halves of block ``rb`` and how many of each half exist
__device__ __forceinline__ void block_rows(const Job& j, int rb, int& rowA, int& rowB, int& nA, int& nB) {
    if (j.pair) {
        const int o0 = rb * 8;
        rowA = (o0 / j.pair) * 2 * j.pair + (o0 % j.pair);
        rowB = rowA + j.pair;
        const int left = j.N / 2 - o0;
        nA = nB = left >= 8 ? 8 : (left > 0 ? left : 0);
    } else {
        rowA = rb * 16;
        rowB = rowA + 8;
        const int la = j.N - rowA, lb = j.N - rowB;
        nA = la >= 8 ? 8 : (la > 0 ? la : 0);
        nB = lb >= 8 ? 8 : (lb > 0 ? lb : 0);
    }
}

struct Shared {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    float rstd[MAXT];
    float ssq[128];
    float warp_sum[CWARPS];
    int tok_pos[MAXT];     // position of each token, and the cache page that holds it
    int tok_page[MAXT];
    int ptc[2][64];        // per attention group: page-table entries of its last item (the table is the same in every layer)
    int ptc_key[2][3];     // whose they are: sequence, first and last page
    int aborted;
    uint64_t pair_bar;     // arrivals of the four attention groups of a CTA pair (used in the pair's first CTA)
};
static_assert(sizeof(Shared) <= STATIC_SMEM, "the static shared memory is counted as STATIC_SMEM bytes");

// Grid-barrier arrivals are counted in sync[0]; an abort sets ABORT_BIT there, which lets every waiter through.
constexpr unsigned ABORT_BIT = 0x40000000u;

__device__ __forceinline__ void raise_abort(const Params& p, Shared* sh, int code) {
    if (p.status) atomicCAS(p.status, 0, code);
    atomicOr(&p.sync[0], ABORT_BIT);
    *(volatile int*)&sh->aborted = 1;
}
__device__ __forceinline__ bool is_aborted(Shared* sh) { return *(volatile int*)&sh->aborted != 0; }

// ---------------------------------------------------------------- the copy warp
template <int HD>
__device__ void copy_warp(const Params& p, Shared* sh, uint32_t ring, int lane) {
    const int G = gridDim.x, cta = blockIdx.x, S = p.n_stages;
    uint32_t n = 0, phase = 0;
    int cursor = 0, slot = 0;
    for (int l = 0; l < p.n_layers; ++l) {
        const LayerDesc L = p.layers[l];
        for (int which = 0; which < 4; ++which) {
            const Job j = job_of<HD>(L, which, p.H);
            const int nkt = (j.K + KC - 1) / KC;
            const CUtensorMap* map = p.maps + (size_t)l * 4 + which;
            const int pr = j.pair ? j.pair : 8;
            for (int rb = (cta - cursor + G) % G; rb < j.n_blocks; rb += G) {
                const int o0 = rb * 8;                              // first of the block's 8 rows within each half
                for (int kt = 0; kt < nkt; ++kt, ++n) {
                    const uint32_t full = smem_u32(&sh->full[slot]), empty = smem_u32(&sh->empty[slot]);
                    if (!is_aborted(sh) && !mbar_wait(empty, phase ^ 1u, nullptr, 0)) raise_abort(p, sh, 201);
                    if (lane == 0) {
                        // columns beyond K and rows beyond N arrive as zeros and count as bytes all the same
                        mbar_expect_tx(full, (uint32_t)STAGE_BYTES);
#pragma unroll
                        for (int c = 0; c < KC / BOXC; ++c)
                            tma_load_4d(ring + slot * STAGE_BYTES + c * BOX_BYTES, map, kt * KC + c * BOXC, o0 % pr, 0, o0 / pr, full);
                    }
                    __syncwarp();
                    if (++slot == S) { slot = 0; phase ^= 1u; }
                }
            }
            cursor = (cursor + j.n_blocks) % G;
        }
    }
    if (p.head_mode) {                                          // the head's rows, walked as the consumers walk them
        const int n_blocks = (p.head_rows + 15) / 16, nkt = (p.H + KC - 1) / KC;
        const CUtensorMap* map = p.maps + (size_t)p.n_layers * 4;
        for (int rb = (cta - cursor + G) % G; rb < n_blocks; rb += G) {
            const int o0 = rb * 8;
            for (int kt = 0; kt < nkt; ++kt, ++n) {
                const uint32_t full = smem_u32(&sh->full[slot]), empty = smem_u32(&sh->empty[slot]);
                if (!is_aborted(sh) && !mbar_wait(empty, phase ^ 1u, nullptr, 0)) raise_abort(p, sh, 201);
                if (lane == 0) {
                    mbar_expect_tx(full, (uint32_t)STAGE_BYTES);
#pragma unroll
                    for (int c = 0; c < KC / BOXC; ++c)
                        tma_load_4d(ring + slot * STAGE_BYTES + c * BOX_BYTES, map, kt * KC + c * BOXC, o0 % 8, 0, o0 / 8, full);
                }
                __syncwarp();
                if (++slot == S) { slot = 0; phase ^= 1u; }
            }
        }
    }
    // after an abort tiles may still be in flight into this CTA's shared memory: let them land
    if (is_aborted(sh)) {
        for (uint32_t back = 1; back <= (uint32_t)S && back <= n; ++back) {
            const uint32_t i = n - back;
            mbar_wait(smem_u32(&sh->full[i % S]), (i / S) & 1u, nullptr, 0);
        }
    }
}

// ---------------------------------------------------------------- consumers: one product
// The 16 rows of a block are the M of the mma (rows 0-7 the first half, 8-15 the second), eight tokens its N;
// tokens 8-15, when there are any, are a second N block. Lane (g, t) holds row g of both halves and token g,
// eight consecutive columns each: K is permuted the same way in both operands, which a dot product allows.
// ``aload(kt, a)``: starts the loads of the warp's activation fragments for tile kt: a[s][0] token g, a[s][1] token g + 8, eight
// consecutive columns from kt·KC + warp·64 + s·32 + 8t. ``epi(rb, m, c, a, b, rowA, rowB, nA, nB, held)``: token m,
// column c (0..7) of both halves of block rb; ``held`` is what ``pre(rb, m, c, rowA, rowB, nA, nB)`` returned when
// the block began (loads that the epilogue needs, issued before the tiles so that they cost no waiting).
struct Walk {
    int slot;          // stage of the next tile (the copy warp walks the ring the same way)
    uint32_t phase;    // how often the ring has been walked, mod 2
    int cursor;        // which CTA gets block 0 of the next product
    int red_par;
};

template <bool WIDE, class ALoad, class Pre, class Epi>
__device__ __forceinline__ void product(const Params& p, Shared* sh, const Job& j, Walk& w, uint32_t ring, float* red,
                                        ALoad aload, Pre pre, Epi epi) {
    constexpr int NF = WIDE ? 2 : 1;                              // token blocks of 8
    constexpr int DEPTH = WIDE ? 1 : 2;                           // tiles whose activation fragments are in flight (as registers allow)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = gridDim.x, S = p.n_stages;
    const int nkt = (j.K + KC - 1) / KC;
    const int first = ((int)blockIdx.x - w.cursor + G) % G;
    if (first < j.n_blocks) {
        // slot u of the ring holds the fragments of tile kt0 + u; after its use it is refilled for its next use
        uint4 fr[DEPTH][SS][NF];
#pragma unroll
        for (int u = 0; u < DEPTH; ++u) aload(u < nkt ? u : 0, fr[u]);
        for (int rb = first; rb < j.n_blocks; rb += G) {
            int rowA, rowB, nA, nB;
            block_rows(j, rb, rowA, rowB, nA, nB);
            // what the epilogue will need from global memory is asked for now and arrives during the tiles
            const int e_m = 8 * (tid >> 6) + 2 * ((tid >> 1) & 3) + (tid & 1), e_c = (tid >> 3) & 7;
            float4 held = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tid < 64 * NF) held = pre(rb, e_m, e_c, rowA, rowB, nA, nB);
            float acc[NF][2][4];                                  // [token block][half of the lane's columns][c0..c3]
#pragma unroll
            for (int i = 0; i < NF; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h) acc[i][h][0] = acc[i][h][1] = acc[i][h][2] = acc[i][h][3] = 0.0f;
            for (int kt0 = 0; kt0 < nkt; kt0 += DEPTH) {
#pragma unroll
                for (int u = 0; u < DEPTH; ++u) {
                    const int kt = kt0 + u;
                    if (kt >= nkt) break;
                    const int slot = w.slot;
                    if (!is_aborted(sh) && !mbar_wait(smem_u32(&sh->full[slot]), w.phase, nullptr, 0)) raise_abort(p, sh, 202);
                    const int kc = min(KC, j.K - kt * KC);
                    const uint32_t base = ring + slot * STAGE_BYTES;
                    if (warp * WSL < kc) {
                        uint4 wa[SS], wb[SS];
#pragma unroll
                        for (int s = 0; s < SS; ++s) {
                            const int kl = warp * WSL + s * 32 + 8 * t;
                            const uint32_t at = base + (kl / BOXC) * BOX_BYTES + (kl % BOXC) * 2;
                            wa[s] = lds128(at + g * (BOXC * 2));                 // zeros where W ends
                            wb[s] = lds128(at + (8 + g) * (BOXC * 2));
                        }
#pragma unroll
                        for (int s = 0; s < SS; ++s)
#pragma unroll
                            for (int i = 0; i < NF; ++i) {
                                mma16816(acc[i][0], wa[s].x, wb[s].x, wa[s].y, wb[s].y, fr[u][s][i].x, fr[u][s][i].y);
                                mma16816(acc[i][1], wa[s].z, wb[s].z, wa[s].w, wb[s].w, fr[u][s][i].z, fr[u][s][i].w);
                            }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sh->empty[slot]));
                    if (++w.slot == S) { w.slot = 0; w.phase ^= 1u; }
                    aload(kt + DEPTH < nkt ? kt + DEPTH : (u < nkt ? u : 0), fr[u]);     // harmless after the last block
                }
            }
            // the warps' K slices, added in warp order
            float* buf = red + w.red_par * RED_FLOATS;
#pragma unroll
            for (int i = 0; i < NF; ++i)
                *(float4*)(buf + ((warp * 2 + i) * 32 + lane) * 4) =
                    make_float4(acc[i][0][0] + acc[i][1][0], acc[i][0][1] + acc[i][1][1], acc[i][0][2] + acc[i][1][2],
                                acc[i][0][3] + acc[i][1][3]);
            bar_sync(1, CTHREADS);
            // thread (token block i, lane slot lp, v): token 8i + 2t + v, column g: c[v] is the first half, c[v + 2] the second
            if (tid < 64 * NF) {
                const int i = tid >> 6, lp = (tid >> 1) & 31, v = tid & 1;
                float a = 0.0f, b = 0.0f;
#pragma unroll
                for (int ww = 0; ww < CWARPS; ++ww) {
                    a += buf[((ww * 2 + i) * 32 + lp) * 4 + v];
                    b += buf[((ww * 2 + i) * 32 + lp) * 4 + v + 2];
                }
                epi(rb, e_m, e_c, a, b, rowA, rowB, nA, nB, held);
            }
            w.red_par ^= 1;          // the other warps may run one block ahead of the epilogue: two buffers
        }
    }
    w.cursor = (w.cursor + j.n_blocks) % G;
}

// ---------------------------------------------------------------- grid barrier
__device__ __forceinline__ void grid_sync(const Params& p, Shared* sh, unsigned& epoch) {
    bar_sync(1, CTHREADS);
    ++epoch;
    if (threadIdx.x == 0) {
        const bool traced = p.trace && (blockIdx.x == 0 || blockIdx.x == 77) && epoch < 200u;
        if (traced) p.trace[(blockIdx.x ? 400 : 0) + 2 * epoch] = global_ns();
        // release: what this CTA wrote (seen by this thread through the CTA barrier) is visible before the count
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");
        const unsigned target = epoch * gridDim.x;
        if (!is_aborted(sh)) {
            unsigned long long t0 = 0;
            unsigned spins = 0, seen;
            while ((seen = ld_acquire_u32(p.sync)) < target) {
                if ((++spins & 255u) == 0u) {
                    const unsigned long long now = global_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > WAIT_LIMIT_NS) { raise_abort(p, sh, 203); break; }
                }
            }
            if (seen & ABORT_BIT) *(volatile int*)&sh->aborted = 1;
        }
        if (traced) p.trace[(blockIdx.x ? 400 : 0) + 2 * epoch + 1] = global_ns();
    }
    bar_sync(1, CTHREADS);
}

// ---------------------------------------------------------------- the product's input and its statistics
// The residual reaches a product already multiplied by the norm's weight and rounded (``xw``, written by whoever
// last added into the residual); 1/rms, which needs every CTA's sum of squares, multiplies the product's result
// in the epilogue instead: y = rstd · (x ⊙ w)·Wᵀ. Here: xw into shared memory (one asynchronous copy) and
// rstd[m] from the CTAs' sums, added in CTA order. A warp issues in order and a load from L2 takes a
// microsecond or two under load, so all loads are issued before the first use.
__device__ __noinline__ void stage_xw(const Params& p, Shared* sh, const float* ssq_src, float eps, uint32_t xn) {
    constexpr int SSQ = 3;                       // float4 of CTA sums per thread: up to 16 x 3 x 4 = 192 CTAs in one batch
    const int tid = threadIdx.x;
    const int n8 = p.H >> 3;
    for (int c = tid; c < p.T * n8; c += CTHREADS) {
        const int m = c / n8, k8 = c - m * n8;
        cp_async16(xn + m * p.xn_row + k8 * 16, p.xw + (size_t)m * p.H + (size_t)k8 * 8);
    }
    cp_async_commit();
    {
        // token m's sums lie side by side: 16 threads fetch them four at a time (every CTA reads all of them, so
        // few, wide requests matter here)
        const int m = tid >> 4, jj = tid & 15;
        const int gp4 = ((int)gridDim.x + 3) >> 2;
        const float4* row = (const float4*)(ssq_src + (size_t)m * gp4 * 4);
        float4 part[SSQ];
#pragma unroll
        for (int u = 0; u < SSQ; ++u) {
            const int c = jj + 16 * u;
            part[u] = (m < p.T && c < gp4) ? __ldcg(row + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float s = 0.0f;
#pragma unroll
        for (int u = 0; u < SSQ; ++u) s += (part[u].x + part[u].y) + (part[u].z + part[u].w);
        if (m < p.T)
            for (int c = jj + 16 * SSQ; c < gp4; c += 16) { const float4 v = __ldcg(row + c); s += (v.x + v.y) + (v.z + v.w); }
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (jj == 0) sh->rstd[m] = 1.0f / sqrtf(s / (float)p.H + eps);
    }
    cp_async_wait<0>();
    bar_sync(1, CTHREADS);
}

// the sums of squares that the epilogue threads (tid < 128) gathered while adding into the residual, per token,
// in a fixed order: token m sits in threads 64·(m / 8) + 8g + 2·((m % 8) / 2) + m % 2, g = 0..7
__device__ __forceinline__ void publish_ssq(Shared* sh, float mine, float* dst, int stride) {
    const int tid = threadIdx.x;
    sh->ssq[tid] = mine;
    bar_sync(2, 128);
    if (tid < MAXT) {
        const int m = tid;
        float s = 0.0f;
#pragma unroll
        for (int gg = 0; gg < 8; ++gg) s += sh->ssq[64 * (m >> 3) + 8 * gg + 2 * ((m & 7) >> 1) + (m & 1)];
        __stcg(dst + (size_t)m * stride, s);
    }
}

// ---------------------------------------------------------------- attention: chunks of keys, then their combination
// GROUPS groups of four warps, each with tiles of its own, work on different (sequence, kv head, chunk) items.
// PAIRED: there is at most one item per group, all chunks of a (sequence, kv head) lie in one CTA pair, and the
// groups' partial results go to ``xch`` ([group][8 heads][HD + 2] floats in this CTA's shared memory) instead of global
// memory; a single chunk is finished here (divided by its sum and stored).
constexpr int XCH_ROWS = 8;
template <int HD, int ST, int GROUPS, int NH, bool PAIRED>
__device__ __noinline__ void attention_chunks(const Params& p, Shared* sh, const LayerDesc& L, uint8_t* scratch_all,
                                              int chunk_pages, int n_chunks, float* xch) {
    using TL = Tile<HD>;
    constexpr int GROUP_BYTES = 16 * TL::ROW + 2 * ST * TL::BYTES + MAX_CHUNK_PAGES * 4;
    constexpr int MS = HD + 2;
    static_assert(4 * 16 * MS * 4 <= ST * TL::BYTES, "the merge buffer reuses the key tiles");
    const int wg = (threadIdx.x >> 5) >> 2;                        // warp group
    const int tid = threadIdx.x & 127, warp = tid >> 5, lane = tid & 31;
    const int bar = 2 + wg;
    uint8_t* scratch = scratch_all + (size_t)wg * GROUP_BYTES;
    const uint32_t q_tile = smem_u32(scratch);                     // 16 rows
    const uint32_t k_tiles = q_tile + 16 * TL::ROW;
    const uint32_t v_tiles = k_tiles + ST * TL::BYTES;
    float* merge = (float*)(scratch + 16 * TL::ROW);               // [4 warps][16 rows][HD + 2], over the key tiles once they are used up
    int* pt_s = (int*)(scratch + 16 * TL::ROW + 2 * ST * TL::BYTES);         // the chunk's page-table entries
    const int Gq = L.nh / L.nkv;
    const int n_items = p.T * L.nkv * n_chunks;
    for (int it = blockIdx.x * GROUPS + wg; it < n_items; it += gridDim.x * GROUPS) {
        const int b = it / (L.nkv * n_chunks), g = (it / n_chunks) % L.nkv, chunk = it % n_chunks;
        const int pos = p.positions[b];
        const int j_first = chunk * chunk_pages;
        const int j_last = min(pos / KT, j_first + chunk_pages - 1);
        const size_t part_base = ((size_t)b * L.nh + (size_t)g * Gq) * n_chunks + chunk;
        if (j_first > j_last) {                                    // no keys in this chunk (the same for all 128 threads)
            for (int i = tid; i < Gq; i += 128) {
                if (PAIRED) {
                    xch[((size_t)wg * XCH_ROWS + i) * MS + HD] = -INFINITY;
                    xch[((size_t)wg * XCH_ROWS + i) * MS + HD + 1] = 0.0f;
                } else {
                    p.part_ml[(part_base + (size_t)i * n_chunks) * 2] = -INFINITY;
                    p.part_ml[(part_base + (size_t)i * n_chunks) * 2 + 1] = 0.0f;
                }
            }
            if (PAIRED) break;
            continue;
        }
        // The table entries first, all at once: a load inside the loop would stall the warp for its whole way to
        // L2. A short list stays in shared memory for the layers to come, which ask for the same entries.
        const int cnt = j_last - j_first + 1;
        int* key = sh->ptc_key[wg];
        const bool small = cnt <= 64;
        const bool hit = small && key[0] == b && key[1] == j_first && key[2] == j_last;
        const int* pts = small ? sh->ptc[wg] : pt_s;
        if (!hit) {
            const int* pt = p.page_table + (size_t)sp_checked_row(p.seq_row[b], p.rg) * p.max_pages;
            int* dst = small ? sh->ptc[wg] : pt_s;
            for (int i = tid; i < cnt; i += 128)
                dst[i] = sp_checked_page(pt[sp_checked_entry(j_first + i, p.max_pages, p.rg)], p.rg);
        }
        for (int c = tid; c < 16 * TL::CHUNKS; c += 128) {
            const int r = c / TL::CHUNKS, k = c % TL::CHUNKS;
            const uint32_t d = q_tile + r * TL::ROW + k * 16;
            if (r < Gq) cp_async16(d, p.q + (size_t)b * L.nh * HD + (size_t)(g * Gq + r) * HD + k * 8);
            else asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(d), "r"(0u) : "memory");
        }
        cp_async_commit();

        uint32_t qb[HD / 16][NH][2];
        float o[HD / 16][NH][4], m[NH][2], l[NH][2];
#pragma unroll
        for (int i = 0; i < NH; ++i) {
            m[i][0] = m[i][1] = -INFINITY;
            l[i][0] = l[i][1] = 0.0f;
#pragma unroll
            for (int dt = 0; dt < HD / 16; ++dt) o[dt][i][0] = o[dt][i][1] = o[dt][i][2] = o[dt][i][3] = 0.0f;
        }
        // each warp fetches and uses its own 16 keys of every page: no barrier among the warps inside the loop
        // the warp's 16 keys of a page are 16·HD consecutive elements: lane takes 16-byte pieces lane, lane + 32, ...
        constexpr int PIECES = 16 * TL::CHUNKS / 32;
        const uint32_t lane_dst = warp * 16 * TL::ROW + (lane / TL::CHUNKS) * TL::ROW + (lane % TL::CHUNKS) * 16;
        const size_t lane_src = ((size_t)g * KT + (size_t)warp * 16) * HD + (size_t)lane * 8;
        auto fetch = [&](int j, int stage) {
            const size_t off = (size_t)pts[j - j_first] * L.nkv * KT * HD + lane_src;
            const uint32_t kd = k_tiles + stage * TL::BYTES + lane_dst, vd = v_tiles + stage * TL::BYTES + lane_dst;
#pragma unroll
            for (int u = 0; u < PIECES; ++u) {
                cp_async16(kd + u * (32 / TL::CHUNKS) * TL::ROW, L.k_pool + off + (size_t)u * 256);
                cp_async16(vd + u * (32 / TL::CHUNKS) * TL::ROW, L.v_pool + off + (size_t)u * 256);
            }
        };
        bar_sync(bar, 128);                                        // the table entries are in place
        if (tid == 0 && !hit) { key[0] = small ? b : -1; key[1] = j_first; key[2] = j_last; }
#pragma unroll
        for (int s = 0; s < ST - 1; ++s) {
            if (j_first + s <= j_last) fetch(j_first + s, s);
            cp_async_commit();
        }
        cp_async_wait<ST - 1>();
        bar_sync(bar, 128);
        // Qᵀ as the B operand: lane (g, t) holds dims 2t, 2t+1 and 2t+8, 2t+9 of head g of each head tile
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
            for (int i = 0; i < NH; ++i) {
                const uint32_t a = q_tile + (i * 8 + (lane >> 2)) * TL::ROW + (kk * 16 + 2 * (lane & 3)) * 2;
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(qb[kk][i][0]) : "r"(a));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(qb[kk][i][1]) : "r"(a + 16));
            }
        for (int j = j_first; j <= j_last; ++j) {
            const int i = j - j_first, stage = i % ST;
            if (j + ST - 1 <= j_last) fetch(j + ST - 1, (i + ST - 1) % ST);
            cp_async_commit();
            cp_async_wait<ST - 1>();
            __syncwarp();
            if (j * KT + KT - 1 <= pos)
                decode_step_t<HD, NH, false>(qb, k_tiles + stage * TL::BYTES, v_tiles + stage * TL::BYTES, warp * 16, j * KT, 0,
                                             pos, L.scale_log2, o, m, l, lane);
            else
                decode_step_t<HD, NH, true>(qb, k_tiles + stage * TL::BYTES, v_tiles + stage * TL::BYTES, warp * 16, j * KT, 0,
                                            pos, L.scale_log2, o, m, l, lane);
            __syncwarp();
        }
        cp_async_wait<0>();
#pragma unroll
        for (int i = 0; i < NH; ++i)
#pragma unroll
            for (int c = 0; c < 2; ++c) {                          // the lanes that share t hold the same head's other keys
                l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], 4);
                l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], 8);
                l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], 16);
            }
        bar_sync(bar, 128);                                        // every warp is done with the key tiles: they become the merge buffer
        const int lg = lane >> 2, lt = lane & 3;
#pragma unroll
        for (int i = 0; i < NH; ++i)
#pragma unroll
            for (int c = 0; c < 2; ++c) {                          // head 8i + 2·lt + c: dims lg and lg + 8 of every 16
                float* dst = merge + ((size_t)warp * 16 + i * 8 + 2 * lt + c) * MS;
#pragma unroll
                for (int dt = 0; dt < HD / 16; ++dt) {
                    dst[dt * 16 + lg] = o[dt][i][c];
                    dst[dt * 16 + lg + 8] = o[dt][i][c + 2];
                }
                if (lg == 0) { dst[HD] = m[i][c]; dst[HD + 1] = l[i][c]; }
            }
        bar_sync(bar, 128);
        for (int e = tid; e < Gq * HD; e += 128) {
            const int row = e / HD, d = e % HD;
            float mm = -INFINITY;
#pragma unroll
            for (int ww = 0; ww < 4; ++ww) mm = fmaxf(mm, merge[((size_t)ww * 16 + row) * MS + HD]);
            const float msafe = (mm == -INFINITY) ? 0.0f : mm;
            float acc = 0.0f, ll = 0.0f;
#pragma unroll
            for (int ww = 0; ww < 4; ++ww) {
                const float* src = merge + ((size_t)ww * 16 + row) * MS;
                const float f = exp2f(src[HD] - msafe);
                acc += src[d] * f;
                ll += src[HD + 1] * f;
            }
            if (PAIRED) {
                if (n_chunks == 1) {
                    // the only chunk: what the combination would do with it (factor 2^0 = 1)
                    p.attn[((size_t)b * L.nh + (size_t)g * Gq + row) * HD + d] = __float2bfloat16_rn(acc / ll);
                } else {
                    float* dst = xch + ((size_t)wg * XCH_ROWS + row) * MS;
                    dst[d] = acc;
                    if (d == 0) { dst[HD] = mm; dst[HD + 1] = ll; }
                }
            } else {
                const size_t pi = part_base + (size_t)row * n_chunks;
                p.part_o[pi * HD + d] = acc;
                if (d == 0) { p.part_ml[pi * 2] = mm; p.part_ml[pi * 2 + 1] = ll; }
            }
        }
        bar_sync(bar, 128);                                        // the tiles are free for the next item
        if (PAIRED) break;
    }
}

// ---------------------------------------------------------------- the pair-wise combination
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
    return ra;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// After attention_chunks<PAIRED>: out[b, heads of g, :] from the chunks' partial results in the pair's shared memory,
// with the arithmetic and the order of attention_combine. Two chunks lie in the two groups of one CTA (a barrier of
// the CTA's consumer warps is enough); four lie in the four groups of the pair: every group announces its result on
// the first CTA's barrier (release, cluster scope), that CTA waits (acquire) and reads its partner's two through
// distributed shared memory. Called by all consumer warps of every CTA; ``pair_phase`` counts the uses of the barrier.
template <int HD>
__device__ __noinline__ void attention_pair_combine(const Params& p, Shared* sh, const LayerDesc& L, float* xch,
                                                       int n_chunks, uint32_t& pair_phase) {
    constexpr int MS = HD + 2;
    const int tid = threadIdx.x;
    const int Gq = L.nh / L.nkv;
    const int n_items = p.T * L.nkv * n_chunks;
    if (n_chunks == 1) return;
    if (n_chunks == 2) {
        const int it0 = (int)blockIdx.x * 2;
        bar_sync(1, CTHREADS);
        if (it0 >= n_items) return;
        const int b = it0 / (L.nkv * 2), g = (it0 / 2) % L.nkv;
        for (int e = tid; e < Gq * HD; e += CTHREADS) {
            const int row = e / HD, d = e % HD;
            const float* c0 = xch + (size_t)row * MS;
            const float* c1 = xch + ((size_t)XCH_ROWS + row) * MS;
            const float mm = fmaxf(c0[HD], c1[HD]);
            const float msafe = (mm == -INFINITY) ? 0.0f : mm;
            float ll = 0.0f, acc = 0.0f;
            if (c0[HD + 1] > 0.0f) { const float f = exp2f(c0[HD] - msafe); ll += c0[HD + 1] * f; acc += c0[d] * f; }
            if (c1[HD + 1] > 0.0f) { const float f = exp2f(c1[HD] - msafe); ll += c1[HD + 1] * f; acc += c1[d] * f; }
            p.attn[((size_t)b * L.nh + (size_t)g * Gq + row) * HD + d] = __float2bfloat16_rn(acc / ll);
        }
        return;
    }
    // four chunks: the pair's four groups
    const uint32_t rank = cluster_rank();
    const int it0 = ((int)blockIdx.x & ~1) * 2;
    if (it0 >= n_items) return;                                    // an idle pair (the same decision in both CTAs)
    const uint32_t bar_local = smem_u32(&sh->pair_bar);
    bar_sync(1, CTHREADS);                                         // both groups of this CTA have written their results
    if (tid == 0) {
        const uint32_t target = map_to_rank(bar_local, 0u);
        // one arrival per group: this thread arrives for both groups of its CTA
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0], 2;" ::"r"(target) : "memory");
    }
    if (rank != 0) return;
    if (!is_aborted(sh)) {
        const uint32_t parity = pair_phase & 1u;
        const unsigned long long t0 = global_ns();
        while (true) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred q;\n\t"
                "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 q, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, q;\n\t}"
                : "=r"(ok) : "r"(bar_local), "r"(parity) : "memory");
            if (ok || is_aborted(sh)) break;
            if (global_ns() - t0 > WAIT_LIMIT_NS) { raise_abort(p, sh, 205); break; }
        }
    }
    ++pair_phase;
    const int b = it0 / (L.nkv * 4), g = (it0 / 4) % L.nkv;
    const uint32_t xch_local = smem_u32(xch), xch_peer = map_to_rank(xch_local, 1u);
    for (int e = tid; e < Gq * HD; e += CTHREADS) {
        const int row = e / HD, d = e % HD;
        float mc[4], lc[4], oc[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {                              // chunk c: CTA c / 2 of the pair, group c % 2
            const uint32_t at = (uint32_t)((((c & 1) * XCH_ROWS + row) * MS) * 4);
            if (c < 2) {
                const float* src = xch + (size_t)((c & 1) * XCH_ROWS + row) * MS;
                mc[c] = src[HD]; lc[c] = src[HD + 1]; oc[c] = src[d];
            } else {
                mc[c] = ld_cluster_f32(xch_peer + at + HD * 4);
                lc[c] = ld_cluster_f32(xch_peer + at + (HD + 1) * 4);
                oc[c] = ld_cluster_f32(xch_peer + at + d * 4);
            }
        }
        const float mm = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
        const float msafe = (mm == -INFINITY) ? 0.0f : mm;
        float ll = 0.0f, acc = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (lc[c] > 0.0f) {                                    // chunks in order
                const float f = exp2f(mc[c] - msafe);
                ll += lc[c] * f;
                acc += oc[c] * f;
            }
        }
        p.attn[((size_t)b * L.nh + (size_t)g * Gq + row) * HD + d] = __float2bfloat16_rn(acc / ll);
    }
}

// out[b, head, :] = sum_c o_c·2^(m_c - M) / sum_c l_c·2^(m_c - M), chunks in order; one warp per (token, head).
// Lane c holds (m, l) of chunk c (there are at most 32 chunks) and hands them round by shuffles; the partial outputs
// of up to CB chunks are asked for in one go, the first batch before the maximum is known: with head size 64 the
// whole combination costs one round trip to L2.
template <int HD>
__device__ __noinline__ void attention_combine(const Params& p, const LayerDesc& L, int n_chunks) {
    static_assert(MAX_CHUNKS <= 32, "a lane per chunk");
    constexpr int DPL = HD / 32;                                   // output dims per lane
    constexpr int CB = DPL <= 2 ? 32 : 16;                         // chunks whose loads are issued together
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nc = n_chunks;
    for (int r = blockIdx.x * CWARPS + warp; r < p.T * L.nh; r += gridDim.x * CWARPS) {
        const size_t bh = (size_t)r;
        float2 ml = make_float2(-INFINITY, 0.0f);
        if (lane < nc) ml = __ldcg((const float2*)&p.part_ml[(bh * nc + lane) * 2]);
        float oc[CB][DPL];
        auto ask = [&](int c0) {
#pragma unroll
            for (int u = 0; u < CB; ++u) {
                const int c = c0 + u;
#pragma unroll
                for (int i = 0; i < DPL; ++i) oc[u][i] = c < nc ? __ldcg(&p.part_o[(bh * nc + c) * HD + lane + 32 * i]) : 0.0f;
            }
        };
        ask(0);
        const float mm = sp_warp_max(ml.x);
        const float msafe = (mm == -INFINITY) ? 0.0f : mm;
        const float f_mine = ml.y > 0.0f ? exp2f(ml.x - msafe) : 0.0f;   // this lane's chunk: its weight, 0 if it saw no key
        float ll = 0.0f, acc[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
        for (int c0 = 0; c0 < nc; c0 += CB) {
            if (c0 > 0) ask(c0);
#pragma unroll
            for (int u = 0; u < CB; ++u) {                          // chunks in order
                const float f = __shfl_sync(0xffffffffu, f_mine, (c0 + u) & 31);
                const float lc = __shfl_sync(0xffffffffu, ml.y, (c0 + u) & 31);
                if (c0 + u < nc && lc > 0.0f) {
                    ll += lc * f;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) acc[i] += oc[u][i] * f;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < DPL; ++i) p.attn[bh * HD + lane + 32 * i] = __float2bfloat16_rn(acc[i] / ll);
    }
}

// ---------------------------------------------------------------- the consumer warps' walk through the layers
template <int HD, int ST, int AG, bool WIDE, bool PAIRS>
__device__ void consumers(const Params& p, Shared* sh, uint32_t ring, float* red, uint8_t* uni) {
    constexpr int NF = WIDE ? 2 : 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = gridDim.x, cta = blockIdx.x, T = p.T, H = p.H;
    unsigned epoch = 0;
    Walk w{0, 0u, 0, 0};
    const int gp = ((G + 3) >> 2) << 2;                        // floats per token in the table of sums
    float* ssq_a = p.ssq;                                      // written by the output projection
    float* ssq_b = p.ssq + (size_t)gp * 16;                    // written by the down projection (and here, first)

    // the split of the keys: launch arguments, or two words on the device that the host refreshes before a replay
    // of a captured launch (the same graph then serves every context length)
    int chunk_pages = p.chunk_pages, n_chunks = p.n_chunks;
    if (p.plan) {
        chunk_pages = __ldg(p.plan);
        n_chunks = __ldg(p.plan + 1);
        if (chunk_pages < 1 || chunk_pages > MAX_CHUNK_PAGES || n_chunks < 1 || n_chunks > MAX_CHUNKS) {
            if (tid == 0 && p.status) atomicCAS(p.status, 0, 204);          // refuse a split the scratch was not sized for
            chunk_pages = MAX_CHUNK_PAGES;
            n_chunks = 1;
        }
    }
    // all chunks of a (sequence, kv head) in one CTA pair: see attention_pair_combine
    const bool pair_split = PAIRS && AG == 2 && chunk_pages <= 64 && (n_chunks == 1 || n_chunks == 2 || n_chunks == 4);
    uint32_t pair_phase = 0;
    if (tid < 2) sh->ptc_key[tid][0] = -1;
    if (tid < T) {
        const int pos = p.positions[tid];
        sh->tok_pos[tid] = pos;
        // a bad page is kept as it is (the cache write checks it again and leaves the write out)
        sh->tok_page[tid] = p.page_table[(size_t)sp_checked_row(p.seq_row[tid], p.rg) * p.max_pages +
                                         sp_checked_entry(pos / KT, p.max_pages, p.rg)];
    }
    // sums of squares of the incoming residual and its product with the first norm's weight: CTA m does token m
    {
        float s = 0.0f;
        if (cta < T) {
            const __nv_bfloat16* w0 = p.layers[0].norm1;
            const __nv_bfloat16* row = nullptr;                  // the token's row of the embedding table, if the kernel embeds
            bool embed = p.embed_w != nullptr, known = true;
            if (embed) {
                const int id = __ldg(p.embed_ids + cta);
                known = id >= 0 && id < p.embed_rows;
                if (!known && tid == 0 && p.status) atomicCAS(p.status, 0, 301);
                row = p.embed_w + (size_t)(known ? id : 0) * H;
            }
            for (int k = tid; k < H; k += CTHREADS) {
                float v;
                if (embed) {
                    v = known ? __bfloat162float(row[k]) : 0.0f;
                    __stcg(p.x + (size_t)cta * H + k, v);
                } else {
                    v = __ldcg(p.x + (size_t)cta * H + k);
                }
                s = fmaf(v, v, s);
                p.xw[(size_t)cta * H + k] = __float2bfloat16_rn(v * __bfloat162float(w0[k]));
            }
        }
        s = sp_warp_sum(s);
        if (lane == 0) sh->warp_sum[warp] = s;
        bar_sync(1, CTHREADS);
        if (tid < MAXT) {
            float tot = 0.0f;
            for (int ww = 0; ww < CWARPS; ++ww) tot += sh->warp_sum[ww];
            __stcg(ssq_b + (size_t)tid * gp + cta, (tid == cta) ? tot : 0.0f);
        }
        grid_sync(p, sh, epoch);
    }

    const uint32_t xn = smem_u32(uni);
    // activation fragments from the normalised residual in shared memory
    auto aload_xn = [&](int kt, uint4 (&a)[SS][NF]) {
#pragma unroll
        for (int s = 0; s < SS; ++s) {
            const int k = kt * KC + warp * WSL + s * 32 + 8 * t;
#pragma unroll
            for (int i = 0; i < NF; ++i) lds128_if(a[s][i], xn + (g + 8 * i) * p.xn_row + k * 2, k < H && g + 8 * i < T);
        }
    };
    // the same from a bfloat16 matrix [T, K] that other CTAs wrote in the phase before
    auto aload_global = [&](const __nv_bfloat16* src, int K, int kt, uint4 (&a)[SS][NF]) {
#pragma unroll
        for (int s = 0; s < SS; ++s) {
            const int k = kt * KC + warp * WSL + s * 32 + 8 * t;
#pragma unroll
            for (int i = 0; i < NF; ++i) ld_cg_u4_if(a[s][i], src + (size_t)(g + 8 * i) * K + k, k < K && g + 8 * i < T);
        }
    };

    auto no_pre = [](int, int, int, int, int, int, int) { return make_float4(0.f, 0.f, 0.f, 0.f); };

    for (int l = 0; l < p.n_layers; ++l) {
        const LayerDesc L = p.layers[l];
        const int nqk = L.nh + L.nkv;

        // ---- QKV, rotation, cache write
        stage_xw(p, sh, ssq_b, L.eps1, xn);
        product<WIDE>(p, sh, job_of<HD>(L, 0, H), w, ring, red, aload_xn, no_pre,
                [&](int rb, int m, int c, float a, float b, int rowA, int rowB, int nA, int nB, const float4&) {
                    if (m >= T || c >= nA) return;
                    const int row = rowA + c, blk = row / HD, d = row % HD;     // d < HD / 2; its partner is HD / 2 on
                    const int pos = sh->tok_pos[m];
                    a *= sh->rstd[m];
                    b *= sh->rstd[m];
                    float lo = a, hi = b;
                    if (blk < nqk) {
                        const float ang = (float)pos * L.inv_freq[d];
                        const float cs = cosf(ang), sn = sinf(ang);
                        lo = a * cs - b * sn;
                        hi = b * cs + a * sn;
                    }
                    __nv_bfloat16* dst;
                    if (blk < L.nh) {
                        dst = p.q + (size_t)m * L.nh * HD + (size_t)blk * HD;
                    } else {
                        const bool is_k = blk < nqk;
                        const int kvh = is_k ? blk - L.nh : blk - nqk;
                        const int page = sh->tok_page[m];
                        if (!sp_index_ok(page, p.rg.n_pages, p.rg, 401)) return;      // debug build: reported, not written
                        dst = (is_k ? L.k_pool : L.v_pool) + (((size_t)page * L.nkv + kvh) * KT + pos % KT) * HD;
                    }
                    dst[d] = __float2bfloat16_rn(lo);
                    dst[d + HD / 2] = __float2bfloat16_rn(hi);
                });
        grid_sync(p, sh, epoch);

        // ---- attention
        const bool paired = PAIRS && pair_split && L.nh <= 8 * L.nkv && p.T * L.nkv * n_chunks <= G * AG;
        if (PAIRS && paired) {
            // (AG == 2: every consumer warp belongs to an attention group) partial results through shared memory
            attention_chunks<HD, ST, AG, 1, true>(p, sh, L, uni, chunk_pages, n_chunks, red);
            attention_pair_combine<HD>(p, sh, L, red, n_chunks, pair_phase);
            grid_sync(p, sh, epoch);
        } else {
            if (warp < 4 * AG) {                     // head tiles of 8: one for up to 8 query heads per kv head, else two
                if (L.nh <= 8 * L.nkv) attention_chunks<HD, ST, AG, 1, false>(p, sh, L, uni, chunk_pages, n_chunks, nullptr);
                else attention_chunks<HD, ST, AG, 2, false>(p, sh, L, uni, chunk_pages, n_chunks, nullptr);
            }
            grid_sync(p, sh, epoch);
            attention_combine<HD>(p, L, n_chunks);
            grid_sync(p, sh, epoch);
        }

        // ---- output projection into the residual
        // residual += product; its square for the next norm's statistics; residual times the next norm's weight
        float ssq = 0.0f;
        const __nv_bfloat16* next_w = L.norm2;
        auto x_pre = [&](int rb, int m, int c, int rowA, int rowB, int nA, int nB) {
            float4 h = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < T && c < nA) { h.x = __ldcg(p.x + (size_t)m * H + rowA + c); h.z = next_w ? __bfloat162float(next_w[rowA + c]) : 0.0f; }
            if (m < T && c < nB) { h.y = __ldcg(p.x + (size_t)m * H + rowB + c); h.w = next_w ? __bfloat162float(next_w[rowB + c]) : 0.0f; }
            return h;
        };
        auto add_into_x = [&](int rb, int m, int c, float a, float b, int rowA, int rowB, int nA, int nB, const float4& h) {
            if (m >= T) return;
            if (c < nA) {
                const float v = h.x + a;
                __stcg(p.x + (size_t)m * H + rowA + c, v);
                p.xw[(size_t)m * H + rowA + c] = __float2bfloat16_rn(v * h.z);
                ssq = fmaf(v, v, ssq);
            }
            if (c < nB) {
                const float v = h.y + b;
                __stcg(p.x + (size_t)m * H + rowB + c, v);
                p.xw[(size_t)m * H + rowB + c] = __float2bfloat16_rn(v * h.w);
                ssq = fmaf(v, v, ssq);
            }
        };
        {
            const int Ko = L.nh * HD;
            product<WIDE>(p, sh, job_of<HD>(L, 1, H), w, ring, red,
                    [&](int kt, uint4 (&a)[SS][NF]) { aload_global(p.attn, Ko, kt, a); },
                    x_pre, add_into_x);
        }
        if (warp < 4) publish_ssq(sh, ssq, ssq_a + cta, gp);
        grid_sync(p, sh, epoch);

        // ---- gate and up with silu(gate)·up
        stage_xw(p, sh, ssq_a, L.eps2, xn);
        product<WIDE>(p, sh, job_of<HD>(L, 2, H), w, ring, red, aload_xn, no_pre,
                [&](int rb, int m, int c, float a, float b, int rowA, int rowB, int nA, int nB, const float4&) {
                    if (m >= T || c >= nA) return;
                    a *= sh->rstd[m];
                    b *= sh->rstd[m];
                    p.act[(size_t)m * L.I + rb * 8 + c] = __float2bfloat16_rn((a / (1.0f + expf(-a))) * b);
                });
        grid_sync(p, sh, epoch);

        // ---- down projection into the residual
        ssq = 0.0f;
        next_w = l + 1 < p.n_layers ? p.layers[l + 1].norm1 : (p.head_mode ? p.final_norm : nullptr);
        {
            const int Kd = L.I;
            product<WIDE>(p, sh, job_of<HD>(L, 3, H), w, ring, red,
                    [&](int kt, uint4 (&a)[SS][NF]) { aload_global(p.act, Kd, kt, a); },
                    x_pre, add_into_x);
        }
        if (warp < 4) publish_ssq(sh, ssq, ssq_b + cta, gp);
        if (l + 1 < p.n_layers || p.head_mode) grid_sync(p, sh, epoch);
    }

    // ---- the output head on the final norm of the residual
    if (p.head_mode) {
        stage_xw(p, sh, ssq_b, p.final_eps, xn);
        Job j;
        j.W = p.head_w; j.N = p.head_rows; j.K = H; j.pair = 0; j.n_blocks = (p.head_rows + 15) / 16;
        float best_v = -INFINITY;                 // of this thread's token and column, over the CTA's blocks
        int best_i = 0x7fffffff;
        const bool logits = p.head_mode == 1;
        product<WIDE>(p, sh, j, w, ring, red, aload_xn, no_pre,
                [&](int rb, int m, int c, float a, float b, int rowA, int rowB, int nA, int nB, const float4&) {
                    if (m >= T) return;
                    a *= sh->rstd[m];
                    b *= sh->rstd[m];
                    if (logits) {
                        float* out = (float*)p.head_out + (size_t)m * p.head_ld;
                        if (c < nA) __stcs(out + rowA + c, a);
                        if (c < nB) __stcs(out + rowB + c, b);
                    } else {
                        if (c < nA) candidate_take(best_v, best_i, a, rowA + c);
                        if (c < nB) candidate_take(best_v, best_i, b, rowB + c);
                    }
                });
        if (!logits) {
            // the epilogue threads of a token (eight columns) leave their finds in shared memory; one thread per token
            // takes the best of them: this CTA's candidate
            Candidate* finds = (Candidate*)red;                  // [16 tokens][8 columns], the K-slice sums are spent
            bar_sync(1, CTHREADS);
            if (tid < 64 * NF) {
                const int e_m = 8 * (tid >> 6) + 2 * ((tid >> 1) & 3) + (tid & 1), e_c = (tid >> 3) & 7;
                finds[e_m * 8 + e_c] = Candidate{best_v, best_i};
            }
            bar_sync(1, CTHREADS);
            if (tid < T) {
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int c = 0; c < 8; ++c) {
                    const Candidate f = finds[tid * 8 + c];
                    if (f.index != 0x7fffffff) candidate_take(bv, bi, f.value, f.index);
                }
                ((Candidate*)p.head_out)[(size_t)tid * p.head_ld + cta] = Candidate{bv, bi};
            }
        }
    }
}

// ---------------------------------------------------------------- the kernel
// HD: head size; ST: stages of the attention's key/value tiles; AG: warp groups that work on attention; PAIRS: launched
// as clusters of two CTAs, with the pair-wise combination of the attention's chunks compiled in
template <int HD, int ST, int AG, bool PAIRS>
__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ Shared sh_;
    Shared* sh = &sh_;
    const uint32_t ring = smem_u32(smem);
    float* red = (float*)(smem + (size_t)p.n_stages * STAGE_BYTES);
    uint8_t* uni = (uint8_t*)(red + 2 * RED_FLOATS);               // normalised residual, or attention tiles
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, cta = blockIdx.x;

    if (tid == 0) {
        for (int s = 0; s < p.n_stages; ++s) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), CWARPS);
        }
        sh->aborted = 0;
        mbar_init(smem_u32(&sh->pair_bar), 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (p.trace && (cta == 0 || cta == 77) && tid == 0) p.trace[cta ? 401 : 1] = global_ns();
    if (warp == CWARPS) {
        copy_warp<HD>(p, sh, ring, lane);
    } else if (p.T > 8) {
        consumers<HD, ST, AG, true, PAIRS>(p, sh, ring, red, uni);
    } else {
        consumers<HD, ST, AG, false, PAIRS>(p, sh, ring, red, uni);
    }
    __syncthreads();
    // the last CTA to finish hands the counters back at zero for the next launch
    __shared__ int is_last;
    if (tid == 0) {
        if (p.trace && cta == 0) p.trace[1023] = global_ns();
        __threadfence();
        const unsigned prev = atomicAdd(&p.sync[1], 1u);
        is_last = prev == (unsigned)G - 1u;
        if (is_last) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            __threadfence();
        }
    }
    __syncthreads();
    // ... and, for a greedy step, takes the best of every token's candidates (one per CTA, all written by now): the
    // largest value, the lowest row among equal values, as a serial scan with a strict ``>`` would
    // (crates/spissa-runtime/src/ops.rs:309-324)
    if (is_last && p.head_mode == 2 && p.tokens && !is_aborted(sh)) {
        __threadfence();
        const Candidate* cand = (const Candidate*)p.head_out;
        for (int m = warp; m < p.T; m += THREADS / 32) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int c = lane; c < G; c += 32) {
                const float v = __ldcg(&cand[(size_t)m * p.head_ld + c].value);
                const int i = __ldcg(&cand[(size_t)m * p.head_ld + c].index);
                if (i != 0x7fffffff) candidate_take(bv, bi, v, i);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                candidate_take(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
            if (lane == 0) {
                const int tok = bi == 0x7fffffff ? 0 : bi;
                p.tokens[m] = tok;
                if (p.header) {
                    const int slot = p.seq_slot[m];
                    if (slot >= 0 && slot < p.n_slots) {
                        int* h = p.header + (size_t)slot * 4;
                        h[0] = p.seq_len[m];
                        h[1] += 1;
                        h[2] = tok;
                    }
                }
            }
        }
    }
}

template <int HD>
constexpr int attention_bytes(int st, int groups) {
    return groups * (16 * Tile<HD>::ROW + 2 * st * Tile<HD>::BYTES + MAX_CHUNK_PAGES * 4);
}
constexpr int ATT_BYTES_64 = attention_bytes<64>(2, 2), ATT_BYTES_128 = attention_bytes<128>(2, 1);

int sm_count() { return sp_sm_count(); }

unsigned long long* trace_buffer = nullptr;

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

// The split of the keys: about one (sequence, kv head, chunk) item per warp group of the grid. Where 1, 2 or 4 chunks
// keep at least three quarters of the groups busy (and the CTAs can be launched as pairs) that split is taken, even if
// the last chunks of a short sequence are empty: the pair-wise combination then saves a phase and a grid barrier.
// chunks per (sequence, kv head) for the pair-wise combination with T sequences, or 0 where it does not pay
int pair_chunks(int G, int T, int hd, int max_nkv) {
    if (hd != 64 || (G % 2) != 0) return 0;
    const int groups = G * 2, items = T * (max_nkv > 0 ? max_nkv : 1);
    const int want = groups / items;
    const int c = want >= 4 ? 4 : (want >= 2 ? 2 : (want >= 1 ? 1 : 0));
    return (c > 0 && 4 * items * c >= 3 * groups) ? c : 0;
}

int plan_split(int G, int T, int hd, int len_pages, int max_nkv, int* chunk_pages, int* n_chunks) {
    if (len_pages < 1) len_pages = 1;
    const int groups = G * (hd == 64 ? 2 : 1);
    int want = groups / (T * (max_nkv > 0 ? max_nkv : 1));
    if (want < 1) want = 1;
    if (const int c = pair_chunks(G, T, hd, max_nkv)) {
        const int per = (len_pages + c - 1) / c;
        if (per <= 64) {
            *chunk_pages = per;
            *n_chunks = c;
            return 0;
        }
    }
    if (want > MAX_CHUNKS) want = MAX_CHUNKS;
    if (want > len_pages) want = len_pages;
    if (want * MAX_CHUNK_PAGES < len_pages) want = (len_pages + MAX_CHUNK_PAGES - 1) / MAX_CHUNK_PAGES;
    if (want > MAX_CHUNKS) SP_FAIL("decode_layers: %d pages per sequence are more than %d chunks of %d hold", len_pages, MAX_CHUNKS, MAX_CHUNK_PAGES);
    *chunk_pages = (len_pages + want - 1) / want;
    *n_chunks = (len_pages + *chunk_pages - 1) / *chunk_pages;
    return 0;
}

}  // namespace

// Optional: 1024 64-bit words on the device into which CTA 0 writes the global timer: [1] at its start, [2e] as it
// enters grid barrier e (e = 1, 2, ...), [2e + 1] as it leaves it, [1023] at its end; CTA 77 does the same from
// word 400 on. Null (the default) switches it off.
SP_API void sp_decode_layers_set_trace(void* buffer) { trace_buffer = (unsigned long long*)buffer; }

// The TMA view of one weight matrix W [N, K] (bfloat16, rows contiguous) as the kernel walks it: row
// blk·2·pair + h·pair + r is element (r, h, blk) of a 4-dimensional tensor [N / (2 pair)][2][pair][K], from which
// one box takes 8 rows of both halves x 256 columns. ``pair`` 0 means plain rows (8 and 8). Writes the 128 bytes of
// the map to ``out`` (host memory); the host copies the maps of all layers to the device, 64-byte aligned.
SP_API int sp_decode_layers_encode_map(void* out, const void* W, int N, int K, int pair) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) SP_FAIL("decode_layers: the driver does not offer cuTensorMapEncodeTiled");
    const int pr = pair > 0 ? pair : 8;
    if ((pr % 8) || (N % (2 * pr)) || (K % 8) || ((uintptr_t)W & 15))
        SP_FAIL("decode_layers: a matrix of %d x %d in row pairs %d apart does not fit the tile walk", N, K, pr);
    cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)pr, 2u, (cuuint64_t)(N / (2 * pr))};
    cuuint64_t strides[3] = {(cuuint64_t)K * 2, (cuuint64_t)pr * K * 2, (cuuint64_t)2 * pr * K * 2};
    cuuint32_t box[4] = {(cuuint32_t)BOXC, 8u, 2u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap map;
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(W), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) SP_FAIL("decode_layers: cuTensorMapEncodeTiled failed with code %d (N %d, K %d, pair %d)", (int)r, N, K, pr);
    memcpy(out, &map, sizeof(map));
    return 0;
}
SP_API int sp_decode_layers_map_bytes() { return (int)sizeof(CUtensorMap); }

// CTAs of the kernel = SMs of the device: the host sizes ``ssq`` ([2][CTAs][16] floats) with it.
SP_API int sp_decode_layers_ctas() { return sm_count(); }
// out[0] = pages per chunk, out[1] = chunks, for ``T`` sequences of at most ``len_pages`` pages
SP_API int sp_decode_layers_plan(int T, int hd, int len_pages, int max_nkv, int* out) {
    const int G = sm_count();
    if (G <= 0) SP_FAIL("decode_layers: cannot read the number of SMs");
    if (T < 1) T = 1;
    return plan_split(G, T, hd, len_pages, max_nkv, out, out + 1);
}
SP_API int sp_decode_layers_max_chunks() { return MAX_CHUNKS; }
SP_API int sp_decode_layers_max_pages() { return MAX_CHUNKS * MAX_CHUNK_PAGES; }
SP_API int sp_decode_layers_desc_bytes() { return (int)sizeof(LayerDesc); }

// Whether the kernel takes these sizes (1) or the layers have to run part by part (0, with the reason as the
// library's last error). ``max_i``, ``max_qdim`` are the largest feed-forward width and heads·head_dim of any layer.
SP_API int sp_decode_layers_supported(int T, int H, int hd, int page_size, int max_heads_per_kv) {
    if (T <= 0 || T > MAXT) { snprintf(sp_error_text, sizeof(sp_error_text), "decode_layers: 1 to %d tokens, got %d", MAXT, T); return 0; }
    if (hd != 64 && hd != 128) { snprintf(sp_error_text, sizeof(sp_error_text), "decode_layers: head_dim %d is not built (64 and 128 are)", hd); return 0; }
    if (page_size != KT) { snprintf(sp_error_text, sizeof(sp_error_text), "decode_layers: pages of %d tokens, built for %d", page_size, KT); return 0; }
    if (H % 8) { snprintf(sp_error_text, sizeof(sp_error_text), "decode_layers: width %d is no multiple of 8", H); return 0; }
    if (max_heads_per_kv > 16) { snprintf(sp_error_text, sizeof(sp_error_text), "decode_layers: %d query heads per kv head, at most 16 fit one tile", max_heads_per_kv); return 0; }
    const int xn = T * (((H * 2 + 127) / 128) * 128 + 64);
    const int att = hd == 64 ? ATT_BYTES_64 : ATT_BYTES_128;
    const int uni = xn > att ? xn : att;
    if ((SMEM_LIMIT - STATIC_SMEM - 2 * RED_FLOATS * 4 - uni) / STAGE_BYTES < 2) {
        snprintf(sp_error_text, sizeof(sp_error_text), "decode_layers: width %d with %d tokens leaves no room for the weight ring", H, T);
        return 0;
    }
    return 1;
}

// ``layers``: n_layers descriptors on the device. ``len_pages``: pages that the longest sequence of the step
// may hold (it only shapes the split of the keys; any actual length is handled). ``max_nkv``: most kv heads of
// any layer. part_o / part_ml hold T·max(nh)·MAX_CHUNKS·(hd + 2) floats together; sync: 3 zeroed words.
// ``plan`` (optional, two int32 on the device: what sp_decode_layers_plan gives) replaces the split made from
// ``len_pages``: a captured launch then serves every length, the host refreshing the two words before a replay.
// The output head for the NEXT call of sp_decode_layers only (mode 0: none): its weight [rows, H] (its tensor map is
// the one behind the layers' in ``maps``), the final norm's weight and eps, and where the result goes: mode 1 logits
// [T, ld] float32, mode 2 candidates [T, ld] pairs of (float32, int32), one per CTA (ld at least sp_decode_layers_ctas()).
namespace {
struct HeadArgs { int mode; const void* w; const void* norm; float eps; int rows; void* out; int ld; } next_head = {0, nullptr, nullptr, 0.f, 0, nullptr, 0};
struct GreedyArgs { int* tokens; int* header; int n_slots; const int* seq_slot; const int* seq_len; } next_greedy = {nullptr, nullptr, 0, nullptr, nullptr};
struct EmbedArgs { const void* w; const int* ids; int rows; } next_embed = {nullptr, nullptr, 0};
}
// For the NEXT call only: the kernel fills the residual itself, x[m] = table[ids[m]] (bfloat16 table [rows, H], ids
// on the device); an id outside the table gives a zero row and code 301 in the status word.
SP_API int sp_decode_layers_set_embedding(const void* table, int rows, const int* ids) {
    if (table && (!ids || rows <= 0)) SP_FAIL("decode_layers: the embedding needs its table's rows and the token ids");
    next_embed = EmbedArgs{table, ids, rows};
    return 0;
}
// With head mode 2, for the NEXT call only: the kernel's last CTA also writes the greedy tokens [T] and, with
// ``header`` [n_slots, 4], notes them in the headers of the step's sequences (slots ``seq_slot``, lengths ``seq_len``).
SP_API int sp_decode_layers_set_greedy_out(int* tokens, int* header, int n_slots, const int* seq_slot, const int* seq_len) {
    if (header && (!seq_slot || !seq_len || n_slots <= 0)) SP_FAIL("decode_layers: noting tokens needs the step's slots and lengths");
    next_greedy = GreedyArgs{tokens, header, n_slots, seq_slot, seq_len};
    return 0;
}
SP_API int sp_decode_layers_set_head(int mode, const void* w, const void* norm, float eps, int rows, void* out, int ld) {
    if (mode < 0 || mode > 2) SP_FAIL("decode_layers: unknown head mode %d", mode);
    if (mode && (!w || !norm || !out || rows <= 0 || ld <= 0)) SP_FAIL("decode_layers: the head needs its weight, the final norm and a place for the result");
    if (mode == 1 && ld < rows) SP_FAIL("decode_layers: logits rows of %d floats do not hold %d", ld, rows);
    if (mode == 2 && ld < sm_count()) SP_FAIL("decode_layers: %d candidates per token, one per CTA (%d) are written", ld, sm_count());
    next_head = HeadArgs{mode, w, norm, eps, rows, out, ld};
    return 0;
}

SP_API int sp_decode_layers(const void* layers, const void* maps, int n_layers, int T, int H, int hd, float* x, void* q, void* attn,
                            void* act, void* xw, float* ssq, float* part_o, float* part_ml, const int* positions,
                            const int* seq_row, const int* page_table, int max_pages, int page_size, int len_pages,
                            int max_nkv, int max_heads_per_kv, const int* plan, unsigned* sync, int* status,
                            cudaStream_t stream) {
    if (n_layers <= 0) return 0;
    if (!sp_decode_layers_supported(T, H, hd, page_size, max_heads_per_kv)) return 1;
    const int G = sm_count();
    if (G <= 0) SP_FAIL("decode_layers: cannot read the number of SMs");
    if (((uintptr_t)x & 15) || ((uintptr_t)q & 15) || ((uintptr_t)attn & 15) || ((uintptr_t)act & 15))
        SP_FAIL("decode_layers: buffers must start on a 16-byte boundary");
    Params p;
    if ((uintptr_t)maps & 63) SP_FAIL("decode_layers: the tensor maps must start on a 64-byte boundary");
    p.layers = (const LayerDesc*)layers;
    p.maps = (const CUtensorMap*)maps;
    p.x = x; p.q = (__nv_bfloat16*)q; p.attn = (__nv_bfloat16*)attn; p.act = (__nv_bfloat16*)act; p.xw = (__nv_bfloat16*)xw;
    p.ssq = ssq; p.part_o = part_o; p.part_ml = part_ml;
    p.positions = positions; p.seq_row = seq_row; p.page_table = page_table;
    p.sync = sync; p.status = status; p.trace = trace_buffer;
    p.n_layers = n_layers; p.T = T; p.H = H; p.max_pages = max_pages;
    p.xn_row = ((H * 2 + 127) / 128) * 128 + 64;
    const int xn = T * p.xn_row;
    const int att = hd == 64 ? ATT_BYTES_64 : ATT_BYTES_128;
    const int uni = xn > att ? xn : att;
    int stages = (SMEM_LIMIT - STATIC_SMEM - 2 * RED_FLOATS * 4 - uni) / STAGE_BYTES;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    p.n_stages = stages;
    p.plan = plan;
    p.pairs = pair_chunks(G, T, hd, max_nkv) > 0 ? 1 : 0;      // CTA pairs only where that split can occur with T sequences
    p.head_mode = next_head.mode;
    p.head_w = (const __nv_bfloat16*)next_head.w;
    p.final_norm = (const __nv_bfloat16*)next_head.norm;
    p.head_out = next_head.out;
    p.final_eps = next_head.eps;
    p.head_rows = next_head.rows;
    p.head_ld = next_head.ld;
    p.tokens = p.head_mode == 2 ? next_greedy.tokens : nullptr;
    p.header = next_greedy.header;
    p.n_slots = next_greedy.n_slots;
    p.seq_slot = next_greedy.seq_slot;
    p.seq_len = next_greedy.seq_len;
    p.embed_w = (const __nv_bfloat16*)next_embed.w;
    p.embed_ids = next_embed.ids;
    p.embed_rows = next_embed.rows;
    p.pad4 = 0;
    next_embed = EmbedArgs{nullptr, nullptr, 0};
    next_head.mode = 0;                                        // for this call only
    next_greedy = GreedyArgs{nullptr, nullptr, 0, nullptr, nullptr};
    p.rg = sp_range_host;
    if (plan_split(G, T, hd, len_pages, max_nkv, &p.chunk_pages, &p.n_chunks)) return 1;
    const int smem = stages * STAGE_BYTES + 2 * RED_FLOATS * 4 + uni;

    void* args[] = {(void*)&p};
    const void* fn = hd == 64 ? (p.pairs ? (const void*)decode_layers_kernel<64, 2, 2, true> : (const void*)decode_layers_kernel<64, 2, 2, false>)
                              : (const void*)decode_layers_kernel<128, 2, 1, false>;
    static SpPerDevice configured[3];
    const int which = hd == 64 ? (p.pairs ? 2 : 0) : 1;
    if (!configured[which].done()) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT - STATIC_SMEM);
        if (e != cudaSuccess) SP_FAIL("decode_layers: cannot reserve shared memory: %s", cudaGetErrorString(e));
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, THREADS, smem);
        if (e != cudaSuccess || per_sm < 1) SP_FAIL("decode_layers: one CTA of %d bytes does not fit an SM", smem);
        configured[which].mark();
    }
    // cooperative (the CTAs wait for one another at the grid barrier), and as clusters of two where the grid is even
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(G);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeCooperative;
    attrs[0].val.cooperative = 1;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = p.pairs ? 2 : 1;
    attrs[1].val.clusterDim.y = 1;
    attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    SP_CHECK_CALL("decode_layers", cudaLaunchKernelExC(&cfg, fn, args));
    return 0;
}
