// The host side of a short prompt step in C++: the launch sequence of every layer in one call.
//
// A prompt of a few dozen tokens is bound by the host: a layer is eight launches (norm, QKV product, rotate and
// store, attention, output projection, norm, gate/up product, down projection: the phases of the reference's block,
// crates/spissa-runtime/src/models/llama/generate.rs:190-778), the kernels take a few microseconds each, and issued
// from Python every launch costs the interpreter ten microseconds or more of argument conversion. Here the sequence
// of all layers runs as one call over a table of layer descriptors that the host part of the library built once from
// what the model's parts say of themselves (weights, sizes, constants: this file knows no model). The kernels are
// the other libraries' own entry points; their addresses are handed over once (sp_host_step_bind) and the choice of
// product kernel by the number of tokens is the same as in the Python path (the thresholds come with the binding).
//
// From 17 to 64 tokens (and head sizes 64 and 128) a layer is five launches instead of eight: the RMS norms, the
// rotation and the cache write ride in the epilogues of the products (sp_tc_stream_fused: see EpiArgs there), as in
// the Python runner of larger prompt steps.
//
// There are no kernels in this file. It allocates nothing: the step's activations live in buffers of the caller.
#include "common.cuh"
#include <string.h>

SP_API const char* sp_host_step_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(host_step)

extern "C" {
typedef int (*RmsnormFn)(const float*, const void*, int, void*, int, const int*, int, int, float, cudaStream_t);
typedef int (*GemvFn)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, cudaStream_t);
typedef int (*GemvSupportedFn)(const void*, const void*, int, int, int, int);
typedef int (*TcStreamFn)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, int*, cudaStream_t);
typedef int (*TcStreamSupportedFn)(const void*, const void*, int, int, int, int, int, int, int);
typedef int (*TcGemmFn)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, int*, cudaStream_t);
typedef int (*TcGemmSupportedFn)(const void*, const void*, int, int, int);
typedef int (*GemmGenericFn)(const void*, int, const void*, int, void*, int, int, int, int, int, int, int, int, cudaStream_t);
typedef int (*SiluMulFn)(const void*, void*, int, int, int, cudaStream_t);
typedef int (*RopeKvWriteFn)(const void*, int, void*, int, void*, void*, int, const int*, const int*, const int*, const int*,
                             int, int, const float*, int, int, int, int, int, int, cudaStream_t);
typedef int (*FlashPrefillFn)(const void*, void*, const void*, const void*, const int*, const int*, const int*, const int*,
                              int, int, int, int, int, int, int, int, float, cudaStream_t);
typedef int (*TcStreamFusedFn)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, const void*, int*, cudaStream_t);
typedef int (*RopeTableFn)(const int*, const int*, const int*, const int*, int, int, const float*, int, int, void*, int*, cudaStream_t);
typedef int (*NormPrepareFn)(const float*, const void*, void*, float*, int, int, cudaStream_t);
typedef const char* (*LastErrorFn)();
}

// The fused epilogues' arguments: the layout of EpiArgs in tc_stream.cu and tc_gemm.cu.
struct EpiArgs {
    const float* row_ssq;
    int n_ssq, norm_width;
    float eps;
    int pad0;
    void* xw;
    const void* next_w;
    float* ssq_out;
    const void* cs;
    const int* tok_page;
    const int* positions;
    void* q_out;
    void* kpool;
    void* vpool;
    int nh, nkv, hd, page_size;
};
static_assert(sizeof(EpiArgs) == 112, "the kernels' libraries read this layout");

// The other libraries' entry points and the thresholds of the kernel choice; the host mirrors this layout.
struct HostKernels {
    RmsnormFn rmsnorm;
    GemvFn gemv;
    GemvSupportedFn gemv_supported;
    TcStreamFn tc_stream;
    TcStreamSupportedFn tc_stream_supported;
    TcGemmFn tc_gemm;
    TcGemmSupportedFn tc_gemm_supported;
    GemmGenericFn gemm_generic;
    SiluMulFn silu_mul;
    RopeKvWriteFn rope_kv_write;
    FlashPrefillFn flash_prefill;
    LastErrorFn err_generic, err_gemv, err_tc_stream, err_tc_gemm, err_attention;
    TcStreamFusedFn tc_stream_fused;
    RopeTableFn rope_table;
    NormPrepareFn norm_prepare;
    int gemv_tokens;           // up to this many tokens the weight-streaming kernel takes a product
    int stream_tokens;         // up to this many the tensor-core kernel that streams the weight
    int flash_query_tile;      // query rows per CTA of the prompt attention
    int pad;
};
static_assert(sizeof(HostKernels) == 19 * 8 + 16, "the host packs this layout");

// One layer: a pre-norm block of an RMS norm, a rotary grouped-query attention and a SwiGLU. All pointers are device
// addresses; weights are bfloat16 [out, in] row-major, the gate/up weight interleaves ``gu_pair`` gate rows and their
// ``gu_pair`` up rows.
struct HostLayer {
    const void* w_qkv;
    const void* w_o;
    const void* w_gu;
    const void* w_down;
    const void* norm1;
    const void* norm2;
    void* k_pool;
    void* v_pool;
    const float* inv_freq;
    int nh, nkv, hd, I;
    int gu_pair, rotary_dim, window, pad;
    float eps1, eps2, scale, padf;
};
static_assert(sizeof(HostLayer) == 9 * 8 + 8 * 4 + 4 * 4, "the host packs this layout");

// The step's arrays (device) and the caller's activation buffers (device, bfloat16 unless marked).
struct HostStep {
    float* h;                  // [T, H] the 32-bit residual stream, in and out
    void* x;                   // [T, H] normed rows
    float* qkv;                // [T, (nh + 2 nkv) hd] float32: the rotation reads unrounded products
    void* q;                   // [T, nh hd]
    void* ctx;                 // [T, nh hd]
    void* act;                 // [T, I]
    void* gu;                  // [T, 2 I] only where no kernel applies silu(gate)·up itself
    const int* token_seq;
    const int* positions;
    const int* seq_row;
    const int* page_table;
    const int* seq_start;
    int* status;
    // the fused sequence (17 tokens or more) only: two buffers each of residual ⊙ norm weight [T, H] bfloat16 and of
    // the rows' partial sums of squares [T, (H + 127) / 128] float32, the step's (cos, sin) table [T, hd / 2] and the
    // tokens' cache pages [T]
    void* xw[2];
    float* ssq[2];
    void* cs;
    int* tok_page;
    int T, H, n_seqs, max_pages, page_size, n_q_tiles, fused, pad1;
};
static_assert(sizeof(HostStep) == 19 * 8 + 8 * 4, "the host packs this layout");

namespace {

HostKernels kernels;
bool bound = false;
int launches = 0;

int fail_from(LastErrorFn f, const char* what) {
    const char* t = f ? f() : nullptr;
    snprintf(sp_error_text, sizeof(sp_error_text), "%s: %s", what, (t && *t) ? t : "the kernel library refused the call");
    return 1;
}

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SILU_MUL = 2, MODE_STREAM_QKV_ROPE = 4 };
enum { DT_F32 = 0, DT_BF16 = 1 };

// y = x · Wᵀ for bfloat16 x [M, K] and W [N, K]: the kernel by the number of tokens, as the Python path chooses it
int linear(const void* x, const void* W, void* out, int out_dt, int M, int N, int K, int ldo, int mode, int pair, int* status,
           cudaStream_t stream) {
    const HostKernels& k = kernels;
    ++launches;
    if (M <= k.gemv_tokens && k.gemv_supported(x, W, M, K, K, K) == 0) {
        if (k.gemv(x, W, out, out_dt, M, N, K, K, K, ldo, mode, pair, stream)) return fail_from(k.err_gemv, "host step");
        return 0;
    }
    if (M <= k.stream_tokens && k.tc_stream_supported(x, W, M, N, K, K, K, mode, pair) == 0) {
        if (k.tc_stream(x, W, out, out_dt, M, N, K, K, K, ldo, mode, pair, status, stream)) return fail_from(k.err_tc_stream, "host step");
        return 0;
    }
    if (k.tc_gemm_supported(x, W, K, K, K) == 0) {
        // one row of tiles (at most 128 tokens here): 128-wide tiles, or the gate/up pair's width
        const int bn = mode == MODE_SILU_MUL ? 2 * pair : 128;
        if (k.tc_gemm(x, W, out, out_dt, M, N, K, K, K, ldo, mode, bn, status, stream)) return fail_from(k.err_tc_gemm, "host step");
        return 0;
    }
    if (mode == MODE_SILU_MUL) SP_FAIL("host step: no kernel applies silu(gate)·up for these sizes");
    if (k.gemm_generic(x, DT_BF16, W, DT_BF16, out, out_dt, M, N, K, K, K, ldo, mode == MODE_ACCUMULATE, stream))
        return fail_from(k.err_generic, "host step");
    return 0;
}

// One layer of the fused sequence. ``n_ssq``: partial sums per row that st.ssq[0] holds for this layer's first norm.
int fused_layer(const HostLayer& L, const HostLayer* next, const HostStep& st, int& n_ssq, cudaStream_t stream) {
    const HostKernels& k = kernels;
    const int nq = L.nh * L.hd, nqkv = (L.nh + 2 * L.nkv) * L.hd;
    const int tiles = (st.H + 127) / 128;
    EpiArgs ep;
    // QKV on residual ⊙ norm weight, scaled by 1/rms, rotated; q stored, k and v into the cache
    memset(&ep, 0, sizeof(ep));
    ep.row_ssq = st.ssq[0]; ep.n_ssq = n_ssq; ep.norm_width = st.H; ep.eps = L.eps1;
    ep.cs = st.cs; ep.tok_page = st.tok_page; ep.positions = st.positions;
    ep.q_out = st.q; ep.kpool = L.k_pool; ep.vpool = L.v_pool;
    ep.nh = L.nh; ep.nkv = L.nkv; ep.hd = L.hd; ep.page_size = st.page_size;
    ++launches;
    if (k.tc_stream_fused(st.xw[0], L.w_qkv, nullptr, DT_BF16, st.T, nqkv, st.H, st.H, st.H, 0, MODE_STREAM_QKV_ROPE, 0, &ep,
                          st.status, stream)) return fail_from(k.err_tc_stream, "host step");
    ++launches;
    if (k.flash_prefill(st.q, st.ctx, L.k_pool, L.v_pool, st.seq_start, st.positions, st.seq_row, st.page_table, st.max_pages,
                        st.page_size, st.n_seqs, st.n_q_tiles, L.nh, L.nkv, L.hd, L.window, L.scale, stream))
        return fail_from(k.err_attention, "host step");
    // output projection into the residual; the same epilogue writes residual ⊙ second norm weight and its statistics
    memset(&ep, 0, sizeof(ep));
    ep.xw = st.xw[1]; ep.next_w = L.norm2; ep.ssq_out = st.ssq[1];
    ++launches;
    if (k.tc_stream_fused(st.ctx, L.w_o, st.h, DT_F32, st.T, st.H, nq, nq, nq, st.H, MODE_ACCUMULATE, 0, &ep, st.status, stream))
        return fail_from(k.err_tc_stream, "host step");
    // gate/up on it, scaled by 1/rms, with silu(gate)·up
    memset(&ep, 0, sizeof(ep));
    ep.row_ssq = st.ssq[1]; ep.n_ssq = tiles; ep.norm_width = st.H; ep.eps = L.eps2;
    ++launches;
    if (k.tc_stream_fused(st.xw[1], L.w_gu, st.act, DT_BF16, st.T, 2 * L.I, st.H, st.H, st.H, L.I, MODE_SILU_MUL, L.gu_pair, &ep,
                          st.status, stream)) return fail_from(k.err_tc_stream, "host step");
    // down projection into the residual, preparing the next layer's first norm
    ++launches;
    if (next) {
        memset(&ep, 0, sizeof(ep));
        ep.xw = st.xw[0]; ep.next_w = next->norm1; ep.ssq_out = st.ssq[0];
        if (k.tc_stream_fused(st.act, L.w_down, st.h, DT_F32, st.T, st.H, L.I, L.I, L.I, st.H, MODE_ACCUMULATE, 0, &ep, st.status,
                              stream)) return fail_from(k.err_tc_stream, "host step");
        n_ssq = tiles;
    } else if (k.tc_stream(st.act, L.w_down, st.h, DT_F32, st.T, st.H, L.I, L.I, L.I, st.H, MODE_ACCUMULATE, 0, st.status, stream)) {
        return fail_from(k.err_tc_stream, "host step");
    }
    return 0;
}

}  // namespace

SP_API int sp_host_step_bind(const void* table, int bytes) {
    if (bytes != (int)sizeof(HostKernels)) SP_FAIL("host step: the kernel table has %d bytes, %d are expected", bytes, (int)sizeof(HostKernels));
    memcpy(&kernels, table, sizeof(kernels));
    if (!kernels.rmsnorm || !kernels.gemv || !kernels.tc_stream || !kernels.tc_gemm || !kernels.rope_kv_write ||
        !kernels.flash_prefill || !kernels.tc_stream_fused || !kernels.rope_table || !kernels.norm_prepare)
        SP_FAIL("host step: an entry point is missing from the kernel table");
    bound = true;
    return 0;
}
SP_API int sp_host_step_layer_bytes() { return (int)sizeof(HostLayer); }
SP_API int sp_host_step_step_bytes() { return (int)sizeof(HostStep); }
SP_API int sp_host_step_kernels_bytes() { return (int)sizeof(HostKernels); }
// Launches that the last call of sp_host_step_prompt_layers made.
SP_API int sp_host_step_launches() { return launches; }

// Every layer of a prompt step (several tokens per sequence, at most 128 in all) on the residual ``st->h``, in place:
// ``layers`` are n_layers descriptors in host memory, run in order. Returns 0, or 1 with the reason as the last error.
SP_API int sp_host_step_prompt_layers(const void* layers_raw, int n_layers, const void* step_raw, cudaStream_t stream) {
    if (!bound) SP_FAIL("host step: sp_host_step_bind has not been called");
    const HostLayer* layers = (const HostLayer*)layers_raw;
    const HostStep& st = *(const HostStep*)step_raw;
    const HostKernels& k = kernels;
    launches = 0;
    if (st.T <= 0 || n_layers <= 0) return 0;
    if (st.fused) {
        if (!st.xw[0] || !st.xw[1] || !st.ssq[0] || !st.ssq[1] || !st.cs || !st.tok_page)
            SP_FAIL("host step: the fused sequence needs its buffers");
        ++launches;
        if (k.norm_prepare(st.h, layers[0].norm1, st.xw[0], st.ssq[0], st.T, st.H, stream)) return fail_from(k.err_generic, "host step");
        int n_ssq = 1;
        const float* table_of = nullptr;                 // layers with the same frequency table share the step's angles
        for (int l = 0; l < n_layers; ++l) {
            const HostLayer& L = layers[l];
            if (L.hd != layers[0].hd) SP_FAIL("host step: the fused sequence takes one head size, got %d and %d", layers[0].hd, L.hd);
            if (L.inv_freq != table_of) {
                ++launches;
                if (k.rope_table(st.positions, st.token_seq, st.seq_row, st.page_table, st.max_pages, st.page_size, L.inv_freq,
                                 L.hd / 2, st.T, st.cs, st.tok_page, stream)) return fail_from(k.err_generic, "host step");
                table_of = L.inv_freq;
            }
            if (fused_layer(L, l + 1 < n_layers ? &layers[l + 1] : nullptr, st, n_ssq, stream)) return 1;
        }
        return 0;
    }
    for (int l = 0; l < n_layers; ++l) {
        const HostLayer& L = layers[l];
        const int nq = L.nh * L.hd, nqkv = (L.nh + 2 * L.nkv) * L.hd;
        // norm, QKV (unrounded), rotation and cache write
        ++launches;
        if (k.rmsnorm(st.h, L.norm1, DT_BF16, st.x, DT_BF16, nullptr, st.T, st.H, L.eps1, stream)) return fail_from(k.err_generic, "host step");
        if (linear(st.x, L.w_qkv, st.qkv, DT_F32, st.T, nqkv, st.H, nqkv, MODE_STORE, 0, st.status, stream)) return 1;
        ++launches;
        if (k.rope_kv_write(st.qkv, DT_F32, st.q, DT_BF16, L.k_pool, L.v_pool, DT_BF16, st.token_seq, st.positions, st.seq_row,
                            st.page_table, st.max_pages, st.page_size, L.inv_freq, st.T, L.nh, L.nkv, L.hd, L.rotary_dim, 1, stream))
            return fail_from(k.err_generic, "host step");
        // attention over the cache, then the output projection into the residual
        ++launches;
        if (k.flash_prefill(st.q, st.ctx, L.k_pool, L.v_pool, st.seq_start, st.positions, st.seq_row, st.page_table, st.max_pages,
                            st.page_size, st.n_seqs, st.n_q_tiles, L.nh, L.nkv, L.hd, L.window, L.scale, stream))
            return fail_from(k.err_attention, "host step");
        if (linear(st.ctx, L.w_o, st.h, DT_F32, st.T, st.H, nq, st.H, MODE_ACCUMULATE, 0, st.status, stream)) return 1;
        // norm, gate/up with silu(gate)·up, down projection into the residual
        ++launches;
        if (k.rmsnorm(st.h, L.norm2, DT_BF16, st.x, DT_BF16, nullptr, st.T, st.H, L.eps2, stream)) return fail_from(k.err_generic, "host step");
        if (linear(st.x, L.w_gu, st.act, DT_BF16, st.T, 2 * L.I, st.H, L.I, MODE_SILU_MUL, L.gu_pair, st.status, stream)) return 1;
        if (linear(st.act, L.w_down, st.h, DT_F32, st.T, st.H, L.I, st.H, MODE_ACCUMULATE, 0, st.status, stream)) return 1;
    }
    return 0;
}
