// Shared helpers for every kernel file: element loads and stores by storage type,
// warp and block reductions with a fixed order, launch-error reporting.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define SP_DT_F32 0
#define SP_DT_BF16 1

#define SP_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------- error text
// Each library keeps the text of its last refusal; the host reads it after a
// non-zero return code. Nothing here aborts the process.
static thread_local char sp_error_text[512];

#define SP_FAIL(...)                                              \
    do {                                                          \
        snprintf(sp_error_text, sizeof(sp_error_text), __VA_ARGS__); \
        return 1;                                                 \
    } while (0)

#define SP_CHECK_LAUNCH(name)                                                      \
    do {                                                                           \
        cudaError_t e_ = cudaGetLastError();                                       \
        if (e_ != cudaSuccess) SP_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

// ---------------------------------------------------------------- element access
__device__ __forceinline__ float sp_ld(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float sp_ld(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void sp_st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void sp_st(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// two neighbouring elements at an even index (the arrays' rows have even length)
__device__ __forceinline__ void sp_st2(float* p, size_t i, float a, float b) { *(float2*)(p + i) = make_float2(a, b); }
__device__ __forceinline__ void sp_st2(__nv_bfloat16* p, size_t i, float a, float b) {
    *(__nv_bfloat162*)(p + i) = __floats2bfloat162_rn(a, b);
}

__device__ __forceinline__ float sp_ld_dt(const void* p, int dt, size_t i) {
    return dt == SP_DT_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void sp_st_dt(void* p, int dt, size_t i, float v) {
    if (dt == SP_DT_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------- reductions
__device__ __forceinline__ float sp_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float sp_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. ``scratch``
// holds 32 floats. The order of additions depends only on blockDim.
__device__ __forceinline__ float sp_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = sp_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? scratch[lane] : 0.0f;
    r = sp_warp_sum(r);
    return r;
}
__device__ __forceinline__ float sp_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = sp_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? scratch[lane] : -INFINITY;
    r = sp_warp_max(r);
    return r;
}

// ---------------------------------------------------------------- launches with a cluster dimension
// ``cluster_x`` CTAs that follow one another in x form a thread-block cluster (1 = none).
// negative ``cluster_x``: |cluster_x| CTAs per cluster AND launched as a programmatic dependent (see below)
template <typename... KArgs, typename... Args>
static inline cudaError_t sp_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, int cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n = 0;
    if (cluster_x < 0) {
        cluster_x = -cluster_x;
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = (unsigned)cluster_x;
        attrs[n].val.clusterDim.y = 1;
        attrs[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with sp_launch_dependent may become resident while the kernel before it in the stream is still
// running (on SMs whose CTAs of that kernel have left): it sets up (barriers, tensor memory) and then waits in
// sp_wait_for_predecessor() until the predecessor has finished and its writes are visible; it touches no global
// memory before that. The predecessor allows it by sp_allow_dependents() (the launch happens once every CTA of it
// has said so or has left, so no CTA of the predecessor is ever kept from an SM). Between long kernels this hides the
// launch gap and the dependent's set-up.
__device__ __forceinline__ void sp_allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void sp_wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t sp_launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

#define SP_CHECK_CALL(name, call)                                                   \
    do {                                                                           \
        cudaError_t e_ = (call);                                                   \
        if (e_ != cudaSuccess) SP_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)


// ---------------------------------------------------------------- once per device
// cudaFuncSetAttribute and the like hold for the device that is current when they are called, so "done once" has
// to be remembered per device: a bit per device index (devices beyond 63 are set up at every call). Two host threads
// that make the first call on a device at the same time both do the set-up, with the same values.
struct SpPerDevice {
    unsigned long long mask = 0;
    int device() const {
        int d = -1;
        return cudaGetDevice(&d) == cudaSuccess ? d : -1;
    }
    bool done() const {
        const int d = device();
        return d >= 0 && d < 64 && ((mask >> d) & 1ull);
    }
    void mark() {
        const int d = device();
        if (d >= 0 && d < 64) mask |= 1ull << d;
    }
};

// streaming multiprocessors of the current device (0 when it cannot be read)
static inline int sp_sm_count() {
    static int count[64];
    int d = -1;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0) return 0;
    if (d < 64 && count[d] > 0) return count[d];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) return 0;
    if (d < 64) count[d] = n;
    return n;
}


// ---------------------------------------------------------------- range checks of the debug build
// Built with -DSP_RANGE_CHECK, every kernel that takes an index from a table that the host packed (a page from a
// page table, a row of that table from ``seq_row``, a page slot from a position) compares it with the bounds the
// host declared for the call, records a code in the status word when it lies outside and leaves the access out (a
// write is skipped, a read goes to page or row 0 instead): no trap, no assert, the kernel ends normally and the host
// raises. It stands in for a memory checker where none can be run. In the regular build the checks compile to
// nothing. Codes: 401 a page beyond the pools, 402 a row beyond the page table, 403 a position beyond the table's width.
struct SpRange {
    int n_pages;      // pages the key/value pools hold
    int n_rows;       // rows of the page table
    int* status;
};
static SpRange sp_range_host = {0, 0, nullptr};        // one per library: what the next launches are given

#ifdef SP_RANGE_CHECK
#define SP_RANGE_CHECKED 1
#else
#define SP_RANGE_CHECKED 0
#endif

__device__ __forceinline__ bool sp_index_ok(long long v, long long n, const SpRange& rg, int code) {
#ifdef SP_RANGE_CHECK
    if (v < 0 || v >= n) {
        if (rg.status) atomicCAS(rg.status, 0, code);
        return false;
    }
#endif
    return true;
}
__device__ __forceinline__ int sp_checked_page(int page, const SpRange& rg) { return sp_index_ok(page, rg.n_pages, rg, 401) ? page : 0; }
__device__ __forceinline__ int sp_checked_row(int row, const SpRange& rg) { return sp_index_ok(row, rg.n_rows, rg, 402) ? row : 0; }
__device__ __forceinline__ int sp_checked_entry(int entry, int width, const SpRange& rg) { return sp_index_ok(entry, width, rg, 403) ? entry : 0; }

// Every library exports whether it is the debug build and takes the bounds for its next launches.
#define SP_DEFINE_RANGE_API(module)                                                                  \
    SP_API int sp_##module##_range_checked() { return SP_RANGE_CHECKED; }                            \
    SP_API void sp_##module##_set_bounds(int n_pages, int n_rows, int* status) {                     \
        sp_range_host.n_pages = n_pages;                                                             \
        sp_range_host.n_rows = n_rows;                                                               \
        sp_range_host.status = status;                                                               \
    }
