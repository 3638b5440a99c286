// Temperature / top-k / top-p sampling on the device, one block per row of logits.
//
// Meaning, as in the reference (crates/spissa-runtime/src/ops.rs:377-430):
//   probs = softmax(logits / temperature); tokens ordered by falling probability,
//   equal ones by rising index (a stable sort); keep the first top_k (0 = all); of
//   those keep the shortest prefix whose mass reaches top_p; draw u·(kept mass) and
//   walk the kept list until the running mass reaches it. If nothing is hit, the most
//   probable token is returned (ops.rs:429).
// The order is made with a bitonic sort of 64-bit keys (inverted probability bits,
// then index) in caller-provided scratch memory of rows · n2 keys, n2 the next power
// of two ≥ V. Sums are 32-bit block scans; they differ from a serial walk by rounding.
#include "common.cuh"

SP_API const char* sp_sampling_last_error() { return sp_error_text; }

#define SS_THREADS 1024
#define SS_CHUNK 4096          // keys sorted in shared memory at a time (32 KB)

__device__ __forceinline__ void ss_cmpswap(unsigned long long& a, unsigned long long& b, bool asc) {
    if ((a > b) == asc) { const unsigned long long t = a; a = b; b = t; }
}

// all passes with stride < SS_CHUNK of merge size k, for the chunk starting at base
__device__ void ss_chunk_passes(unsigned long long* keys, unsigned long long* sh, size_t base,
                                unsigned k, unsigned j_from, unsigned chunk) {
    for (unsigned i = threadIdx.x; i < chunk; i += blockDim.x) sh[i] = keys[base + i];
    __syncthreads();
    for (unsigned j = j_from; j > 0; j >>= 1) {
        for (unsigned i = threadIdx.x; i < chunk; i += blockDim.x) {
            const unsigned x = i ^ j;
            if (x > i) {
                const bool asc = (((unsigned)base + i) & k) == 0;
                unsigned long long a = sh[i], b = sh[x];
                if ((a > b) == asc) { sh[i] = b; sh[x] = a; }
            }
        }
        __syncthreads();
    }
    for (unsigned i = threadIdx.x; i < chunk; i += blockDim.x) keys[base + i] = sh[i];
    __syncthreads();
}

// inclusive block scan of one value per thread; returns the thread's inclusive sum
__device__ __forceinline__ float ss_block_scan(float v, float* warp_tot, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += n;
        }
        warp_tot[lane] = w;
    }
    __syncthreads();
    if (warp > 0) v += warp_tot[warp - 1];
    *total = warp_tot[31];
    return v;
}

__device__ __forceinline__ float ss_key_prob(unsigned long long key) {
    return __uint_as_float(~(unsigned)(key >> 32));
}

// first r in [0, n) whose running mass reaches target, or n; also the mass of [0, n)
__device__ unsigned ss_first_reaching(const unsigned long long* keys, unsigned n, float target,
                                      float* warp_tot, unsigned* found, float* mass_out) {
    if (threadIdx.x == 0) *found = n;
    float carry = 0.0f;
    __syncthreads();
    for (unsigned base = 0; base < n; base += blockDim.x) {
        const unsigned r = base + threadIdx.x;
        const float p = r < n ? ss_key_prob(keys[r]) : 0.0f;
        float tile_total;
        const float cum = carry + ss_block_scan(p, warp_tot, &tile_total);
        if (r < n && cum >= target) atomicMin(found, r);
        carry += tile_total;
        __syncthreads();
        if (*found < n) break;          // uniform: read after the barrier
        __syncthreads();
    }
    __syncthreads();
    if (mass_out) *mass_out = carry;
    return *found;
}

__global__ void __launch_bounds__(SS_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int ld, int V, unsigned n2, float temperature, int top_k,
                   float top_p, const float* __restrict__ u, unsigned long long* __restrict__ scratch,
                   int* __restrict__ out) {
    __shared__ unsigned long long sh[SS_CHUNK];
    __shared__ float red[32];
    __shared__ unsigned found;
    const int row_id = blockIdx.x;
    const float* row = logits + (size_t)row_id * ld;
    unsigned long long* keys = scratch + (size_t)row_id * n2;

    // softmax of logits / temperature: exp(x - max), then divided by the sum
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, row[c] / temperature);
    mx = sp_block_max(mx, red);
    float sum = 0.0f;
    for (int c = threadIdx.x; c < V; c += blockDim.x) sum += expf(row[c] / temperature - mx);
    sum = sp_block_sum(sum, red);
    for (unsigned c = threadIdx.x; c < n2; c += blockDim.x) {
        unsigned long long key = ~0ull;
        if (c < (unsigned)V) {
            float p = expf(row[c] / temperature - mx) / sum;
            if (!(p >= 0.0f)) p = 0.0f;                       // NaN logits never win
            key = ((unsigned long long)(~__float_as_uint(p)) << 32) | c;
        }
        keys[c] = key;
    }
    __syncthreads();

    // bitonic sort, ascending keys = falling probability, rising index
    const unsigned chunk = n2 < SS_CHUNK ? n2 : SS_CHUNK;
    for (size_t base = 0; base < n2; base += chunk) {
        // every merge size up to the chunk, in shared memory
        for (unsigned i = threadIdx.x; i < chunk; i += blockDim.x) sh[i] = keys[base + i];
        __syncthreads();
        for (unsigned k = 2; k <= chunk; k <<= 1) {
            for (unsigned j = k >> 1; j > 0; j >>= 1) {
                for (unsigned i = threadIdx.x; i < chunk; i += blockDim.x) {
                    const unsigned x = i ^ j;
                    if (x > i) {
                        const bool asc = (((unsigned)base + i) & k) == 0;
                        unsigned long long a = sh[i], b = sh[x];
                        if ((a > b) == asc) { sh[i] = b; sh[x] = a; }
                    }
                }
                __syncthreads();
            }
        }
        for (unsigned i = threadIdx.x; i < chunk; i += blockDim.x) keys[base + i] = sh[i];
        __syncthreads();
    }
    for (unsigned k = chunk << 1; k <= n2 && k != 0; k <<= 1) {
        unsigned j = k >> 1;
        for (; j >= chunk; j >>= 1) {
            for (unsigned i = threadIdx.x; i < n2; i += blockDim.x) {
                const unsigned x = i ^ j;
                if (x > i) {
                    const bool asc = (i & k) == 0;
                    unsigned long long a = keys[i], b = keys[x];
                    if ((a > b) == asc) { keys[i] = b; keys[x] = a; }
                }
            }
            __syncthreads();
        }
        for (size_t base = 0; base < n2; base += chunk) ss_chunk_passes(keys, sh, base, k, j, chunk);
    }

    unsigned kept = (top_k > 0 && top_k < V) ? (unsigned)top_k : (unsigned)V;
    // shortest prefix whose mass reaches top_p
    {
        const unsigned r = ss_first_reaching(keys, kept, top_p, red, &found, nullptr);
        if (r < kept) kept = r + 1;
    }
    __shared__ float mass;
    {
        // mass of the kept prefix
        float m = 0.0f;
        for (unsigned r = threadIdx.x; r < kept; r += blockDim.x) m += ss_key_prob(keys[r]);
        m = sp_block_sum(m, red);
        if (threadIdx.x == 0) mass = m;
        __syncthreads();
    }
    const float target = u[row_id] * mass;
    const unsigned r = ss_first_reaching(keys, kept, target, red, &found, nullptr);
    if (threadIdx.x == 0) out[row_id] = (int)(unsigned)(keys[r < kept ? r : 0] & 0xffffffffu);
}

SP_API long long sp_sample_scratch_keys(int rows, int V) {
    unsigned n2 = 1;
    while (n2 < (unsigned)V) n2 <<= 1;
    return (long long)rows * n2;
}

SP_API int sp_sample_rows(const float* logits, int ld, int rows, int V, float temperature, int top_k,
                          float top_p, const float* u, void* scratch, long long scratch_keys, int* out,
                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0) SP_FAIL("sample: empty rows");
    if (!(temperature > 0.0f)) SP_FAIL("sample: temperature must be positive here (greedy rows use argmax)");
    if (!(top_p > 0.0f && top_p <= 1.0f)) SP_FAIL("sample: top_p must be in (0, 1], got %g", (double)top_p);
    if (top_k < 0) SP_FAIL("sample: top_k must not be negative");
    if (V > (1 << 30)) SP_FAIL("sample: vocabulary %d is beyond this kernel's limit", V);
    unsigned n2 = 1;
    while (n2 < (unsigned)V) n2 <<= 1;
    if (scratch_keys < (long long)rows * n2)
        SP_FAIL("sample: scratch holds %lld keys, %lld are needed", scratch_keys, (long long)rows * n2);
    sample_rows_kernel<<<rows, SS_THREADS, 0, stream>>>(logits, ld, V, n2, temperature, top_k, top_p, u,
                                                        (unsigned long long*)scratch, out);
    SP_CHECK_LAUNCH("sample_rows");
    return 0;
}
