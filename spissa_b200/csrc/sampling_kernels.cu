// Temperature / top-k / top-p sampling on the device, without sorting: a thread-block cluster per row of logits.
//
// Meaning, as in the reference (crates/spissa-runtime/src/ops.rs:377-430):
//   probs = softmax(logits / temperature); tokens ordered by falling probability,
//   equal ones by rising index (a stable sort); keep the first top_k (0 = all); of
//   those keep the shortest prefix whose mass reaches top_p; draw u·(kept mass) and
//   walk the kept list until the running mass reaches it. If nothing is hit, the most
//   probable token is returned (ops.rs:429).
//
// Every step of that walk asks the same question: which is the first token, in that order, at which a
// running total (a count for top-k, a mass for top-p and for the draw) reaches a target? The order is the
// rising order of a 64-bit key (inverted probability bits, then index), keys are unique, and the total up
// to a key is a plain sum over the tokens with smaller or equal keys. So the token is found by descending
// the key four bits at a time: one pass over the row adds every token that is still in question into one
// of 16 sums by its next four key bits, the sums are added up in rising order until the target is
// reached, and the search goes on inside that one. A pass touches only tokens that share the bits chosen
// so far; once a single token is left it is looked up and the search ends (a peaked distribution is done
// after a few passes; equal probabilities are told apart by the index bits of the key).
//
// Sums are integers: a probability counts as floor(p · 2^44) and a token as 1 in the high bits of the same
// 64-bit word, so every total is exact and independent of the order of addition (the same draw always
// gives the same token), and finer than the 32-bit running sum of a serial walk. Each thread adds into
// words of its own in shared memory (no atomics); the CTAs of the cluster take slices of the row and add
// their 16 sums through distributed shared memory, so every CTA takes every decision alike.
#include "common.cuh"

SP_API const char* sp_sampling_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(sampling)

namespace {

constexpr int SS_CLUSTER = 8;                      // CTAs per row; 256 threads each, 1024 when few rows leave SMs idle
constexpr int SS_SEGS = 16;                        // sums per pass: four key bits
constexpr int MASS_BITS = 45;                      // low bits: mass in units of 2^-44 (a row's total stays below 2^45)
constexpr unsigned long long MASS_MASK = (1ull << MASS_BITS) - 1;
constexpr unsigned long long ONE_TOKEN = 1ull << MASS_BITS;      // the count lives in the 19 bits above
constexpr float MASS_UNIT = 17592186044416.0f;     // 2^44
constexpr int SS_MAX_V = (1 << (64 - MASS_BITS)) - 1;

__device__ __forceinline__ unsigned ss_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void ss_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned ss_peer_addr(const void* local, unsigned rank) {
    unsigned ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
    return ra;
}
__device__ __forceinline__ unsigned long long ss_ld_peer_u64(const void* local, unsigned rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(ss_peer_addr(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ float ss_ld_peer_f32(const void* local, unsigned rank) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ss_peer_addr(local, rank)) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long ss_key(unsigned prob_bits, unsigned idx) {
    return ((unsigned long long)(~prob_bits) << 32) | idx;
}
// One token and its mass floor(p · 2^44), p in [0, 1], from the float's fields: (1.m) · 2^(e - 127 + 44 - 23).
__device__ __forceinline__ unsigned long long ss_weight(unsigned prob_bits) {
    const int e = (int)(prob_bits >> 23);                     // the sign bit is clear
    const unsigned long long m = (unsigned long long)((prob_bits & 0x7fffffu) | 0x800000u);
    const int up = e - 106;                                    // e - 127 + 21
    const unsigned long long q = e == 0 ? 0ull : (up >= 0 ? m << up : (up > -24 ? m >> -up : 0ull));
    return ONE_TOKEN + q;
}

struct Shared {
    unsigned long long* acc;                       // [16][threads]: every thread's own 16 sums (dynamic shared memory)
    unsigned long long seg[2][SS_SEGS];            // this CTA's sums of a pass (two buffers: peers read one while the next fills)
    unsigned long long total[SS_SEGS];             // the cluster's sums
    unsigned long long loc;                        // this CTA's find of a lookup (0: none)
    float stat[2];                                 // this CTA's maximum / sum of exponentials
    float red[32];
};

struct Row {
    const unsigned* bits;      // probability bits of this CTA's slice of the row: bits[i - i0], in shared memory when it fits
    int i0, i1;                // the slice
    int idx_digits;            // four-bit digits that hold an index
};

// The first key (rising) among those ≤ ``limit`` at which the running count (by_mass false) or mass reaches
// ``target``. Returns false when even the total does not; ``upto`` is then that total. Else ``key`` is the
// token's key and ``upto`` the packed total up to and including it. Every thread of the cluster runs this alike.
template <int THREADS>
__device__ bool ss_descend(Shared* sh, const Row& row, bool by_mass, unsigned long long target, unsigned long long limit,
                           unsigned& parity, unsigned long long& key, unsigned long long& upto) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned long long* acc = sh->acc;
    unsigned long long prefix = 0, below = 0;
    const int n_digits = 8 + row.idx_digits;
    for (int d = 0; d < n_digits; ++d) {
        const int shift = d < 8 ? 60 - 4 * d : 4 * (n_digits - 1 - d);
        // bits above this digit that a token must share with the prefix (all of them; none in the first pass)
        const unsigned long long above = d == 0 ? 0ull : ~0ull << (shift + 4 > 63 ? 63 : shift + 4);
#pragma unroll
        for (int s = 0; s < SS_SEGS; ++s) acc[s * THREADS + tid] = 0ull;
        if (d < 8) {
            // a digit of the probability: 32-bit arithmetic on the key's upper half; the index only settles
            // whether a token with the limit's own probability is still inside
            const unsigned lim_hi = (unsigned)(limit >> 32), lim_lo = (unsigned)limit;
            const unsigned pre_hi = (unsigned)(prefix >> 32), above_hi = (unsigned)(above >> 32);
            const int sh_hi = shift - 32;
            for (int i = row.i0 + tid; i < row.i1; i += THREADS) {
                const unsigned b = row.bits[i - row.i0];
                const unsigned kb = ~b;
                if (((kb ^ pre_hi) & above_hi) == 0u && (kb < lim_hi || (kb == lim_hi && (unsigned)i <= lim_lo)))
                    acc[((kb >> sh_hi) & 15u) * THREADS + tid] += ss_weight(b);
            }
        } else {
            for (int i = row.i0 + tid; i < row.i1; i += THREADS) {
                const unsigned b = row.bits[i - row.i0];
                const unsigned long long k = ss_key(b, (unsigned)i);
                if (k <= limit && ((k ^ prefix) & above) == 0ull) acc[((k >> shift) & 15u) * THREADS + tid] += ss_weight(b);
            }
        }
        __syncthreads();
        // this CTA's 16 sums: the first 16 warps (or 8, two segments each) add up a segment's words
        constexpr int WARPS = THREADS / 32, PER_WARP = WARPS >= SS_SEGS ? 1 : SS_SEGS / WARPS;
        if (warp * PER_WARP < SS_SEGS) {
#pragma unroll
            for (int h = 0; h < PER_WARP; ++h) {
                const int s = PER_WARP * warp + h;
                unsigned long long v = 0ull;
#pragma unroll 8
                for (int k = 0; k < THREADS / 32; ++k) v += acc[s * THREADS + lane + 32 * k];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) sh->seg[parity][s] = v;
            }
        }
        ss_cluster_sync();                                     // every CTA's sums are written (and the acc reads are done)
        if (tid < SS_SEGS) {
            unsigned long long v = 0ull;
#pragma unroll
            for (unsigned r = 0; r < SS_CLUSTER; ++r) v += ss_ld_peer_u64(&sh->seg[parity][tid], r);
            sh->total[tid] = v;
        }
        parity ^= 1u;
        __syncthreads();
        int chosen = -1;
        unsigned long long cum = below;
        for (int s = 0; s < SS_SEGS; ++s) {
            const unsigned long long t = sh->total[s];
            if (t >= ONE_TOKEN) {                               // tokens in this segment
                const unsigned long long with = cum + t;
                if ((by_mass ? (with & MASS_MASK) : (with >> MASS_BITS)) >= target) { chosen = s; break; }
                cum = with;
            }
        }
        if (chosen < 0) {                                      // only the first pass can fail: later ones search a segment that reached
            upto = cum;
            __syncthreads();
            return false;
        }
        below = cum;
        prefix |= (unsigned long long)chosen << shift;
        const unsigned long long in_segment = sh->total[chosen];
        __syncthreads();                                       // sh->total is read by all before the next pass rewrites it
        if ((in_segment >> MASS_BITS) == 1ull || d == n_digits - 1) {
            // one token left: look it up (its remaining key bits are not known yet)
            const unsigned long long fixed = ~0ull << shift;
            if (tid == 0) sh->loc = 0ull;
            __syncthreads();
            for (int i = row.i0 + tid; i < row.i1; i += THREADS) {
                const unsigned long long k = ss_key(row.bits[i - row.i0], (unsigned)i);
                if (k <= limit && ((k ^ prefix) & fixed) == 0ull) sh->loc = k + 1ull;       // at most one thread of the cluster
            }
            __syncthreads();
            ss_cluster_sync();
            unsigned long long found = 0ull;
#pragma unroll
            for (unsigned r = 0; r < SS_CLUSTER; ++r) found += ss_ld_peer_u64(&sh->loc, r);
            ss_cluster_sync();                                 // all have read before anyone's loc is reset
            key = found - 1ull;
            upto = below + in_segment;
            return true;
        }
    }
    return false;                                              // not reached: the last digit always ends above
}

// ``cached`` tokens of a slice fit the dynamic shared memory: the passes then read the probabilities from there,
// else from the scratch row in global memory (``scratch`` may be null when every slice fits).
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
sample_rows_kernel(const float* __restrict__ logits, int ld, int V, float temperature, int top_k, float top_p,
                   const float* __restrict__ u, unsigned* __restrict__ scratch, int cached, int* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ Shared sh_;
    Shared* sh = &sh_;
    sh->acc = (unsigned long long*)dyn_smem;                   // every thread writes the same value
    unsigned* slice_cache = (unsigned*)(dyn_smem + (size_t)SS_SEGS * THREADS * 8);
    const int tid = threadIdx.x;
    const unsigned rank = ss_cluster_rank();
    const int row_id = blockIdx.x / SS_CLUSTER;
    const float* x = logits + (size_t)row_id * ld;
    const int per = (V + SS_CLUSTER - 1) / SS_CLUSTER;
    Row row;
    row.i0 = min(V, (int)rank * per);
    row.i1 = min(V, row.i0 + per);
    unsigned* bits = per <= cached ? slice_cache : scratch + (size_t)row_id * V + row.i0;
    row.bits = bits;
    row.idx_digits = 1;
    while (row.idx_digits < 8 && (V - 1) >> (4 * row.idx_digits)) ++row.idx_digits;
    const int n = row.i1 - row.i0;

    // softmax of logits / temperature: exp(x - max) divided by the sum; every thread keeps to its own tokens, so
    // what it wrote to the slice it reads back itself
    float mx = -INFINITY;
    for (int j = tid; j < n; j += THREADS) {
        const float v = x[row.i0 + j] / temperature;
        bits[j] = __float_as_uint(v);
        mx = fmaxf(mx, v);
    }
    mx = sp_block_max(mx, sh->red);
    if (tid == 0) sh->stat[0] = mx;
    ss_cluster_sync();
    mx = -INFINITY;
#pragma unroll
    for (unsigned r = 0; r < SS_CLUSTER; ++r) mx = fmaxf(mx, ss_ld_peer_f32(&sh->stat[0], r));
    float sum = 0.0f;
    for (int j = tid; j < n; j += THREADS) {
        const float e = expf(__uint_as_float(bits[j]) - mx);
        bits[j] = __float_as_uint(e);
        sum += e;
    }
    sum = sp_block_sum(sum, sh->red);
    if (tid == 0) sh->stat[1] = sum;
    ss_cluster_sync();
    sum = 0.0f;
#pragma unroll
    for (unsigned r = 0; r < SS_CLUSTER; ++r) sum += ss_ld_peer_f32(&sh->stat[1], r);       // in rank order, alike in every CTA
    for (int j = tid; j < n; j += THREADS) {
        float p = __uint_as_float(bits[j]) / sum;
        if (!(p >= 0.0f)) p = 0.0f;                           // NaN logits never win
        if (p > 1.0f) p = 1.0f;
        bits[j] = __float_as_uint(p);
    }

    unsigned parity = 0;
    unsigned long long limit = ~0ull, key = 0ull, upto = 0ull;
    if (top_k > 0 && top_k < V) {                              // the first top_k tokens
        if (ss_descend<THREADS>(sh, row, false, (unsigned long long)top_k, limit, parity, key, upto)) limit = key;
    }
    // of those the shortest prefix whose mass reaches top_p; its mass
    unsigned long long kept_mass;
    if (ss_descend<THREADS>(sh, row, true, __float2ull_rz(top_p * MASS_UNIT), limit, parity, key, upto)) limit = key;
    kept_mass = upto & MASS_MASK;
    // the draw: u is a multiple of 2^-24, the target u · mass is taken exactly
    const unsigned long long n_u = (unsigned long long)(u[row_id] * 16777216.0f);
    const unsigned long long target = (__umul64hi(kept_mass, n_u) << 40) | ((kept_mass * n_u) >> 24);
    if (!ss_descend<THREADS>(sh, row, true, target, limit, parity, key, upto))
        ss_descend<THREADS>(sh, row, true, 0ull, limit, parity, key, upto);                          // the most probable token
    if (rank == 0 && tid == 0) out[row_id] = (int)(unsigned)(key & 0xffffffffu);
    ss_cluster_sync();                                         // no CTA leaves while a peer may still read its shared memory
}

}  // namespace

constexpr int SS_CACHE_BYTES = 128 * 1024;         // of a slice's probabilities in shared memory

// 64-bit words of scratch: one 32-bit probability per token (unused when a slice fits the shared memory)
SP_API long long sp_sample_scratch_keys(int rows, int V) {
    return ((long long)rows * V + 1) / 2;
}

SP_API int sp_sample_rows(const float* logits, int ld, int rows, int V, float temperature, int top_k,
                          float top_p, const float* u, void* scratch, long long scratch_keys, int* out,
                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0) SP_FAIL("sample: empty rows");
    if (!(temperature > 0.0f)) SP_FAIL("sample: temperature must be positive here (greedy rows use argmax)");
    if (!(top_p > 0.0f && top_p <= 1.0f)) SP_FAIL("sample: top_p must be in (0, 1], got %g", (double)top_p);
    if (top_k < 0) SP_FAIL("sample: top_k must not be negative");
    if (V > SS_MAX_V) SP_FAIL("sample: a vocabulary of %d is beyond this kernel's counters (%d at most)", V, SS_MAX_V);
    const int per = (V + SS_CLUSTER - 1) / SS_CLUSTER;
    const bool fits = (long long)per * 4 <= SS_CACHE_BYTES;
    if (!fits && scratch_keys < sp_sample_scratch_keys(rows, V))
        SP_FAIL("sample: scratch holds %lld words, %lld are needed", scratch_keys, sp_sample_scratch_keys(rows, V));
    const int cached = fits ? per : 0;
    const size_t cache_bytes = fits ? (((size_t)per * 4 + 15) / 16) * 16 : 0;
    static SpPerDevice configured;
    if (!configured.done()) {
        cudaError_t e = cudaFuncSetAttribute(sample_rows_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SS_CACHE_BYTES + SS_SEGS * 256 * 8);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(sample_rows_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     SS_CACHE_BYTES / 2 + SS_SEGS * 1024 * 8);
        if (e != cudaSuccess) SP_FAIL("sample: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured.mark();
    }
    // few rows: 1,024 threads per CTA (one CTA per SM, a quarter of the tokens per thread); many rows: 256, several CTAs per SM
    if (rows * SS_CLUSTER <= 128 && cache_bytes <= SS_CACHE_BYTES / 2)
        SP_CHECK_CALL("sample_rows", sp_launch_cluster(sample_rows_kernel<1024>, dim3(rows * SS_CLUSTER), dim3(1024),
                                                       cache_bytes + SS_SEGS * 1024 * 8, stream, SS_CLUSTER, logits, ld, V,
                                                       temperature, top_k, top_p, u, (unsigned*)scratch, cached, out));
    else
        SP_CHECK_CALL("sample_rows", sp_launch_cluster(sample_rows_kernel<256>, dim3(rows * SS_CLUSTER), dim3(256),
                                                       cache_bytes + SS_SEGS * 256 * 8, stream, SS_CLUSTER, logits, ld, V,
                                                       temperature, top_k, top_p, u, (unsigned*)scratch, cached, out));
    return 0;
}
