// Token selection on the device: arg-max, and the reference's sampler
// (src/generate.rs:122-210): repetition penalty, temperature, top-k, top-p, min-p and an
// inverse-CDF draw over the candidates ordered by logit, highest first.
//
// Nothing is sorted.  Candidates are ordered by a composite key (logit descending, then
// index), and "the first place where the running count / mass reaches x" is found by a
// radix descent over that key, eight bits a pass.  Masses are 40-bit fixed point, so their
// sums do not depend on the order threads add them in: the same logits and the same uniform
// number always give the same token.  A bucket's 64-bit sum is kept as two 32-bit words, added
// with the hardware's 32-bit shared-memory atomics and an explicit carry (a 64-bit atomic add
// on shared memory is a compare-and-swap loop, and the first passes put the whole vocabulary
// into a handful of buckets: that loop was most of the kernel's four milliseconds).
#include "api.h"
#include "common.cuh"

namespace dlmk {

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned int desc_key(float v) {
    unsigned int u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending order of floats
    return ~u;                                        // larger float -> smaller key
}

// (max value, first index holding it) over the block; result valid in every thread.
__device__ void block_argmax(float v, int i, float* sv, int* si, float& out_v, int& out_i) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    float bv = sv[0];
    int bi = si[0];
    for (int w = 1; w < nwarp; ++w)
        if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    out_v = bv;
    out_i = bi;
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* logits, int32_t* out,
                                                         int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    dep_wait();
    dep_launch_next();
    const float* row = logits + (long long)blockIdx.x * V;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }
    }
    if (bi == 0x7fffffff && threadIdx.x == 0) bi = 0;   // a row of -inf / NaN: index 0, as the reference
    float rv;
    int ri;
    block_argmax(bv, bi, sv, si, rv, ri);
    if (threadIdx.x == 0) out[blockIdx.x] = ri == 0x7fffffff ? 0 : ri;
}

// Two stages for a large vocabulary: every block finds the first maximum of its chunk, then one
// warp per row picks among the chunks (lower chunk first on ties, so the first maximum overall).
constexpr int ARGMAX_CHUNKS = 32;

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* logits, float* pv,
                                                             int32_t* pi, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    dep_wait();
    dep_launch_next();
    const int row = blockIdx.x, c = blockIdx.y;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = c * per, hi = min(V, lo + per);
    const float* r = logits + (long long)row * V;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = r[i];
        if (v > bv) { bv = v; bi = i; }
    }
    float rv;
    int ri;
    block_argmax(bv, bi, sv, si, rv, ri);
    if (threadIdx.x == 0) { pv[row * ARGMAX_CHUNKS + c] = rv; pi[row * ARGMAX_CHUNKS + c] = ri; }
}

__global__ void argmax_final_kernel(const float* pv, const int32_t* pi,
                                    int32_t* out) {
    dep_wait();
    dep_launch_next();
    const int row = blockIdx.x, lane = threadIdx.x;
    float v = pv[row * ARGMAX_CHUNKS + lane];
    int i = pi[row * ARGMAX_CHUNKS + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    if (lane == 0) out[row] = i == 0x7fffffff ? 0 : i;
}

enum SelectMode { COUNT = 0, MASS_GE = 1, MASS_GT = 2 };

struct RowView {
    const float* z;       // penalised logits [V]
    int V;
    int idx_bits;
    float mx, inv_temp, minp_thr;
    unsigned long long cut;   // candidates have composite key <= cut
    __device__ unsigned long long ckey(int i, float v) const {
        return ((unsigned long long)desc_key(v) << idx_bits) | (unsigned long long)i;
    }
    __device__ float prob(float v) const { return expf((v - mx) * inv_temp); }
    __device__ unsigned long long mass(float p) const { return (unsigned long long)((double)p * 1099511627776.0); }
};

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned int lo = __shfl_xor_sync(0xffffffffu, (unsigned int)v, o);
        const unsigned int hi = __shfl_xor_sync(0xffffffffu, (unsigned int)(v >> 32), o);
        v += ((unsigned long long)hi << 32) | lo;
    }
    return v;
}

// bucket[b] += m, the sum kept as (low word, high word)
__device__ __forceinline__ void bucket_add(unsigned int* lo, unsigned int* hi, int b, unsigned long long m) {
    const unsigned int add = (unsigned int)m;
    const unsigned int old = atomicAdd(&lo[b], add);
    const unsigned int up = (unsigned int)(m >> 32) + ((old + add < old) ? 1u : 0u);
    if (up != 0u) atomicAdd(&hi[b], up);
}

// Sum of masses (or count) of the candidates.
__device__ unsigned long long block_total(const RowView& rv, bool count, unsigned long long* s_part) {
    unsigned long long local = 0ull;
#pragma unroll 4
    for (int i = threadIdx.x; i < rv.V; i += blockDim.x) {
        const float v = rv.z[i];
        const float p = rv.prob(v);
        if (rv.ckey(i, v) <= rv.cut && p >= rv.minp_thr) local += count ? 1ull : rv.mass(p);
    }
    local = warp_sum_u64(local);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = local;
    __syncthreads();
    unsigned long long r = 0ull;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) r += s_part[w];
    __syncthreads();
    return r;
}

// Composite key of the first candidate (in key order) at which the running count / mass reaches `target`.
__device__ unsigned long long block_select(const RowView& rv, int mode, unsigned long long target,
                                           unsigned int* bucket_lo, unsigned int* bucket_hi,
                                           unsigned long long* s_state) {
    const int total_bits = 32 + rv.idx_bits;
    const int passes = (total_bits + 7) / 8;
    unsigned long long prefix = 0ull, before = 0ull;
    for (int pass = 0; pass < passes; ++pass) {
        const int shift = (passes - 1 - pass) * 8;
        for (int b = threadIdx.x; b < 256; b += blockDim.x) { bucket_lo[b] = 0u; bucket_hi[b] = 0u; }
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < rv.V; i += blockDim.x) {
            const float v = rv.z[i];
            const unsigned long long ck = rv.ckey(i, v);
            if (ck > rv.cut) continue;
            if (pass > 0 && (ck >> (shift + 8)) != (prefix >> (shift + 8))) continue;
            const float p = rv.prob(v);
            if (p < rv.minp_thr) continue;
            bucket_add(bucket_lo, bucket_hi, (int)((ck >> shift) & 255ull), mode == COUNT ? 1ull : rv.mass(p));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long run = before;
            int pick = -1, last = -1;
            unsigned long long last_sum = 0ull;
            for (int b = 0; b < 256; ++b) {
                const unsigned long long sum = ((unsigned long long)bucket_hi[b] << 32) | bucket_lo[b];
                if (sum == 0ull) continue;
                last = b;
                last_sum = sum;
                const unsigned long long nxt = run + sum;
                const bool hit = mode == MASS_GT ? (nxt > target) : (nxt >= target);
                if (hit) { pick = b; break; }
                run = nxt;
            }
            if (pick < 0) {            // rounding left the target just beyond the total: the last candidate
                pick = last < 0 ? 0 : last;
                run -= (last >= 0 ? last_sum : 0ull);
            }
            s_state[0] = prefix | ((unsigned long long)pick << shift);
            s_state[1] = run;
        }
        __syncthreads();
        prefix = s_state[0];
        before = s_state[1];
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int V, const float* __restrict__ params,
              const int32_t* __restrict__ top_k, const float* __restrict__ u, const int32_t* __restrict__ seen_offsets,
              const int32_t* __restrict__ seen_tokens, float* __restrict__ scratch) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ unsigned int bucket_lo[256], bucket_hi[256];
    __shared__ unsigned long long s_state[2];
    __shared__ unsigned long long s_part[32];
    const int row = blockIdx.x;
    const float temperature = params[row * 4 + 0], top_p = params[row * 4 + 1], min_p = params[row * 4 + 2],
                penalty = params[row * 4 + 3];
    const float* lg = logits + (long long)row * V;
    // the penalised logits: a copy in the scratch when there is a penalty, else the logits themselves
    const float* z = lg;
    if (penalty != 1.0f && seen_offsets != nullptr) {
        float* zc = scratch + (long long)row * V;
        for (int i = threadIdx.x; i < V; i += blockDim.x) zc[i] = lg[i];
        __syncthreads();
        for (int s = seen_offsets[row] + threadIdx.x; s < seen_offsets[row + 1]; s += blockDim.x) {
            const int t = seen_tokens[s];
            if (t >= 0 && t < V) {
                const float v = zc[t];
                zc[t] = v > 0.f ? v / penalty : v * penalty;
            }
        }
        __syncthreads();
        z = zc;
    }
    // the maximum and its first index (the greedy answer)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = z[i];
        if (v > bv) { bv = v; bi = i; }
    }
    float mx;
    int mi;
    block_argmax(bv, bi, sv, si, mx, mi);
    if (mi == 0x7fffffff) mi = 0;
    if (!(temperature > 0.f)) {
        if (threadIdx.x == 0) out[row] = mi;
        return;
    }
    RowView rv;
    rv.z = z;
    rv.V = V;
    rv.idx_bits = 1;
    while ((1 << rv.idx_bits) < V) ++rv.idx_bits;
    rv.mx = mx;
    rv.inv_temp = 1.0f / temperature;
    rv.minp_thr = 0.f;
    rv.cut = ~0ull;
    const int k = top_k[row];
    if (k > 0 && k < V) rv.cut = block_select(rv, COUNT, (unsigned long long)k, bucket_lo, bucket_hi, s_state);
    if (top_p > 0.f && top_p < 1.f) {
        const unsigned long long Z = block_total(rv, false, s_part);
        unsigned long long target = (unsigned long long)((double)top_p * (double)Z);
        if (target < 1ull) target = 1ull;
        rv.cut = block_select(rv, MASS_GE, target, bucket_lo, bucket_hi, s_state);
    }
    if (min_p > 0.f) rv.minp_thr = fminf(min_p, 1.0f);   // the top candidate (probability 1 before scaling) stays
    const unsigned long long Z = block_total(rv, false, s_part);
    const unsigned long long target = (unsigned long long)((double)u[row] * (double)Z);
    const unsigned long long pick = block_select(rv, MASS_GT, target, bucket_lo, bucket_hi, s_state);
    if (threadIdx.x == 0) {
        int tok = (int)(pick & ((1ull << rv.idx_bits) - 1ull));
        if (tok >= V) tok = mi;
        out[row] = tok;
    }
}

}  // namespace

size_t argmax_scratch_bytes(int N, int V) { return V >= 16384 ? (size_t)N * ARGMAX_CHUNKS * 8 : 0; }

void argmax(const float* logits, int32_t* out, int N, int V, void* scratch, cudaStream_t stream) {
    if (N <= 0) return;
    DLM_CHECK(V > 0, "argmax: empty vocabulary");
    static_assert(ARGMAX_CHUNKS == 32, "the final stage is one warp");
    if (V >= 16384 && scratch != nullptr) {
        float* pv = static_cast<float*>(scratch);
        int32_t* pi = reinterpret_cast<int32_t*>(pv + (size_t)N * ARGMAX_CHUNKS);
        launch_dep(argmax_partial_kernel, dim3(N, ARGMAX_CHUNKS), 256, 0, stream, logits, pv, pi, V);
        launch_dep(argmax_final_kernel, N, 32, 0, stream, pv, pi, out);
    } else {
        launch_dep(argmax_kernel, N, THREADS, 0, stream, logits, out, V);
    }
    check_launch("argmax");
}

void sample(const float* logits, int32_t* out, int N, int V, const float* params, const int32_t* top_k,
            const float* u, const int32_t* seen_offsets, const int32_t* seen_tokens, float* scratch,
            cudaStream_t stream) {
    if (N <= 0) return;
    DLM_CHECK(V > 0 && V <= (1 << 30), "sample: vocabulary size out of range");
    sample_kernel<<<N, THREADS, 0, stream>>>(logits, out, V, params, top_k, u, seen_offsets, seen_tokens, scratch);
    check_launch("sample");
}

}  // namespace dlmk
