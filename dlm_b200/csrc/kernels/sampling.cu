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
// into a handful of buckets: that loop was most of the kernel's four milliseconds).  A row of a large
// vocabulary is shared by the blocks of a cluster, see team_rank() below.
#include "api.h"
#include "common.cuh"

namespace dlmk {

namespace {

constexpr int THREADS = 1024;
constexpr int SAMPLE_TEAM = 8;          // most blocks that share a row of a large vocabulary

__device__ __forceinline__ unsigned int desc_key(float v) {
    unsigned int u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending order of floats
    return ~u;                                        // larger float -> smaller key
}

// A row's candidates are shared out over a TEAM: the blocks of a thread-block cluster (one block when the
// vocabulary is small).  A block keeps its partial results in its own shared memory; after a cluster barrier
// every block reads all the partial results (distributed shared memory) and combines them in the same order,
// so all blocks of a team reach the same decisions without a word being sent back.
__device__ __forceinline__ unsigned int team_rank() {
    unsigned int r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned int team_size() {
    unsigned int r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void team_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// reads of what block `rank` of the team holds at `p` (an address in this block's own shared memory)
__device__ __forceinline__ uint32_t team_addr(const void* p, unsigned int rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ unsigned int team_load_u32(const void* p, unsigned int rank) {
    unsigned int v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(team_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long team_load_u64(const void* p, unsigned int rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(team_addr(p, rank)) : "memory");
    return v;
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
    unsigned int rank, team;  // this block's place in its team, the team's size
    bool vec;             // V is a multiple of 4 and z is 16-byte aligned: the row is read four logits at a time
    __device__ unsigned long long ckey(int i, float v) const {
        return ((unsigned long long)desc_key(v) << idx_bits) | (unsigned long long)i;
    }
    __device__ float prob(float v) const { return expf((v - mx) * inv_temp); }
    __device__ unsigned long long mass(float p) const { return (unsigned long long)((double)p * 1099511627776.0); }
};

// Calls f(i, z[i]) for the elements of the row that this thread of this block of the team takes.  A pass over the row is bound by the
// latency of its loads (one block reads 600 KB): 16-byte loads, four of them in flight, not one logit at a time.
template <typename F>
__device__ __forceinline__ void for_each_logit(const RowView& rv, F f) {
    const int first = (int)(rv.rank * blockDim.x + threadIdx.x), step = (int)(rv.team * blockDim.x);
    if (rv.vec) {
        const float4* z4 = reinterpret_cast<const float4*>(rv.z);
        const int n4 = rv.V >> 2;
#pragma unroll 4
        for (int j = first; j < n4; j += step) {
            const float4 v = z4[j];
            f(4 * j, v.x); f(4 * j + 1, v.y); f(4 * j + 2, v.z); f(4 * j + 3, v.w);
        }
    } else {
#pragma unroll 4
        for (int i = first; i < rv.V; i += step) f(i, rv.z[i]);
    }
}

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

// Sum of masses (or count) of the candidates, over the team.  `s_part`: 33 words; [32] is the block's sum, which
// the other blocks read.
__device__ unsigned long long team_total(const RowView& rv, bool count, unsigned long long* s_part) {
    unsigned long long local = 0ull;
    for_each_logit(rv, [&](int i, float v) {
        const float p = rv.prob(v);
        if (rv.ckey(i, v) <= rv.cut && p >= rv.minp_thr) local += count ? 1ull : rv.mass(p);
    });
    local = warp_sum_u64(local);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long r = 0ull;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) r += s_part[w];
        s_part[32] = r;
    }
    team_sync();
    unsigned long long total = 0ull;
    for (unsigned int c = 0; c < rv.team; ++c) total += team_load_u64(&s_part[32], c);
    team_sync();                 // everyone has read before anyone writes the slots again
    return total;
}

// Composite key of the first candidate (in key order) at which the running count / mass reaches `target`.
__device__ unsigned long long block_select(const RowView& rv, int mode, unsigned long long target,
                                           unsigned int* bucket_lo, unsigned int* bucket_hi,
                                           unsigned long long* merged, unsigned long long* s_state) {
    const int total_bits = 32 + rv.idx_bits;
    const int passes = (total_bits + 7) / 8;
    unsigned long long prefix = 0ull, before = 0ull;
    for (int pass = 0; pass < passes; ++pass) {
        const int shift = (passes - 1 - pass) * 8;
        for (int b = threadIdx.x; b < 256; b += blockDim.x) { bucket_lo[b] = 0u; bucket_hi[b] = 0u; }
        __syncthreads();
        for_each_logit(rv, [&](int i, float v) {
            const unsigned long long ck = rv.ckey(i, v);
            if (ck > rv.cut) return;
            if (pass > 0 && (ck >> (shift + 8)) != (prefix >> (shift + 8))) return;
            const float p = rv.prob(v);
            if (p < rv.minp_thr) return;
            bucket_add(bucket_lo, bucket_hi, (int)((ck >> shift) & 255ull), mode == COUNT ? 1ull : rv.mass(p));
        });
        // every block of the team adds up all the blocks' buckets and scans the sums: the same answer everywhere
        team_sync();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned long long sum = 0ull;
            for (unsigned int c = 0; c < rv.team; ++c)
                sum += ((unsigned long long)team_load_u32(&bucket_hi[b], c) << 32) | team_load_u32(&bucket_lo[b], c);
            merged[b] = sum;
        }
        team_sync();                 // all reads of the buckets are done: the next pass may clear them
        if (threadIdx.x == 0) {
            unsigned long long run = before;
            int pick = -1, last = -1;
            unsigned long long last_sum = 0ull;
            for (int b = 0; b < 256; ++b) {
                const unsigned long long sum = merged[b];
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
    __shared__ unsigned long long merged[256];
    __shared__ unsigned long long s_state[2];
    __shared__ unsigned long long s_part[33];
    __shared__ float s_best_v;
    __shared__ int s_best_i;
    const unsigned int rank = team_rank(), team = team_size();
    const int row = (int)(blockIdx.x / team);
    const float temperature = params[row * 4 + 0], top_p = params[row * 4 + 1], min_p = params[row * 4 + 2],
                penalty = params[row * 4 + 3];
    const float* lg = logits + (long long)row * V;
    // the penalised logits: a copy in the scratch when there is a penalty, else the logits themselves
    const float* z = lg;
    if (penalty != 1.0f && seen_offsets != nullptr) {
        float* zc = scratch + (long long)row * V;
        const int first = (int)(rank * blockDim.x + threadIdx.x), step = (int)(team * blockDim.x);
        for (int i = first; i < V; i += step) zc[i] = lg[i];
        __threadfence();
        team_sync();
        for (int s = seen_offsets[row] + first; s < seen_offsets[row + 1]; s += step) {
            const int t = seen_tokens[s];
            if (t >= 0 && t < V) {
                const float v = __ldcg(zc + t);     // (not through L1: the line holds other blocks' elements too,
                                                    //  which they may be changing, and this block reads it later)
                zc[t] = v > 0.f ? v / penalty : v * penalty;
            }
        }
        __threadfence();
        team_sync();
        z = zc;
    }
    // the maximum and its first index (the greedy answer): per block, then over the team
    RowView rv;
    rv.z = z;
    rv.V = V;
    rv.rank = rank;
    rv.team = team;
    rv.vec = (V & 3) == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for_each_logit(rv, [&](int i, float v) {
        if (v > bv) { bv = v; bi = i; }         // a thread's indices ascend: the first maximum stays
    });
    float mx;
    int mi;
    block_argmax(bv, bi, sv, si, mx, mi);
    if (threadIdx.x == 0) { s_best_v = mx; s_best_i = mi; }
    team_sync();
    for (unsigned int c = 0; c < team; ++c) {
        const float ov = __uint_as_float(team_load_u32(&s_best_v, c));
        const int oi = (int)team_load_u32(&s_best_i, c);
        if (ov > mx || (ov == mx && oi < mi)) { mx = ov; mi = oi; }
    }
    team_sync();
    if (mi == 0x7fffffff) mi = 0;
    if (!(temperature > 0.f)) {                 // (the same for every block of the team)
        if (threadIdx.x == 0 && rank == 0) out[row] = mi;
        return;
    }
    rv.idx_bits = 1;
    while ((1 << rv.idx_bits) < V) ++rv.idx_bits;
    rv.mx = mx;
    rv.inv_temp = 1.0f / temperature;
    rv.minp_thr = 0.f;
    rv.cut = ~0ull;
    const int k = top_k[row];
    if (k > 0 && k < V) rv.cut = block_select(rv, COUNT, (unsigned long long)k, bucket_lo, bucket_hi, merged, s_state);
    if (top_p > 0.f && top_p < 1.f) {
        const unsigned long long Z = team_total(rv, false, s_part);
        unsigned long long target = (unsigned long long)((double)top_p * (double)Z);
        if (target < 1ull) target = 1ull;
        rv.cut = block_select(rv, MASS_GE, target, bucket_lo, bucket_hi, merged, s_state);
    }
    if (min_p > 0.f) rv.minp_thr = fminf(min_p, 1.0f);   // the top candidate (probability 1 before scaling) stays
    const unsigned long long Z = team_total(rv, false, s_part);
    const unsigned long long target = (unsigned long long)((double)u[row] * (double)Z);
    const unsigned long long pick = block_select(rv, MASS_GT, target, bucket_lo, bucket_hi, merged, s_state);
    if (threadIdx.x == 0 && rank == 0) {
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
    // a large vocabulary is shared out over a cluster of blocks (one block walks 150,000 logits in 26 us a pass,
    // and a draw takes nine passes)
    // (as many blocks a row as leave the rows of one launch a block each at the same time: 64 rows with 8 blocks
    // each took longer than with one)
    int team = 1;
    if (V >= 32768)
        while (team < SAMPLE_TEAM && (long long)N * team * 2 <= sm_count()) team *= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)N * team);
    cfg.blockDim = dim3(THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = team;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, sample_kernel, logits, out, V, params, top_k, u, seen_offsets, seen_tokens, scratch);
    check_launch("sample");
}

}  // namespace dlmk
