// Routing: router logits, softmax, top-k and the grouping of (token, expert) pairs by expert.
#include "api.h"
#include "common.cuh"

namespace dlmk {

namespace {

constexpr int ROUTER_THREADS = 256;

// 4 consecutive elements of a row as floats (one 8-byte load for bfloat16, one 16-byte load for float32).
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
    v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
}
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}

// Asks for a row of the router's matrix to be brought into L2 (one 128-byte line a lane and round).  The matrix
// is never written by a kernel, so this may run before dep_wait(): the row is then near when the dot product
// starts.
template <typename T>
__device__ __forceinline__ void prefetch_row_l2(const T* row, int H, int lane) {
    const char* base = reinterpret_cast<const char*>(row);
    const int bytes = H * (int)sizeof(T);
    for (int off = lane * 128; off < bytes; off += 32 * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

// Router logits: blockIdx.x = token, blockIdx.y = a block of ROUTER_WARPS experts, one warp per
// expert.  Each logit is one warp's dot product summed in a fixed order (lane l takes elements
// 4l..4l+3 and 128+4l..128+4l+3 of every 256, so that a quarter warp reads 128 consecutive bytes of the
// staged row and no two lanes meet in a bank; then a shuffle tree), so routing does not depend on what
// else is in the batch.  VEC: rows are 16-byte aligned and H is a multiple of 8.
// With norm_w != nullptr the input is the 32-bit residual and the RMS norm (weight norm_w, eps)
// is applied here, in 32-bit, so that the router never sees a rounded activation.
constexpr int ROUTER_WARPS = ROUTER_THREADS / 32;

template <typename TX, typename T, bool VEC>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_logits_kernel(const TX* h, const T* __restrict__ w, const float* __restrict__ norm_w, float eps,
                     float* logits, int H, int rows) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    {
        const int e_mine = blockIdx.y * ROUTER_WARPS + (threadIdx.x >> 5);
        if (e_mine < rows) prefetch_row_l2(w + (long long)e_mine * H, H, threadIdx.x & 31);
    }
    dep_wait();
    dep_launch_next();
    float* x = smem;            // [H]
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float ss = 0.f;
    for (int i = tid; i < H; i += blockDim.x) {
        const float v = to_f32(h[(long long)t * H + i]);
        x[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (norm_w != nullptr) {
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (int i = tid; i < H; i += blockDim.x) x[i] = (x[i] * inv) * norm_w[i];
    }
    __syncthreads();
    const int e = blockIdx.y * ROUTER_WARPS + warp;
    if (e >= rows) return;
    const T* wr = w + (long long)e * H;
    float s = 0.f;
    if (VEC) {
#pragma unroll 4
        for (int b = 0; b < H; b += 256) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = b + 128 * half + lane * 4;
                if (i < H) {
                    float wv[4];
                    load4(wr + i, wv);
                    const float4 xa = *reinterpret_cast<const float4*>(x + i);
                    s = fmaf(xa.x, wv[0], s); s = fmaf(xa.y, wv[1], s); s = fmaf(xa.z, wv[2], s); s = fmaf(xa.w, wv[3], s);
                }
            }
        }
    } else {
        for (int i = lane; i < H; i += 32) s = fmaf(x[i], to_f32(wr[i]), s);
    }
    s = warp_sum(s);
    if (lane == 0) logits[(long long)t * rows + e] = s;
}

// The same for many tokens: a block takes ROUTER_TB tokens, so that a weight row read from memory meets all
// of them.  Per token the sums run in exactly the order of router_logits_kernel, so a token's logits do not
// depend on which of the two kernels computed them.
constexpr int ROUTER_TB = 8;

constexpr int ROUTER_EW = 4;     // experts per warp in the many-token kernel

template <typename TX, typename T>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_logits_multi_kernel(const TX* h, const T* __restrict__ w, const float* __restrict__ norm_w,
                           float eps, float* logits, int T_, int H, int rows, int x_settled) {
    extern __shared__ float smem[];               // [ROUTER_TB][H]
    // x_settled: the activations are older than the kernel launched just before this one; the tokens are
    // staged and a warp's first sums worked out while that kernel ends, and nothing is stored before the wait
    bool waited = x_settled == 0;
    if (waited) {
        dep_wait();
        dep_launch_next();
    }
    const int t0 = blockIdx.x * ROUTER_TB, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nt = min(ROUTER_TB, T_ - t0);
    // Staging: warp j brings token t0 + j into shared memory and normalises it.  The sum of squares is taken
    // in the order of router_logits_kernel's block_sum over ROUTER_THREADS threads: lane l keeps one partial sum
    // for each of that kernel's warps v (its thread 32 v + l takes elements 32 v + l, + ROUTER_THREADS, ...),
    // every partial sum goes through the same shuffle tree, and the warps' sums are added in order.
    static_assert(ROUTER_TB == ROUTER_WARPS, "one staging warp per token");
    {
        const int j = warp;
        float* x = smem + (size_t)j * H;
        if (j >= nt) {
            for (int i = lane; i < H; i += 32) x[i] = 0.f;
        } else {
            const TX* src = h + (long long)(t0 + j) * H;
            float part[ROUTER_WARPS];
#pragma unroll
            for (int v = 0; v < ROUTER_WARPS; ++v) part[v] = 0.f;
            for (int base = 0; base < H; base += ROUTER_THREADS) {
#pragma unroll
                for (int v = 0; v < ROUTER_WARPS; ++v) {
                    const int i = base + 32 * v + lane;
                    if (i < H) {
                        const float val = to_f32(src[i]);
                        x[i] = val;
                        part[v] = fmaf(val, val, part[v]);
                    }
                }
            }
            if (norm_w != nullptr) {
                float ss = 0.f;
#pragma unroll
                for (int v = 0; v < ROUTER_WARPS; ++v) ss += warp_sum(part[v]);
                const float inv = 1.0f / sqrtf(ss / (float)H + eps);
                for (int i = lane; i < H; i += 32) x[i] = (x[i] * inv) * norm_w[i];
            }
        }
    }
    __syncthreads();
    // a warp takes ROUTER_EW experts x ROUTER_TB tokens at a time: every activation read from shared memory
    // meets ROUTER_EW weight rows, every weight meets ROUTER_TB tokens
    for (int e0 = warp * ROUTER_EW; e0 < rows; e0 += ROUTER_WARPS * ROUTER_EW) {
        float s[ROUTER_EW][ROUTER_TB];
#pragma unroll
        for (int a = 0; a < ROUTER_EW; ++a)
#pragma unroll
            for (int j = 0; j < ROUTER_TB; ++j) s[a][j] = 0.f;
        for (int b = 0; b < H; b += 256) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = b + 128 * half + lane * 4;       // the elements of router_logits_kernel's lane
                if (i < H) {
                    float wv[ROUTER_EW][4];
#pragma unroll
                    for (int a = 0; a < ROUTER_EW; ++a) {
                        const int e = min(e0 + a, rows - 1);    // rows beyond the table repeat the last one (not stored)
                        load4(w + (long long)e * H + i, wv[a]);
                    }
#pragma unroll
                    for (int j = 0; j < ROUTER_TB; ++j) {
                        const float4 xa = *reinterpret_cast<const float4*>(smem + (size_t)j * H + i);
#pragma unroll
                        for (int a = 0; a < ROUTER_EW; ++a) {
                            s[a][j] = fmaf(xa.x, wv[a][0], s[a][j]); s[a][j] = fmaf(xa.y, wv[a][1], s[a][j]);
                            s[a][j] = fmaf(xa.z, wv[a][2], s[a][j]); s[a][j] = fmaf(xa.w, wv[a][3], s[a][j]);
                        }
                    }
                }
            }
        }
        if (!waited) {
            dep_wait();
            dep_launch_next();
            waited = true;
        }
#pragma unroll
        for (int a = 0; a < ROUTER_EW; ++a)
#pragma unroll
            for (int j = 0; j < ROUTER_TB; ++j) {
                const float v = warp_sum(s[a][j]);
                if (lane == 0 && j < nt && e0 + a < rows) logits[(long long)(t0 + j) * rows + e0 + a] = v;
            }
    }
    if (!waited) {
        dep_wait();
        dep_launch_next();
    }
}

// One token's choice, by one warp: scores from the logits (score_fn 0: softmax over the experts; 1: a sigmoid
// of each logit), the k best (ties: lower index; with select_bias the choice is made on score + bias, the
// weight stays the score), optional renormalisation of the chosen weights, a constant factor, and the shared
// expert's sigmoid gate.  `prob`: 2 * (E + 1) floats of shared memory of this warp's own.
template <bool COHERENT>
__device__ __forceinline__ void select_token(float* prob, const float* logits, int32_t* ids, float* wts, float* gate,
                                             int t, int E, int k, int norm, int has_gate, int score_fn, float scale,
                                             const float* __restrict__ select_bias) {
    const int lane = threadIdx.x & 31;
    const int rows = E + (has_gate ? 1 : 0);
    float* pick = prob + (E + 1);                // what the choice is made on (score, or score + bias)
    // COHERENT: the logits were written by other blocks of this launch; read them where those writes are
    for (int e = lane; e < rows; e += 32)
        prob[e] = COHERENT ? __ldcg(logits + (long long)t * rows + e) : logits[(long long)t * rows + e];
    __syncwarp();
    if (has_gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-prob[E]));
    if (score_fn == 0) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, prob[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(prob[e] - mx);
            prob[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        __syncwarp();
        if (sum > 0.f)
            for (int e = lane; e < E; e += 32) prob[e] = prob[e] / sum;
    } else {
        for (int e = lane; e < E; e += 32) prob[e] = 1.0f / (1.0f + expf(-prob[e]));
    }
    for (int e = lane; e < E; e += 32) pick[e] = prob[e] + (select_bias != nullptr ? select_bias[e] : 0.f);
    __syncwarp();
    float chosen_sum = 0.f;
    for (int j = 0; j < k; ++j) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float p = pick[e];
            if (p > bv) { bv = p; bi = e; }     // ascending e per lane: ties keep the lower index
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        const float w = prob[bi];               // every lane reads it before lane 0 marks the expert as taken
        __syncwarp();
        if (lane == 0) {
            ids[t * k + j] = bi;
            wts[t * k + j] = w;
            pick[bi] = -INFINITY;               // taken
        }
        chosen_sum += w;
        __syncwarp();
    }
    if (lane == 0) {
        const float div = (norm && chosen_sum > 0.f) ? chosen_sum : 1.0f;
        if (div != 1.0f || scale != 1.0f)
            for (int j = 0; j < k; ++j) wts[t * k + j] = (wts[t * k + j] / div) * scale;
    }
}

// One warp per token.
__global__ void __launch_bounds__(128)
router_select_kernel(const float* logits, int32_t* ids, float* wts,
                     float* gate, int T, int E, int k, int norm, int has_gate, int score_fn, float scale,
                     const float* __restrict__ select_bias) {
    extern __shared__ float smem[];
    dep_wait();
    dep_launch_next();
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    select_token<false>(smem + warp * 2 * (E + 1), logits, ids, wts, gate, t, E, k, norm, has_gate, score_fn, scale,
                        select_bias);
}

// Groups n (token, choice) pairs by expert with the threads of one block: counts, an exclusive scan, and the
// rows.  `sm`: 2 * E ints of shared memory.  Every thread of the block calls it.
template <bool COHERENT = false>
__device__ __forceinline__ void permute_block(int* sm, const int32_t* ids, int n, int k, int E, int32_t* offsets,
                                              int32_t* rows, int32_t* dest, int* err) {
    int* count = sm;          // [E]
    int* cursor = sm + E;     // [E]
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
        const int e = COHERENT ? __ldcg(ids + i) : ids[i];      // COHERENT: written by other blocks of this launch
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
        else *err = 4;
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = acc;
            cursor[e] = acc;
            acc += count[e];
        }
        offsets[E] = acc;
    }
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
        const int e = COHERENT ? __ldcg(ids + i) : ids[i];
        if (e >= 0 && e < E) {
            const int pos = atomicAdd(&cursor[e], 1);
            rows[pos] = i / k;
            dest[i] = pos;
        } else {
            dest[i] = 0;
        }
    }
}

constexpr int PERMUTE_THREADS = 1024;

__global__ void __launch_bounds__(PERMUTE_THREADS)
moe_permute_kernel(const int32_t* ids, int n, int k, int E, int32_t* offsets,
                   int32_t* rows, int32_t* dest, int* err) {
    extern __shared__ int sm[];
    dep_wait();
    dep_launch_next();
    permute_block(sm, ids, n, k, E, offsets, rows, dest, err);
}

// Few tokens (a decode step of at most 16): logits, choice and grouping in ONE launch.  Blocks compute logits as
// router_logits_kernel does (blockIdx.x = token, blockIdx.y = a block of experts, the same sums in the same
// order); the block that finishes last (a counter in global memory, put back to zero by that block, so
// launches of this kernel must not overlap) then chooses for every token and groups the pairs by expert.
__device__ unsigned int g_router_blocks_done;

template <typename TX, typename T, bool VEC>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_fused_kernel(const TX* h, const T* __restrict__ w, const float* __restrict__ norm_w, float eps,
                    float* logits, int32_t* ids, float* wts, float* gate, int32_t* offsets, int32_t* rows_out,
                    int32_t* dest, int T_, int H, int E, int k, int norm, int has_gate, int score_fn, float scale,
                    const float* __restrict__ select_bias, int x_settled, int* err) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    __shared__ int s_last;
    const int rows = E + (has_gate ? 1 : 0);
    {
        const int e_mine = blockIdx.y * ROUTER_WARPS + (threadIdx.x >> 5);
        if (e_mine < rows) prefetch_row_l2(w + (long long)e_mine * H, H, threadIdx.x & 31);
    }
    // x_settled: the activations are older than the kernel launched just before this one (the caller says so),
    // and the logits are worked out while that kernel ends; nothing is written before the wait.
    if (!x_settled) {
        dep_wait();
        dep_launch_next();
    }
    float* x = smem;            // [H]
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float ss = 0.f;
    for (int i = tid; i < H; i += blockDim.x) {
        const float v = to_f32(h[(long long)t * H + i]);
        x[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (norm_w != nullptr) {
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (int i = tid; i < H; i += blockDim.x) x[i] = (x[i] * inv) * norm_w[i];
    }
    __syncthreads();
    const int e = blockIdx.y * ROUTER_WARPS + warp;
    float s = 0.f;
    if (e < rows) {
        const T* wr = w + (long long)e * H;
        if (VEC) {
#pragma unroll 4
            for (int b = 0; b < H; b += 256) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int i = b + 128 * half + lane * 4;
                    if (i < H) {
                        float wv[4];
                        load4(wr + i, wv);
                        const float4 xa = *reinterpret_cast<const float4*>(x + i);
                        s = fmaf(xa.x, wv[0], s); s = fmaf(xa.y, wv[1], s); s = fmaf(xa.z, wv[2], s); s = fmaf(xa.w, wv[3], s);
                    }
                }
            }
        } else {
            for (int i = lane; i < H; i += 32) s = fmaf(x[i], to_f32(wr[i]), s);
        }
        s = warp_sum(s);
    }
    if (x_settled) {
        dep_wait();
        dep_launch_next();
    }
    if (e < rows && lane == 0) __stcg(logits + (long long)t * rows + e, s);
    // the last block to get here does the rest
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned total = gridDim.x * gridDim.y;
        s_last = atomicAdd(&g_router_blocks_done, 1u) == total - 1 ? 1 : 0;
        if (s_last) g_router_blocks_done = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int tt = warp; tt < T_; tt += ROUTER_WARPS)
        select_token<true>(smem + warp * 2 * (E + 1), logits, ids, wts, gate, tt, E, k, norm, has_gate, score_fn,
                           scale, select_bias);
    __syncthreads();
    permute_block(reinterpret_cast<int*>(smem), ids, T_ * k, k, E, offsets, rows_out, dest, err);
}

// A few dozen tokens (17 to 48): logits, choice and grouping in ONE launch, one block per token.  Warp v
// takes the rows v, v + 8, ... of the router's matrix (each logit the same sum in the same order as in
// router_logits_kernel), warp 0 then chooses for the token, and the block that finishes last groups the pairs by
// expert (the counter of router_fused_kernel: launches of the two must not overlap either).
constexpr int TOKEN_WARPS = 8;      // (16 warps a token: no faster)

template <typename TX, typename T, bool VEC>
__global__ void __launch_bounds__(TOKEN_WARPS * 32)
router_token_kernel(const TX* h, const T* __restrict__ w, const float* __restrict__ norm_w, float eps,
                    float* logits, int32_t* ids, float* wts, float* gate, int32_t* offsets, int32_t* rows_out,
                    int32_t* dest, int T_, int H, int E, int k, int norm, int has_gate, int score_fn, float scale,
                    const float* __restrict__ select_bias, int* err) {
    extern __shared__ float smem[];            // [H] the token, then [2 (E + 1)] for the choice
    __shared__ float scratch[32];
    __shared__ int s_last;
    const int rows = E + (has_gate ? 1 : 0);
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (blockIdx.x < 4)        // a few blocks ask for the whole matrix; the others find it in L2
        for (int e = (int)blockIdx.x * TOKEN_WARPS + warp; e < rows; e += 4 * TOKEN_WARPS)
            prefetch_row_l2(w + (long long)e * H, H, lane);
    // (working the logits out before the wait, as router_fused_kernel does, was slower here: 1 % of a step)
    dep_wait();
    dep_launch_next();
    float* x = smem;
    // the sum of squares in router_logits_kernel's order: its 256 threads' partial sums, the other warps add zeros
    float ss = 0.f;
    if (tid < ROUTER_THREADS)
        for (int i = tid; i < H; i += ROUTER_THREADS) {
            const float v = to_f32(h[(long long)t * H + i]);
            x[i] = v;
            ss = fmaf(v, v, ss);
        }
    if (norm_w != nullptr) {
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (int i = tid; i < H; i += blockDim.x) x[i] = (x[i] * inv) * norm_w[i];
    }
    __syncthreads();
    for (int e = warp; e < rows; e += TOKEN_WARPS) {
        const T* wr = w + (long long)e * H;
        float s = 0.f;
        if (VEC) {
#pragma unroll 4
            for (int b = 0; b < H; b += 256) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int i = b + 128 * half + lane * 4;
                    if (i < H) {
                        float wv[4];
                        load4(wr + i, wv);
                        const float4 xa = *reinterpret_cast<const float4*>(x + i);
                        s = fmaf(xa.x, wv[0], s); s = fmaf(xa.y, wv[1], s); s = fmaf(xa.z, wv[2], s); s = fmaf(xa.w, wv[3], s);
                    }
                }
            }
        } else {
            for (int i = lane; i < H; i += 32) s = fmaf(x[i], to_f32(wr[i]), s);
        }
        s = warp_sum(s);
        if (lane == 0) logits[(long long)t * rows + e] = s;
    }
    __syncthreads();
    if (warp == 0)
        select_token<false>(smem + H, logits, ids, wts, gate, t, E, k, norm, has_gate, score_fn, scale, select_bias);
    // the last block to get here groups the pairs of all tokens
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        s_last = atomicAdd(&g_router_blocks_done, 1u) == gridDim.x - 1 ? 1 : 0;
        if (s_last) g_router_blocks_done = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    permute_block<true>(reinterpret_cast<int*>(smem), ids, T_ * k, k, E, offsets, rows_out, dest, err);
}

}  // namespace

void router_topk(const void* h, const void* w, const float* norm_w, float eps, float* logits, int32_t* ids, float* wts,
                 float* gate, int T, int H, int E, int k, int norm, int has_gate, int dtype, int h_is_f32,
                 int score_fn, float scale, const float* select_bias, int x_settled, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(score_fn == 0 || score_fn == 1, "router: score function must be 0 (softmax) or 1 (sigmoid)");
    const bool x32 = norm_w != nullptr || h_is_f32 != 0;      // the activations are 32-bit whatever the weights are
    DLM_CHECK(E >= 1 && k >= 1 && k <= E, "router: top-k must be in 1..num_experts");
    const size_t smem = sizeof(float) * (size_t)H;
    DLM_CHECK(smem <= 200 * 1024, "router: hidden_size does not fit in shared memory");
    DLM_CHECK(E <= 8192, "router: more than 8192 experts");
    const int rows = E + (has_gate ? 1 : 0);
    const bool vec = H % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    const size_t smem_multi = sizeof(float) * (size_t)H * ROUTER_TB;
    // (with few tokens the one-token kernel has more blocks: tokens x groups of experts)
    if (vec && T >= 512 && smem_multi <= 200 * 1024) {
        dim3 mgrid((T + ROUTER_TB - 1) / ROUTER_TB);
#define DLM_ROUTER_MULTI(TX, TW)                                                                              \
    {                                                                                                         \
        auto kern = router_logits_multi_kernel<TX, TW>;                                                       \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_multi);             \
        launch_dep(kern, mgrid, ROUTER_THREADS, smem_multi, stream, static_cast<const TX*>(h),                \
                   static_cast<const TW*>(w), norm_w, eps, logits, T, H, rows, x_settled);                    \
    }
        if (dtype == F32) DLM_ROUTER_MULTI(float, float)
        else if (x32) DLM_ROUTER_MULTI(float, __nv_bfloat16)
        else DLM_ROUTER_MULTI(__nv_bfloat16, __nv_bfloat16)
#undef DLM_ROUTER_MULTI
        check_launch("router_logits_multi");
    } else {
    dim3 grid(T, (rows + ROUTER_WARPS - 1) / ROUTER_WARPS);
#define DLM_ROUTER(TX, TW, VEC)                                                                               \
    {                                                                                                         \
        auto kern = router_logits_kernel<TX, TW, VEC>;                                                        \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
        launch_dep(kern, grid, ROUTER_THREADS, smem, stream, static_cast<const TX*>(h),                       \
                   static_cast<const TW*>(w), norm_w, eps, logits, H, rows);                                  \
    }
    // with norm_w the activations are the 32-bit residual whatever the weights' dtype
    if (dtype == F32) { if (vec) DLM_ROUTER(float, float, true) else DLM_ROUTER(float, float, false) }
    else if (x32) { if (vec) DLM_ROUTER(float, __nv_bfloat16, true) else DLM_ROUTER(float, __nv_bfloat16, false) }
    else { if (vec) DLM_ROUTER(__nv_bfloat16, __nv_bfloat16, true) else DLM_ROUTER(__nv_bfloat16, __nv_bfloat16, false) }
#undef DLM_ROUTER
    check_launch("router_logits");
    }
    const int wpb = 4;
    const size_t smem2 = sizeof(float) * (size_t)wpb * 2 * (E + 1);
    cudaFuncSetAttribute(router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    launch_dep(router_select_kernel, (T + wpb - 1) / wpb, wpb * 32, smem2, stream, logits, ids, wts, gate, T, E, k,
               norm, has_gate, score_fn, scale, select_bias);
    check_launch("router_select");
}

void moe_permute(const int32_t* ids, int n, int k, int E, int32_t* offsets, int32_t* rows, int32_t* dest,
                 cudaStream_t stream) {
    DLM_CHECK(E >= 1 && E <= 4096, "moe_permute: num_experts must be in 1..4096");
    DLM_CHECK(k >= 1, "moe_permute: k must be >= 1");
    launch_dep(moe_permute_kernel, 1, PERMUTE_THREADS, sizeof(int) * 2 * E, stream, ids, n < 0 ? 0 : n, k, E, offsets,
               rows, dest, error_flag_ptr());
    check_launch("moe_permute");
}

int router_topk_permute(const void* h, const void* w, const float* norm_w, float eps, float* logits, int32_t* ids,
                         float* wts, float* gate, int32_t* offsets, int32_t* rows_out, int32_t* dest, int T, int H,
                         int E, int k, int norm, int has_gate, int dtype, int h_is_f32, int score_fn, float scale,
                         const float* select_bias, int x_settled, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int rows = E + (has_gate ? 1 : 0);
    const size_t need = sizeof(float) * (size_t)H;
    const size_t need2 = sizeof(float) * (size_t)ROUTER_WARPS * 2 * (E + 1);
    const size_t smem = need > need2 ? need : need2;
    const size_t smem_token = sizeof(float) * ((size_t)H + 2 * (size_t)(E + 1));
    // (measured, 60 experts of 2,048: 24 / 32 / 48 tokens 3 % / 2 % / 2 % faster a decode step than the three
    // launches, 64 tokens 1.4 % slower: a block then reads the whole matrix for one token, on 64 multiprocessors)
    const bool per_token = T > 16 && T <= 48 && smem_token <= 200 * 1024 && E <= 4096;
    if ((T > 16 && !per_token) || smem > 200 * 1024 || E > 4096) {
        router_topk(h, w, norm_w, eps, logits, ids, wts, gate, T, H, E, k, norm, has_gate, dtype, h_is_f32, score_fn,
                    scale, select_bias, x_settled, stream);
        moe_permute(ids, T * k, k, E, offsets, rows_out, dest, stream);
        return 3;
    }
    DLM_CHECK(E >= 1 && k >= 1 && k <= E, "router: top-k must be in 1..num_experts");
    DLM_CHECK(score_fn == 0 || score_fn == 1, "router: score function must be 0 (softmax) or 1 (sigmoid)");
    const bool x32 = norm_w != nullptr || h_is_f32 != 0;
    const bool vec = H % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    if (per_token) {
#define DLM_ROUTER_TOKEN(TX, TW, VEC)                                                                         \
    {                                                                                                         \
        auto kern = router_token_kernel<TX, TW, VEC>;                                                         \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_token);             \
        launch_dep(kern, T, TOKEN_WARPS * 32, smem_token, stream, static_cast<const TX*>(h),                  \
                   static_cast<const TW*>(w), norm_w, eps, logits, ids, wts, gate, offsets, rows_out, dest, T, H, E, \
                   k, norm, has_gate, score_fn, scale, select_bias, error_flag_ptr());                        \
    }
        if (dtype == F32) { if (vec) DLM_ROUTER_TOKEN(float, float, true) else DLM_ROUTER_TOKEN(float, float, false) }
        else if (x32) { if (vec) DLM_ROUTER_TOKEN(float, __nv_bfloat16, true) else DLM_ROUTER_TOKEN(float, __nv_bfloat16, false) }
        else { if (vec) DLM_ROUTER_TOKEN(__nv_bfloat16, __nv_bfloat16, true) else DLM_ROUTER_TOKEN(__nv_bfloat16, __nv_bfloat16, false) }
#undef DLM_ROUTER_TOKEN
        check_launch("router_token");
        return 1;
    }
    dim3 grid(T, (rows + ROUTER_WARPS - 1) / ROUTER_WARPS);
#define DLM_ROUTER_FUSED(TX, TW, VEC)                                                                         \
    {                                                                                                         \
        auto kern = router_fused_kernel<TX, TW, VEC>;                                                         \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
        launch_dep(kern, grid, ROUTER_THREADS, smem, stream, static_cast<const TX*>(h),                       \
                   static_cast<const TW*>(w), norm_w, eps, logits, ids, wts, gate, offsets, rows_out, dest, T, H, E, \
                   k, norm, has_gate, score_fn, scale, select_bias, x_settled, error_flag_ptr());             \
    }
    if (dtype == F32) { if (vec) DLM_ROUTER_FUSED(float, float, true) else DLM_ROUTER_FUSED(float, float, false) }
    else if (x32) { if (vec) DLM_ROUTER_FUSED(float, __nv_bfloat16, true) else DLM_ROUTER_FUSED(float, __nv_bfloat16, false) }
    else { if (vec) DLM_ROUTER_FUSED(__nv_bfloat16, __nv_bfloat16, true) else DLM_ROUTER_FUSED(__nv_bfloat16, __nv_bfloat16, false) }
#undef DLM_ROUTER_FUSED
    check_launch("router_fused");
    return 1;
}

}  // namespace dlmk
