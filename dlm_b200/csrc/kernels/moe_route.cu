// Routing: router logits, softmax, top-k and the grouping of (token, expert) pairs by expert.
#include "api.h"
#include "common.cuh"

namespace dlmk {

namespace {

constexpr int ROUTER_THREADS = 128;

// One block per token.  Each expert's logit is one warp's dot product summed in a fixed order,
// so routing does not depend on what else is in the batch.
template <typename T>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_topk_kernel(const T* __restrict__ h, const T* __restrict__ w, int32_t* __restrict__ ids,
                   float* __restrict__ wts, float* __restrict__ gate, int H, int E, int k, int norm, int has_gate) {
    extern __shared__ float smem[];
    float* x = smem;            // [H]
    float* prob = x + H;        // [E + 1]
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nwarp = blockDim.x >> 5;
    for (int i = tid; i < H; i += blockDim.x) x[i] = to_f32(h[(long long)t * H + i]);
    __syncthreads();
    const int rows = E + (has_gate ? 1 : 0);
    for (int e = warp; e < rows; e += nwarp) {
        const T* wr = w + (long long)e * H;
        float s = 0.f;
        for (int i = lane; i < H; i += 32) s = fmaf(x[i], to_f32(wr[i]), s);
        s = warp_sum(s);
        if (lane == 0) prob[e] = s;
    }
    __syncthreads();
    if (warp != 0) return;
    if (has_gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-prob[E]));
    // softmax over the E experts
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
    __syncwarp();
    // k rounds of arg-max; equal probabilities: the lower index wins
    float chosen_sum = 0.f;
    for (int j = 0; j < k; ++j) {
        float bv = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float p = prob[e];
            if (p > bv) { bv = p; bi = e; }     // ascending e per lane: ties keep the lower index
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            ids[t * k + j] = bi;
            wts[t * k + j] = bv;
            prob[bi] = -2.f;                    // taken
        }
        chosen_sum += bv;
        __syncwarp();
    }
    if (norm && chosen_sum > 0.f && lane == 0)
        for (int j = 0; j < k; ++j) wts[t * k + j] = wts[t * k + j] / chosen_sum;
}

constexpr int PERMUTE_THREADS = 1024;

__global__ void __launch_bounds__(PERMUTE_THREADS)
moe_permute_kernel(const int32_t* __restrict__ ids, int n, int k, int E, int32_t* __restrict__ offsets,
                   int32_t* __restrict__ rows, int32_t* __restrict__ dest, int* err) {
    extern __shared__ int sm[];
    int* count = sm;          // [E]
    int* cursor = sm + E;     // [E]
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
        const int e = ids[i];
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
        const int e = ids[i];
        if (e >= 0 && e < E) {
            const int pos = atomicAdd(&cursor[e], 1);
            rows[pos] = i / k;
            dest[i] = pos;
        } else {
            dest[i] = 0;
        }
    }
}

}  // namespace

void router_topk(const void* h, const void* w, int32_t* ids, float* wts, float* gate, int T, int H, int E, int k,
                 int norm, int has_gate, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(E >= 1 && k >= 1 && k <= E, "router: top-k must be in 1..num_experts");
    const size_t smem = sizeof(float) * (size_t)(H + E + 1);
    DLM_CHECK(smem <= 200 * 1024, "router: hidden_size + num_experts does not fit in shared memory");
    if (dtype == F32) {
        auto kern = router_topk_kernel<float>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<T, ROUTER_THREADS, smem, stream>>>(static_cast<const float*>(h), static_cast<const float*>(w), ids,
                                                  wts, gate, H, E, k, norm, has_gate);
    } else {
        auto kern = router_topk_kernel<__nv_bfloat16>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<T, ROUTER_THREADS, smem, stream>>>(static_cast<const __nv_bfloat16*>(h),
                                                  static_cast<const __nv_bfloat16*>(w), ids, wts, gate, H, E, k, norm,
                                                  has_gate);
    }
    check_launch("router_topk");
}

void moe_permute(const int32_t* ids, int n, int k, int E, int32_t* offsets, int32_t* rows, int32_t* dest,
                 cudaStream_t stream) {
    DLM_CHECK(E >= 1 && E <= 4096, "moe_permute: num_experts must be in 1..4096");
    DLM_CHECK(k >= 1, "moe_permute: k must be >= 1");
    moe_permute_kernel<<<1, PERMUTE_THREADS, sizeof(int) * 2 * E, stream>>>(ids, n < 0 ? 0 : n, k, E, offsets, rows,
                                                                            dest, error_flag_ptr());
    check_launch("moe_permute");
}

}  // namespace dlmk
