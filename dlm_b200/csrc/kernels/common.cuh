// Shared device helpers: element conversion, warp/block reductions, error checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

namespace dlmk {

enum DType : int { F32 = 0, BF16 = 1 };

#define DLM_CHECK(cond, msg)                                                        \
    do {                                                                            \
        if (!(cond)) throw std::invalid_argument(std::string("dlm_b200 kernels: ") + (msg)); \
    } while (0)

inline void check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        throw std::runtime_error(std::string("dlm_b200 kernels: launch of ") + what + " failed: " +
                                 cudaGetErrorString(e));
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block in a fixed order (per-thread partials -> warp trees -> serial over warps).
// `scratch` holds at least 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nwarp; ++i) t += scratch[i];
    return t;
}

// Device pointer of the host-mapped error flag (see take_error_flag in api.h).
int* error_flag_ptr();

// silu(z) = z / (1 + exp(-z)), as the reference writes it
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

}  // namespace dlmk
