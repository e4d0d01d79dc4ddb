// Shared device helpers: element conversion, warp/block reductions, error checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>

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

// Programmatic dependent launch.  A kernel launched through launch_dep() may be made resident
// while the kernel before it in the stream is still running, as soon as every block of that kernel
// has called dep_launch_next() or ended.  It must call dep_wait() before it reads anything an earlier
// kernel wrote and before it writes anything at all; dep_wait() returns when the earlier kernel
// has ended and its writes are visible.  Every block calls dep_wait() before it ends, so that
// "this kernel has ended" implies "all earlier kernels have ended".  What a kernel does before
// dep_wait() (index arithmetic, loads of weights, which no kernel writes) overlaps the end of the
// kernel before it.  Launched in the ordinary way both calls do nothing.  Pointers to what earlier
// kernels write (and to what this kernel writes) are not declared __restrict__ in such kernels:
// the compiler may move an access through a __restrict__ pointer across dep_wait(), which is an
// assembly statement that clobbers memory and so orders every other access.
__device__ __forceinline__ void dep_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Whether launch_dep() asks for the early launch (off: DLM_B200_NO_PDL=1, or set_dep_launch(false)).
bool dep_launch_enabled();
void set_dep_launch(bool on);

template <typename... P, typename... A>
inline void launch_dep(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dep_launch_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);   // an error shows in check_launch()
}

// Multiprocessors of the current device (asked once).
int sm_count();

// Device pointer of the host-mapped error flag (see take_error_flag in api.h).
int* error_flag_ptr();

// silu(z) = z / (1 + exp(-z)), as the reference writes it
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

}  // namespace dlmk
