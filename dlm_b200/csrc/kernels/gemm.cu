// Chooses the kernel of a matrix product.
#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"

namespace dlmk {

void gemm(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
          const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N, int K,
          int in_dtype, int out_dtype, int epilogue, int fast, cudaStream_t stream) {
    (void)fast;
    gemm_simt(a, lda, a_rows, w, ldw, w_expert_stride, expert_offsets, num_experts, bias, out, ldo, M, N, K, in_dtype,
              out_dtype, epilogue, stream);
}

}  // namespace dlmk
