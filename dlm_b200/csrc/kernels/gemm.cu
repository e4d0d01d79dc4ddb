// Chooses the kernel of a matrix product.
#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"

namespace dlmk {

void gemm(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
          const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N, int K,
          int in_dtype, int out_dtype, int epilogue, int fast, cudaStream_t stream) {
    // more rows than the weight-streaming kernel takes in one pass, or experts with more than a row or two
    // each: the tcgen05 kernel (rows of A must be contiguous)
    if (fast && a_rows == nullptr && gemm_tc_enabled() &&
        gemm_tc_ok(a, lda, w, ldw, w_expert_stride, M, N, K, in_dtype) &&
        ((expert_offsets == nullptr && M > 16) ||
         (expert_offsets != nullptr && bias == nullptr && grouped_rows_are_many(M, num_experts)))) {
        if (gemm_tc(a, lda, w, ldw, expert_offsets, num_experts, bias, out, ldo, M, N, K, out_dtype, epilogue, stream))
            return;
    }
    if (fast && gemm_smallm_ok(a, lda, w, ldw, w_expert_stride, M, N, K, in_dtype)) {
        const bool stream_ok = gemm_stream_enabled() &&
            gemm_stream_ok(a, lda, w, ldw, w_expert_stride, expert_offsets, num_experts, M, N, K, in_dtype);
        if (expert_offsets == nullptr) {
            if (M <= 16 && stream_ok) {
                gemm_stream(a, lda, a_rows, w, ldw, w_expert_stride, nullptr, 0, bias, out, ldo, M, N, K, out_dtype,
                            epilogue, M, stream);
                return;
            }
            if (M <= 64) {
                gemm_smallm(a, lda, a_rows, w, ldw, w_expert_stride, nullptr, 0, bias, out, ldo, M, N, K, out_dtype,
                            epilogue, M, stream);
                return;
            }
            gemm_mma(a, lda, a_rows, w, ldw, w_expert_stride, nullptr, 0, bias, out, ldo, M, N, K, out_dtype, epilogue,
                     stream);
            return;
        } else if (bias == nullptr && (long long)M <= 16LL * num_experts) {
            // few rows per expert on average (and the tcgen05 kernel did not take them): stream each active
            // expert's weights once
            const int avg2 = (2 * M + num_experts - 1) / num_experts;     // twice the mean rows per expert
            if (stream_ok) {
                gemm_stream(a, lda, a_rows, w, ldw, w_expert_stride, expert_offsets, num_experts, nullptr, out, ldo,
                            M, N, K, out_dtype, epilogue, avg2 <= 4 ? 8 : (avg2 <= 16 ? 16 : 32), stream);
                return;
            }
            gemm_smallm(a, lda, a_rows, w, ldw, w_expert_stride, expert_offsets, num_experts, nullptr, out, ldo, M, N,
                        K, out_dtype, epilogue, avg2 <= 4 ? 8 : (avg2 <= 16 ? 16 : 32), stream);
            return;
        } else if (bias == nullptr) {
            gemm_mma(a, lda, a_rows, w, ldw, w_expert_stride, expert_offsets, num_experts, nullptr, out, ldo, M, N, K,
                     out_dtype, epilogue, stream);
            return;
        }
    }
    gemm_simt(a, lda, a_rows, w, ldw, w_expert_stride, expert_offsets, num_experts, bias, out, ldo, M, N, K, in_dtype,
              out_dtype, epilogue, stream);
}

}  // namespace dlmk
