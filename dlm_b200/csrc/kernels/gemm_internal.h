// Kernels behind dlmk::gemm (see api.h for the meaning of the arguments).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace dlmk {

// FMA-unit kernel: any sizes, both dtypes.
void gemm_simt(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
               const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
               int K, int in_dtype, int out_dtype, int epilogue, cudaStream_t stream);

// Weight-streaming tensor-core kernel for few rows of A (bfloat16 inputs only).  rows_per_pass: how many
// rows of A (of one group) meet the weights in one pass over them: up to 8, 16 or 32.
bool gemm_smallm_ok(const void* a, int lda, const void* w, int ldw, long long w_expert_stride, int M, int N, int K,
                    int in_dtype);
void gemm_smallm(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
                 const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
                 int K, int out_dtype, int epilogue, int rows_per_pass, cudaStream_t stream);

// The same job with bulk asynchronous copies into shared memory, one persistent block per multiprocessor
// (bfloat16 inputs only; grouped: at most 1,024 experts can have rows).  Off with DLM_B200_NO_STREAM=1.
bool gemm_stream_enabled();
bool gemm_stream_ok(const void* a, int lda, const void* w, int ldw, long long w_expert_stride,
                    const int32_t* expert_offsets, int num_experts, int M, int N, int K, int in_dtype);
void gemm_stream(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
                 const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
                 int K, int out_dtype, int epilogue, int rows_per_pass, cudaStream_t stream);

// Warp-level tensor-core kernel for many rows of A (bfloat16 inputs; same alignment needs as gemm_smallm).
void gemm_mma(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
              const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
              int K, int out_dtype, int epilogue, cudaStream_t stream);

// tcgen05 / TMA kernel for many rows of A (bfloat16 inputs, rows of A contiguous: no gather).  gemm_tc returns
// false when the tensor maps cannot be made (the caller then takes another kernel).
// Grouped products go to the tcgen05 kernel from a little more than one row per expert on average.  (Measured
// on a decode step of 60 experts, top 4, rows of 2,048 and 1,408 elements, tok/s on the streaming kernel against
// this one: 56 rows over the experts 3,106 : 2,945; 64 rows 3,390 : 3,204; 72 rows 3,325 : 3,440; 80 rows
// 3,394 : 3,493; 96 rows 3,690 : 3,930; 256 rows 7,180 : 8,010.  64 experts, top 8, rows of 3,584 elements, 512
// rows: 1,980 : 3,140.)
inline bool grouped_rows_are_many(long long M, long long num_experts) { return 8 * M > 9 * num_experts; }
bool gemm_tc_enabled();
bool gemm_tc_ok(const void* a, int lda, const void* w, int ldw, long long w_expert_stride, int M, int N, int K,
                int in_dtype);
bool gemm_tc(const void* a, int lda, const void* w, int ldw, const int32_t* expert_offsets, int num_experts,
             const float* bias, void* out, int ldo, int M, int N, int K, int out_dtype, int epilogue,
             cudaStream_t stream);

// The same on pairs of multiprocessors (tcgen05.mma.cta_group::2: 256 weight rows a tile); gemm_tc tries it
// first when N > 128.  Off with DLM_B200_NO_PAIR=1.
bool gemm_tc_pair_enabled();
bool gemm_tc_pair(const void* a, int lda, const void* w, int ldw, const int32_t* expert_offsets, int num_experts,
                  const float* bias, void* out, int ldo, int M, int N, int K, int out_dtype, int epilogue,
                  cudaStream_t stream);

}  // namespace dlmk
