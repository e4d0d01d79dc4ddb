// Kernels behind dlmk::attention (see api.h for the meaning of the arguments).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace dlmk {

// FMA-unit kernel for any mix of query lengths.  skip_single != 0: requests with exactly one query token are
// left to the decode kernel.
void attention_simt(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                    int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                    int nkv, int hd, int page_size, int total_pages, int window, float scale, int skip_single,
                    int dtype, cudaStream_t stream);

// Tensor-core kernel (bfloat16) for the head sizes attention_prefill_ok names.
bool attention_prefill_ok(int hd);
void attention_prefill(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                       int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                       int nkv, int hd, int page_size, int total_pages, int window, float scale, int skip_single,
                       cudaStream_t stream);

// The same on the fifth-generation tensor cores (tcgen05, TMA): head size 128, pages of a power of two of at
// least 64 tokens.  attention_prefill_tc returns false when the tensor maps cannot be made (the caller then
// takes another kernel).  Off with DLM_B200_NO_TCGEN05=1.
bool attention_prefill_tc_enabled();
bool attention_prefill_tc_ok(const void* q, const void* k_cache, const void* v_cache, int nh, int nkv, int hd,
                             int page_size, float scale);
bool attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                          int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                          int nkv, int hd, int page_size, int total_pages, int window, float scale, int skip_single,
                          cudaStream_t stream);

// Split-key decode kernel for requests with exactly one query token (bfloat16 and float32).
bool attention_decode_ok(int hd);
void attention_decode_plan(int R, int nkv, int max_kv_len, int* n_splits, int* chunk);
size_t attention_decode_scratch_floats(int R, int nh, int hd, int n_splits);
void attention_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                      int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, float* scratch, int R,
                      int nh, int nkv, int hd, int page_size, int total_pages, int window, float scale, int n_splits,
                      int chunk, int dtype, cudaStream_t stream);

void attention_decode_merge(const float* part_o, const float* part_ml, const int32_t* cu_q, void* out, int R, int nh,
                            int hd, int n_splits, int dtype, cudaStream_t stream);
// The same on the tensor-core path (bfloat16, head sizes of attention_prefill_ok); same scratch, same plan.
void attention_decode_mma(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                          int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, float* scratch,
                          int R, int nh, int nkv, int hd, int page_size, int total_pages, int window, float scale,
                          int n_splits, int chunk, cudaStream_t stream);

}  // namespace dlmk
