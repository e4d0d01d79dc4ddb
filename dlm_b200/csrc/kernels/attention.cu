// Chooses the attention kernels of a step.
#include "api.h"
#include "attention_internal.h"
#include "common.cuh"

namespace dlmk {

size_t attention_scratch_floats(int R, int nh, int nkv, int hd, int max_kv_len) {
    if (R <= 0 || !attention_decode_ok(hd)) return 0;
    int n_splits, chunk;
    attention_decode_plan(R, nkv, max_kv_len < 1 ? 1 : max_kv_len, &n_splits, &chunk);
    return attention_decode_scratch_floats(R, nh, hd, n_splits);
}

void attention(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table, int table_width,
               const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh, int nkv, int hd,
               int page_size, int total_pages, int window, float scale, int max_q_len, int max_kv_len,
               int num_single, float* scratch, int dtype, int fast, cudaStream_t stream) {
    if (T <= 0 || R <= 0) return;
    const bool decode = fast && num_single > 0 && scratch != nullptr && attention_decode_ok(hd);
    if (decode) {
        int n_splits, chunk;
        attention_decode_plan(R, nkv, max_kv_len < 1 ? 1 : max_kv_len, &n_splits, &chunk);
        if (dtype == BF16 && attention_prefill_ok(hd))
            attention_decode_mma(q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, out, scratch, R, nh, nkv,
                                 hd, page_size, total_pages, window, scale, n_splits, chunk, stream);
        else
            attention_decode(q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, out, scratch, R, nh, nkv, hd,
                             page_size, total_pages, window, scale, n_splits, chunk, dtype, stream);
    }
    if (!decode || num_single < R) {
        if (fast && dtype == BF16 && attention_prefill_tc_enabled() &&
            attention_prefill_tc_ok(q, k_cache, v_cache, nh, nkv, hd, page_size, scale) &&
            attention_prefill_tc(q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, out, T, R, nh, nkv, hd,
                                 page_size, total_pages, window, scale, decode ? 1 : 0, stream)) {
            // done on the tcgen05 path
        } else if (fast && dtype == BF16 && attention_prefill_ok(hd))
            attention_prefill(q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, out, T, R, nh, nkv, hd,
                              page_size, total_pages, window, scale, decode ? 1 : 0, stream);
        else
            attention_simt(q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, out, T, R, nh, nkv, hd,
                           page_size, total_pages, window, scale, decode ? 1 : 0, dtype, stream);
    }
    (void)max_q_len;
}

}  // namespace dlmk
