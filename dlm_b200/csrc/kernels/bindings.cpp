// Python bindings of the kernel launchers.  Pointers and the stream arrive as integers
// (tensor.data_ptr(), stream.cuda_stream); shapes are checked on the Python side.
#include <pybind11/pybind11.h>

#include "api.h"

namespace py = pybind11;
using u64 = uintptr_t;

namespace {
template <typename T> T* ptr(u64 p) { return reinterpret_cast<T*>(p); }
cudaStream_t st(u64 s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

PYBIND11_MODULE(_dlm_kernels, m) {
    m.doc() = "dlm_b200 sm_100a kernels";
    m.attr("EPI_STORE") = (int)dlmk::EPI_STORE;
    m.attr("EPI_ADD") = (int)dlmk::EPI_ADD;
    m.attr("EPI_SWIGLU") = (int)dlmk::EPI_SWIGLU;

    m.def("embed", [](u64 tokens, u64 table, u64 out, int T, int H, int V, int dtype, u64 stream) {
        dlmk::embed(ptr<const int32_t>(tokens), ptr<const void>(table), ptr<float>(out), T, H, V, dtype, st(stream));
    });
    m.def("rmsnorm", [](u64 x, u64 w, u64 out, u64 rows, int n_rows, int H, float eps, int out_dtype, u64 stream) {
        dlmk::rmsnorm(ptr<const float>(x), ptr<const float>(w), ptr<void>(out), ptr<const int32_t>(rows), n_rows, H,
                      eps, out_dtype, st(stream));
    });
    m.def("gemm", [](u64 a, int lda, u64 a_rows, u64 w, int ldw, long long w_expert_stride, u64 expert_offsets,
                     int num_experts, u64 bias, u64 out, int ldo, int M, int N, int K, int in_dtype, int out_dtype,
                     int epilogue, int fast, u64 stream) {
        dlmk::gemm(ptr<const void>(a), lda, ptr<const int32_t>(a_rows), ptr<const void>(w), ldw, w_expert_stride,
                   ptr<const int32_t>(expert_offsets), num_experts, ptr<const float>(bias), ptr<void>(out), ldo, M, N,
                   K, in_dtype, out_dtype, epilogue, fast, st(stream));
    });
    m.def("rope_kv_write", [](u64 qkv, u64 positions, u64 inv_freq, int rotary_dim, int interleaved, u64 slots,
                              u64 q_out, u64 k_cache, u64 v_cache, int T, int nh, int nkv, int hd, int page_size,
                              int total_pages, int dtype, u64 stream) {
        dlmk::rope_kv_write(ptr<const float>(qkv), ptr<const int32_t>(positions), ptr<const float>(inv_freq),
                            rotary_dim, interleaved, ptr<const int32_t>(slots), ptr<void>(q_out), ptr<void>(k_cache),
                            ptr<void>(v_cache), T, nh, nkv, hd, page_size, total_pages, dtype, st(stream));
    });
    m.def("attention", [](u64 q, u64 k_cache, u64 v_cache, u64 block_table, int table_width, u64 cu_q, u64 kv_len,
                          u64 out, int T, int R, int nh, int nkv, int hd, int page_size, int total_pages, int window,
                          float scale, int max_q_len, int max_kv_len, int num_single, u64 scratch, int dtype, int fast,
                          u64 stream) {
        dlmk::attention(ptr<const void>(q), ptr<const void>(k_cache), ptr<const void>(v_cache),
                        ptr<const int32_t>(block_table), table_width, ptr<const int32_t>(cu_q),
                        ptr<const int32_t>(kv_len), ptr<void>(out), T, R, nh, nkv, hd, page_size, total_pages, window,
                        scale, max_q_len, max_kv_len, num_single, ptr<float>(scratch), dtype, fast, st(stream));
    });
    m.def("attention_scratch_floats", [](int R, int nh, int nkv, int hd, int max_kv_len) {
        return dlmk::attention_scratch_floats(R, nh, nkv, hd, max_kv_len);
    });
    m.def("router_topk", [](u64 h, u64 w, u64 norm_w, float eps, u64 logits, u64 ids, u64 wts, u64 gate, int T, int H,
                            int E, int k, int norm, int has_gate, int dtype, int h_is_f32, int score_fn, float scale,
                            u64 select_bias, u64 stream) {
        dlmk::router_topk(ptr<const void>(h), ptr<const void>(w), ptr<const float>(norm_w), eps, ptr<float>(logits),
                          ptr<int32_t>(ids), ptr<float>(wts), ptr<float>(gate), T, H, E, k, norm, has_gate, dtype,
                          h_is_f32, score_fn, scale, ptr<const float>(select_bias), 0, st(stream));
    });
    m.def("router_topk_permute", [](u64 h, u64 w, u64 norm_w, float eps, u64 logits, u64 ids, u64 wts, u64 gate,
                                    u64 offsets, u64 rows, u64 dest, int T, int H, int E, int k, int norm, int has_gate,
                                    int dtype, int h_is_f32, int score_fn, float scale, u64 select_bias, int x_settled,
                                    u64 stream) {
        return dlmk::router_topk_permute(ptr<const void>(h), ptr<const void>(w), ptr<const float>(norm_w), eps,
                                  ptr<float>(logits), ptr<int32_t>(ids), ptr<float>(wts), ptr<float>(gate),
                                  ptr<int32_t>(offsets), ptr<int32_t>(rows), ptr<int32_t>(dest), T, H, E, k, norm,
                                  has_gate, dtype, h_is_f32, score_fn, scale, ptr<const float>(select_bias),
                                  x_settled, st(stream));
    });
    m.def("moe_permute", [](u64 ids, int n, int k, int E, u64 offsets, u64 rows, u64 dest, u64 stream) {
        dlmk::moe_permute(ptr<const int32_t>(ids), n, k, E, ptr<int32_t>(offsets), ptr<int32_t>(rows),
                          ptr<int32_t>(dest), st(stream));
    });
    m.def("moe_combine", [](u64 y, u64 dest, u64 wts, u64 shared, u64 gate, u64 resid, int T, int H, int k,
                            u64 stream) {
        dlmk::moe_combine(ptr<const float>(y), ptr<const int32_t>(dest), ptr<const float>(wts),
                          ptr<const float>(shared), ptr<const float>(gate), ptr<float>(resid), T, H, k, st(stream));
    });
    m.def("argmax", [](u64 logits, u64 out, int N, int V, u64 scratch, u64 stream) {
        dlmk::argmax(ptr<const float>(logits), ptr<int32_t>(out), N, V, ptr<void>(scratch), st(stream));
    });
    m.def("argmax_scratch_bytes", [](int N, int V) { return dlmk::argmax_scratch_bytes(N, V); });
    m.def("sample", [](u64 logits, u64 out, int N, int V, u64 params, u64 top_k, u64 u, u64 seen_offsets,
                       u64 seen_tokens, u64 scratch, u64 stream) {
        dlmk::sample(ptr<const float>(logits), ptr<int32_t>(out), N, V, ptr<const float>(params),
                     ptr<const int32_t>(top_k), ptr<const float>(u), ptr<const int32_t>(seen_offsets),
                     ptr<const int32_t>(seen_tokens), ptr<float>(scratch), st(stream));
    });
    m.def("gemm_tc_enabled", &dlmk::gemm_tc_enabled);
    m.def("gather_rows", [](u64 src, u64 rows, u64 out, int n_rows, int width, int dtype, u64 stream) {
        dlmk::gather_rows(ptr<const void>(src), ptr<const int32_t>(rows), ptr<void>(out), n_rows, width, dtype,
                          st(stream));
    });
    m.def("take_error_flag", &dlmk::take_error_flag);
    m.def("reset_decode_merge_counters", [](u64 stream) { dlmk::reset_decode_merge_counters(st(stream)); });
    m.def("dep_launch_enabled", &dlmk::dep_launch_enabled);
    m.def("set_dep_launch", &dlmk::set_dep_launch);
}
