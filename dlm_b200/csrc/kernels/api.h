// Launchers of every kernel.  All pointers are device pointers; `stream` is the
// CUDA stream to launch on.  dtype: 0 = float32, 1 = bfloat16 (dlmk::DType).
// Launchers validate sizes and throw std::invalid_argument for what a kernel
// cannot take; none of them allocates memory.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace dlmk {

enum Epilogue : int {
    EPI_STORE = 0,    // out[m, n] = acc (+ bias[n]), stored as the output dtype
    EPI_ADD = 1,      // out[m, n] += acc, out is float32 (the residual stream)
    EPI_SWIGLU = 2    // out[m, n/2] = silu(acc[m, n]) * acc[m, n+1] for even n (interleaved weight rows)
};

// out[T, H] (f32) = table[tokens[t], :]
void embed(const int32_t* tokens, const void* table, float* out, int T, int H, int V, int dtype, cudaStream_t stream);

// out[i, :] = x[rows ? rows[i] : i, :] * rsqrt(mean(x^2) + eps) * w      (x, w f32; out dtype given)
void rmsnorm(const float* x, const float* w, void* out, const int32_t* rows, int n_rows, int H, float eps,
             int out_dtype, cudaStream_t stream);

// C[M, N] = A[M, K] · W[N, K]^T with an epilogue.  Dense: expert_offsets == nullptr.
// Grouped: rows [expert_offsets[e], expert_offsets[e+1]) use W + e * w_expert_stride elements.
// a_rows (optional) gathers the rows of A: row m of the product reads A[a_rows[m], :].
// `fast` != 0 allows tensor-core kernels (bfloat16 inputs only); 0 forces the plain FMA kernel.
// expert_offsets are read before the kernel launched just before this one has ended (the tensor-core kernel lists
// its tiles while it is set up): that kernel must not be the one that writes them (in a layer a gather or the
// experts' first product lies in between).
void gemm(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
          const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N, int K,
          int in_dtype, int out_dtype, int epilogue, int fast, cudaStream_t stream);

// True when the tcgen05 / TMA matrix kernel can be used (it needs the driver's tensor-map encoder; the
// environment variable DLM_B200_NO_TCGEN05=1 switches it off).
bool gemm_tc_enabled();

// out[i, :] = src[rows[i], :] for bfloat16 / float32 rows of `width` elements (width * element size a multiple
// of 16 bytes): the gather that puts an expert's rows side by side before a grouped product.
void gather_rows(const void* src, const int32_t* rows, void* out, int n_rows, int width, int dtype,
                 cudaStream_t stream);

// Rotates q and k heads of qkv[T, (nh + 2 nkv) * hd] (f32) by position * inv_freq within the first rotary_dim
// dims (pair i is dims (i, i + rotary_dim / 2), or (2i, 2i + 1) with interleaved != 0; inv_freq == nullptr: no
// rotation), writes q to q_out[T, nh * hd] and, where slots != nullptr and slots[t] >= 0, k and v to the paged
// caches [pages, nkv, page_size, hd].  positions, slots and inv_freq are read before the kernel launched just
// before this one has ended (they are a step's inputs): that kernel must not be the one that writes them.
void rope_kv_write(const float* qkv, const int32_t* positions, const float* inv_freq, int rotary_dim, int interleaved,
                   const int32_t* slots, void* q_out, void* k_cache, void* v_cache, int T, int nh, int nkv, int hd,
                   int page_size, int total_pages, int dtype, cudaStream_t stream);

// Causal (optionally windowed) attention of every token of the step over its request's paged keys and values.
// num_single: how many requests have exactly one query token.  With fast != 0 and a scratch buffer of
// attention_scratch_floats(...) floats those go to the split-key decode kernel.
void attention(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table, int table_width,
               const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh, int nkv, int hd,
               int page_size, int total_pages, int window, float scale, int max_q_len, int max_kv_len,
               int num_single, float* scratch, int dtype, int fast, cudaStream_t stream);
// Floats of scratch the decode kernel needs for a step of R requests whose longest holds max_kv_len tokens.
size_t attention_scratch_floats(int R, int nh, int nkv, int hd, int max_kv_len);

// Router: logits = h · w^T (32-bit); scores = softmax over E (score_fn 0) or sigmoid of each logit (score_fn 1);
// the k best scores (ties: lower index; with select_bias[E] the choice is made on score + bias and the weight
// stays the score); norm != 0: the chosen weights are divided by their sum; all are multiplied by `scale`.
// has_gate: w has E + 1 rows and gate[t] = sigmoid(h · w[E]).  The input h is: activations of the weights' dtype
// (default); the 32-bit residual, with rmsnorm(h, norm_w, eps) applied first in 32-bit (norm_w != nullptr); or
// 32-bit activations that are already normalised (h_is_f32 != 0).  dtype is the weights' dtype.
// logits: scratch of T * (E + has_gate) floats (the router logits are left there).
void router_topk(const void* h, const void* w, const float* norm_w, float eps, float* logits, int32_t* ids, float* wts,
                 float* gate, int T, int H, int E, int k, int norm, int has_gate, int dtype, int h_is_f32,
                 int score_fn, float scale, const float* select_bias, int x_settled, cudaStream_t stream);

// router_topk followed by moe_permute (below).  One launch up to 16 tokens (blocks of 8 experts per token, the
// block that finishes last chooses for every token and groups) and from 17 to 48 tokens (a block per token
// computes all its logits and chooses; the last block groups); three launches from 49 tokens on.  Returns the
// number of launches.  x_settled != 0: `h` was written before the kernel launched just before this one began its
// work (a step's residual, with a norm kernel in between): the logits of at most 16 tokens, or the first of 512
// and more, are then worked out while that kernel ends (`router_topk` takes the same flag).
int router_topk_permute(const void* h, const void* w, const float* norm_w, float eps, float* logits, int32_t* ids,
                         float* wts, float* gate, int32_t* offsets, int32_t* rows, int32_t* dest, int T, int H, int E,
                         int k, int norm, int has_gate, int dtype, int h_is_f32, int score_fn, float scale,
                         const float* select_bias, int x_settled, cudaStream_t stream);

// Groups the n = T * k (token, choice) pairs by expert: offsets[E + 1], rows[n] = token of each sorted row,
// dest[n] = sorted row of pair (t, j).
void moe_permute(const int32_t* ids, int n, int k, int E, int32_t* offsets, int32_t* rows, int32_t* dest,
                 cudaStream_t stream);

// resid[t, :] += sum_j wts[t, j] * y[dest[t, j], :] (+ gate[t] * shared[t, :]); gate == nullptr: 1.
void moe_combine(const float* y, const int32_t* dest, const float* wts, const float* shared, const float* gate,
                 float* resid, int T, int H, int k, cudaStream_t stream);

// out[i] = index of the first maximum of logits[i, :].  scratch: argmax_scratch_bytes(N, V) bytes (may be
// nullptr when that is 0; a large vocabulary is then searched by one block per row).
void argmax(const float* logits, int32_t* out, int N, int V, void* scratch, cudaStream_t stream);
size_t argmax_scratch_bytes(int N, int V);

// Per row: repetition penalty over seen tokens, then greedy (temperature <= 0) or temperature / top-k / top-p /
// min-p sampling with the uniform number u[i] (candidates ordered by logit descending, ties by index).
// seen_offsets[N + 1] indexes seen_tokens; params[i] = {temperature, top_p, min_p, repetition_penalty}; top_k[i].
// scratch: N * V floats.
void sample(const float* logits, int32_t* out, int N, int V, const float* params, const int32_t* top_k,
            const float* u, const int32_t* seen_offsets, const int32_t* seen_tokens, float* scratch,
            cudaStream_t stream);

// A device-side error flag kernels set instead of touching memory they must not (a page id outside the pool,
// an expert id outside the table).  Returns the flag and clears it.
int take_error_flag();

// Clears what a decode attention launch that ended through a bounded wait's give-up path (error 5) may have
// left in the split-merge counters, so that later steps merge correctly.  Call after take_error_flag() == 5.
void reset_decode_merge_counters(cudaStream_t stream);

// Whether the small kernels are launched so that each may start while the one before it ends
// (programmatic dependent launch; on unless DLM_B200_NO_PDL=1).
bool dep_launch_enabled();
void set_dep_launch(bool on);

}  // namespace dlmk
