// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference (vedantnimbarte/dlm); it exists for embedders of this
// library.  Some hosts drive the kernels from places where cudaMalloc is off limits: a real-time
// loop that must not take the allocator's locks or trigger a device synchronisation, a process
// whose device memory was handed out once at start-up and is now fully owned by another allocator,
// a plug-in whose host forbids calls that change the address space.  The engine's normal path lets
// PyTorch's caching allocator provide the decode-attention kernel's scratch buffer; this entry
// point instead keeps that scratch in a fixed array inside the library's own device image.
//
// dlm_b200_decode_attention_noalloc: decode attention (one query token per request, bfloat16)
// over paged keys and values, the same computation as dlmk::attention_decode, with these terms:
//
//  * It calls no cudaMalloc, cudaFree, cudaHostAlloc or any other allocating routine.  Inputs and
//    the output are the caller's buffers.
//  * The split-key partial results live in a file-scope __device__ array of
//    DLM_B200_NOALLOC_SCRATCH_FLOATS floats (4 MiB) plus a 256-byte status block.  Every GPU on
//    which the library's image is loaded holds these bytes until the process exits.
//  * A call whose partial results would not fit (requests x heads x splits x (head_dim + 2) floats
//    beyond the maximum) is refused: the return value is non-zero and `err_msg` (if given) says why.
//    Nothing is launched in that case.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and remembers it.  Make that first call outside of any stream capture.
//  * All calls share the one array, and it keeps whatever the last call left in it.  The kernels
//    write every partial result they later read, so nothing needs to start at zero except the
//    status word, which each call clears on `stream` before launching.  Two calls that overlap on
//    the GPU (different streams, or graphs replayed concurrently) race on the array: serialise them.
//
//  * A return value of 0 means "launched", not "correct".  The kernels never read through a page id
//    that is missing (-1) or outside the pool for a key the query must see: they skip that key's page,
//    the output is then computed without it, and they record code 3 in the status word.  A caller
//    that cannot rule such tables out asks for the word with dlm_b200_noalloc_status after the call.
//
// Returns 0 once everything is launched; 1 for arguments the kernel cannot take (message in err_msg);
// a CUDA error code otherwise.
//
// dlm_b200_noalloc_status: copies the status word of the calls made on this device so far (0: every
// visible key had a page; 3: some call skipped a visible key that had no page) to `host_status` with one
// cudaMemcpyAsync on `stream`; the value is there once the stream has reached that point (synchronise
// the stream or an event recorded after it; use pinned memory if the copy must not block).  Each
// attention call clears the word before it launches, so ask after each call whose answer matters.
// Allocates nothing.  Returns 0, 1 for a null pointer, or a CUDA error code.
#pragma once
#include <cuda_runtime.h>

#include <stddef.h>
#include <stdint.h>

#define DLM_B200_NOALLOC_SCRATCH_FLOATS (1u << 20)

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int dlm_b200_decode_attention_noalloc(
    const void* q,                 // bf16 [T, nh * hd]; request r's only query row is cu_q[r]
    const void* k_cache,           // bf16 [total_pages, nkv, page_size, hd]
    const void* v_cache,           // bf16, same shape
    const int32_t* block_table,    // [R, table_width] logical page -> physical page (-1: none)
    int table_width,
    const int32_t* cu_q,           // [R + 1]; requests with cu_q[r + 1] - cu_q[r] != 1 are skipped
    const int32_t* kv_len,         // [R] tokens each request holds (the query is the last one)
    void* out,                     // bf16 [T, nh * hd]
    int R, int nh, int nkv, int hd, int page_size, int total_pages,
    int window,                    // 0: all keys; W: the last W keys
    float scale,
    int max_kv_len,                // upper bound of kv_len (sizes the split)
    cudaStream_t stream,
    char* err_msg, size_t err_msg_len);

__attribute__((visibility("default"))) int dlm_b200_noalloc_status(int* host_status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
