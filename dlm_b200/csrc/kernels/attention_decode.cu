// Decode attention: one query token per request against its paged keys and values.
// Memory-bound, so the work is cut for bandwidth: the keys of a request are split into
// chunks, one block per (request, kv head, chunk) streams its chunk once with 16-byte
// loads and serves every query head of the kv head's group from the same registers; the
// chunks' partial results (maximum, sum, weighted values) are merged by a second kernel.
// Requests with more than one query token in the step are skipped (the prefill kernel has them).
#include "api.h"
#include "attention_internal.h"
#include "common.cuh"
#include "mma_sync.cuh"

namespace dlmk {

namespace {

constexpr int WARPS = 4;
constexpr int UNROLL = 4;

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// LPK lanes share a key (each holds 8 head dims); GT query heads of the group are served together.
// Keys and values arrive in shared memory in tiles of `tile` keys, two tiles in flight
// (asynchronous 16-byte copies), so that the loads of the next tile overlap the arithmetic of this one.
template <typename T, int LPK, int GT>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ cu_q,
                        const int32_t* __restrict__ kv_len, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int nh, int nkv, int hd, int page_size, int total_pages, int window, float scale, int chunk,
                        int n_splits, int head_passes, int tile, int max_pages, int* err) {
    constexpr int KPW = 32 / LPK;                 // keys per warp per iteration
    constexpr int STREAMS = WARPS * KPW;
    constexpr int EPC = 16 / (int)sizeof(T);      // elements per 16-byte chunk
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* Ks = reinterpret_cast<T*>(smem_raw);                       // [2][tile][hd]
    T* Vs = Ks + 2 * tile * hd;                                   // [2][tile][hd]
    float* sm_m = reinterpret_cast<float*>(Vs + 2 * tile * hd);   // [STREAMS][GT]
    float* sm_l = sm_m + STREAMS * GT;                            // [STREAMS][GT]
    float* sm_o = sm_l + STREAMS * GT;                            // [STREAMS][GT][LPK * 8]
    int* s_table = reinterpret_cast<int*>(sm_o + STREAMS * GT * LPK * 8);   // [max_pages]

    const int r = blockIdx.x;
    const int kvh = blockIdx.y / head_passes, pass = blockIdx.y % head_passes;
    const int sp = blockIdx.z;
    if (cu_q[r + 1] - cu_q[r] != 1) return;
    const int group = nh / nkv;
    const int h0 = kvh * group + pass * GT;                       // first query head of this block
    const int n_heads = min(GT, group - pass * GT);
    const int len = kv_len[r], p = len - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    // the request's own visible keys [lo, len) are cut into n_splits shares (multiples of 64 keys, at most
    // `chunk`), so that a request far shorter than the longest, or one with a window, still uses every block
    int share = (len - lo + n_splits - 1) / n_splits;
    share = min(chunk, (share + 63) / 64 * 64);
    const int j_begin = min(len, lo + sp * share), j_end = min(len, lo + (sp + 1) * share);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int li = lane % LPK, ks = lane / LPK;
    const int d0 = li * 8;
    const bool dim_ok = d0 < hd;                                   // hd is a multiple of 8
    const int token = cu_q[r];

    float m[GT], l[GT], acc[GT][8];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    }

    if (j_begin < j_end) {
        float qv[GT][8];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[g][i] = 0.f;
            if (g < n_heads && dim_ok) Vec8<T>::load(q + (long long)token * nh * hd + (h0 + g) * hd + d0, qv[g]);
        }
        // the pages this block touches
        const int first_page = j_begin / page_size, last_page = (j_end - 1) / page_size;
        const int32_t* table = block_table + (long long)r * table_width;
        for (int i = tid; i <= last_page - first_page && i < max_pages; i += blockDim.x) {
            const int lp = first_page + i;
            int page = lp < table_width ? table[lp] : -1;
            if (page < 0 || page >= total_pages) { *err = 3; page = -1; }
            s_table[i] = page;
        }
        __syncthreads();

        const int cpr = hd / EPC;                                  // 16-byte chunks per key row
        auto fill = [&](int stage, int j0) {
            T* kd = Ks + (size_t)stage * tile * hd;
            T* vd = Vs + (size_t)stage * tile * hd;
            for (int idx = tid; idx < tile * cpr; idx += WARPS * 32) {
                const int key = idx / cpr, c = idx % cpr;
                const int j = j0 + key;
                int page = -1;
                if (j >= j_begin && j < j_end) page = s_table[j / page_size - first_page];
                if (page >= 0) {
                    const long long off = (((long long)page * nkv + kvh) * page_size + (j % page_size)) * hd + c * EPC;
                    cp_async16(kd + key * hd + c * EPC, k_cache + off);
                    cp_async16(vd + key * hd + c * EPC, v_cache + off);
                } else {                                           // nothing to see: zeros, so that 0 * v stays 0
                    *reinterpret_cast<uint4*>(kd + key * hd + c * EPC) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vd + key * hd + c * EPC) = make_uint4(0, 0, 0, 0);
                }
            }
            cp_async_commit();
        };

        const int t_begin = (j_begin / tile) * tile;
        const int n_tiles = (j_end - t_begin + tile - 1) / tile;
        fill(0, t_begin);
        for (int it = 0; it < n_tiles; ++it) {
            const int stage = it & 1;
            const int j0 = t_begin + it * tile;
            if (it + 1 < n_tiles) {
                fill(stage ^ 1, j0 + tile);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            const T* kt = Ks + (size_t)stage * tile * hd;
            const T* vt = Vs + (size_t)stage * tile * hd;
            // every lane of a warp runs the same number of rounds (the shuffles name all 32 lanes)
            for (int kb = warp * KPW; kb < tile; kb += STREAMS * UNROLL) {
                float kf[UNROLL][8], vf[UNROLL][8];
                bool ok[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int key = kb + ks + u * STREAMS;
                    const int j = j0 + key;
                    ok[u] = key < tile && j >= j_begin && j < j_end;
#pragma unroll
                    for (int i = 0; i < 8; ++i) { kf[u][i] = 0.f; vf[u][i] = 0.f; }
                    if (ok[u] && dim_ok) {
                        Vec8<T>::load(kt + key * hd + d0, kf[u]);
                        Vec8<T>::load(vt + key * hd + d0, vf[u]);
                    }
                }
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    if (g >= n_heads) break;
                    float s[UNROLL];
                    float mx = m[g];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        float d = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) d = fmaf(qv[g][i], kf[u][i], d);
#pragma unroll
                        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                        s[u] = ok[u] ? d * scale : -INFINITY;
                        mx = fmaxf(mx, s[u]);
                    }
                    if (mx != -INFINITY) {
                        const float alpha = expf(m[g] - mx);
                        float lsum = l[g] * alpha;
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][i] *= alpha;
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u) {
                            const float pu = ok[u] ? expf(s[u] - mx) : 0.f;
                            lsum += pu;
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(pu, vf[u][i], acc[g][i]);
                        }
                        l[g] = lsum;
                        m[g] = mx;
                    }
                }
            }
            __syncthreads();                                      // the stage may be refilled now
        }
    }

    // merge the block's streams (fixed order)
    const int stream = warp * KPW + ks;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        if (li == 0) { sm_m[stream * GT + g] = m[g]; sm_l[stream * GT + g] = l[g]; }
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_o[(stream * GT + g) * (LPK * 8) + d0 + i] = acc[g][i];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_heads * hd; idx += blockDim.x) {
        const int g = idx / hd, d = idx % hd;
        float mx = -INFINITY;
        for (int s2 = 0; s2 < STREAMS; ++s2) mx = fmaxf(mx, sm_m[s2 * GT + g]);
        float o = 0.f, ls = 0.f;
        if (mx != -INFINITY) {
            for (int s2 = 0; s2 < STREAMS; ++s2) {
                const float ms = sm_m[s2 * GT + g];
                if (ms == -INFINITY) continue;
                const float a = expf(ms - mx);
                o = fmaf(a, sm_o[(s2 * GT + g) * (LPK * 8) + d], o);
                ls = fmaf(a, sm_l[s2 * GT + g], ls);
            }
        }
        const long long base = ((long long)r * nh + (h0 + g)) * n_splits + sp;
        part_o[base * hd + d] = o;
        if (d == 0) { part_ml[base * 2] = mx; part_ml[base * 2 + 1] = ls; }
    }
}

template <typename T>
__global__ void attention_decode_merge_kernel(const float* part_o, const float* part_ml,
                                              const int32_t* __restrict__ cu_q, T* out, int nh, int hd,
                                              int n_splits) {
    dep_wait();
    dep_launch_next();
    const int r = blockIdx.x, h = blockIdx.y;
    if (cu_q[r + 1] - cu_q[r] != 1) return;
    const long long base = ((long long)r * nh + h) * n_splits;
    float mx = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_ml[(base + s) * 2]);
    T* o = out + (long long)cu_q[r] * nh * hd + h * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f, ls = 0.f;
        if (mx != -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float ms = part_ml[(base + s) * 2];
                if (ms == -INFINITY) continue;
                const float a = expf(ms - mx);
                acc = fmaf(a, part_o[(base + s) * hd + d], acc);
                ls = fmaf(a, part_ml[(base + s) * 2 + 1], ls);
            }
        }
        o[d] = from_f32<T>(ls > 0.f ? acc / ls : 0.f);
    }
}

template <typename T, int LPK>
void launch_decode(int gt, dim3 grid, size_t smem_bytes, cudaStream_t stream, const void* q, const void* k_cache,
                   const void* v_cache, const int32_t* block_table, int table_width, const int32_t* cu_q,
                   const int32_t* kv_len, float* part_o, float* part_ml, int nh, int nkv, int hd, int page_size,
                   int total_pages, int window, float scale, int chunk, int n_splits, int head_passes, int* err) {
    // a tile of keys is about 16 KB per stage and tensor, and a multiple of the keys a block handles per round
    const int streams = WARPS * (32 / LPK);
    int tile = 16384 / (hd * (int)sizeof(T));
    tile = tile > 64 ? 64 : tile;
    tile = tile < streams ? streams : tile / streams * streams;
    const int max_pages = chunk / page_size + 2;
    smem_bytes = (size_t)4 * tile * hd * sizeof(T) + sizeof(float) * ((size_t)streams * gt * 2 +
                 (size_t)streams * gt * LPK * 8) + sizeof(int) * max_pages;
#define DLM_LAUNCH(GT)                                                                                         \
    {                                                                                                          \
        auto kern = attention_decode_kernel<T, LPK, GT>;                                                       \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);              \
        kern<<<grid, WARPS * 32, smem_bytes, stream>>>(                                                        \
            static_cast<const T*>(q), static_cast<const T*>(k_cache), static_cast<const T*>(v_cache),          \
            block_table, table_width, cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages,      \
            window, scale, chunk, n_splits, head_passes, tile, max_pages, err);                                \
    }
    if (gt == 1) DLM_LAUNCH(1)
    else if (gt == 2) DLM_LAUNCH(2)
    else if (gt == 4) DLM_LAUNCH(4)
    else DLM_LAUNCH(8)
#undef DLM_LAUNCH
}

}  // namespace

bool attention_decode_ok(int hd) { return hd % 8 == 0 && hd >= 16 && hd <= 256; }

void attention_decode_plan(int R, int nkv, int max_kv_len, int* n_splits, int* chunk) {
    // one resident wave of blocks (three per multiprocessor), chunks of at least 64 keys
    int splits = 3 * sm_count() / (R * nkv);
    const int max_splits = (max_kv_len + 63) / 64;
    splits = splits < 1 ? 1 : (splits > max_splits ? max_splits : splits);
    if (splits > 64) splits = 64;
    int c = (max_kv_len + splits - 1) / splits;
    c = (c + 63) / 64 * 64;
    *chunk = c;
    *n_splits = (max_kv_len + c - 1) / c;
}

size_t attention_decode_scratch_floats(int R, int nh, int hd, int n_splits) {
    return (size_t)R * nh * n_splits * (hd + 2);
}

void attention_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                      int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, float* scratch, int R,
                      int nh, int nkv, int hd, int page_size, int total_pages, int window, float scale, int n_splits,
                      int chunk, int dtype, cudaStream_t stream) {
    if (R <= 0) return;
    DLM_CHECK(attention_decode_ok(hd), "decode attention: head_dim must be a multiple of 8, at most 256");
    DLM_CHECK(nh % nkv == 0, "attention: heads must be a multiple of kv heads");
    const int group = nh / nkv;
    const int gt = group >= 8 ? 8 : (group > 2 ? (group > 4 ? 8 : 4) : group);
    const int head_passes = (group + gt - 1) / gt;
    int lpk = 1;
    while (lpk * 8 < hd) lpk <<= 1;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)R * nh * n_splits * hd;
    dim3 grid(R, nkv * head_passes, n_splits);
    int* err = error_flag_ptr();
    const int streams = WARPS * (32 / lpk);
    const size_t smem_bytes = sizeof(float) * ((size_t)streams * gt * 2 + (size_t)streams * gt * lpk * 8);
#define DLM_DISPATCH(T)                                                                                            \
    switch (lpk) {                                                                                                 \
        case 1: launch_decode<T, 1>(gt, grid, smem_bytes, stream, q, k_cache, v_cache, block_table, table_width,   \
                    cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,      \
                    n_splits, head_passes, err); break;                                                            \
        case 2: launch_decode<T, 2>(gt, grid, smem_bytes, stream, q, k_cache, v_cache, block_table, table_width,   \
                    cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,      \
                    n_splits, head_passes, err); break;                                                            \
        case 4: launch_decode<T, 4>(gt, grid, smem_bytes, stream, q, k_cache, v_cache, block_table, table_width,   \
                    cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,      \
                    n_splits, head_passes, err); break;                                                            \
        case 8: launch_decode<T, 8>(gt, grid, smem_bytes, stream, q, k_cache, v_cache, block_table, table_width,   \
                    cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,      \
                    n_splits, head_passes, err); break;                                                            \
        case 16: launch_decode<T, 16>(gt, grid, smem_bytes, stream, q, k_cache, v_cache, block_table, table_width, \
                    cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,      \
                    n_splits, head_passes, err); break;                                                            \
        default: launch_decode<T, 32>(gt, grid, smem_bytes, stream, q, k_cache, v_cache, block_table, table_width, \
                    cu_q, kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,      \
                    n_splits, head_passes, err); break;                                                            \
    }
    if (dtype == F32) { DLM_DISPATCH(float) } else { DLM_DISPATCH(__nv_bfloat16) }
#undef DLM_DISPATCH
    check_launch("attention_decode");
    dim3 mgrid(R, nh);
    if (dtype == F32)
        launch_dep(attention_decode_merge_kernel<float>, mgrid, 128, 0, stream, part_o, part_ml, cu_q, static_cast<float*>(out), nh, hd, n_splits);
    else
        launch_dep(attention_decode_merge_kernel<__nv_bfloat16>, mgrid, 128, 0, stream, part_o, part_ml, cu_q, static_cast<__nv_bfloat16*>(out), nh, hd, n_splits);
    check_launch("attention_decode_merge");
}

}  // namespace dlmk

namespace dlmk {

// The second stage alone (shared with the tensor-core decode kernel): merges the chunks' partial results.
void attention_decode_merge(const float* part_o, const float* part_ml, const int32_t* cu_q, void* out, int R, int nh,
                            int hd, int n_splits, int dtype, cudaStream_t stream) {
    if (R <= 0) return;
    dim3 mgrid(R, nh);
    if (dtype == F32)
        launch_dep(attention_decode_merge_kernel<float>, mgrid, 128, 0, stream, part_o, part_ml, cu_q, static_cast<float*>(out), nh, hd, n_splits);
    else
        launch_dep(attention_decode_merge_kernel<__nv_bfloat16>, mgrid, 128, 0, stream, part_o, part_ml, cu_q, static_cast<__nv_bfloat16*>(out), nh, hd, n_splits);
    check_launch("attention_decode_merge");
}

}  // namespace dlmk

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (see no_alloc.h for its terms).  It launches the same
// kernels as attention_decode above; only the home of the scratch differs.
#include <atomic>
#include <cstdio>

#include "no_alloc.h"

namespace {

// Partial results of the split-key kernel, and a status block whose first word the kernels set when
// they refuse an access.  In host code this name is only a handle for cudaGetSymbolAddress; it is
// not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) float g_noalloc_scratch[DLM_B200_NOALLOC_SCRATCH_FLOATS + 64];

// The array's device address, per device.  Threads that make their first call on a device at the same
// time each look the address up and store the same value, so a plain atomic is enough.
constexpr int kMaxDevices = 64;
std::atomic<float*> g_noalloc_ptr[kMaxDevices];

// Device address of the array on the current device (looked up at the first call there), or nullptr.
float* noalloc_scratch(cudaError_t* e) {
    int dev = -1;
    *e = cudaGetDevice(&dev);
    if (*e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    float* p = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        *e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
        if (*e != cudaSuccess) return nullptr;
        g_noalloc_ptr[dev].store(p, std::memory_order_release);
    }
    return p;
}

void noalloc_fail(char* msg, size_t len, const char* text) {
    if (msg != nullptr && len > 0) snprintf(msg, len, "%s", text);
}

}  // namespace

extern "C" int dlm_b200_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                                 const int32_t* block_table, int table_width, const int32_t* cu_q,
                                                 const int32_t* kv_len, void* out, int R, int nh, int nkv, int hd,
                                                 int page_size, int total_pages, int window, float scale,
                                                 int max_kv_len, cudaStream_t stream, char* err_msg,
                                                 size_t err_msg_len) {
    using namespace dlmk;
    if (err_msg != nullptr && err_msg_len > 0) err_msg[0] = '\0';
    if (R <= 0) return 0;
    if (!attention_decode_ok(hd) || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || max_kv_len < 1) {
        noalloc_fail(err_msg, err_msg_len, "decode attention: head_dim must be a multiple of 8 in 16..256, heads a "
                                           "multiple of kv heads, page_size and max_kv_len positive");
        return 1;
    }
    int n_splits = 0, chunk = 0;
    attention_decode_plan(R, nkv, max_kv_len, &n_splits, &chunk);
    const size_t need = attention_decode_scratch_floats(R, nh, hd, n_splits);
    if (need > (size_t)DLM_B200_NOALLOC_SCRATCH_FLOATS) {
        char text[200];
        snprintf(text, sizeof(text), "decode attention without allocation: %zu floats of partial results exceed the "
                 "built-in maximum of %u (requests x heads x splits x (head_dim + 2))", need,
                 (unsigned)DLM_B200_NOALLOC_SCRATCH_FLOATS);
        noalloc_fail(err_msg, err_msg_len, text);
        return 1;
    }
    // set-up, once per device, with that device current: the array's device address
    cudaError_t e = cudaSuccess;
    float* scratch = noalloc_scratch(&e);
    if (scratch == nullptr) {
        noalloc_fail(err_msg, err_msg_len, "decode attention without allocation: the built-in array's device "
                                           "address could not be found (cudaGetSymbolAddress)");
        return e != cudaSuccess ? (int)e : 1;
    }
    int* status = reinterpret_cast<int*>(scratch + DLM_B200_NOALLOC_SCRATCH_FLOATS);
    e = cudaMemsetAsync(status, 0, sizeof(int), stream);      // the one word that must start at zero
    if (e != cudaSuccess) return (int)e;

    const int group = nh / nkv;
    const int gt = group >= 8 ? 8 : (group > 2 ? (group > 4 ? 8 : 4) : group);
    const int head_passes = (group + gt - 1) / gt;
    int lpk = 1;
    while (lpk * 8 < hd) lpk <<= 1;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)R * nh * n_splits * hd;
    dim3 grid(R, nkv * head_passes, n_splits);
    using T = __nv_bfloat16;
#define DLM_NOALLOC_CASE(L)                                                                                      \
    case L: launch_decode<T, L>(gt, grid, 0, stream, q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, \
                                part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale, chunk,       \
                                n_splits, head_passes, status); break;
    switch (lpk) {
        DLM_NOALLOC_CASE(2)
        DLM_NOALLOC_CASE(4)
        DLM_NOALLOC_CASE(8)
        DLM_NOALLOC_CASE(16)
        default: launch_decode<T, 32>(gt, grid, 0, stream, q, k_cache, v_cache, block_table, table_width, cu_q,
                                      kv_len, part_o, part_ml, nh, nkv, hd, page_size, total_pages, window, scale,
                                      chunk, n_splits, head_passes, status); break;
    }
#undef DLM_NOALLOC_CASE
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    attention_decode_merge_kernel<T><<<dim3(R, nh), 128, 0, stream>>>(part_o, part_ml, cu_q, static_cast<T*>(out), nh,
                                                                      hd, n_splits);
    e = cudaGetLastError();
    return (int)e;
}

extern "C" int dlm_b200_noalloc_status(int* host_status, cudaStream_t stream) {
    if (host_status == nullptr) return 1;
    cudaError_t e = cudaSuccess;
    float* scratch = noalloc_scratch(&e);
    if (scratch == nullptr) return e != cudaSuccess ? (int)e : 1;
    return (int)cudaMemcpyAsync(host_status, scratch + DLM_B200_NOALLOC_SCRATCH_FLOATS, sizeof(int),
                                cudaMemcpyDeviceToHost, stream);
}
