// Memory-bound kernels: embedding gather, RMSNorm, rotary + paged key/value write,
// combination of expert outputs into the residual.
#include "api.h"
#include <cstdlib>

#include "common.cuh"

namespace dlmk {

// ------------------------------------------------------------------ error flag
namespace {
int* g_flag_host = nullptr;
int* g_flag_dev = nullptr;
}  // namespace

// Device pointer of a host-mapped flag (allocated once per process, at the first launch that needs it).
int* error_flag_ptr() {
    if (g_flag_dev == nullptr) {
        if (cudaHostAlloc(reinterpret_cast<void**>(&g_flag_host), sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
            cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_flag_dev), g_flag_host, 0) != cudaSuccess)
            throw std::runtime_error("dlm_b200 kernels: cannot allocate the error flag");
        *g_flag_host = 0;
    }
    return g_flag_dev;
}

namespace {
int g_dep_launch = -1;
}

bool dep_launch_enabled() {
    if (g_dep_launch < 0) {
        const char* off = std::getenv("DLM_B200_NO_PDL");
        g_dep_launch = (off != nullptr && off[0] != '\0' && off[0] != '0') ? 0 : 1;
    }
    return g_dep_launch == 1;
}
void set_dep_launch(bool on) { g_dep_launch = on ? 1 : 0; }

int take_error_flag() {
    if (g_flag_host == nullptr) return 0;
    int v = *reinterpret_cast<volatile int*>(g_flag_host);
    *reinterpret_cast<volatile int*>(g_flag_host) = 0;
    return v;
}

// ------------------------------------------------------------------- embedding
namespace {

template <typename T>
__global__ void embed_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ table, float* out,
                             int H, int V, int* err) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (long long)t * H;
    if (tok < 0 || tok >= V) {   // never read outside the table
        if (threadIdx.x == 0) *err = 1;
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (long long)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

// ---------------------------------------------------------------------- rmsnorm
template <typename TOut>
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w, TOut* out,
                               const int32_t* rows, int H, float eps) {
    __shared__ float scratch[32];
    dep_wait();
    dep_launch_next();
    const int r = blockIdx.x;
    const float* xr = x + (long long)(rows ? rows[r] : r) * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TOut* o = out + (long long)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TOut>((xr[i] * inv) * w[i]);
}

// ------------------------------------------------------- rotary + cache write
// blockIdx.x = token, blockIdx.y = slice of the token's work.  The rotation angles of a token depend on the
// pair index only, so each block computes the rotary_dim / 2 sines and cosines once (in shared memory); then
// threads run over (head, pair) of the q and k heads, over the unrotated dims, and over the v elements.
template <typename T>
__global__ void rope_kv_write_kernel(const float* qkv, const int32_t* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     const int32_t* __restrict__ slots, T* q_out, T* k_cache,
                                     T* v_cache, int nh, int nkv, int hd, int page_size, int total_pages,
                                     int* err) {
    extern __shared__ float sc[];                  // [2][rotary_dim / 2]: sines, cosines
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    const int Q = nh * hd, KV = nkv * hd;
    const float* row = qkv + (long long)t * (Q + 2 * KV);
    const float pos = (float)positions[t];
    const int half = inv_freq != nullptr ? rotary_dim / 2 : 0;
    const int rd = 2 * half;                       // dims that are rotated
    int in_page = 0, page = -1;
    if (slots != nullptr) {
        const int s = slots[t];
        if (s >= 0) {
            page = s / page_size;
            in_page = s % page_size;
            if (page >= total_pages) {
                if (threadIdx.x == 0) *err = 2;
                page = -1;
            }
        }
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        sc[i] = sn;
        sc[half + i] = cs;
    }
    __syncthreads();
    const int rot_heads = nh + nkv;
    const int tpt = blockDim.x * gridDim.y, tid0 = blockIdx.y * blockDim.x + threadIdx.x;
    // rotated pairs (i, i + half) of every q and k head
    for (int idx = tid0; idx < rot_heads * half; idx += tpt) {
        const int h = idx / half, i = idx % half;
        const float* src = row + (long long)h * hd;          // q heads then k heads are contiguous in qkv
        const float a = src[i], b = src[i + half];
        const float sn = sc[i], cs = sc[half + i];
        const float lo = a * cs - b * sn, hi = a * sn + b * cs;
        if (h < nh) {
            T* o = q_out + (long long)t * Q + h * hd;
            o[i] = from_f32<T>(lo);
            o[i + half] = from_f32<T>(hi);
        } else if (page >= 0) {
            T* o = k_cache + (((long long)page * nkv + (h - nh)) * page_size + in_page) * hd;
            o[i] = from_f32<T>(lo);
            o[i + half] = from_f32<T>(hi);
        }
    }
    // dims from rotary_dim on pass through
    const int rest = hd - rd;
    for (int idx = tid0; idx < rot_heads * rest; idx += tpt) {
        const int h = idx / rest, d = rd + idx % rest;
        const float val = row[(long long)h * hd + d];
        if (h < nh) q_out[(long long)t * Q + h * hd + d] = from_f32<T>(val);
        else if (page >= 0)
            k_cache[(((long long)page * nkv + (h - nh)) * page_size + in_page) * hd + d] = from_f32<T>(val);
    }
    if (page >= 0) {
        const float* vsrc = row + Q + KV;
        for (int idx = tid0; idx < KV; idx += tpt) {
            const int kh = idx / hd, d = idx % hd;
            v_cache[(((long long)page * nkv + kh) * page_size + in_page) * hd + d] = from_f32<T>(vsrc[idx]);
        }
    }
}

// ------------------------------------------------------------------ row gather
__global__ void gather_rows_kernel(const uint4* src, const int32_t* rows,
                                   uint4* out, int chunks) {
    dep_wait();
    dep_launch_next();
    const int r = blockIdx.x;
    const uint4* s = src + (long long)rows[r] * chunks;
    uint4* o = out + (long long)r * chunks;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) o[i] = s[i];
}

// ------------------------------------------------------------------ moe combine
__global__ void moe_combine_kernel(const float* y, const int32_t* dest,
                                   const float* wts, const float* shared,
                                   const float* gate, float* resid, int H, int k) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    float* r = resid + (long long)t * H;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += blockDim.x * gridDim.y) {
        float acc = 0.f;
        for (int j = 0; j < k; ++j)
            acc = fmaf(wts[t * k + j], y[(long long)dest[t * k + j] * H + i], acc);
        if (shared != nullptr) {
            const float g = gate ? gate[t] : 1.0f;
            acc = fmaf(g, shared[(long long)t * H + i], acc);
        }
        r[i] += acc;
    }
}

}  // namespace

int* error_flag_ptr();

void embed(const int32_t* tokens, const void* table, float* out, int T, int H, int V, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    int* err = error_flag_ptr();
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == F32) launch_dep(embed_kernel<float>, T, threads, 0, stream, tokens, static_cast<const float*>(table), out, H, V, err);
    else launch_dep(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, tokens, static_cast<const __nv_bfloat16*>(table), out, H, V, err);
    check_launch("embed");
}

void rmsnorm(const float* x, const float* w, void* out, const int32_t* rows, int n_rows, int H, float eps,
             int out_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (out_dtype == F32) launch_dep(rmsnorm_kernel<float>, n_rows, threads, 0, stream, x, w, static_cast<float*>(out), rows, H, eps);
    else launch_dep(rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, x, w, static_cast<__nv_bfloat16*>(out), rows, H, eps);
    check_launch("rmsnorm");
}

void rope_kv_write(const float* qkv, const int32_t* positions, const float* inv_freq, int rotary_dim,
                   const int32_t* slots, void* q_out, void* k_cache, void* v_cache, int T, int nh, int nkv, int hd,
                   int page_size, int total_pages, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(inv_freq == nullptr || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= hd),
              "rope: rotary_dim must be even and in 2..head_dim");
    int* err = error_flag_ptr();
    const int threads = 256;
    const int work = (nh + nkv) * hd;
    int slices = (work + threads - 1) / threads;
    if (T >= 512) slices = 1; else if (slices > 16) slices = 16;
    dim3 grid(T, slices);
    const size_t smem = inv_freq != nullptr ? sizeof(float) * rotary_dim : 0;
    if (dtype == F32)
        launch_dep(rope_kv_write_kernel<float>, grid, threads, smem, stream, qkv, positions, inv_freq, rotary_dim, slots,
            static_cast<float*>(q_out), static_cast<float*>(k_cache), static_cast<float*>(v_cache), nh, nkv, hd,
            page_size, total_pages, err);
    else
        launch_dep(rope_kv_write_kernel<__nv_bfloat16>, grid, threads, smem, stream, qkv, positions, inv_freq, rotary_dim, slots,
            static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
            static_cast<__nv_bfloat16*>(v_cache), nh, nkv, hd, page_size, total_pages, err);
    check_launch("rope_kv_write");
}

void gather_rows(const void* src, const int32_t* rows, void* out, int n_rows, int width, int dtype,
                 cudaStream_t stream) {
    if (n_rows <= 0) return;
    const int bytes = width * (dtype == F32 ? 4 : 2);
    DLM_CHECK(bytes % 16 == 0, "gather_rows: a row must be a multiple of 16 bytes");
    launch_dep(gather_rows_kernel, n_rows, 128, 0, stream, static_cast<const uint4*>(src), rows,
               static_cast<uint4*>(out), bytes / 16);
    check_launch("gather_rows");
}

void moe_combine(const float* y, const int32_t* dest, const float* wts, const float* shared, const float* gate,
                 float* resid, int T, int H, int k, cudaStream_t stream) {
    if (T <= 0) return;
    int slices = (H + 255) / 256;
    if (T >= 512) slices = 1; else if (slices > 16) slices = 16;
    launch_dep(moe_combine_kernel, dim3(T, slices), 256, 0, stream, y, dest, wts, shared, gate, resid, H, k);
    check_launch("moe_combine");
}

}  // namespace dlmk
