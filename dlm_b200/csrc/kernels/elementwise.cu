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

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

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
// Two passes over a row; the second finds it in the L1 cache.
template <typename TOut> struct Out4;
template <> struct Out4<float> {
    static __device__ __forceinline__ void store(float* o, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
    }
};
template <> struct Out4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* o, float a, float b, float c, float d) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<const uint32_t*>(&lo);
        v.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(o) = v;
    }
};

// The sum of squares of a row has one order, whoever computes it: the row's elements (VEC: its groups of four)
// are dealt round-robin to 8 x 32 partial sums, partial sum (v, l) takes items 32 v + l, + 256, + 512, ...; each
// v's 32 partial sums go through a shuffle tree; the eight results are added in order.  The eight warps of a
// block share one row, warp v keeps the partial sums (v, .).  (A warp per row, eight rows to a block, was
// measured for launches of 2,048 rows: 2 us slower a launch.)
template <typename TOut, bool VEC>
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w, TOut* out,
                               const int32_t* rows, int n_rows, int H, float eps) {
    __shared__ float s_part[8];
    // the norm's weight is no kernel's output: ask for it before waiting for the kernel before this one
    for (int off = threadIdx.x * 128; off < H * (int)sizeof(float); off += blockDim.x * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(w) + off));
    dep_wait();
    dep_launch_next();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const float* xr = x + (long long)(rows ? rows[r] : r) * H;
    TOut* o = out + (long long)r * H;
    const int items = VEC ? H / 4 : H;
    auto square = [&](int i, float acc) -> float {
        if (VEC) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            acc = fmaf(v.x, v.x, acc); acc = fmaf(v.y, v.y, acc); acc = fmaf(v.z, v.z, acc); acc = fmaf(v.w, v.w, acc);
        } else {
            acc = fmaf(xr[i], xr[i], acc);
        }
        return acc;
    };
    // VEC: a thread's first NORM_KEEP groups of four stay in registers between the two passes (rows of up to
    // 1,024 NORM_KEEP columns are read once), and so do their weights, asked for before the sum is known
    constexpr int NORM_KEEP = 4;
    float4 kept[NORM_KEEP], wk[NORM_KEEP];
    float part = 0.f;
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
        for (int n = 0; n < NORM_KEEP; ++n) {
            const int i = (int)threadIdx.x + 256 * n;
            kept[n] = make_float4(0.f, 0.f, 0.f, 0.f);
            wk[n] = kept[n];
            if (i < items) { kept[n] = x4[i]; wk[n] = __ldg(w4 + i); }
        }
#pragma unroll
        for (int n = 0; n < NORM_KEEP; ++n) {
            const int i = (int)threadIdx.x + 256 * n;
            if (i < items) {
                const float4 v = kept[n];
                part = fmaf(v.x, v.x, part); part = fmaf(v.y, v.y, part); part = fmaf(v.z, v.z, part); part = fmaf(v.w, v.w, part);
            }
        }
        for (int i = (int)threadIdx.x + 256 * NORM_KEEP; i < items; i += 256) part = square(i, part);
    } else {
        for (int i = 32 * warp + lane; i < items; i += 256) part = square(i, part);
    }
    part = warp_sum(part);
    if (lane == 0) s_part[warp] = part;
    __syncthreads();
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < 8; ++v) ss += s_part[v];
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
        for (int n = 0; n < NORM_KEEP; ++n) {
            const int i = (int)threadIdx.x + 256 * n;
            if (i < items) {
                const float4 v = kept[n], g = wk[n];
                Out4<TOut>::store(o + 4 * i, (v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
            }
        }
        for (int i = (int)threadIdx.x + 256 * NORM_KEEP; i < items; i += 256) {
            const float4 v = x4[i], g = __ldg(w4 + i);
            Out4<TOut>::store(o + 4 * i, (v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
        }
    } else {
        for (int i = (int)threadIdx.x; i < items; i += 256) o[i] = from_f32<TOut>((xr[i] * inv) * w[i]);
    }
}

// ------------------------------------------------------- rotary + cache write
// blockIdx.x = token, blockIdx.y = slice of the token's work.  The rotation angles of a token depend on the
// pair index only, so each block computes the rotary_dim / 2 sines and cosines once (in shared memory); then
// threads run over (head, pair) of the q and k heads, over the unrotated dims, and over the v elements.
template <typename T>
__global__ void rope_kv_write_kernel(const float* qkv, const int32_t* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int rotary_dim, int interleaved,
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
    // rotated pairs of every q and k head: dims (i, i + half), or (2i, 2i + 1) when interleaved
    for (int idx = tid0; idx < rot_heads * half; idx += tpt) {
        const int h = idx / half, i = idx % half;
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const float* src = row + (long long)h * hd;          // q heads then k heads are contiguous in qkv
        const float a = src[ia], b = src[ib];
        const float sn = sc[i], cs = sc[half + i];
        const float lo = a * cs - b * sn, hi = a * sn + b * cs;
        if (h < nh) {
            T* o = q_out + (long long)t * Q + h * hd;
            o[ia] = from_f32<T>(lo);
            o[ib] = from_f32<T>(hi);
        } else if (page >= 0) {
            T* o = k_cache + (((long long)page * nkv + (h - nh)) * page_size + in_page) * hd;
            o[ia] = from_f32<T>(lo);
            o[ib] = from_f32<T>(hi);
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

// The same in steps of four elements (16-byte loads, 8- or 16-byte stores), for head sizes, rotary sizes and
// addresses that allow it.  Per element the arithmetic is that of rope_kv_write_kernel.
template <typename T>
__global__ void rope_kv_write_vec_kernel(const float* qkv, const int32_t* __restrict__ positions,
                                         const float* __restrict__ inv_freq, int rotary_dim, int /*interleaved: never*/,
                                         const int32_t* __restrict__ slots, T* q_out, T* k_cache,
                                         T* v_cache, int nh, int nkv, int hd, int page_size, int total_pages,
                                         int* err) {
    extern __shared__ float sc[];                  // [2][rotary_dim / 2]: sines, cosines
    // Positions, slots and frequencies are the step's inputs, not a kernel's output: the angles are ready
    // before the kernel that writes q, k and v has ended.
    const int t = blockIdx.x;
    const int Q = nh * hd, KV = nkv * hd;
    const float* row = qkv + (long long)t * (Q + 2 * KV);
    const float pos = (float)positions[t];
    const int half = inv_freq != nullptr ? rotary_dim / 2 : 0;
    const int rd = 2 * half;
    int in_page = 0, page = -1;
    bool bad_slot = false;
    if (slots != nullptr) {
        const int s = slots[t];
        if (s >= 0) {
            page = s / page_size;
            in_page = s % page_size;
            if (page >= total_pages) {
                bad_slot = true;
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
    dep_wait();
    dep_launch_next();
    if (bad_slot && threadIdx.x == 0) *err = 2;
    __syncthreads();
    const int rot_heads = nh + nkv;
    const int tpt = blockDim.x * gridDim.y, tid0 = blockIdx.y * blockDim.x + threadIdx.x;
    // where head h of this token goes: a q row, or a k row of the cache (nullptr: not stored)
    auto dst_of = [&](int h) -> T* {
        if (h < nh) return q_out + (long long)t * Q + (long long)h * hd;
        if (page < 0) return nullptr;
        return k_cache + (((long long)page * nkv + (h - nh)) * page_size + in_page) * hd;
    };
    const int hq = half / 4;
    for (int idx = tid0; idx < rot_heads * hq; idx += tpt) {
        const int h = idx / hq, i = (idx % hq) * 4;
        T* o = dst_of(h);
        if (o == nullptr) continue;
        const float* src = row + (long long)h * hd;
        const float4 a = *reinterpret_cast<const float4*>(src + i), b = *reinterpret_cast<const float4*>(src + i + half);
        const float4 sn = *reinterpret_cast<const float4*>(sc + i), cs = *reinterpret_cast<const float4*>(sc + half + i);
        Out4<T>::store(o + i, a.x * cs.x - b.x * sn.x, a.y * cs.y - b.y * sn.y, a.z * cs.z - b.z * sn.z,
                       a.w * cs.w - b.w * sn.w);
        Out4<T>::store(o + i + half, a.x * sn.x + b.x * cs.x, a.y * sn.y + b.y * cs.y, a.z * sn.z + b.z * cs.z,
                       a.w * sn.w + b.w * cs.w);
    }
    const int rq = (hd - rd) / 4;
    for (int idx = tid0; idx < rot_heads * rq; idx += tpt) {
        const int h = idx / rq, d = rd + (idx % rq) * 4;
        T* o = dst_of(h);
        if (o == nullptr) continue;
        const float4 v = *reinterpret_cast<const float4*>(row + (long long)h * hd + d);
        Out4<T>::store(o + d, v.x, v.y, v.z, v.w);
    }
    if (page >= 0) {
        const float* vsrc = row + Q + KV;
        for (int idx = tid0; idx < KV / 4; idx += tpt) {
            const int kh = (idx * 4) / hd, d = (idx * 4) % hd;
            const float4 v = *reinterpret_cast<const float4*>(vsrc + idx * 4);
            Out4<T>::store(v_cache + (((long long)page * nkv + kh) * page_size + in_page) * hd + d, v.x, v.y, v.z, v.w);
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
template <bool VEC>
__global__ void moe_combine_kernel(const float* y, const int32_t* dest,
                                   const float* wts, const float* shared,
                                   const float* gate, float* resid, int H, int k) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    float* r = resid + (long long)t * H;
    if constexpr (VEC) {
        // four columns a thread; per element the same sums in the same order as below
        const float g = (shared != nullptr && gate != nullptr) ? gate[t] : 1.0f;
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H / 4; i += blockDim.x * gridDim.y) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < k; ++j) {
                const float wj = wts[t * k + j];
                const float4 v = *reinterpret_cast<const float4*>(y + (long long)dest[t * k + j] * H + 4 * i);
                acc.x = fmaf(wj, v.x, acc.x); acc.y = fmaf(wj, v.y, acc.y);
                acc.z = fmaf(wj, v.z, acc.z); acc.w = fmaf(wj, v.w, acc.w);
            }
            if (shared != nullptr) {
                const float4 v = *reinterpret_cast<const float4*>(shared + (long long)t * H + 4 * i);
                acc.x = fmaf(g, v.x, acc.x); acc.y = fmaf(g, v.y, acc.y);
                acc.z = fmaf(g, v.z, acc.z); acc.w = fmaf(g, v.w, acc.w);
            }
            float4 cur = *reinterpret_cast<float4*>(r + 4 * i);
            cur.x += acc.x; cur.y += acc.y; cur.z += acc.z; cur.w += acc.w;
            *reinterpret_cast<float4*>(r + 4 * i) = cur;
        }
    } else {
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
    const int grid = n_rows, threads = 256;
    const bool vec = H % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
                                     reinterpret_cast<uintptr_t>(out)) & 15) == 0;
#define DLM_NORM(TOUT, VEC)                                                                              \
    launch_dep(rmsnorm_kernel<TOUT, VEC>, grid, threads, 0, stream, x, w, static_cast<TOUT*>(out), rows, \
               n_rows, H, eps)
    if (out_dtype == F32) { if (vec) DLM_NORM(float, true); else DLM_NORM(float, false); }
    else { if (vec) DLM_NORM(__nv_bfloat16, true); else DLM_NORM(__nv_bfloat16, false); }
#undef DLM_NORM
    check_launch("rmsnorm");
}

void rope_kv_write(const float* qkv, const int32_t* positions, const float* inv_freq, int rotary_dim, int interleaved,
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
    const size_t smem = inv_freq != nullptr ? sizeof(float) * rotary_dim : 0;
    const int half = inv_freq != nullptr ? rotary_dim / 2 : 0;
    const bool vec = hd % 4 == 0 && half % 4 == 0 && !interleaved &&
                     ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                       reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
    if (vec) {
        slices = (work / 4 + threads - 1) / threads;
        if (T >= 512) slices = 1; else if (slices > 16) slices = 16;
    }
    dim3 grid(T, slices);
    if (dtype == F32) {
        auto kern = vec ? rope_kv_write_vec_kernel<float> : rope_kv_write_kernel<float>;
        launch_dep(kern, grid, threads, smem, stream, qkv, positions, inv_freq, rotary_dim, interleaved, slots,
            static_cast<float*>(q_out), static_cast<float*>(k_cache), static_cast<float*>(v_cache), nh, nkv, hd,
            page_size, total_pages, err);
    } else {
        auto kern = vec ? rope_kv_write_vec_kernel<__nv_bfloat16> : rope_kv_write_kernel<__nv_bfloat16>;
        launch_dep(kern, grid, threads, smem, stream, qkv, positions, inv_freq, rotary_dim, interleaved, slots,
            static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
            static_cast<__nv_bfloat16*>(v_cache), nh, nkv, hd, page_size, total_pages, err);
    }
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
    const bool vec = H % 4 == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(shared) |
                                     reinterpret_cast<uintptr_t>(resid)) & 15) == 0;
    const int cols = vec ? H / 4 : H;
    int slices = (cols + 255) / 256;
    if (T >= 512) slices = 1; else if (slices > 16) slices = 16;
    if (vec) launch_dep(moe_combine_kernel<true>, dim3(T, slices), 256, 0, stream, y, dest, wts, shared, gate, resid, H, k);
    else launch_dep(moe_combine_kernel<false>, dim3(T, slices), 256, 0, stream, y, dest, wts, shared, gate, resid, H, k);
    check_launch("moe_combine");
}

}  // namespace dlmk
