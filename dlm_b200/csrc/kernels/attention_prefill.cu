// Prefill attention on the warp-level tensor-core path (bfloat16): portions of prompts, each
// query attending to its request's paged keys up to its own position (optionally only the
// last `window` of them).
//
// One block = 128 consecutive query tokens of one request x one query head; 8 warps of 16 rows,
// two blocks a multiprocessor.  Keys and values come in tiles of 64 (aligned to absolute
// positions), two tiles in flight through asynchronous 16-byte copies; S = Q K^T and O += P V are
// mma.sync m16n8k16 with 32-bit accumulation; the softmax runs in 32-bit on the accumulator
// registers, whose layout is already that of the next product's left operand.  A warp skips tiles
// none of its rows can see, and tiles that all of its rows see in full take a path without the
// mask.  Blocks are numbered so that the longest (latest queries) start first.  Requests with a
// single query token are left to the decode kernel when it runs.
#include "api.h"
#include "attention_internal.h"
#include "common.cuh"
#include "mma_sync.cuh"

namespace dlmk {

namespace {

constexpr int BQ = 128, BKV = 64, WARPS = 8, THREADS = WARPS * 32;

// 2^x on the special-function unit (32-bit in and out; 2^-inf = 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const int32_t* __restrict__ block_table,
                         int table_width, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ kv_len,
                         __nv_bfloat16* __restrict__ out, int R, int nh, int nkv, int page_size, int total_pages,
                         int page_shift, int window, float scale_log2, int skip_single, int n_sm, int* err) {
    constexpr int PITCH = HD + 8;              // elements per shared-memory row (16 bytes of padding)
    constexpr int KS = HD / 16;                // k16 steps over the head dimension
    constexpr int DT = HD / 8;                 // n8 tiles of the output
    constexpr int CPR = HD / 8;                // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [BQ][PITCH]
    __nv_bfloat16* Ks = Qs + BQ * PITCH;                                 // [2][BKV][PITCH]
    __nv_bfloat16* Vs = Ks + 2 * BKV * PITCH;                            // [2][BKV][PITCH]
    __shared__ int s_map[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Work order.  Blocks start in the order of their linear index; with two blocks per multiprocessor the
    // first n_sm blocks take the heaviest tiles (the latest queries see the most keys), the next n_sm the
    // lightest in ascending order, so that a multiprocessor's two first blocks add up to about the same work;
    // the rest follows from heavy to light as blocks end.
    const int linear = (int)(blockIdx.y * gridDim.x + blockIdx.x), total = (int)(gridDim.x * gridDim.y);
    int rank = linear;
    if (linear >= n_sm) rank = linear < 2 * n_sm ? total - 1 - (linear - n_sm) : linear - n_sm;
    const int head = rank % nh, kvh = head / (nh / nkv);
    const int bx = (int)gridDim.y - 1 - rank / nh;              // late tiles (most keys) have the low ranks
    if (tid == 0) {
        int acc = 0;
        s_map[0] = -1;
        for (int r = 0; r < R; ++r) {
            const int ql = cu_q[r + 1] - cu_q[r];
            const int tiles = (skip_single && ql == 1) ? 0 : (ql + BQ - 1) / BQ;
            if (bx < acc + tiles) {
                s_map[0] = r;
                s_map[1] = (bx - acc) * BQ;
                break;
            }
            acc += tiles;
        }
    }
    __syncthreads();
    const int r = s_map[0];
    if (r < 0) return;
    const int q0 = s_map[1];
    const int q_begin = cu_q[r], q_len = cu_q[r + 1] - q_begin;
    const int n_q = min(BQ, q_len - q0);
    const int len = kv_len[r];
    const int pos0 = len - q_len + q0;
    const int Q = nh * HD;
    const int32_t* table = block_table + (long long)r * table_width;

    // the query tile (rows beyond the portion are zero)
    for (int idx = tid; idx < BQ * CPR; idx += THREADS) {
        const int row = idx / CPR, c = idx % CPR;
        if (row < n_q) cp_async16(Qs + row * PITCH + c * 8, q + (long long)(q_begin + q0 + row) * Q + head * HD + c * 8);
        else *reinterpret_cast<uint4*>(Qs + row * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    const int hi = pos0 + n_q - 1;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int t_begin = (lo / BKV) * BKV;
    const int n_tiles = (hi - t_begin) / BKV + 1;
    // a tile lies within one page when pages are a power of two of at least a tile (tiles are aligned)
    const bool one_page = page_shift >= 0 && page_size >= BKV;

    auto fill = [&](int stage, int j0) {
        __nv_bfloat16* kd = Ks + (size_t)stage * BKV * PITCH;
        __nv_bfloat16* vd = Vs + (size_t)stage * BKV * PITCH;
        int tile_page = -1;
        if (one_page) {
            const int lp = j0 >> page_shift;
            tile_page = lp < table_width ? table[lp] : -1;
        }
        for (int idx = tid; idx < BKV * CPR; idx += THREADS) {
            const int key = idx / CPR, c = idx % CPR;
            const int j = j0 + key;
            int page = -1, in_page = 0;
            if (j >= lo && j <= hi) {
                if (one_page) {
                    page = tile_page;
                    in_page = j & (page_size - 1);
                } else {
                    const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
                    in_page = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
                    page = lp < table_width ? table[lp] : -1;
                }
                if (page < 0 || page >= total_pages) { *err = 3; page = -1; }
            }
            if (page >= 0) {
                const long long off = (((long long)page * nkv + kvh) * page_size + in_page) * HD + c * 8;
                cp_async16(kd + key * PITCH + c * 8, k_cache + off);
                cp_async16(vd + key * PITCH + c * 8, v_cache + off);
            } else {
                *reinterpret_cast<uint4*>(kd + key * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + key * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fill(0, t_begin);

    const int g = lane >> 2, t = lane & 3;
    const int lm_row = lane & 15, lm_col = (lane >> 4) * 8;
    const int row_a = warp * 16 + g, row_b = row_a + 8;          // this thread's two query rows in the tile
    const int pa = pos0 + row_a, pb = pos0 + row_b;
    const int w_lo = pos0 + warp * 16, w_hi = w_lo + 15;         // positions of the warp's rows
    const bool warp_live = warp * 16 < n_q;                      // a warp of padding rows computes nothing
    const __nv_bfloat16* q_frag = Qs + (warp * 16 + lm_row) * PITCH + lm_col;

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it & 1;
        const int j0 = t_begin + it * BKV;
        if (it + 1 < n_tiles) {
            fill(stage ^ 1, j0 + BKV);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* kt = Ks + (size_t)stage * BKV * PITCH;
        const __nv_bfloat16* vt = Vs + (size_t)stage * BKV * PITCH;
        // does any row of this warp see any key of the tile?
        const bool seen = warp_live && j0 <= w_hi && (window <= 0 || j0 + BKV - 1 > w_lo - window);
        if (seen) {
            // S = Q K^T for 16 rows x 64 keys
            float s[BKV / 8][4];
#pragma unroll
            for (int j = 0; j < BKV / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                uint32_t qf[4];
                ldsm_x4(qf, q_frag + kk * 16);
#pragma unroll
                for (int jn = 0; jn < BKV / 16; ++jn) {
                    uint32_t kf[4];
                    ldsm_x4(kf, kt + (jn * 16 + lm_row) * PITCH + kk * 16 + lm_col);
                    mma16816(s[2 * jn], qf, kf[0], kf[2]);
                    mma16816(s[2 * jn + 1], qf, kf[1], kf[3]);
                }
            }
            // scale (to base 2), mask where needed, running maximum
            float mx_a = m_a, mx_b = m_b;
            const bool all_visible = j0 + BKV - 1 <= w_lo && (window <= 0 || w_hi - j0 < window);
            if (all_visible) {
#pragma unroll
                for (int j = 0; j < BKV / 8; ++j) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float v = s[j][c] * scale_log2;
                        s[j][c] = v;
                        if (c < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < BKV / 8; ++j) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int key = j0 + j * 8 + 2 * t + (c & 1);
                        const int p = (c < 2) ? pa : pb;
                        const bool vis = key <= p && (window <= 0 || p - key < window);
                        const float v = vis ? s[j][c] * scale_log2 : -INFINITY;
                        s[j][c] = v;
                        if (c < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                    }
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            // a row that has seen nothing yet keeps its state (2^(-inf - -inf) must not appear)
            const float base_a = mx_a == -INFINITY ? 0.f : mx_a, base_b = mx_b == -INFINITY ? 0.f : mx_b;
            const float al_a = ex2(m_a - base_a), al_b = ex2(m_b - base_b);     // m = -inf: 0
            float sum_a = 0.f, sum_b = 0.f;
            uint32_t pf[BKV / 16][4];
#pragma unroll
            for (int j = 0; j < BKV / 8; ++j) {
                const float p0 = ex2(s[j][0] - base_a), p1 = ex2(s[j][1] - base_a);
                const float p2 = ex2(s[j][2] - base_b), p3 = ex2(s[j][3] - base_b);
                sum_a += p0 + p1;
                sum_b += p2 + p3;
                // accumulator tiles 2k and 2k + 1 are the left operand of the k-th 16-key step of P V
                pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
            sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
            sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
            sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
            l_a = l_a * al_a + sum_a;
            l_b = l_b * al_b + sum_b;
            m_a = mx_a;
            m_b = mx_b;
            if (__any_sync(0xffffffffu, al_a != 1.0f || al_b != 1.0f)) {
#pragma unroll
                for (int i = 0; i < DT; ++i) {
                    o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b;
                }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
                for (int dn = 0; dn < HD / 16; ++dn) {
                    uint32_t vf[4];
                    ldsm_x4_trans(vf, vt + (kk * 16 + lm_row) * PITCH + dn * 16 + lm_col);
                    mma16816(o[2 * dn], pf[kk], vf[0], vf[1]);
                    mma16816(o[2 * dn + 1], pf[kk], vf[2], vf[3]);
                }
            }
        }
        __syncthreads();
    }

    const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
    for (int i = 0; i < DT; ++i) {
        const int d = i * 8 + 2 * t;
        if (row_a < n_q)
            *reinterpret_cast<uint32_t*>(out + (long long)(q_begin + q0 + row_a) * Q + head * HD + d) =
                pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < n_q)
            *reinterpret_cast<uint32_t*>(out + (long long)(q_begin + q0 + row_b) * Q + head * HD + d) =
                pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

template <int HD>
void launch(dim3 grid, cudaStream_t stream, const void* q, const void* k_cache, const void* v_cache,
            const int32_t* block_table, int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int R,
            int nh, int nkv, int page_size, int total_pages, int window, float scale, int skip_single) {
    const size_t smem = (size_t)(BQ + 4 * BKV) * (HD + 8) * sizeof(__nv_bfloat16);
    int shift = -1;
    if ((page_size & (page_size - 1)) == 0) { shift = 0; while ((1 << shift) < page_size) ++shift; }
    auto kern = attention_prefill_kernel<HD>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, THREADS, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
        static_cast<const __nv_bfloat16*>(v_cache), block_table, table_width, cu_q, kv_len,
        static_cast<__nv_bfloat16*>(out), R, nh, nkv, page_size, total_pages, shift, window,
        scale * 1.4426950408889634f, skip_single, sm_count(), error_flag_ptr());
}

}  // namespace

bool attention_prefill_ok(int hd) {
    return hd == 16 || hd == 32 || hd == 48 || hd == 64 || hd == 96 || hd == 128;
}

void attention_prefill(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                       int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                       int nkv, int hd, int page_size, int total_pages, int window, float scale, int skip_single,
                       cudaStream_t stream) {
    if (T <= 0 || R <= 0) return;
    DLM_CHECK(attention_prefill_ok(hd), "prefill attention: this head_dim has no tensor-core kernel");
    DLM_CHECK(nh % nkv == 0, "attention: heads must be a multiple of kv heads");
    dim3 grid(nh, (T + BQ - 1) / BQ + R);
#define DLM_PREFILL(HD)                                                                                             \
    launch<HD>(grid, stream, q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, out, R, nh, nkv, page_size, \
               total_pages, window, scale, skip_single)
    switch (hd) {
        case 16: DLM_PREFILL(16); break;
        case 32: DLM_PREFILL(32); break;
        case 48: DLM_PREFILL(48); break;
        case 64: DLM_PREFILL(64); break;
        case 96: DLM_PREFILL(96); break;
        default: DLM_PREFILL(128); break;
    }
#undef DLM_PREFILL
    check_launch("attention_prefill");
}

}  // namespace dlmk
