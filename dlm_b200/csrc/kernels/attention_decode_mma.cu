// Decode attention on the warp-level tensor-core path (bfloat16): one query token per request,
// the query heads of one kv head's group stacked as the rows of a 16-row MMA tile (rows beyond the
// group are zero).  The arithmetic per byte of keys and values read drops to a few instructions,
// which is what lets the kernel follow memory bandwidth; the FMA version in attention_decode.cu
// spends its time on conversions and multiply-adds instead.
//
// One block = (request, kv head [x pass of 16 heads], chunk of keys).  Keys and values arrive in
// tiles of 64 through asynchronous 16-byte copies, two tiles in flight; each of the 4 warps takes
// 16 keys of a tile, keeps a running maximum / sum / output of its own, and the four are merged at
// the end.  Partial results go to the same scratch layout as the FMA version; the merge kernel is
// shared.  With head sizes of 64 or 128 and pages of at least a tile, the second kernel of this file
// takes over: the same arithmetic, the tiles brought by the TMA unit (off with DLM_B200_NO_TCGEN05=1).
#include <cstdlib>

#include "api.h"
#include "attention_internal.h"
#include "common.cuh"
#include "mma_sync.cuh"
#include "tcgen05.cuh"

namespace dlmk {

namespace {

constexpr int WARPS = 4, BKV = 64, ROWS = 16;


// How many blocks of a (request, kv head, pass of heads) have written their partial results: the block that
// comes last merges them, so no second kernel is needed.  The counters are zero between launches (the last
// block puts its counter back), so launches must not overlap (one stream at a time in a process); a launch that
// gave up on a wait leaves counters behind, which reset_decode_merge_counters() clears before the next step.
// MERGE_SLOTS bounds requests x kv heads x passes.
constexpr int MERGE_SLOTS = 1 << 16;
__device__ int g_merge_counters[MERGE_SLOTS];

// The end of a block, shared by the two kernels below: the warps' streams are merged through shared memory
// (`smem_raw`, free by now), the block's partial result goes to the scratch, and the block that finishes a
// (request, kv head, pass) last merges its key splits into the output.  Every thread of the block calls it;
// `warp < WARPS` are the warps that hold streams.
template <int HD>
__device__ __forceinline__ void finish_block(unsigned char* smem_raw, const float (&o)[HD / 8][4], float m_a, float m_b,
                                             float l_a, float l_b, int r, int h0, int n_heads, int sp, int token,
                                             float* part_o, float* part_ml, int nh, int n_splits,
                                             __nv_bfloat16* out, int fuse_merge) {
    constexpr int DT = HD / 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // merge the four warps' streams; the tiles' shared memory is free now
    float* sm_m = reinterpret_cast<float*>(smem_raw);             // [WARPS][ROWS]
    float* sm_l = sm_m + WARPS * ROWS;                            // [WARPS][ROWS]
    float* sm_o = sm_l + WARPS * ROWS;                            // [WARPS][ROWS][HD]
    __syncthreads();
    if (warp < WARPS && t == 0) {
        sm_m[warp * ROWS + g] = m_a; sm_m[warp * ROWS + g + 8] = m_b;
        sm_l[warp * ROWS + g] = l_a; sm_l[warp * ROWS + g + 8] = l_b;
    }
#pragma unroll
    for (int i = 0; i < DT; ++i) {
        if (warp >= WARPS) break;
        const int d = i * 8 + 2 * t;
        sm_o[(warp * ROWS + g) * HD + d] = o[i][0];
        sm_o[(warp * ROWS + g) * HD + d + 1] = o[i][1];
        sm_o[(warp * ROWS + g + 8) * HD + d] = o[i][2];
        sm_o[(warp * ROWS + g + 8) * HD + d + 1] = o[i][3];
    }
    __syncthreads();
    for (int idx = tid; idx < n_heads * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx % HD;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, sm_m[w * ROWS + row]);
        float acc = 0.f, ls = 0.f;
        if (mx != -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float ms = sm_m[w * ROWS + row];
                if (ms == -INFINITY) continue;
                const float a = exp2f(ms - mx);
                acc = fmaf(a, sm_o[(w * ROWS + row) * HD + d], acc);
                ls = fmaf(a, sm_l[w * ROWS + row], ls);
            }
        }
        const long long base = ((long long)r * nh + (h0 + row)) * n_splits + sp;
        part_o[base * HD + d] = acc;
        // the merge kernel works with natural-base maxima
        if (d == 0) { part_ml[base * 2] = mx * 0.6931471805599453f; part_ml[base * 2 + 1] = ls; }
    }
    if (!fuse_merge) return;
    // the last of this (request, kv head, pass)'s blocks merges all splits, with the merge kernel's arithmetic
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int slot = r * (int)gridDim.y + (int)blockIdx.y;
        s_last = atomicAdd(&g_merge_counters[slot], 1) == n_splits - 1 ? 1 : 0;
        if (s_last) g_merge_counters[slot] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = tid; idx < n_heads * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx % HD;
        const long long base = ((long long)r * nh + (h0 + row)) * n_splits;
        float mx = -INFINITY;
        for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, __ldcg(part_ml + (base + s) * 2));
        float acc = 0.f, ls = 0.f;
        if (mx != -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float ms = __ldcg(part_ml + (base + s) * 2);
                if (ms == -INFINITY) continue;
                const float a = expf(ms - mx);
                acc = fmaf(a, __ldcg(part_o + (base + s) * HD + d), acc);
                ls = fmaf(a, __ldcg(part_ml + (base + s) * 2 + 1), ls);
            }
        }
        out[(long long)token * nh * HD + (long long)(h0 + row) * HD + d] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
    }
}

template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_mma_kernel(const __nv_bfloat16* q, const __nv_bfloat16* k_cache,
                            const __nv_bfloat16* v_cache, const int32_t* __restrict__ block_table,
                            int table_width, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ kv_len,
                            float* part_o, float* part_ml, int nh, int nkv, int page_size,
                            int page_shift, int total_pages, int window, float scale_log2, int chunk, int n_splits,
                            int head_passes, __nv_bfloat16* out, int fuse_merge, int* err) {
    constexpr int PITCH = HD + 8;
    constexpr int KS = HD / 16, DT = HD / 8, CPR = HD / 8;
    dep_wait();
    dep_launch_next();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [ROWS][PITCH]
    __nv_bfloat16* Ks = Qs + ROWS * PITCH;                               // [2][BKV][PITCH]
    __nv_bfloat16* Vs = Ks + 2 * BKV * PITCH;                            // [2][BKV][PITCH]

    const int r = blockIdx.x;
    const int kvh = blockIdx.y / head_passes, pass = blockIdx.y % head_passes;
    const int sp = blockIdx.z;
    if (cu_q[r + 1] - cu_q[r] != 1) return;
    const int group = nh / nkv;
    const int h0 = kvh * group + pass * ROWS;
    const int n_heads = min(ROWS, group - pass * ROWS);
    const int len = kv_len[r], p = len - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    // the request's own visible keys, cut into n_splits equal shares (multiples of 16 keys): every split of a
    // request has the same work, whatever the longest request of the batch is
    const int share = (((len - lo) + n_splits - 1) / n_splits + 15) & ~15;
    const int j_begin = lo + sp * share, j_end = min(len, j_begin + share);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = lane & 3;
    const int token = cu_q[r];

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    if (j_begin < j_end) {
        const int32_t* table = block_table + (long long)r * table_width;
        for (int idx = tid; idx < ROWS * CPR; idx += WARPS * 32) {
            const int row = idx / CPR, c = idx % CPR;
            if (row < n_heads) cp_async16(Qs + row * PITCH + c * 8, q + ((long long)token * nh + h0 + row) * HD + c * 8);
            else *reinterpret_cast<uint4*>(Qs + row * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");

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
            for (int idx = tid; idx < BKV * CPR; idx += WARPS * 32) {
                const int key = idx / CPR, c = idx % CPR;         // CPR is a compile-time constant
                const int j = j0 + key;
                int page = -1, in_page = 0;
                if (j >= j_begin && j < j_end) {
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

        const int t_begin = (j_begin / BKV) * BKV;
        const int n_tiles = (j_end - t_begin + BKV - 1) / BKV;
        fill(0, t_begin);
        const int lm_row = lane & 15, lm_col = (lane >> 4) * 8;
        uint32_t qf[KS][4];
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
            if (it == 0) {
#pragma unroll
                for (int kk = 0; kk < KS; ++kk) ldsm_x4(qf[kk], Qs + lm_row * PITCH + kk * 16 + lm_col);
            }
            const __nv_bfloat16* kt = Ks + (size_t)stage * BKV * PITCH + (warp * 16) * PITCH;
            const __nv_bfloat16* vt = Vs + (size_t)stage * BKV * PITCH + (warp * 16) * PITCH;
            const int jw = j0 + warp * 16;                        // this warp's 16 keys
            if (jw < j_end && jw + 16 > j_begin) {                // warp-uniform
                float s[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
#pragma unroll
                for (int kk = 0; kk < KS; ++kk) {
                    uint32_t kf[4];
                    ldsm_x4(kf, kt + lm_row * PITCH + kk * 16 + lm_col);
                    mma16816(s[0], qf[kk], kf[0], kf[2]);
                    mma16816(s[1], qf[kk], kf[1], kf[3]);
                }
                float mx_a = m_a, mx_b = m_b;
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = jw + n * 8 + 2 * t + (c & 1);
                        const float v = (j >= j_begin && j < j_end) ? s[n][c] * scale_log2 : -INFINITY;
                        s[n][c] = v;
                        if (c < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                    }
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                const float base_a = mx_a == -INFINITY ? 0.f : mx_a, base_b = mx_b == -INFINITY ? 0.f : mx_b;
                const float al_a = exp2f(m_a - base_a), al_b = exp2f(m_b - base_b);
                const float p00 = exp2f(s[0][0] - base_a), p01 = exp2f(s[0][1] - base_a);
                const float p02 = exp2f(s[0][2] - base_b), p03 = exp2f(s[0][3] - base_b);
                const float p10 = exp2f(s[1][0] - base_a), p11 = exp2f(s[1][1] - base_a);
                const float p12 = exp2f(s[1][2] - base_b), p13 = exp2f(s[1][3] - base_b);
                float sum_a = (p00 + p01) + (p10 + p11), sum_b = (p02 + p03) + (p12 + p13);
                sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
                sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
                sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
                sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
                l_a = l_a * al_a + sum_a;
                l_b = l_b * al_b + sum_b;
                m_a = mx_a;
                m_b = mx_b;
                const uint32_t pf[4] = {pack_bf16(p00, p01), pack_bf16(p02, p03), pack_bf16(p10, p11),
                                        pack_bf16(p12, p13)};
#pragma unroll
                for (int dn = 0; dn < HD / 16; ++dn) {
                    uint32_t vf[4];
                    ldsm_x4_trans(vf, vt + lm_row * PITCH + dn * 16 + lm_col);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        o[2 * dn][c] *= (c < 2) ? al_a : al_b;
                        o[2 * dn + 1][c] *= (c < 2) ? al_a : al_b;
                    }
                    mma16816(o[2 * dn], pf, vf[0], vf[1]);
                    mma16816(o[2 * dn + 1], pf, vf[2], vf[3]);
                }
            }
            __syncthreads();
        }
    }

    finish_block<HD>(smem_raw, o, m_a, m_b, l_a, l_b, r, h0, n_heads, sp, token, part_o, part_ml, nh, n_splits, out,
                     fuse_merge);
}

// ------------------------------------------------------------------------------------------ with TMA
// The same kernel with the keys and values brought by the TMA unit: a producer warp asks for each tile of 64
// keys as boxes of 64 keys x 64 dims straight from the page (128-byte swizzle, so that ldmatrix reads without
// bank conflicts), NST tiles in flight on mbarriers; the four consumer warps neither compute addresses nor
// meet at a block-wide barrier per tile.  Needs head sizes of 64 or 128 and pages of a power of two of at
// least 64 tokens.  Keys outside the block's share are masked, not zeroed: the cache holds finite numbers
// everywhere (it starts as zeros and only kernels write it); a page that is not there is read as zeros.

struct DecodeTmaParams {
    const __nv_bfloat16* q;
    const int32_t* block_table; int table_width;
    const int32_t* cu_q; const int32_t* kv_len;
    float* part_o; float* part_ml;
    int nh, nkv, page_size, page_shift, total_pages, window;
    float scale_log2;
    int n_splits, head_passes;
    __nv_bfloat16* out; int fuse_merge;
    int* err;
};

template <int HD, int NST>
__global__ void __launch_bounds__((WARPS + 1) * 32)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            DecodeTmaParams p) {
    using namespace tc5;
    constexpr int PITCH = HD + 8;
    constexpr int KS = HD / 16, DT = HD / 8, CPR = HD / 8, NHALF = HD / 64;
    constexpr uint32_t HALF_BYTES = BKV * 128;                      // 64 keys x 64 dims
    constexpr uint32_t STAGE_BYTES = 2 * NHALF * HALF_BYTES;        // keys then values
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full_bar[NST], empty_bar[NST];
    __shared__ int s_abort;
    const uint32_t raw_addr = smem_u32(smem_dyn);
    unsigned char* smem_raw = smem_dyn + (((raw_addr + 1023u) & ~1023u) - raw_addr);     // the tiles want 1024-byte alignment
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw + NST * STAGE_BYTES);  // [ROWS][PITCH]

    const int r = blockIdx.x;
    const int kvh = blockIdx.y / p.head_passes, pass = blockIdx.y % p.head_passes;
    const int sp = blockIdx.z;
    if (p.cu_q[r + 1] - p.cu_q[r] != 1) {      // (the step's lengths and tables were there before the step began)
        dep_wait();
        return;
    }
    const int group = p.nh / p.nkv;
    const int h0 = kvh * group + pass * ROWS;
    const int n_heads = min(ROWS, group - pass * ROWS);
    const int len = p.kv_len[r], pos = len - 1;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int share = (((len - lo) + p.n_splits - 1) / p.n_splits + 15) & ~15;
    const int j_begin = lo + sp * share, j_end = min(len, j_begin + share);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = lane & 3;
    const int token = p.cu_q[r];
    const int t_begin = (j_begin / BKV) * BKV;
    const int n_tiles = j_begin < j_end ? (j_end - t_begin + BKV - 1) / BKV : 0;
    volatile int* abort_flag = &s_abort;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < NST; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The kernel before this one wrote the step's new key and value (position len - 1) and the queries.
    // Everything older in the cache, the block table and the lengths were there before the step began, so the
    // producer asks for every tile that does not hold position len - 1 before it waits for that kernel;
    // everybody else waits first.
    const int tiles_before_wait = (t_begin + n_tiles * BKV > pos) ? max(n_tiles - 1, 0) : n_tiles;
    if (warp != WARPS) {
        dep_wait();
        dep_launch_next();
    }

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    if (warp == WARPS) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            const int32_t* table = p.block_table + (long long)r * p.table_width;
            const int rows_total = p.total_pages * p.nkv * p.page_size;
            bool waited = false;
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it % NST;
                // (a stage is given back only after the consumers, who have waited, have read it)
                if (it >= tiles_before_wait && !waited) { dep_wait(); waited = true; }
                if (it >= NST && !mbar_wait(&empty_bar[s], ((it / NST) & 1) ^ 1, abort_flag)) break;
                const int key0 = t_begin + it * BKV;
                const int lp = key0 >> p.page_shift;
                int page = lp < p.table_width ? table[lp] : -1;
                if (page < 0 || page >= p.total_pages) { *p.err = 3; page = -1; }       // the tile holds keys of this block's share
                const int y = page >= 0 ? (page * p.nkv + kvh) * p.page_size + (key0 & (p.page_size - 1)) : rows_total;
                unsigned char* dst = smem_raw + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
#pragma unroll
                for (int h = 0; h < NHALF; ++h) {
                    tma_load_2d(dst + h * HALF_BYTES, &map_k, 64 * h, y, &full_bar[s]);
                    tma_load_2d(dst + (NHALF + h) * HALF_BYTES, &map_v, 64 * h, y, &full_bar[s]);
                }
            }
        }
        dep_wait();        // every thread has waited for the kernel before this one when the block ends
    } else if (n_tiles > 0) {
        // ----------------------------------------------------------------- consumers
        for (int idx = tid; idx < ROWS * CPR; idx += WARPS * 32) {
            const int row = idx / CPR, c = idx % CPR;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < n_heads) v = *reinterpret_cast<const uint4*>(p.q + ((long long)token * p.nh + h0 + row) * HD + c * 8);
            *reinterpret_cast<uint4*>(Qs + row * PITCH + c * 8) = v;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");      // the four consumer warps only
        const int lm_row = lane & 15, lm_col = (lane >> 4) * 8;
        uint32_t qf[KS][4];
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) ldsm_x4(qf[kk], Qs + lm_row * PITCH + kk * 16 + lm_col);
        // this lane's row of a tile (a key) and its place in the 128-byte swizzle
        const int krow = warp * 16 + lm_row;
        const uint32_t row_off = (uint32_t)krow * 128, sw = (uint32_t)(krow & 7);
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % NST;
            const int j0 = t_begin + it * BKV;
            if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (it / NST) & 1, abort_flag))) break;
            const unsigned char* kt = smem_raw + (size_t)s * STAGE_BYTES;
            const unsigned char* vt = kt + NHALF * HALF_BYTES;
            const int jw = j0 + warp * 16;                        // this warp's 16 keys
            if (jw < j_end && jw + 16 > j_begin) {                // warp-uniform
                float sc[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int c = 0; c < 4; ++c) sc[n][c] = 0.f;
#pragma unroll
                for (int kk = 0; kk < KS; ++kk) {
                    const uint32_t chunk = (uint32_t)(kk * 2 + (lm_col >> 3));      // 16-byte chunk of the key's row
                    uint32_t kf[4];
                    ldsm_x4(kf, kt + (chunk >> 3) * HALF_BYTES + row_off + (((chunk & 7) ^ sw) << 4));
                    mma16816(sc[0], qf[kk], kf[0], kf[2]);
                    mma16816(sc[1], qf[kk], kf[1], kf[3]);
                }
                float mx_a = m_a, mx_b = m_b;
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = jw + n * 8 + 2 * t + (c & 1);
                        const float v = (j >= j_begin && j < j_end) ? sc[n][c] * p.scale_log2 : -INFINITY;
                        sc[n][c] = v;
                        if (c < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                    }
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                const float base_a = mx_a == -INFINITY ? 0.f : mx_a, base_b = mx_b == -INFINITY ? 0.f : mx_b;
                const float al_a = exp2f(m_a - base_a), al_b = exp2f(m_b - base_b);
                const float p00 = exp2f(sc[0][0] - base_a), p01 = exp2f(sc[0][1] - base_a);
                const float p02 = exp2f(sc[0][2] - base_b), p03 = exp2f(sc[0][3] - base_b);
                const float p10 = exp2f(sc[1][0] - base_a), p11 = exp2f(sc[1][1] - base_a);
                const float p12 = exp2f(sc[1][2] - base_b), p13 = exp2f(sc[1][3] - base_b);
                float sum_a = (p00 + p01) + (p10 + p11), sum_b = (p02 + p03) + (p12 + p13);
                sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
                sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
                sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
                sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
                l_a = l_a * al_a + sum_a;
                l_b = l_b * al_b + sum_b;
                m_a = mx_a;
                m_b = mx_b;
                const uint32_t pf[4] = {pack_bf16(p00, p01), pack_bf16(p02, p03), pack_bf16(p10, p11),
                                        pack_bf16(p12, p13)};
#pragma unroll
                for (int dn = 0; dn < HD / 16; ++dn) {
                    const uint32_t chunk = (uint32_t)(dn * 2 + (lm_col >> 3));
                    uint32_t vf[4];
                    ldsm_x4_trans(vf, vt + (chunk >> 3) * HALF_BYTES + row_off + (((chunk & 7) ^ sw) << 4));
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        o[2 * dn][c] *= (c < 2) ? al_a : al_b;
                        o[2 * dn + 1][c] *= (c < 2) ? al_a : al_b;
                    }
                    mma16816(o[2 * dn], pf, vf[0], vf[1]);
                    mma16816(o[2 * dn + 1], pf, vf[2], vf[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
    }
    __syncthreads();                    // every copy has landed and been read (or a wait ran out)
    if (s_abort) {
        if (tid == 0) *p.err = 5;
        for (int i = 0; i < 200; ++i) __nanosleep(1000);       // copies that may still be in flight
        __syncthreads();
    }
    finish_block<HD>(smem_raw, o, m_a, m_b, l_a, l_b, r, h0, n_heads, sp, token, p.part_o, p.part_ml, p.nh, p.n_splits,
                     p.out, p.fuse_merge);
}

bool make_kv_map(CUtensorMap* map, const void* base, long long rows, int hd) {
    tc5::EncodeTiledFn fn = tc5::encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)BKV};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD, int NST>
bool launch_tma(dim3 grid, cudaStream_t stream, const void* k_cache, const void* v_cache, const DecodeTmaParams& p) {
    CUtensorMap mk, mv;
    const long long rows = (long long)p.total_pages * p.nkv * p.page_size;
    if (!make_kv_map(&mk, k_cache, rows, HD) || !make_kv_map(&mv, v_cache, rows, HD)) return false;
    size_t smem = (size_t)NST * 2 * (HD / 64) * BKV * 128 + (size_t)ROWS * (HD + 8) * sizeof(__nv_bfloat16) + 1024;
    const size_t merge = sizeof(float) * (size_t)(2 * WARPS * ROWS + WARPS * ROWS * HD) + 1024;
    if (merge > smem) smem = merge;
    auto kern = attention_decode_tma_kernel<HD, NST>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_dep(kern, grid, (WARPS + 1) * 32, smem, stream, mk, mv, p);
    return true;
}

template <int HD>
void launch(dim3 grid, cudaStream_t stream, const void* q, const void* k_cache, const void* v_cache,
            const int32_t* block_table, int table_width, const int32_t* cu_q, const int32_t* kv_len, float* part_o,
            float* part_ml, int nh, int nkv, int page_size, int total_pages, int window, float scale, int chunk,
            int n_splits, int head_passes, void* out, int fuse_merge) {
    size_t smem = (size_t)(ROWS + 4 * BKV) * (HD + 8) * sizeof(__nv_bfloat16);
    const size_t merge = sizeof(float) * (size_t)(2 * WARPS * ROWS + WARPS * ROWS * HD);
    if (merge > smem) smem = merge;
    int shift = -1;
    if ((page_size & (page_size - 1)) == 0) { shift = 0; while ((1 << shift) < page_size) ++shift; }
    auto kern = attention_decode_mma_kernel<HD>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_dep(kern, grid, WARPS * 32, smem, stream,
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
        static_cast<const __nv_bfloat16*>(v_cache), block_table, table_width, cu_q, kv_len, part_o, part_ml, nh, nkv,
        page_size, shift, total_pages, window, scale * 1.4426950408889634f, chunk, n_splits, head_passes,
        static_cast<__nv_bfloat16*>(out), fuse_merge, error_flag_ptr());
}

}  // namespace

void attention_decode_mma(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                          int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, float* scratch,
                          int R, int nh, int nkv, int hd, int page_size, int total_pages, int window, float scale,
                          int n_splits, int chunk, cudaStream_t stream) {
    if (R <= 0) return;
    DLM_CHECK(attention_prefill_ok(hd), "decode attention: this head_dim has no tensor-core kernel");
    DLM_CHECK(nh % nkv == 0, "attention: heads must be a multiple of kv heads");
    const int group = nh / nkv;
    const int head_passes = (group + ROWS - 1) / ROWS;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)R * nh * n_splits * hd;
    dim3 grid(R, nkv * head_passes, n_splits);
    const int fuse_merge = (long long)R * nkv * head_passes <= MERGE_SLOTS ? 1 : 0;
    static const bool tma_on = []() {
        const char* off = std::getenv("DLM_B200_NO_TCGEN05");
        return !(off != nullptr && off[0] != '\0' && off[0] != '0') && tc5::encode_tiled() != nullptr;
    }();
    if (tma_on && (hd == 64 || hd == 128) && page_size >= 64 && (page_size & (page_size - 1)) == 0 &&
        ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(q)) & 15) == 0) {
        int shift = 0;
        while ((1 << shift) < page_size) ++shift;
        // This kernel is fastest with one block per multiprocessor and as few key splits as that allows (a
        // block's start and the merge of splits cost more than a second wave saves); never more splits than
        // the plan, whose scratch it uses.
        const int n_sm = sm_count();
        const long long per_split = (long long)R * nkv * head_passes;
        int splits = (int)(n_sm / per_split);
        splits = splits < 1 ? 1 : (splits > n_splits ? n_splits : splits);
        const dim3 tma_grid(R, nkv * head_passes, splits);
        DecodeTmaParams p{static_cast<const __nv_bfloat16*>(q), block_table, table_width, cu_q, kv_len, part_o, part_ml, nh,
                          nkv, page_size, shift, total_pages, window, scale * 1.4426950408889634f, splits, head_passes,
                          static_cast<__nv_bfloat16*>(out), fuse_merge, error_flag_ptr()};
        // Blocks that have a multiprocessor to themselves keep six tiles in flight instead of three (8 requests
        // of 8,192 tokens: 4.72 -> 4.57 ms a step; of 1,030: 3.245 -> 3.235).
        const bool alone = per_split * splits <= n_sm;
        const bool done = hd == 64 ? (alone ? launch_tma<64, 6>(tma_grid, stream, k_cache, v_cache, p)
                                            : launch_tma<64, 3>(tma_grid, stream, k_cache, v_cache, p))
                                   : (alone ? launch_tma<128, 6>(tma_grid, stream, k_cache, v_cache, p)
                                            : launch_tma<128, 3>(tma_grid, stream, k_cache, v_cache, p));
        if (done) {
            check_launch("attention_decode_tma");
            if (!fuse_merge) attention_decode_merge(part_o, part_ml, cu_q, out, R, nh, hd, splits, BF16, stream);
            return;
        }
    }
#define DLM_DECODE(HD)                                                                                              \
    launch<HD>(grid, stream, q, k_cache, v_cache, block_table, table_width, cu_q, kv_len, part_o, part_ml, nh, nkv, \
               page_size, total_pages, window, scale, chunk, n_splits, head_passes, out, fuse_merge)
    switch (hd) {
        case 16: DLM_DECODE(16); break;
        case 32: DLM_DECODE(32); break;
        case 48: DLM_DECODE(48); break;
        case 64: DLM_DECODE(64); break;
        case 96: DLM_DECODE(96); break;
        default: DLM_DECODE(128); break;
    }
#undef DLM_DECODE
    check_launch("attention_decode_mma");
    if (!fuse_merge) attention_decode_merge(part_o, part_ml, cu_q, out, R, nh, hd, n_splits, BF16, stream);
}

}  // namespace dlmk

namespace dlmk {

void reset_decode_merge_counters(cudaStream_t stream) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_merge_counters) == cudaSuccess && p != nullptr)
        cudaMemsetAsync(p, 0, sizeof(int) * MERGE_SLOTS, stream);
}

}  // namespace dlmk
