// Paged causal attention on the FMA units, for any head size up to 256 and both dtypes.
// It is the 32-bit path's attention and the reference every faster kernel is checked against.
//
// One block = 16 consecutive query tokens of one request x one query head.  Keys are walked
// in tiles of 32 that start at absolute positions divisible by 32, and a tile in which a
// query sees nothing leaves that query's running maximum, sum and output untouched; so a
// query's result does not depend on how its request was cut into steps, on the other
// requests of the batch, or on which pages hold its keys.
#include "api.h"
#include "attention_internal.h"
#include "common.cuh"

namespace dlmk {

namespace {

constexpr int BQ = 16;        // queries per block
constexpr int BKV = 32;       // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int QPW = BQ / WARPS;
constexpr int MAX_HD = 256;
constexpr int DPL = MAX_HD / 32;   // head dims per lane

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ cu_q,
                      const int32_t* __restrict__ kv_len, T* __restrict__ out, int R, int nh, int nkv, int hd,
                      int page_size, int total_pages, int window, float scale, int skip_single, int* err) {
    extern __shared__ float smem[];
    float* Qs = smem;                               // [BQ][hd]
    float* Ks = Qs + BQ * hd;                       // [BKV][hd + 1]
    float* Vs = Ks + BKV * (hd + 1);                // [BKV][hd]
    float* Ps = Vs + BKV * hd;                      // [WARPS][QPW][BKV]
    __shared__ int s_map[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.y;
    const int kvh = head / (nh / nkv);

    // which request and which of its query tiles this block has
    if (tid == 0) {
        int acc = 0;
        s_map[0] = -1;
        for (int r = 0; r < R; ++r) {
            const int ql = cu_q[r + 1] - cu_q[r];
            const int tiles = (skip_single && ql == 1) ? 0 : (ql + BQ - 1) / BQ;
            if ((int)blockIdx.x < acc + tiles) {
                s_map[0] = r;
                s_map[1] = ((int)blockIdx.x - acc) * BQ;
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
    const int pos0 = len - q_len + q0;              // position of the tile's first query
    const int Q = nh * hd;

    for (int idx = tid; idx < BQ * hd; idx += blockDim.x) {
        const int qi = idx / hd, d = idx % hd;
        Qs[idx] = qi < n_q ? to_f32(q[(long long)(q_begin + q0 + qi) * Q + head * hd + d]) : 0.f;
    }

    float m[QPW], l[QPW], o[QPW][DPL];
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) o[i][j] = 0.f;
    }

    const int hi = pos0 + n_q - 1;                  // last key any query of the tile sees
    int lo = 0;
    if (window > 0) lo = max(0, pos0 - window + 1);
    const int tile_lo = (lo / BKV) * BKV;
    const int* table = block_table + (long long)r * table_width;

    for (int kv0 = tile_lo; kv0 <= hi; kv0 += BKV) {
        __syncthreads();
        // load the tile: key j = kv0 + jj
        for (int idx = tid; idx < BKV * hd; idx += blockDim.x) {
            const int jj = idx / hd, d = idx % hd;
            const int j = kv0 + jj;
            float kvv = 0.f, vvv = 0.f;
            if (j <= hi && j >= lo) {
                const int lp = j / page_size;
                const int page = lp < table_width ? table[lp] : -1;
                if (page >= 0 && page < total_pages) {
                    const long long off = (((long long)page * nkv + kvh) * page_size + (j % page_size)) * hd + d;
                    kvv = to_f32(k_cache[off]);
                    vvv = to_f32(v_cache[off]);
                } else {
                    *err = 3;    // a visible key without a page: refuse to read, report
                }
            }
            Ks[jj * (hd + 1) + d] = kvv;
            Vs[jj * hd + d] = vvv;
        }
        __syncthreads();

        const int j = kv0 + lane;
#pragma unroll
        for (int i = 0; i < QPW; ++i) {
            const int qi = warp * QPW + i;
            if (qi >= n_q) continue;                // uniform over the warp
            const int p = pos0 + qi;
            const float* qv = Qs + qi * hd;
            const float* kr = Ks + lane * (hd + 1);
            float s = 0.f;
            for (int d = 0; d < hd; ++d) s = fmaf(qv[d], kr[d], s);
            s *= scale;
            const bool visible = (j <= p) && (window <= 0 || p - j < window);
            if (!visible) s = -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            if (m_new == -INFINITY) continue;       // this query sees nothing in the tile
            const float pj = visible ? expf(s - m_new) : 0.f;
            const float alpha = expf(m[i] - m_new); // exp(-inf) = 0 on the first tile with a visible key
            l[i] = l[i] * alpha + warp_sum(pj);
            m[i] = m_new;
            float* pw = Ps + (warp * QPW + i) * BKV;
            pw[lane] = pj;
            __syncwarp();
#pragma unroll
            for (int jd = 0; jd < DPL; ++jd) {
                const int d = lane + 32 * jd;
                if (d < hd) {
                    float acc = o[i][jd] * alpha;
                    for (int kk = 0; kk < BKV; ++kk) acc = fmaf(pw[kk], Vs[kk * hd + d], acc);
                    o[i][jd] = acc;
                }
            }
            __syncwarp();
        }
    }

#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        const int qi = warp * QPW + i;
        if (qi >= n_q) continue;
        const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
        T* orow = out + (long long)(q_begin + q0 + qi) * Q + head * hd;
#pragma unroll
        for (int jd = 0; jd < DPL; ++jd) {
            const int d = lane + 32 * jd;
            if (d < hd) orow[d] = from_f32<T>(o[i][jd] * inv);
        }
    }
}

}  // namespace

void attention_simt(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                    int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                    int nkv, int hd, int page_size, int total_pages, int window, float scale, int skip_single,
                    int dtype, cudaStream_t stream) {
    if (T <= 0 || R <= 0) return;
    DLM_CHECK(hd > 0 && hd <= MAX_HD, "attention: head_dim must be in 1..256");
    DLM_CHECK(nh % nkv == 0, "attention: heads must be a multiple of kv heads");
    const int tiles = (T + BQ - 1) / BQ + R;        // every request may end in a partial tile
    const size_t smem = sizeof(float) * (BQ * hd + BKV * (hd + 1) + BKV * hd + WARPS * QPW * BKV);
    dim3 grid(tiles, nh);
    int* err = error_flag_ptr();
    if (dtype == F32) {
        auto kern = attention_simt_kernel<float>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<grid, WARPS * 32, smem, stream>>>(static_cast<const float*>(q), static_cast<const float*>(k_cache),
            static_cast<const float*>(v_cache), block_table, table_width, cu_q, kv_len, static_cast<float*>(out), R,
            nh, nkv, hd, page_size, total_pages, window, scale, skip_single, err);
    } else {
        auto kern = attention_simt_kernel<__nv_bfloat16>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<grid, WARPS * 32, smem, stream>>>(static_cast<const __nv_bfloat16*>(q),
            static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache), block_table,
            table_width, cu_q, kv_len, static_cast<__nv_bfloat16*>(out), R, nh, nkv, hd, page_size, total_pages,
            window, scale, skip_single, err);
    }
    check_launch("attention_simt");
}

}  // namespace dlmk
