// What the tcgen05 products share: the launch parameters, the walk over token tiles, the token boxes, the
// tensor-map encoder, and the epilogue: one weight tile's accumulator (128 lanes = output columns, the
// tile's tokens as columns of tensor memory) leaves through the warp's staging area as 16-byte stores along
// the rows of the output.  Used by the kernel on single multiprocessors and by the one on pairs.
#pragma once
#include <cuda_bf16.h>

#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace dlmk {
namespace tc5 {

struct TcParams {
    const int32_t* expert_offsets; int num_experts;
    const float* bias;
    void* out; int ldo;
    int M, N, K;
    int* err;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int TT = 256;          // most tokens per tile (the MMA's N)

struct TileInfo { int expert, row_begin, row_end; };

// Token tile `ty` of the launch: dense, rows [ty * tt, ...); grouped, the ty-th tile when every expert's rows
// are cut into tiles of tt (at most TT) tokens.  expert < 0: there is no such tile.
__device__ __forceinline__ TileInfo tile_info(const TcParams& p, int ty, int tt = TT) {
    TileInfo t{0, ty * tt, p.M};
    if (p.expert_offsets != nullptr) {
        t.expert = -1;
        int acc = 0;
        for (int e = 0; e < p.num_experts; ++e) {
            const int r0 = p.expert_offsets[e], r1 = p.expert_offsets[e + 1];
            const int tiles_e = (r1 - r0 + tt - 1) / tt;
            if (ty < acc + tiles_e) {
                t.expert = e;
                t.row_begin = r0 + (ty - acc) * tt;
                t.row_end = r1;
                break;
            }
            acc += tiles_e;
        }
    }
    t.row_end = min(min(t.row_end, t.row_begin + tt), p.M);
    if (t.row_begin >= t.row_end) t.expert = -1;
    return t;
}

// Token tiles are fetched with the smallest of sixteen boxes that holds the tile's tokens (16, 32, ..., 256
// rows; half of that where a pair of multiprocessors shares a tile), so that a short group does not cost the
// bandwidth of a full one.
struct TokenMaps { CUtensorMap m[16]; };

// Warp `hsel` (0 or 1) of a quadrant takes the chunks of CH tokens c0 = CH hsel, CH hsel + 2 CH, ...  (CH = 32,
// or 16 where the staging areas have to be small).  `d_tmem` addresses the accumulator's first column in
// this warp's 32 lanes, `colw` is the warp's first output column, `st` its staging area of CH x 33 floats.
template <int EPI, typename TOut, int CH = 32>
__device__ __forceinline__ void epilogue_tile(const TcParams& p, float* st, uint32_t d_tmem, int colw, int n_mma,
                                              int row_begin, int row_end, int hsel, int lane, bool vec_ok) {
    const int col = colw + lane;
    const bool col_ok = col < p.N;
    const float bias = (EPI == EPI_STORE && p.bias != nullptr && col_ok) ? p.bias[col] : 0.f;
#pragma unroll 1
    for (int c0 = hsel * CH; c0 < n_mma; c0 += 2 * CH) {
        uint32_t v[CH];
        tmem_ld(d_tmem + (uint32_t)c0, v);
        const int tok0 = row_begin + c0;
        const int n_valid = min(CH, row_end - tok0);      // tokens of this chunk that exist
        if (n_valid <= 0) continue;                       // uniform over the warp
        if (EPI == EPI_SWIGLU) {
            // Even lanes hold gate, their odd neighbours up, for the same output.  Per pair of tokens (j, j + 1)
            // the two lanes swap one number: the even lane sends its gate of token j + 1 and gets the up of
            // token j, so the even lane finishes token j and the odd lane token j + 1: one exchange and one
            // SiLU per lane and pair, no lane idle.  The result is rounded to bfloat16: the fast exponential
            // and division are exact enough.
            const bool odd = lane & 1;
#pragma unroll
            for (int j = 0; j < CH; j += 2) {
                const float a0 = __uint_as_float(v[j]), a1 = __uint_as_float(v[j + 1]);
                const float got = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
                const float g = odd ? got : a0, uu = odd ? a1 : got;
                st[(j + (odd ? 1 : 0)) * 17 + (lane >> 1)] = __fdividef(g, 1.0f + __expf(-g)) * uu;
            }
            __syncwarp();
            TOut* o = static_cast<TOut*>(p.out) + (long long)tok0 * p.ldo + (colw >> 1);
            if (vec_ok && sizeof(TOut) == 2) {
                // CH tokens x 16 outputs: a lane stores 8 outputs (16 bytes) of one token, 16 tokens a pass
#pragma unroll
                for (int pass = 0; pass < CH / 16; ++pass) {
                    const int j = pass * 16 + (lane >> 1), seg = (lane & 1) * 8;
                    if (j < n_valid && colw + 2 * seg + 15 < p.N) {
                        const float* r = st + j * 17 + seg;
                        uint4 pk;
                        pk.x = pack2(r[0], r[1]); pk.y = pack2(r[2], r[3]);
                        pk.z = pack2(r[4], r[5]); pk.w = pack2(r[6], r[7]);
                        *reinterpret_cast<uint4*>(o + (long long)j * p.ldo + seg) = pk;
                    }
                }
            } else {
                for (int idx = lane; idx < CH * 16; idx += 32) {
                    const int j = idx >> 4, c = idx & 15;
                    if (j < n_valid && colw + 2 * c + 1 < p.N) o[(long long)j * p.ldo + c] = from_f32<TOut>(st[j * 17 + c]);
                }
            }
            __syncwarp();
        } else {
#pragma unroll
            for (int j = 0; j < CH; ++j) st[j * 33 + lane] = __uint_as_float(v[j]) + bias;
            __syncwarp();
            if (EPI == EPI_ADD) {
                float* o = static_cast<float*>(p.out) + (long long)tok0 * p.ldo + colw;
                if (vec_ok) {
                    // CH tokens x 32 columns: a lane owns 4 columns (16 bytes) of one token, 4 tokens a pass;
                    // all loads of the residual are in flight before the first store
                    const int seg = (lane & 7) * 4;
                    const bool cok = colw + seg + 3 < p.N;
                    float4 old[CH / 4];
#pragma unroll
                    for (int pass = 0; pass < CH / 4; ++pass) {
                        const int j = pass * 4 + (lane >> 3);
                        old[pass] = (cok && j < n_valid)
                                        ? *reinterpret_cast<const float4*>(o + (long long)j * p.ldo + seg)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int pass = 0; pass < CH / 4; ++pass) {
                        const int j = pass * 4 + (lane >> 3);
                        if (cok && j < n_valid) {
                            const float* r = st + j * 33 + seg;
                            float4 nv = old[pass];
                            nv.x += r[0]; nv.y += r[1]; nv.z += r[2]; nv.w += r[3];
                            *reinterpret_cast<float4*>(o + (long long)j * p.ldo + seg) = nv;
                        }
                    }
                } else {
                    for (int j = 0; j < n_valid; ++j)
                        if (col_ok) o[(long long)j * p.ldo + lane] += st[j * 33 + lane];
                }
            } else {
                TOut* o = static_cast<TOut*>(p.out) + (long long)tok0 * p.ldo + colw;
                if (vec_ok && sizeof(TOut) == 4) {
                    const int seg = (lane & 7) * 4;
                    const bool cok = colw + seg + 3 < p.N;
#pragma unroll
                    for (int pass = 0; pass < CH / 4; ++pass) {
                        const int j = pass * 4 + (lane >> 3);
                        if (cok && j < n_valid) {
                            const float* r = st + j * 33 + seg;
                            *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + (long long)j * p.ldo + seg) =
                                make_float4(r[0], r[1], r[2], r[3]);
                        }
                    }
                } else if (vec_ok && sizeof(TOut) == 2) {
                    const int seg = (lane & 3) * 8;
                    const bool cok = colw + seg + 7 < p.N;
#pragma unroll
                    for (int pass = 0; pass < CH / 8; ++pass) {
                        const int j = pass * 8 + (lane >> 2);
                        if (cok && j < n_valid) {
                            const float* r = st + j * 33 + seg;
                            uint4 pk;
                            pk.x = pack2(r[0], r[1]); pk.y = pack2(r[2], r[3]);
                            pk.z = pack2(r[4], r[5]); pk.w = pack2(r[6], r[7]);
                            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(o) + (long long)j * p.ldo + seg) = pk;
                        }
                    }
                } else {
                    for (int j = 0; j < n_valid; ++j)
                        if (col_ok) o[(long long)j * p.ldo + lane] = from_f32<TOut>(st[j * 33 + lane]);
                }
            }
            __syncwarp();
        }
    }
}

// rows x K bfloat16 matrix with `ld` elements between rows; boxes of box_rows x 64 elements, 128-byte swizzle,
// elements outside the matrix read as zero
inline bool make_map(CUtensorMap* map, const void* base, long long rows, int K, int ld, int box_rows,
              CUtensorMapL2promotion promote = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promote,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc5
}  // namespace dlmk
