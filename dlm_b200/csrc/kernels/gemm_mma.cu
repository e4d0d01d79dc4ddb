// C = A · W^T for many rows of A (prompt portions) on the warp-level tensor-core path:
// mma.sync m16n8k16 (bfloat16 in, 32-bit accumulation) fed through a three-stage pipeline of
// asynchronous 16-byte copies and ldmatrix.  Dense or grouped by expert, rows of A optionally
// gathered, with the store / accumulate / SwiGLU epilogues.
//
// Block tile BM x 128 x 32 (BM = 128 or 64), 8 warps in a 2 x 4 arrangement.  Shared-memory rows
// are padded from 64 to 80 bytes so that the eight 16-byte rows an ldmatrix reads fall into
// different banks.  Every output element is summed over k in the same order whatever tile or group
// it lies in.
#include "api.h"
#include "common.cuh"
#include "mma_sync.cuh"
#include "gemm_internal.h"

namespace dlmk {

namespace {

constexpr int BN = 128, BK = 32, STAGES = 3, THREADS = 256;
constexpr int PITCH = BK + 8;      // elements per shared-memory row (80 bytes)

struct MmaParams {
    const __nv_bfloat16* a; int lda; const int32_t* a_rows;
    const __nv_bfloat16* w; int ldw; long long w_expert_stride;
    const int32_t* expert_offsets; int num_experts;
    const float* bias;
    void* out; int ldo;
    int M, N, K;
};

__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    const int bytes = valid ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}

template <int BM, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS) gemm_mma_kernel(MmaParams p) {
    constexpr int WM = BM / 2;                 // rows per warp (2 warps along M)
    constexpr int MT = WM / 16;                // m16 tiles per warp
    constexpr int NTW = 4;                     // n8 tiles per warp (4 warps along N, 32 columns each)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [STAGES][BM][PITCH]
    __nv_bfloat16* Bs = As + STAGES * BM * PITCH;                              // [STAGES][BN][PITCH]
    __shared__ int s_tile[3];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;
    const int n0 = blockIdx.x * BN;
    int row_begin, row_end;
    const __nv_bfloat16* w = p.w;
    if (p.expert_offsets != nullptr) {
        if (tid == 0) {
            int acc = 0;
            s_tile[0] = -1;
            for (int e = 0; e < p.num_experts; ++e) {
                const int r0 = p.expert_offsets[e], r1 = p.expert_offsets[e + 1];
                const int tiles = (r1 - r0 + BM - 1) / BM;
                if ((int)blockIdx.y < acc + tiles) {
                    s_tile[0] = e;
                    s_tile[1] = r0 + ((int)blockIdx.y - acc) * BM;
                    s_tile[2] = r1;
                    break;
                }
                acc += tiles;
            }
        }
        __syncthreads();
        if (s_tile[0] < 0) return;
        row_begin = s_tile[1];
        row_end = min(min(s_tile[2], row_begin + BM), p.M);
        w += (long long)s_tile[0] * p.w_expert_stride;
    } else {
        row_begin = blockIdx.y * BM;
        if (row_begin >= p.M) return;
        row_end = min(p.M, row_begin + BM);
    }

    // copy assignment: a row of 32 elements is 4 chunks of 16 bytes; 256 threads cover 64 rows a pass
    const int c_row = tid >> 2, c_chunk = (tid & 3) * 8;
    const __nv_bfloat16* a_src[BM / 64];
    bool a_ok[BM / 64];
#pragma unroll
    for (int i = 0; i < BM / 64; ++i) {
        const int r = row_begin + c_row + i * 64;
        a_ok[i] = r < row_end;
        const int src = a_ok[i] ? (p.a_rows ? p.a_rows[r] : r) : 0;
        a_src[i] = p.a + (long long)src * p.lda + c_chunk;
    }
    const __nv_bfloat16* b_src[2];
    bool b_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int n = n0 + c_row + i * 64;
        b_ok[i] = n < p.N;
        b_src[i] = w + (long long)(b_ok[i] ? n : 0) * p.ldw + c_chunk;
    }
    const int k_tiles = (p.K + BK - 1) / BK;
    auto load_stage = [&](int stage, int kt) {
        const int k = kt * BK + c_chunk;
        const bool k_ok = k < p.K;                  // K is a multiple of 8: a chunk is all in or all out
#pragma unroll
        for (int i = 0; i < BM / 64; ++i)
            cp_async16_zfill(As + ((size_t)stage * BM + c_row + i * 64) * PITCH + c_chunk, a_src[i] + kt * BK,
                             a_ok[i] && k_ok);
#pragma unroll
        for (int i = 0; i < 2; ++i)
            cp_async16_zfill(Bs + ((size_t)stage * BN + c_row + i * 64) * PITCH + c_chunk, b_src[i] + kt * BK,
                             b_ok[i] && k_ok);
    };

    float acc[MT][NTW][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NTW; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < k_tiles) load_stage(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // ldmatrix addressing: lane l supplies the address of row (l % 16) at column 8 * (l / 16) of a 16 x 16 tile
    const int lm_row = lane & 15, lm_col = (lane >> 4) * 8;
    for (int kt = 0; kt < k_tiles; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();
        const int nxt = kt + STAGES - 1;
        if (nxt < k_tiles) load_stage(nxt % STAGES, nxt);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* at = As + (size_t)(kt % STAGES) * BM * PITCH + (wm * WM) * PITCH;
        const __nv_bfloat16* bt = Bs + (size_t)(kt % STAGES) * BN * PITCH + (wn * 32) * PITCH;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            uint32_t af[MT][4], bf[2][4];
#pragma unroll
            for (int i = 0; i < MT; ++i) ldsm_x4(af[i], at + (i * 16 + lm_row) * PITCH + kk + lm_col);
            // W rows are the product's columns: a 16 (n) x 16 (k) tile gives the B fragments of two n8 tiles:
            // registers {0, 2} = (n 0-7, k 0-7 | k 8-15), {1, 3} = (n 8-15, k 0-7 | k 8-15)
#pragma unroll
            for (int j = 0; j < 2; ++j) ldsm_x4(bf[j], bt + (j * 16 + lm_row) * PITCH + kk + lm_col);
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    mma16816(acc[i][2 * j], af[i], bf[j][0], bf[j][2]);
                    mma16816(acc[i][2 * j + 1], af[i], bf[j][1], bf[j][3]);
                }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // epilogue: thread (g = lane / 4, t = lane % 4) holds rows g, g + 8 and columns 2t, 2t + 1 of each 16 x 8 tile
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = row_begin + wm * WM + i * 16 + g + half * 8;
            if (row >= row_end) continue;
#pragma unroll
            for (int j = 0; j < NTW; ++j) {
                const int col = n0 + wn * 32 + j * 8 + 2 * t;
                const float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
                if (EPI == EPI_SWIGLU) {
                    if (col + 1 < p.N)
                        static_cast<TOut*>(p.out)[(long long)row * p.ldo + (col >> 1)] = from_f32<TOut>(silu_f(v0) * v1);
                } else if (EPI == EPI_ADD) {
                    float* o = static_cast<float*>(p.out) + (long long)row * p.ldo;
                    if (col < p.N) o[col] += v0;
                    if (col + 1 < p.N) o[col + 1] += v1;
                } else {
                    TOut* o = static_cast<TOut*>(p.out) + (long long)row * p.ldo;
                    if (col < p.N) o[col] = from_f32<TOut>(v0 + (p.bias ? p.bias[col] : 0.f));
                    if (col + 1 < p.N) o[col + 1] = from_f32<TOut>(v1 + (p.bias ? p.bias[col + 1] : 0.f));
                }
            }
        }
}

template <int BM, typename TOut>
void launch_bm(const MmaParams& p, int epilogue, dim3 grid, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * (BM + BN) * PITCH * sizeof(__nv_bfloat16);
#define DLM_MMA(EPI, TO)                                                                         \
    {                                                                                            \
        auto kern = gemm_mma_kernel<BM, EPI, TO>;                                                \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        kern<<<grid, THREADS, smem, stream>>>(p);                                                \
    }
    switch (epilogue) {
        case EPI_STORE: DLM_MMA(EPI_STORE, TOut) break;
        case EPI_ADD: DLM_MMA(EPI_ADD, float) break;
        default: DLM_MMA(EPI_SWIGLU, TOut) break;
    }
#undef DLM_MMA
}

}  // namespace

void gemm_mma(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
              const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
              int K, int out_dtype, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return;
    DLM_CHECK(epilogue != EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N");
    DLM_CHECK(epilogue != EPI_ADD || out_dtype == F32, "gemm: the accumulate epilogue needs a float32 output");
    DLM_CHECK(bias == nullptr || epilogue == EPI_STORE, "gemm: a bias goes with the store epilogue only");
    MmaParams p{static_cast<const __nv_bfloat16*>(a), lda, a_rows, static_cast<const __nv_bfloat16*>(w), ldw,
                w_expert_stride, expert_offsets, num_experts, bias, out, ldo, M, N, K};
    // grouped products have ragged groups: smaller row tiles waste less
    const bool small_tile = expert_offsets != nullptr && (long long)M < 192LL * num_experts;
    const int bm = small_tile ? 64 : 128;
    int m_tiles = (M + bm - 1) / bm;
    if (expert_offsets != nullptr) m_tiles += num_experts;
    DLM_CHECK(m_tiles <= 65535, "gemm: too many row tiles for one launch");
    dim3 grid((N + BN - 1) / BN, m_tiles);
    const bool f32 = out_dtype == F32;
    if (bm == 64) { if (f32) launch_bm<64, float>(p, epilogue, grid, stream); else launch_bm<64, __nv_bfloat16>(p, epilogue, grid, stream); }
    else { if (f32) launch_bm<128, float>(p, epilogue, grid, stream); else launch_bm<128, __nv_bfloat16>(p, epilogue, grid, stream); }
    check_launch("gemm_mma");
}

}  // namespace dlmk
