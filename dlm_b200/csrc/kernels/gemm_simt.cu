// C = A · W^T on the FMA units: the true 32-bit matrix product (no tensor cores, no
// reduced-precision mode), also the fallback of every bfloat16 product.
//
// Every output element is one thread's sequential sum over k = 0..K-1 (fused
// multiply-adds in that order), so a row's result does not depend on which tile,
// batch or expert group it was computed in.
#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"

namespace dlmk {

namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

struct GemmParams {
    const void* a; int lda; const int32_t* a_rows;
    const void* w; int ldw; long long w_expert_stride;
    const int32_t* expert_offsets; int num_experts;
    const float* bias;
    void* out; int ldo;
    int M, N, K;
};

template <typename TIn, typename TOut, int EPI>
__global__ void __launch_bounds__(THREADS) gemm_simt_kernel(GemmParams p) {
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    __shared__ int s_tile[3];

    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * BN;
    int row_begin, row_end;
    const TIn* w = static_cast<const TIn*>(p.w);
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
        row_end = min(s_tile[2], row_begin + BM);
        if (row_end > p.M) row_end = p.M;
        w += (long long)s_tile[0] * p.w_expert_stride;
    } else {
        row_begin = blockIdx.y * BM;
        if (row_begin >= p.M) return;
        row_end = min(p.M, row_begin + BM);
    }

    // load assignment: 4 consecutive k of one row per thread
    const int l_row = tid >> 2, l_k = (tid & 3) * 4;
    const TIn* a_base = static_cast<const TIn*>(p.a);
    long long a_off = -1;
    if (row_begin + l_row < row_end) {
        const int r = row_begin + l_row;
        a_off = (long long)(p.a_rows ? p.a_rows[r] : r) * p.lda;
    }
    const long long w_off = (n0 + l_row < p.N) ? (long long)(n0 + l_row) * p.ldw : -1;

    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + l_k + i;
            As[l_k + i][l_row] = (a_off >= 0 && k < p.K) ? to_f32(a_base[a_off + k]) : 0.f;
            Bs[l_k + i][l_row] = (w_off >= 0 && k < p.K) ? to_f32(w[w_off + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float a[4] = {av.x, av.y, av.z, av.w};
            const float b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row_begin + ty * 4 + i;
        if (row >= row_end) continue;
        if (EPI == EPI_SWIGLU) {
            TOut* o = static_cast<TOut*>(p.out) + (long long)row * p.ldo;
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int col = n0 + tx * 4 + j;
                if (col + 1 < p.N) o[col >> 1] = from_f32<TOut>(silu_f(acc[i][j]) * acc[i][j + 1]);
            }
        } else if (EPI == EPI_ADD) {
            float* o = static_cast<float*>(p.out) + (long long)row * p.ldo;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = n0 + tx * 4 + j;
                if (col < p.N) o[col] += acc[i][j];
            }
        } else {
            TOut* o = static_cast<TOut*>(p.out) + (long long)row * p.ldo;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = n0 + tx * 4 + j;
                if (col < p.N) o[col] = from_f32<TOut>(acc[i][j] + (p.bias ? p.bias[col] : 0.f));
            }
        }
    }
}

template <typename TIn, typename TOut>
void launch(const GemmParams& p, int epilogue, dim3 grid, cudaStream_t stream) {
    switch (epilogue) {
        case EPI_STORE: gemm_simt_kernel<TIn, TOut, EPI_STORE><<<grid, THREADS, 0, stream>>>(p); break;
        case EPI_ADD: gemm_simt_kernel<TIn, float, EPI_ADD><<<grid, THREADS, 0, stream>>>(p); break;
        case EPI_SWIGLU: gemm_simt_kernel<TIn, TOut, EPI_SWIGLU><<<grid, THREADS, 0, stream>>>(p); break;
        default: DLM_CHECK(false, "gemm: unknown epilogue");
    }
}

}  // namespace

void gemm_simt(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
               const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
               int K, int in_dtype, int out_dtype, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return;
    DLM_CHECK(K > 0, "gemm: K must be > 0");
    DLM_CHECK(epilogue != EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N");
    DLM_CHECK(epilogue != EPI_ADD || out_dtype == F32, "gemm: the accumulate epilogue needs a float32 output");
    DLM_CHECK(bias == nullptr || epilogue == EPI_STORE, "gemm: a bias goes with the store epilogue only");
    GemmParams p{a, lda, a_rows, w, ldw, w_expert_stride, expert_offsets, num_experts, bias, out, ldo, M, N, K};
    int m_tiles = (M + BM - 1) / BM;
    if (expert_offsets != nullptr) {
        DLM_CHECK(num_experts > 0, "gemm: grouped product without experts");
        m_tiles += num_experts;   // every group may end in a partial tile
    }
    DLM_CHECK(m_tiles <= 65535, "gemm: too many row tiles for one launch");
    dim3 grid((N + BN - 1) / BN, m_tiles);
    if (in_dtype == F32) {
        if (out_dtype == F32) launch<float, float>(p, epilogue, grid, stream);
        else launch<float, __nv_bfloat16>(p, epilogue, grid, stream);
    } else {
        if (out_dtype == F32) launch<__nv_bfloat16, float>(p, epilogue, grid, stream);
        else launch<__nv_bfloat16, __nv_bfloat16>(p, epilogue, grid, stream);
    }
    check_launch("gemm_simt");
}

}  // namespace dlmk
