// C = A · W^T for few rows of A (decode steps, and experts that got a handful of tokens):
// a weight-streaming kernel.  Every weight is read from memory exactly once, 16 bytes a
// lane, and meets all rows of A in tensor-core MMAs with the roles swapped: 16 rows of W
// are the MMA's M, up to 8 rows of A its N (mma.sync m16n8k16, bfloat16 in, 32-bit
// accumulation).
//
// K is walked in blocks of 32.  Lane (g = lane / 4, t = lane % 4) loads the 8 consecutive
// elements 8t..8t+7 of rows g and g + 8 of the weight tile and of row g of A; the two MMAs of
// a block take elements {0,1 | 2,3} and {4,5 | 6,7} of those as their k-slices.  A sum does
// not care in which order its terms are listed, and A and W list them alike.
//
// A block of 8 warps covers R weight tiles x S slices of K (R * S = 8); the S partial sums of
// a tile are added in a fixed order through shared memory, so a result does not depend on
// what else was in the batch.
//
// The kernel may start while the kernel before it ends (see dep_wait in common.cuh): a dense
// product asks its weights into the L2 cache before it waits for its activations.
#include <mma.h>

#include "api.h"
#include "common.cuh"
#include "mma_sync.cuh"
#include "gemm_internal.h"

namespace dlmk {

namespace {

constexpr int WARPS = 8;
constexpr int KB = 32;          // k per block
constexpr int UNROLL = 8;

struct SmallParams {
    const __nv_bfloat16* a; int lda; const int32_t* a_rows;
    const __nv_bfloat16* w; int ldw; long long w_expert_stride;
    const int32_t* expert_offsets; int num_experts;
    const float* bias;
    void* out; int ldo;
    int M, N, K;
    int S;          // slices of K per weight tile (1, 2, 4 or 8)
    int k_chunk;    // k per slice, a multiple of KB
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}


template <int NT, int EPI, typename TOut>
__global__ void __launch_bounds__(WARPS * 32) gemm_smallm_kernel(SmallParams p) {
    constexpr int MP = 8 * NT;                       // rows of A per pass
    __shared__ float red[WARPS][16][MP + 1];
    __shared__ int s_expert;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int S = p.S, R = WARPS / S;
    const int r = warp / S, s = warp % S;
    const int tile = blockIdx.x * R + r;
    const int n_base = tile * 16;
    const bool tile_ok = n_base < p.N;
    const int k_begin = s * p.k_chunk;
    const int k_end = min(p.K, k_begin + p.k_chunk);
    // weight rows of this lane (clamped to a valid row; rows beyond N are never stored)
    const int wr0 = min(n_base + g, p.N - 1), wr1 = min(n_base + g + 8, p.N - 1);

    int row0 = 0, m_count = p.M;
    const __nv_bfloat16* w = p.w;
    if (p.expert_offsets == nullptr) {
        // no kernel writes weights: this warp's share of them is asked into the L2 cache while the
        // kernel before this one ends (one request per 128 bytes, all inside the matrix)
        if (tile_ok) {
            const __nv_bfloat16* r0 = w + (long long)wr0 * p.ldw;
            const __nv_bfloat16* r1 = w + (long long)wr1 * p.ldw;
            for (int k = k_begin + 64 * t; k < k_end; k += 256) {
                prefetch_l2(r0 + k);
                prefetch_l2(r1 + k);
            }
        }
        dep_wait();
        dep_launch_next();
    } else {
        dep_wait();
        dep_launch_next();
        // blockIdx.y counts the experts that have rows: the first warp finds the expert by a scan of the offsets
        if (warp == 0) {
            int found = -1, seen = 0;
            for (int base = 0; base < p.num_experts && found < 0; base += 32) {
                const int e = base + lane;
                const bool has = e < p.num_experts && p.expert_offsets[e + 1] > p.expert_offsets[e];
                const unsigned mask = __ballot_sync(0xffffffffu, has);
                const int c = __popc(mask);
                if ((int)blockIdx.y < seen + c) found = base + (int)__fns(mask, 0, (int)blockIdx.y - seen + 1);
                seen += c;
            }
            if (lane == 0) s_expert = found;
        }
        __syncthreads();
        const int e = s_expert;
        if (e < 0) return;
        row0 = p.expert_offsets[e];
        m_count = p.expert_offsets[e + 1] - row0;
        if (m_count <= 0) return;
        if (row0 + m_count > p.M) m_count = p.M - row0;
        w += (long long)e * p.w_expert_stride;
    }
    const __nv_bfloat16* w0 = w + (long long)wr0 * p.ldw + 8 * t;
    const __nv_bfloat16* w1 = w + (long long)wr1 * p.ldw + 8 * t;

    for (int m0 = 0; m0 < m_count; m0 += MP) {
        // rows of A this lane supplies: one per 8-row tile
        const __nv_bfloat16* arow[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = m0 + nt * 8 + g;
            if (m < m_count) {
                const int src = p.a_rows ? p.a_rows[row0 + m] : row0 + m;
                arow[nt] = p.a + (long long)src * p.lda + 8 * t;
            } else {
                arow[nt] = nullptr;
            }
        }
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

        if (tile_ok) {
            for (int k0 = k_begin; k0 < k_end; k0 += KB * UNROLL) {
                uint4 wa[UNROLL][2];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int k = k0 + u * KB;
                    if (k + 8 * t < k_end) {          // K is a multiple of 8: a lane's 8 elements are all in or all out
                        wa[u][0] = ldg_stream(w0 + k);
                        wa[u][1] = ldg_stream(w1 + k);
                    } else {
                        wa[u][0] = make_uint4(0, 0, 0, 0);
                        wa[u][1] = make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int k = k0 + u * KB;
                    const bool in = k + 8 * t < k_end;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        uint4 xb = make_uint4(0, 0, 0, 0);
                        if (in && arow[nt] != nullptr) xb = __ldg(reinterpret_cast<const uint4*>(arow[nt] + k));
                        mma_bf16(acc[nt], wa[u][0].x, wa[u][1].x, wa[u][0].y, wa[u][1].y, xb.x, xb.y);
                        mma_bf16(acc[nt], wa[u][0].z, wa[u][1].z, wa[u][0].w, wa[u][1].w, xb.z, xb.w);
                    }
                }
            }
        }
        // partial sums to shared memory: red[warp][weight row][row of A]
        __syncthreads();                              // the previous pass's readers are done
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[warp][g][nt * 8 + 2 * t] = acc[nt][0];
            red[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
            red[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
            red[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
        }
        __syncthreads();

        const int m_here = min(MP, m_count - m0);
        if (EPI == EPI_SWIGLU) {
            // element = (tile r', row of A, pair of weight rows)
            for (int i = tid; i < R * MP * 8; i += WARPS * 32) {
                const int pr = i & 7, m = (i >> 3) % MP, rr = i / (8 * MP);
                const int n = (blockIdx.x * R + rr) * 16 + 2 * pr;
                if (m >= m_here || n + 1 >= p.N) continue;
                float gate = 0.f, up = 0.f;
                for (int ss = 0; ss < S; ++ss) {
                    gate += red[rr * S + ss][2 * pr][m];
                    up += red[rr * S + ss][2 * pr + 1][m];
                }
                static_cast<TOut*>(p.out)[(long long)(row0 + m0 + m) * p.ldo + (n >> 1)] =
                    from_f32<TOut>(silu_f(gate) * up);
            }
        } else {
            for (int i = tid; i < R * MP * 16; i += WARPS * 32) {
                const int row = i & 15, m = (i >> 4) % MP, rr = i / (16 * MP);
                const int n = (blockIdx.x * R + rr) * 16 + row;
                if (m >= m_here || n >= p.N) continue;
                float v = 0.f;
                for (int ss = 0; ss < S; ++ss) v += red[rr * S + ss][row][m];
                const long long o = (long long)(row0 + m0 + m) * p.ldo + n;
                if (EPI == EPI_ADD) static_cast<float*>(p.out)[o] += v;
                else static_cast<TOut*>(p.out)[o] = from_f32<TOut>(v + (p.bias ? p.bias[n] : 0.f));
            }
        }
    }
}

template <int NT, typename TOut>
void launch_nt(const SmallParams& p, int epilogue, dim3 grid, cudaStream_t stream) {
    switch (epilogue) {
        case EPI_STORE: launch_dep(gemm_smallm_kernel<NT, EPI_STORE, TOut>, grid, WARPS * 32, 0, stream, p); break;
        case EPI_ADD: launch_dep(gemm_smallm_kernel<NT, EPI_ADD, float>, grid, WARPS * 32, 0, stream, p); break;
        default: launch_dep(gemm_smallm_kernel<NT, EPI_SWIGLU, TOut>, grid, WARPS * 32, 0, stream, p); break;
    }
}

}  // namespace

bool gemm_smallm_ok(const void* a, int lda, const void* w, int ldw, long long w_expert_stride, int M, int N, int K,
                    int in_dtype) {
    return in_dtype == BF16 && M > 0 && N > 0 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
           w_expert_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(w) & 15) == 0;
}

void gemm_smallm(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
                 const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
                 int K, int out_dtype, int epilogue, int rows_per_pass, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return;
    DLM_CHECK(epilogue != EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N");
    DLM_CHECK(epilogue != EPI_ADD || out_dtype == F32, "gemm: the accumulate epilogue needs a float32 output");
    SmallParams p;
    p.a = static_cast<const __nv_bfloat16*>(a); p.lda = lda; p.a_rows = a_rows;
    p.w = static_cast<const __nv_bfloat16*>(w); p.ldw = ldw; p.w_expert_stride = w_expert_stride;
    p.expert_offsets = expert_offsets; p.num_experts = num_experts; p.bias = bias; p.out = out; p.ldo = ldo; p.M = M; p.N = N; p.K = K;
    const int tiles = (N + 15) / 16;
    // no more experts have rows than there are rows
    const int groups = expert_offsets ? (num_experts < M ? num_experts : M) : 1;
    // slices of K: enough blocks to fill the machine, but a slice keeps at least 128 elements
    int S = 8;
    while (S > 1 && ((long long)tiles * groups * S / WARPS > 4096 || K / S < 128)) S >>= 1;
    p.S = S;
    p.k_chunk = ((K + S - 1) / S + KB - 1) / KB * KB;
    const int R = WARPS / S;
    dim3 grid((tiles + R - 1) / R, groups);
    const bool f32 = out_dtype == F32;
    const int nt = rows_per_pass <= 8 ? 1 : (rows_per_pass <= 16 ? 2 : 4);
    if (nt == 1) { if (f32) launch_nt<1, float>(p, epilogue, grid, stream); else launch_nt<1, __nv_bfloat16>(p, epilogue, grid, stream); }
    else if (nt == 2) { if (f32) launch_nt<2, float>(p, epilogue, grid, stream); else launch_nt<2, __nv_bfloat16>(p, epilogue, grid, stream); }
    else { if (f32) launch_nt<4, float>(p, epilogue, grid, stream); else launch_nt<4, __nv_bfloat16>(p, epilogue, grid, stream); }
    check_launch("gemm_smallm");
}

}  // namespace dlmk
