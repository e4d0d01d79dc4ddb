// C = A · W^T for many rows of A on the fifth-generation tensor cores (tcgen05), bfloat16 in,
// 32-bit accumulation in tensor memory.
//
// One block computes one 128 x BN tile of C.  Six warps, three roles:
//   warp 4 (one lane)   the producer: for every 64-wide slice of K it waits for a free stage and asks the
//                       TMA unit for the A tile (128 x 64) and the W tile (BN x 64); the copies land in
//                       shared memory in the 128-byte-swizzled, K-major layout the MMA reads, and complete
//                       a transaction barrier;
//   warp 5 (one lane)   the MMA issuer: waits for a stage, issues four tcgen05.mma (K = 16 each) that
//                       accumulate into the tile's 128 lanes x BN columns of tensor memory, and commits:
//                       the commit frees the stage when the MMAs have read it, and, after the last
//                       slice, tells the epilogue that the accumulator is complete.  Warp 5 also
//                       allocates and frees the tensor memory;
//   warps 0-3           the epilogue: each warp reads its 32 lanes of the accumulator with tcgen05.ld
//                       (one row of the tile per thread), applies the epilogue (bias / accumulate into
//                       the residual / SwiGLU of neighbouring columns) and stores.
//
// Dense, or grouped by expert (rows of one expert are consecutive; the tile list is walked as in the
// other GEMM kernels).  Rows of A must be contiguous in memory (no gather): the caller gathers first.
//
// Every wait on a barrier is bounded.  If a bound is reached the block sets the error flag, stops
// issuing work, gives in-flight copies time to land, frees its tensor memory and returns; the host
// reads the flag after the step (NativeOps.check_errors).
#include <cuda.h>

#include <cstdlib>

#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"

namespace dlmk {

namespace {

constexpr int BM = 128, BK = 64, THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;       // try_wait calls before a wait gives up

struct TcParams {
    const int32_t* expert_offsets; int num_experts;
    const float* bias;
    void* out; int ldo;
    int M, N, K;
    int* err;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait.  Returns false when it gave up (or another role already had): the caller stops.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset: next group of 8 rows
    d |= (uint64_t)1 << 46;                              // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BN, int STAGES, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, TcParams p) {
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    // M = 128, N = BN, bfloat16 x bfloat16 -> float32, both operands K-major
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_tile[3];
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* tiles = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

    if (tid == 0) {
        s_abort = 0;
        s_tile[0] = 0;
        if (p.expert_offsets != nullptr) {
            int acc = 0;
            s_tile[0] = -1;
            for (int e = 0; e < p.num_experts; ++e) {
                const int r0 = p.expert_offsets[e], r1 = p.expert_offsets[e + 1];
                const int tiles_e = (r1 - r0 + BM - 1) / BM;
                if ((int)blockIdx.y < acc + tiles_e) {
                    s_tile[0] = e;
                    s_tile[1] = r0 + ((int)blockIdx.y - acc) * BM;
                    s_tile[2] = r1;
                    break;
                }
                acc += tiles_e;
            }
        } else {
            s_tile[1] = blockIdx.y * BM;
            s_tile[2] = p.M;
        }
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int expert = s_tile[0];
    const int row_begin = s_tile[1];
    const int row_end = min(min(s_tile[2], row_begin + BM), p.M);
    if (expert < 0 || row_begin >= row_end) return;           // uniform over the block; nothing allocated yet

    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_flag = &s_abort;

    const int n0 = blockIdx.x * BN;
    const int k_tiles = (p.K + BK - 1) / BK;

    if (warp == 4) {
        if (lane == 0) {
            const int w_row = (p.expert_offsets != nullptr ? expert * p.N : 0) + n0;
            for (int kt = 0; kt < k_tiles; ++kt) {
                const int s = kt % STAGES;
                if (kt >= STAGES && !mbar_wait(&empty_bar[s], ((kt / STAGES) & 1) ^ 1, abort_flag)) break;
                unsigned char* a_dst = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, kt * BK, row_begin, &full_bar[s]);
                tma_load_2d(a_dst + A_BYTES, &map_w, kt * BK, w_row, &full_bar[s]);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < k_tiles && ok; ++kt) {
                const int s = kt % STAGES;
                ok = mbar_wait(&full_bar[s], (kt / STAGES) & 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)          // 16 elements of K = 32 bytes = 2 address units
                    umma_bf16(tmem_base, da + 2 * k, db + 2 * k, IDESC, (kt > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);                // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(&acc_bar);                 // the accumulator is complete once all MMAs are done
        }
    } else {
        // epilogue: thread = one row of the tile; warp w may read tensor-memory lanes 32w .. 32w + 31
        if (mbar_wait(&acc_bar, 0, abort_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = row_begin + warp * 32 + lane;
            const bool row_ok = row < row_end;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
                if (!row_ok) continue;
                const int col0 = n0 + c0;
                if (EPI == EPI_SWIGLU) {
                    TOut* o = static_cast<TOut*>(p.out) + (long long)row * p.ldo + (col0 >> 1);
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        if (col0 + j + 1 < p.N)
                            o[j >> 1] = from_f32<TOut>(silu_f(__uint_as_float(v[j])) * __uint_as_float(v[j + 1]));
                } else if (EPI == EPI_ADD) {
                    float* o = static_cast<float*>(p.out) + (long long)row * p.ldo + col0;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.N) o[j] += __uint_as_float(v[j]);
                } else {
                    TOut* o = static_cast<TOut*>(p.out) + (long long)row * p.ldo + col0;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.N)
                            o[j] = from_f32<TOut>(__uint_as_float(v[j]) + (p.bias ? p.bias[col0 + j] : 0.f));
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        // a wait ran out: report, and give copies that may still be in flight time to land before the
        // shared memory they target goes away
        if (tid == 0) *p.err = 5;
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN)
                     : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// rows x K bfloat16 matrix with `ld` elements between rows; boxes of box_rows x 64 elements, 128-byte swizzle,
// elements outside the matrix read as zero
bool make_map(CUtensorMap* map, const void* base, long long rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI, typename TOut>
void launch(const CUtensorMap& ma, const CUtensorMap& mw, const TcParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int BN = 128, STAGES = 5;
    const size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
    auto kern = gemm_tc_kernel<BN, STAGES, EPI, TOut>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, THREADS, smem, stream>>>(ma, mw, p);
}

}  // namespace

bool gemm_tc_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* off = std::getenv("DLM_B200_NO_TCGEN05");
        state = (off != nullptr && off[0] == '1') ? 0 : (encode_tiled() != nullptr ? 1 : 0);
    }
    return state == 1;
}

bool gemm_tc_ok(const void* a, int lda, const void* w, int ldw, long long w_expert_stride, int M, int N, int K,
                int in_dtype) {
    // TMA: 16-byte aligned bases and row strides; the grouped form addresses expert e's rows at e * N
    return in_dtype == BF16 && M > 0 && N > 0 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (w_expert_stride == 0 || w_expert_stride == (long long)N * ldw);
}

bool gemm_tc(const void* a, int lda, const void* w, int ldw, const int32_t* expert_offsets, int num_experts,
             const float* bias, void* out, int ldo, int M, int N, int K, int out_dtype, int epilogue,
             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return true;
    DLM_CHECK(epilogue != EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N");
    DLM_CHECK(epilogue != EPI_ADD || out_dtype == F32, "gemm: the accumulate epilogue needs a float32 output");
    DLM_CHECK(bias == nullptr || epilogue == EPI_STORE, "gemm: a bias goes with the store epilogue only");
    constexpr int BN = 128;
    CUtensorMap ma, mw;
    const long long w_rows = expert_offsets ? (long long)num_experts * N : N;
    if (!make_map(&ma, a, M, K, lda, BM) || !make_map(&mw, w, w_rows, K, ldw, BN)) return false;
    TcParams p{expert_offsets, num_experts, bias, out, ldo, M, N, K, error_flag_ptr()};
    int m_tiles = (M + BM - 1) / BM;
    if (expert_offsets != nullptr) m_tiles += num_experts;
    DLM_CHECK(m_tiles <= 65535, "gemm: too many row tiles for one launch");
    dim3 grid((N + BN - 1) / BN, m_tiles);
    const bool f32 = out_dtype == F32;
    switch (epilogue) {
        case EPI_STORE: if (f32) launch<EPI_STORE, float>(ma, mw, p, grid, stream); else launch<EPI_STORE, __nv_bfloat16>(ma, mw, p, grid, stream); break;
        case EPI_ADD: launch<EPI_ADD, float>(ma, mw, p, grid, stream); break;
        default: if (f32) launch<EPI_SWIGLU, float>(ma, mw, p, grid, stream); else launch<EPI_SWIGLU, __nv_bfloat16>(ma, mw, p, grid, stream); break;
    }
    check_launch("gemm_tc");
    return true;
}

}  // namespace dlmk
