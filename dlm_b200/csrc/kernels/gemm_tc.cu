// C = A · W^T on the fifth-generation tensor cores (tcgen05), bfloat16 in, 32-bit accumulation in
// tensor memory, with the operands' roles swapped: 128 rows of W are the MMA's M, the rows of A (tokens)
// its N.  N may be any multiple of 16 up to 256, so an expert that got 137 tokens costs one MMA tile of
// N = 144 instead of two 128-row tiles, and a decode batch of 64 tokens fits as it is.
//
// A tile of C^T is (128 weight rows) x (up to 256 tokens).  Ten warps, three roles:
//   warp 8 (one lane)   the producer: for every 64-wide slice of K it waits for a free stage and asks the
//                       TMA unit for the W tile (128 x 64) and the A tile (tokens x 64); the copies land in
//                       shared memory in the 128-byte-swizzled, K-major layout the MMA reads, and complete
//                       a transaction barrier;
//   warp 9 (one lane)   the MMA issuer: waits for a stage, issues four tcgen05.mma (K = 16 each) that
//                       accumulate into 128 lanes x N columns of tensor memory, and commits: the commit
//                       frees the stage when the MMAs have read it and, after the last slice, tells the
//                       epilogue that the accumulator is complete.  Warp 9 also allocates and frees the
//                       tensor memory;
//   warps 0-7           the epilogue: each warp reads 32 lanes of the accumulator with tcgen05.ld.
//                       A thread holds one output column (weight row) for 32 tokens at a time, so for each
//                       token the warp stores 32 consecutive columns: coalesced without staging.  Bias,
//                       accumulation into the residual, or SwiGLU (gate and up are neighbouring lanes).
// The kernel is persistent: a block walks a strided list of tiles, and two accumulators alternate in tensor
// memory, so that the epilogue of one tile overlaps the MMAs of the next.
//
// Dense, or grouped by expert (rows of one expert are consecutive).  Rows of A must be contiguous in
// memory (no gather): the caller gathers first.
//
// Every wait on a barrier is bounded.  If a bound is reached the block sets the error flag, stops
// issuing work, gives in-flight copies time to land, frees its tensor memory and returns; the host
// reads the flag after the step (NativeOps.check_errors).
#include <cuda.h>

#include <cstdlib>

#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"
#include "gemm_tc_common.cuh"
#include "tcgen05.cuh"

namespace dlmk {

namespace {

using namespace tc5;

constexpr int BM = 128, BK = 64;
constexpr int EPI_WARPS = 8, PRODUCER_WARP = 8, MMA_WARP = 9, THREADS = 320;

// Persistent: a block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Two accumulators in tensor memory
// alternate, so that the epilogue of one tile runs while the MMAs of the next are issued.
template <int STAGES, int G, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ TokenMaps maps_a, TcParams p, int nx,
               int total_tiles) {
    constexpr uint32_t W_BYTES = BM * BK * 2, A_MAX_BYTES = TT * BK * 2, STAGE_BYTES = G * W_BYTES + A_MAX_BYTES;
    // M = 128, bfloat16 x bfloat16 -> float32, both operands K-major; N is filled in per tile
    constexpr uint32_t IDESC0 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    // the block's first tiles, looked up once (the search through the experts' offsets is too slow to stand at
    // the head of every tile in every role)
    constexpr int TABLE = 64;
    __shared__ TileInfo s_tiles[TABLE];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* tiles = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EPI_WARPS * 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < TABLE; i += THREADS) {
        const long long tile = (long long)blockIdx.x + (long long)i * gridDim.x;
        if (tile < total_tiles) s_tiles[i] = tile_info(p, (int)(tile / nx));
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)(2 * TT)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_flag = &s_abort;
    const int k_tiles = (p.K + BK - 1) / BK;
    auto info_of = [&](int tile) -> TileInfo {
        const int i = (tile - (int)blockIdx.x) / (int)gridDim.x;
        return i < TABLE ? s_tiles[i] : tile_info(p, tile / nx);
    };
    // the set-up above may run while the kernel before this one ends (see dep_wait in common.cuh)
    dep_wait();
    dep_launch_next();

    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            uint32_t it = 0;                                  // slices issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const TileInfo ti = info_of(tile);
                if (ti.expert < 0) continue;
                const int n0 = (tile % nx) * (G * BM);
                const int n_w = min(G, (p.N - n0 + BM - 1) / BM);     // weight tiles of this item
                const int n_tok = ti.row_end - ti.row_begin;
                const int bi = (n_tok + 15) / 16 - 1;         // box of 16 * (bi + 1) rows
                const int box = 16 * (bi + 1);
                const CUtensorMap* map_a = &maps_a.m[bi];
                const uint32_t tx = (uint32_t)n_w * W_BYTES + (uint32_t)box * BK * 2;
                const int w_row = (p.expert_offsets != nullptr ? ti.expert * p.N : 0) + n0;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    unsigned char* w_dst = tiles + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], tx);
                    for (int t = 0; t < n_w; ++t)
                        tma_load_2d(w_dst + t * W_BYTES, &map_w, kt * BK, w_row + t * BM, &full_bar[s]);
                    tma_load_2d(w_dst + G * W_BYTES, map_a, kt * BK, ti.row_begin, &full_bar[s]);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            uint32_t it = 0, acc_i = 0;
            bool ok = true;
            // descriptor of stage 0's weight tile; a stage, a weight tile or the token tile further on is a constant
            // added to the address field (in units of 16 bytes): the issuing thread has little else to do per stage
            const uint64_t dw0 = umma_desc(smem_u32(tiles));
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const TileInfo ti = info_of(tile);
                if (ti.expert < 0) continue;
                const int n_mma = max(16, (ti.row_end - ti.row_begin + 15) & ~15);
                const uint32_t idesc = IDESC0 | ((uint32_t)(n_mma >> 3) << 17);
                const int n_w = min(G, (p.N - (tile % nx) * (G * BM) + BM - 1) / BM);
                // G = 1: two accumulators alternate; G = 2: the item's two accumulators fill the tensor memory
                const uint32_t b = G == 1 ? (acc_i & 1) : 0, u = G == 1 ? (acc_i >> 1) : acc_i;
                // the epilogue must have drained this accumulator's previous tile
                if (u >= 1 && !mbar_wait(&acc_empty[b], (u & 1) ^ 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + b * TT;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ds = dw0 + (uint64_t)(s * (STAGE_BYTES >> 4));
                    const uint64_t da = ds + (uint64_t)(G * (W_BYTES >> 4));
                    for (int t = 0; t < n_w; ++t) {
                        const uint64_t dw = ds + (uint64_t)(t * (W_BYTES >> 4));
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)      // 16 elements of K = 32 bytes = 2 address units
                            umma_bf16(d_tmem + t * TT, dw + 2 * k, da + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);            // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[b]);                 // the accumulator is complete once all MMAs are done
                ++acc_i;
            }
        }
    } else {
        // epilogue, eight warps: warp w reads tensor-memory lanes 32q .. 32q + 31 (q = w % 4) = output columns
        // n0 + 32q + lane; the accumulator's columns are the tile's tokens, and the two warps of a quadrant
        // take alternate chunks of 32 tokens.  A thread gets one output column for 32 tokens; the chunk is
        // turned through the warp's own staging area so that it leaves as 16-byte stores along the rows.
        const int q = warp & 3, hsel = warp >> 2;
        float* st = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES) + warp * (32 * 33);
        const bool vec_ok = (p.ldo % 8 == 0) && (p.N % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        uint32_t acc_i = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            TileInfo ti;
            if (lane == 0) ti = info_of(tile);
            ti.expert = __shfl_sync(0xffffffffu, ti.expert, 0);
            ti.row_begin = __shfl_sync(0xffffffffu, ti.row_begin, 0);
            ti.row_end = __shfl_sync(0xffffffffu, ti.row_end, 0);
            if (ti.expert < 0) continue;
            const int n_first = (tile % nx) * (G * BM);
            const int n_w = min(G, (p.N - n_first + BM - 1) / BM);
            const int row_begin = ti.row_begin, row_end = ti.row_end;
            const int n_mma = max(16, (row_end - row_begin + 15) & ~15);
            const uint32_t b = G == 1 ? (acc_i & 1) : 0, u = G == 1 ? (acc_i >> 1) : acc_i;
            if (!mbar_wait(&acc_full[b], u & 1, abort_flag)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int t = 0; t < n_w; ++t) {
                const uint32_t d_tmem = tmem_base + (b + t) * TT + ((uint32_t)(q * 32) << 16);
                const int colw = n_first + t * BM + q * 32;       // first output column of this warp
                epilogue_tile<EPI, TOut>(p, st, d_tmem, colw, n_mma, row_begin, row_end, hsel, lane, vec_ok);
            }
            // this accumulator may be written again
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&acc_empty[b]);
            ++acc_i;
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
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * TT))
                     : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
template <int G, int EPI, typename TOut>
void launch(const CUtensorMap& mw, const TokenMaps& ma, const TcParams& p, int nx, int total_tiles,
            cudaStream_t stream) {
    constexpr int STAGES = G == 1 ? 4 : 3;
    const size_t smem = (size_t)STAGES * (G * BM * BK * 2 + TT * BK * 2) + EPI_WARPS * 32 * 33 * sizeof(float) + 1024;
    auto kern = gemm_tc_kernel<STAGES, G, EPI, TOut>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int grid = total_tiles < sm_count() ? total_tiles : sm_count();
    launch_dep(kern, grid, THREADS, smem, stream, mw, ma, p, nx, total_tiles);
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
    if (N > BM && gemm_tc_pair_enabled() &&
        gemm_tc_pair(a, lda, w, ldw, expert_offsets, num_experts, bias, out, ldo, M, N, K, out_dtype, epilogue, stream))
        return true;
    CUtensorMap mw;
    TokenMaps ma;
    const long long w_rows = expert_offsets ? (long long)num_experts * N : N;
    // (weights: a miss fetches 256 bytes of the row, i.e. the next slice's box too)
    if (!make_map(&mw, w, w_rows, K, ldw, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return false;
    for (int i = 0; i < 16; ++i)
        if (!make_map(&ma.m[i], a, M, K, lda, 16 * (i + 1))) return false;
    TcParams p{expert_offsets, num_experts, bias, out, ldo, M, N, K, error_flag_ptr()};
    int t_tiles = (M + TT - 1) / TT;
    if (expert_offsets != nullptr) t_tiles += num_experts;
    // Grouped: an expert's tokens are few and its weights are read once, so the token tile, which comes from L2
    // again for every weight tile, is most of what a multiprocessor takes in.  With the plain store epilogue two
    // weight tiles (256 rows) share each token stage and fill the tensor memory with their two accumulators
    // (measured: 109 -> 95 us for the experts' down projection of a 2,048-token step).  The SwiGLU epilogue is
    // too long to run without the next tile's MMAs beside it (191 -> 239 us), so it keeps one weight tile and
    // two alternating accumulators, as the dense products do.
    const int g = (expert_offsets != nullptr && epilogue == EPI_STORE) ? 2 : 1;
    const int nx = (N + g * BM - 1) / (g * BM);
    DLM_CHECK((long long)nx * t_tiles < (1LL << 30), "gemm: too many tiles for one launch");
    const int total_tiles = nx * t_tiles;
    const bool f32 = out_dtype == F32;
#define DLM_TC(G)                                                                                           \
    switch (epilogue) {                                                                                     \
        case EPI_STORE: if (f32) launch<G, EPI_STORE, float>(mw, ma, p, nx, total_tiles, stream);           \
                        else launch<G, EPI_STORE, __nv_bfloat16>(mw, ma, p, nx, total_tiles, stream); break; \
        case EPI_ADD: launch<G, EPI_ADD, float>(mw, ma, p, nx, total_tiles, stream); break;                 \
        default: if (f32) launch<G, EPI_SWIGLU, float>(mw, ma, p, nx, total_tiles, stream);                 \
                 else launch<G, EPI_SWIGLU, __nv_bfloat16>(mw, ma, p, nx, total_tiles, stream); break;      \
    }
    if (g == 2) { DLM_TC(2) } else { DLM_TC(1) }
#undef DLM_TC
    check_launch("gemm_tc");
    return true;
}

}  // namespace dlmk
