// C = A · W^T on pairs of multiprocessors: the tcgen05 product of gemm_tc.cu with MMAs of M = 256 that span
// the two blocks of a cluster (tcgen05.mma.cta_group::2).  A tile of C^T is (256 weight rows) x (up to 256
// tokens): each block of the pair holds 128 of the weight rows and half of the tokens in its shared memory,
// and the 128 x N half of the accumulator that belongs to its weight rows in its tensor memory.  One
// instruction does twice the work of the single-block form and reads, per block, only half of the token
// operand from shared memory, which is what bounds the single-block kernel.
//
// Roles per block (ten warps, as in gemm_tc.cu):
//   warp 8 (one lane)   producer: waits for its own block's free stage and asks the TMA unit for its 128
//                       weight rows and its half of the tokens; both blocks' copies complete the transaction
//                       barrier of the pair's first block (the leader), which expects the bytes of both;
//   warp 9 (one lane)   in the leader only: waits for a stage, issues the four MMAs of the slice and commits
//                       to the stage's "empty" barrier of both blocks (multicast commit); after the last slice
//                       commits to both blocks' "accumulator full" barrier.  Warp 9 of both blocks allocates
//                       and frees the tensor memory (a joint operation of the pair);
//   warps 0-7           epilogue of the block's own half (shared with gemm_tc.cu); when a block has drained
//                       an accumulator, one lane per warp arrives at the leader's "accumulator empty" barrier.
// No load uses multicast.  Every wait on an mbarrier is bounded, as in gemm_tc.cu; the two blocks meet at
// cluster barriers after the set-up and before the tensor memory is freed, which every thread of both
// blocks reaches whatever happened in between.
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
constexpr uint32_t W_BYTES = BM * BK * 2;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of `p` (a location in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_address) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
// TMA load into this block's shared memory whose bytes are counted by a barrier that may lie in the pair's
// other block (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
// arrives at the barrier at this address in both blocks of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

// STAGES stages of 128 weight rows and A_ROWS token rows (half of the tile's most tokens, `tt`); CH: tokens per
// pass of the epilogue.  What bounds the kernel is the bytes in flight: a stage comes back to the producer only
// some 4,000 clocks after its copy was issued (copy, wait for the tensor pipe, MMAs, commit), so the ring holds
// all the shared memory there is, and the epilogue's staging areas are small.
template <int STAGES, int A_ROWS, int CH, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ TokenMaps maps_a, TcParams p, int nx,
                    int total_tiles, int tt) {
    constexpr uint32_t STAGE_BYTES = W_BYTES + A_ROWS * BK * 2;
    // M = 256 over the pair, bfloat16 x bfloat16 -> float32, both operands K-major; N is filled in per tile
    constexpr uint32_t IDESC0 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * BM) >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];     // the leader's are used
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];         // the leader's are used
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    constexpr int TABLE = 64;
    __shared__ TileInfo s_tiles[TABLE];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();
    const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* tiles = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < TABLE; i += THREADS) {
        const long long tile = (long long)pair + (long long)i * n_pairs;
        if (tile < total_tiles) s_tiles[i] = tile_info(p, (int)(tile / nx), tt);
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)(2 * TT)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                 // both blocks' barriers are initialised and their tensor memory is there
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_flag = &s_abort;
    const int k_tiles = (p.K + BK - 1) / BK;
    auto info_of = [&](int tile) -> TileInfo {
        const int i = (tile - pair) / n_pairs;
        return i < TABLE ? s_tiles[i] : tile_info(p, tile / nx, tt);
    };
    dep_wait();
    dep_launch_next();

    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const uint32_t leader_full0 = cluster_addr(&full_bar[0], 0);      // barriers are 8 bytes apart
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
                const TileInfo ti = info_of(tile);
                if (ti.expert < 0) continue;
                const int n0 = (tile % nx) * (2 * BM) + (int)rank * BM;      // this block's weight rows
                const int n_mma = max(16, (ti.row_end - ti.row_begin + 15) & ~15);
                const int half = n_mma >> 1;                               // tokens of each block: a multiple of 8
                const CUtensorMap* map_a = &maps_a.m[half / 8 - 1];
                const uint32_t tx = 2u * W_BYTES + 2u * (uint32_t)half * BK * 2;
                const int w_row = (p.expert_offsets != nullptr ? ti.expert * p.N : 0) + n0;
                const int a_row = ti.row_begin + (int)rank * half;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    unsigned char* dst = tiles + (size_t)s * STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], tx);
                    tma_load_2d_pair(dst, &map_w, kt * BK, w_row, leader_full0 + 8 * s);
                    tma_load_2d_pair(dst + W_BYTES, map_a, kt * BK, a_row, leader_full0 + 8 * s);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // The whole warp walks the loop and one elected lane issues, so that addresses and descriptors are the
        // same in every lane (a loop of "wait, four MMAs, commit" walked by one lane of a divergent branch cost
        // that lane 540 clocks an iteration in a probe kernel, walked by the warp 390).  The next slice's
        // barrier is asked before the MMAs of this one are issued, and the answer read after them.
        if (rank == 0) {
            uint32_t it = 0, acc_i = 0;
            bool ok = true;
            const uint64_t dw0 = umma_desc(smem_u32(tiles));
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
                const TileInfo ti = info_of(tile);
                if (ti.expert < 0) continue;
                const int n_mma = max(16, (ti.row_end - ti.row_begin + 15) & ~15);
                const uint32_t idesc = IDESC0 | ((uint32_t)(n_mma >> 3) << 17);
                const uint32_t b = acc_i & 1, u = acc_i >> 1;
                // both blocks' epilogues must have drained this accumulator's previous tile
                if (u >= 1 && !mbar_wait(&acc_empty[b], (u & 1) ^ 1, abort_flag)) { ok = false; break; }
                const uint32_t d_tmem = tmem_base + b * TT;
                if (!mbar_wait(&full_bar[it % STAGES], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const uint32_t s = it % STAGES;
                    const bool has_next = kt + 1 < k_tiles;
                    const uint32_t s_next = (it + 1) % STAGES, parity_next = ((it + 1) / STAGES) & 1;
                    const bool next_ready = has_next ? mbar_try_wait(&full_bar[s_next], parity_next) : true;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (elect_one()) {
                        const uint64_t dw = dw0 + (uint64_t)(s * (STAGE_BYTES >> 4));
                        const uint64_t da = dw + (uint64_t)(W_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_pair_bf16(d_tmem, dw + 2 * k, da + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                        umma_commit_pair(&empty_bar[s]);
                    }
                    __syncwarp();
                    if (!next_ready && !mbar_wait(&full_bar[s_next], parity_next, abort_flag)) { ok = false; break; }
                }
                if (!ok) break;
                if (elect_one()) umma_commit_pair(&acc_full[b]);
                __syncwarp();
                ++acc_i;
            }
        }
    } else {
        const int q = warp & 3, hsel = warp >> 2;
        float* st = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES) + warp * (CH * 33);
        const bool vec_ok = (p.ldo % 8 == 0) && (p.N % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        const uint32_t leader_empty0 = cluster_addr(&acc_empty[0], 0);
        uint32_t acc_i = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
            TileInfo ti;
            if (lane == 0) ti = info_of(tile);
            ti.expert = __shfl_sync(0xffffffffu, ti.expert, 0);
            ti.row_begin = __shfl_sync(0xffffffffu, ti.row_begin, 0);
            ti.row_end = __shfl_sync(0xffffffffu, ti.row_end, 0);
            if (ti.expert < 0) continue;
            const int n0 = (tile % nx) * (2 * BM) + (int)rank * BM;
            const int n_mma = max(16, (ti.row_end - ti.row_begin + 15) & ~15);
            const uint32_t b = acc_i & 1, u = acc_i >> 1;
            if (!mbar_wait(&acc_full[b], u & 1, abort_flag)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (n0 < p.N) {
                const uint32_t d_tmem = tmem_base + b * TT + ((uint32_t)(q * 32) << 16);
                epilogue_tile<EPI, TOut, CH>(p, st, d_tmem, n0 + q * 32, n_mma, ti.row_begin, ti.row_end, hsel, lane, vec_ok);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_empty0 + 8 * b);
            ++acc_i;
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        if (tid == 0) *p.err = 5;
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();                 // neither block reads or signals the other from here on
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * TT))
                     : "memory");
    }
}

template <typename... P, typename... A>
void launch_pair(void (*kernel)(P...), int grid, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dep_launch_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);   // an error shows in check_launch()
}

template <int STAGES, int A_ROWS, int EPI, typename TOut>
void launch(const CUtensorMap& mw, const TokenMaps& ma, const TcParams& p, int nx, int total_tiles, int tt,
            cudaStream_t stream) {
    constexpr int CH = 16;
    constexpr size_t smem = (size_t)STAGES * (W_BYTES + A_ROWS * BK * 2) + EPI_WARPS * CH * 33 * sizeof(float) + 1024;
    static_assert(smem + 1024 <= 227 * 1024, "the ring does not fit in shared memory");
    auto kern = gemm_tc_pair_kernel<STAGES, A_ROWS, CH, EPI, TOut>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int pairs = total_tiles < sm_count() / 2 ? total_tiles : sm_count() / 2;
    launch_pair(kern, 2 * pairs, smem, stream, mw, ma, p, nx, total_tiles, tt);
}

}  // namespace

bool gemm_tc_pair_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* off = std::getenv("DLM_B200_NO_PAIR");
        int dev = 0, clusters = 0;
        cudaGetDevice(&dev);
        const bool can = cudaDeviceGetAttribute(&clusters, cudaDevAttrClusterLaunch, dev) == cudaSuccess && clusters != 0 &&
                         sm_count() >= 2;
        state = (off != nullptr && off[0] != '\0' && off[0] != '0') || !can ? 0 : 1;
    }
    return state == 1;
}

bool gemm_tc_pair(const void* a, int lda, const void* w, int ldw, const int32_t* expert_offsets, int num_experts,
                  const float* bias, void* out, int ldo, int M, int N, int K, int out_dtype, int epilogue,
                  cudaStream_t stream) {
    if (M <= 0 || N <= 0) return true;
    CUtensorMap mw;
    TokenMaps ma;
    const long long w_rows = expert_offsets ? (long long)num_experts * N : N;
    if (!make_map(&mw, w, w_rows, K, ldw, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return false;
    for (int i = 0; i < 16; ++i)
        if (!make_map(&ma.m[i], a, M, K, lda, 8 * (i + 1))) return false;
    TcParams p{expert_offsets, num_experts, bias, out, ldo, M, N, K, error_flag_ptr()};
    // Grouped: tiles of at most 160 tokens, so that a stage is 26 KB and eight of them fit (an expert with more
    // tokens takes several tiles); dense: 256 tokens a tile, six stages of 32 KB.
    // Few tokens (a decode step): the tokens' part of a stage shrinks to 64 (dense) or 32 (grouped) tokens a
    // tile, and the ring holds 10 or 11 stages of weights instead of 6 or 8 (a decode step of 64 requests
    // 8.18 -> 7.99 ms, most of it from the experts' products; the dense products of 24-64 rows gain 8 %).
    const bool grouped = expert_offsets != nullptr;
    const bool few = grouped ? M <= 4 * num_experts : M <= 64;
    const int tt = few ? (grouped ? 32 : 64) : (grouped ? 160 : TT);
    int t_tiles = (M + tt - 1) / tt;
    if (grouped) t_tiles += num_experts;
    const int nx = (N + 2 * BM - 1) / (2 * BM);
    DLM_CHECK((long long)nx * t_tiles < (1LL << 30), "gemm: too many tiles for one launch");
    const int total_tiles = nx * t_tiles;
    const bool f32 = out_dtype == F32;
#define DLM_PAIR(ST, AR)                                                                                          \
    switch (epilogue) {                                                                                           \
        case EPI_STORE: if (f32) launch<ST, AR, EPI_STORE, float>(mw, ma, p, nx, total_tiles, tt, stream);        \
                        else launch<ST, AR, EPI_STORE, __nv_bfloat16>(mw, ma, p, nx, total_tiles, tt, stream); break; \
        case EPI_ADD: launch<ST, AR, EPI_ADD, float>(mw, ma, p, nx, total_tiles, tt, stream); break;              \
        default: if (f32) launch<ST, AR, EPI_SWIGLU, float>(mw, ma, p, nx, total_tiles, tt, stream);              \
                 else launch<ST, AR, EPI_SWIGLU, __nv_bfloat16>(mw, ma, p, nx, total_tiles, tt, stream); break;   \
    }
    if (few) { if (grouped) { DLM_PAIR(11, 16) } else { DLM_PAIR(10, 32) } }
    else if (grouped) { DLM_PAIR(8, 80) } else { DLM_PAIR(6, 128) }
#undef DLM_PAIR
    check_launch("gemm_tc_pair");
    return true;
}

}  // namespace dlmk
