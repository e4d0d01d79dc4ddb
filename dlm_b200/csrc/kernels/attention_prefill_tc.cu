// Prefill attention on the fifth-generation tensor cores (tcgen05), bfloat16, head size 128, pages of a
// multiple of 64 tokens: portions of prompts, each query attending to its request's paged keys up to its
// own position (optionally only the last `window` of them).
//
// One block = 128 consecutive query tokens of one request x one query head.  Seven warps, three roles:
//   warps 4 and 6      the producers (one lane each): the query tile once, then per tile of 128 keys the keys
//                      (warp 4) and the values (warp 6), as TMA boxes of 64 keys x 64 dims straight from the
//                      pages, 128-byte swizzle, two tiles of each in flight;
//   warp 5 (one lane)  the MMA issuer: S = Q K^T (128 x 128, K-major operands) into one of two score buffers
//                      in tensor memory, and O += P V (V is read as it lies in the cache: keys x dims, i.e.
//                      MN-major) into the output accumulator in tensor memory; the scores of tile j + 1 are
//                      issued before P V of tile j, so the tensor cores work while the softmax runs;
//   warps 0-3          the softmax: thread i owns query row i = lane i of tensor memory.  It reads its scores
//                      with tcgen05.ld, keeps the running maximum and sum in 32-bit, rescales its row of O in
//                      tensor memory when the maximum moved far, and writes P (bfloat16) into one of two buffers
//                      in shared memory in the layout the next MMA reads, so that it need not wait for the
//                      product of the tile before.  At the end it reads O, divides and stores.
// Every wait on a barrier is bounded (see tcgen05.cuh); a wait that runs out ends the block with error 5.
//
// Keys a query must not see (later positions, positions outside the window) get probability exactly 0.
// A page that is not there is read as zeros (a box outside the tensor); a page that is missing although a
// query sees it raises error 3.
#include <cstdlib>

#include "api.h"
#include "attention_internal.h"
#include "common.cuh"
#include "mma_sync.cuh"
#include "tcgen05.cuh"

namespace dlmk {

namespace {

using namespace tc5;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int SOFTMAX_WARPS = 4, KEY_WARP = 4, MMA_WARP = 5, VALUE_WARP = 6, THREADS = 224;
constexpr uint32_t HALF_BYTES = 128 * 128;             // 128 rows x 64 elements: one swizzled half of a tile
constexpr uint32_t TILE_BYTES = 2 * HALF_BYTES;        // 128 rows x 128 elements
constexpr uint32_t TMEM_COLS = 512;                    // S0 | S1 | O | unused, 128 columns each

struct PrefillTcParams {
    const int32_t* block_table; int table_width;
    const int32_t* cu_q; const int32_t* kv_len;
    __nv_bfloat16* out;
    int R, nh, nkv, page_size, page_shift, total_pages, window;
    float scale_log2;
    int skip_single;
    int* err;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// tcgen05.ld without its wait, and the wait as a statement that the registers depend on (so that no use of them
// can be placed before it)
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_fence(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :: "memory");
}
// MN-major operand tile with 128-byte swizzle (the contiguous dimension is the MMA's N): rows are K, 128 bytes
// each, groups of 8 rows 1024 bytes apart; the next 64 elements of N lie `n_block_bytes` further.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t n_block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((n_block_bytes >> 4) & 0x3FFF) << 16;      // leading byte offset: next block along N
    d |= (uint64_t)(1024 >> 4) << 32;                          // stride byte offset: next group of 8 rows of K
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PrefillTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full[2], v_full[2], s_full[2], p_ready[2], pv_done[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    __shared__ int s_map[2];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* base = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    unsigned char* Qs = base;                              // [2 halves][128 queries][128 bytes]
    unsigned char* Ks = Qs + TILE_BYTES;                   // [2 stages][2 halves][128 keys][128 bytes]
    unsigned char* Vs = Ks + 2 * TILE_BYTES;               // [2 stages][2 halves][128 keys][128 bytes]
    unsigned char* Ps = Vs + 2 * TILE_BYTES;               // [2 buffers][2 halves of the keys][128 queries][128 bytes]

    // work item: blocks start in the order of their linear index; the latest query tiles (most keys) go first
    const int linear = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    const int head = linear % p.nh, kvh = head / (p.nh / p.nkv);
    const int bx = (int)gridDim.y - 1 - linear / p.nh;
    if (tid == 0) {
        s_abort = 0;
        int acc = 0;
        s_map[0] = -1;
        for (int r = 0; r < p.R; ++r) {
            const int ql = p.cu_q[r + 1] - p.cu_q[r];
            const int tiles = (p.skip_single && ql == 1) ? 0 : (ql + BQ - 1) / BQ;
            if (bx < acc + tiles) {
                s_map[0] = r;
                s_map[1] = (bx - acc) * BQ;
                break;
            }
            acc += tiles;
        }
        mbar_init(&q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_ready[s], SOFTMAX_WARPS * 32);
            mbar_init(&pv_done[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int r = s_map[0];
    if (r < 0) {                                           // uniform over the block; nothing allocated yet
        dep_wait();                                        // (every block waits for the kernel before, see common.cuh)
        return;
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_flag = &s_abort;
    // the set-up above may run while the kernel before this one ends (see dep_wait in common.cuh)
    dep_wait();
    dep_launch_next();

    const int q0 = s_map[1];
    const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
    const int n_q = min(BQ, q_len - q0);
    const int len = p.kv_len[r];
    const int pos0 = len - q_len + q0;
    const int hi = pos0 + n_q - 1;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int t_begin = (lo / BKV) * BKV;
    const int n_tiles = (hi - t_begin) / BKV + 1;

    if (warp == KEY_WARP || warp == VALUE_WARP) {
        // one warp brings the queries and the keys, another the values: a key stage is free as soon as its scores
        // are computed (s_full), a value stage only after its P V product (pv_done), and neither copy waits for
        // the other
        if (lane == 0) {
            const bool keys = warp == KEY_WARP;
            const int32_t* table = p.block_table + (long long)r * p.table_width;
            const int rows_total = p.total_pages * p.nkv * p.page_size;
            const CUtensorMap* map = keys ? &map_k : &map_v;
            uint64_t* full = keys ? k_full : v_full;
            uint64_t* empty = keys ? s_full : pv_done;
            unsigned char* tiles = keys ? Ks : Vs;
            if (keys) {
                mbar_expect_tx(&q_full, TILE_BYTES);
                tma_load_2d(Qs, &map_q, head * HD, q_begin + q0, &q_full);
                tma_load_2d(Qs + HALF_BYTES, &map_q, head * HD + 64, q_begin + q0, &q_full);
            }
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                if (j >= 2 && !mbar_wait(&empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&full[s], TILE_BYTES);
                const int j0 = t_begin + j * BKV;
#pragma unroll
                for (int part = 0; part < 2; ++part) {               // two runs of 64 keys
                    const int key0 = j0 + 64 * part;
                    const int lp = key0 >> p.page_shift;
                    int page = lp < p.table_width ? table[lp] : -1;
                    if (page >= p.total_pages) page = -1;
                    // some query of the tile sees keys of this run: its page must be there
                    if (page < 0 && key0 <= hi && key0 + 63 >= lo) *p.err = 3;
                    // a run without a page is read from outside the tensor: zeros
                    const int y = page >= 0 ? (page * p.nkv + kvh) * p.page_size + (key0 & (p.page_size - 1)) : rows_total;
                    unsigned char* dst = tiles + (size_t)s * TILE_BYTES + part * (64 * 128);
                    tma_load_2d(dst, map, 0, y, &full[s]);
                    tma_load_2d(dst + HALF_BYTES, map, 64, y, &full[s]);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // M = 128, N = 128, bfloat16 x bfloat16 -> float32
            constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) |
                                         ((uint32_t)(BQ >> 4) << 24);
            constexpr uint32_t IDESC_PV = IDESC_S | (1u << 16);          // B (the values) is MN-major
            // operand descriptors of every buffer, made once: a step of 16 along K adds a constant to the
            // address field (in units of 16 bytes)
            const uint64_t dq = umma_desc(smem_u32(Qs));
            const uint64_t dk[2] = {umma_desc(smem_u32(Ks)), umma_desc(smem_u32(Ks + TILE_BYTES))};
            const uint64_t dp[2] = {umma_desc(smem_u32(Ps)), umma_desc(smem_u32(Ps + TILE_BYTES))};
            const uint64_t dv[2] = {umma_desc_mn(smem_u32(Vs), HALF_BYTES), umma_desc_mn(smem_u32(Vs + TILE_BYTES), HALF_BYTES)};
            auto issue_s = [&](int j) {
                const uint64_t dkj = dk[j & 1];
                const uint32_t d_tmem = tmem_base + (uint32_t)(j & 1) * BKV;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t off = (uint64_t)((kk >> 2) * (HALF_BYTES >> 4) + (kk & 3) * 2);
                    umma_bf16(d_tmem, dq + off, dkj + off, IDESC_S, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[j & 1]);         // the scores are there, and the keys of the stage are read
            };
            bool ok = mbar_wait(&q_full, 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(0);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    const int s = (j + 1) & 1;
                    if (!mbar_wait(&k_full[s], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    // (the softmax of tile j - 1 has read this score buffer: it had its scores in registers before
                    // it announced P of tile j - 1, which this thread waited for before that tile's P V)
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(j + 1);
                }
                if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&p_ready[j & 1], (j >> 1) & 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dpj = dp[j & 1], dvj = dv[j & 1];
                const uint32_t o_tmem = tmem_base + 2 * BKV;
                const uint32_t first = j > 0 ? 1u : 0u;
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                    const uint64_t da = dpj + (uint64_t)((kk >> 2) * (HALF_BYTES >> 4) + (kk & 3) * 2);
                    const uint64_t db = dvj + (uint64_t)(kk * (16 * 128 >> 4));          // 16 keys further
                    umma_bf16(o_tmem, da, db, IDESC_PV, kk > 0 ? 1u : first);
                }
                // O holds tiles 0..j; this P buffer may be written again; the values of the stage are read
                umma_commit(&pv_done[j & 1]);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax, one thread per query row
        const int row = tid;                                   // = lane of tensor memory
        const int pos = pos0 + row;
        const uint32_t lane_base = ((uint32_t)(warp * 32) << 16);
        const uint32_t o_tmem = tmem_base + 2 * BKV + lane_base;
        unsigned char* p_row0 = Ps + (size_t)(row >> 3) * 1024 + (size_t)(row & 7) * 128;
        // m is the maximum the probabilities are taken against.  It follows the row's true maximum only when
        // that has grown by more than 2^RESCALE_STEP since (or at the row's first keys): a probability is then
        // at most 2^RESCALE_STEP instead of 1, which neither bfloat16 nor the 32-bit sums mind, the final
        // division makes up for it exactly, and O is seldom rescaled.
        constexpr float RESCALE_STEP = 8.0f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int j0 = t_begin + j * BKV;
            const uint32_t s_tmem = tmem_base + (uint32_t)(j & 1) * BKV + lane_base;
            // (the outcome of a wait is made the same for the whole warp: the collectives below need all lanes)
            if (!__all_sync(0xffffffffu, mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag))) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the row's 128 scores
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32_issue(s_tmem + (uint32_t)(c * 32), v[c]);
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_fence(v[c]);
            // the scores are in registers: once P of this tile is announced, the buffer may be written again
            // does every row of this warp see every key of the tile?  Then nothing is masked.
            const bool row_all = j0 + BKV - 1 <= pos && (p.window <= 0 || pos - j0 < p.window);
            const bool warp_all = __all_sync(0xffffffffu, row_all);
            if (!warp_all) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = j0 + c * 32 + i;
                        const bool vis = key <= pos && (p.window <= 0 || pos - key < p.window);
                        if (!vis) v[c][i] = 0xff800000u;             // -inf
                    }
            }
            // the row's maximum of the raw scores (the scale is positive), four chains
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[c][i]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;   // -inf: nothing seen
            float alpha = 1.0f;
            if (mx > m + RESCALE_STEP || m == -INFINITY) {
                if (mx != -INFINITY) {
                    alpha = ex2(m - mx);                                // m = -inf: 0
                    m = mx;
                }
            }
            const float base_m = m == -INFINITY ? 0.f : m;               // nothing seen yet: every probability is 0
            // O is rescaled only between two P V products: the one of the tile before this must be done
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                {
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(o_tmem + (uint32_t)(c * 32), o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(o_tmem + (uint32_t)(c * 32), o);
                    }
                }
            }
            // this P buffer was read by the P V product of two tiles ago
            if (j >= 2 && !__all_sync(0xffffffffu, mbar_wait(&pv_done[j & 1], ((j >> 1) & 1) ^ 1, abort_flag))) { ok = false; break; }
            unsigned char* p_row = p_row0 + (size_t)(j & 1) * TILE_BYTES;
            // probabilities, their sum (four chains), P in bfloat16 into shared memory (K-major, 128-byte swizzle)
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float pr[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    pr[i] = ex2(fmaf(__uint_as_float(v[c][i]), p.scale_log2, -base_m));     // -inf: 0
                    sum4[i & 3] += pr[i];
                }
                // keys 32c .. 32c + 31 of this row: half c / 2, 16-byte chunks 4 (c % 2) .. + 3 of the row
                unsigned char* dst = p_row + (size_t)(c >> 1) * HALF_BYTES;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c & 1) * 4 + q4;
                    uint4 w;
                    w.x = pack_bf16(pr[8 * q4], pr[8 * q4 + 1]);
                    w.y = pack_bf16(pr[8 * q4 + 2], pr[8 * q4 + 3]);
                    w.z = pack_bf16(pr[8 * q4 + 4], pr[8 * q4 + 5]);
                    w.w = pack_bf16(pr[8 * q4 + 6], pr[8 * q4 + 7]);
                    *reinterpret_cast<uint4*>(dst + ((chunk ^ (row & 7)) << 4)) = w;
                }
            }
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            // P and O are written: hand over to the MMA issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&p_ready[j & 1]);
        }
        if (ok && __all_sync(0xffffffffu, mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag))) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const int Q = p.nh * HD;
            __nv_bfloat16* orow = p.out + (long long)(q_begin + q0 + row) * Q + head * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(o_tmem + (uint32_t)(c * 32), v);
                if (row < n_q) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[8 * q4]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = w;
                    }
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
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// rows x cols bfloat16 matrix with `ld` elements between rows; boxes of box_rows x 64 elements, 128-byte
// swizzle, elements outside the matrix read as zero
bool make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool attention_prefill_tc_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* off = std::getenv("DLM_B200_NO_TCGEN05");
        on = (off != nullptr && off[0] != '\0' && off[0] != '0') ? 0 : 1;
        if (on && encode_tiled() == nullptr) on = 0;
    }
    return on == 1;
}

bool attention_prefill_tc_ok(const void* q, const void* k_cache, const void* v_cache, int nh, int nkv, int hd,
                             int page_size, float scale) {
    // (the row maximum is taken before the scores are scaled: the scale must be positive)
    return scale > 0.f && hd == HD && nkv > 0 && nh % nkv == 0 && page_size >= 64 && (page_size & (page_size - 1)) == 0 &&
           ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
             reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
}

bool attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                          int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                          int nkv, int hd, int page_size, int total_pages, int window, float scale, int skip_single,
                          cudaStream_t stream) {
    if (T <= 0 || R <= 0) return true;
    CUtensorMap mq, mk, mv;
    const long long kv_rows = (long long)total_pages * nkv * page_size;
    if (!make_map(&mq, q, T, nh * hd, (long long)nh * hd, BQ) || !make_map(&mk, k_cache, kv_rows, hd, hd, 64) ||
        !make_map(&mv, v_cache, kv_rows, hd, hd, 64))
        return false;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    PrefillTcParams p{block_table, table_width, cu_q, kv_len, static_cast<__nv_bfloat16*>(out), R, nh, nkv, page_size,
                      shift, total_pages, window, scale * 1.4426950408889634f, skip_single, error_flag_ptr()};
    const size_t smem = (size_t)TILE_BYTES * 7 + 1024;      // Q, 2 x K, 2 x V, 2 x P, and room to align
    cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(nh, (T + BQ - 1) / BQ + R);
    launch_dep(attention_prefill_tc_kernel, grid, THREADS, smem, stream, mq, mk, mv, p);
    check_launch("attention_prefill_tc");
    return true;
}

}  // namespace dlmk
