// C = A · W^T for few rows of A (decode steps, and experts that got a handful of tokens), bound by
// the reading of W: a weight-streaming kernel built on bulk asynchronous copies.
//
// One persistent block per multiprocessor walks a contiguous range of work items; an item is a tile
// of 16 rows of W (of one expert), so that a block reads one long contiguous stretch of memory.
// A producer warp brings the tile into shared memory with bulk copies (cp.async.bulk, completion on an
// mbarrier), three stages deep: the whole tile in ONE copy when its rows lie back to back in memory and fit
// a stage and are shorter than 2,048 elements, else one copy per row and chunk of 2,048 elements.  (Issuing a
// bulk copy costs about 60 ns whatever its size; with one copy per row a tile could not take less than a
// microsecond, which held products with rows shorter than 1,500 elements below the memory's bandwidth.)  Eight consumer warps split a chunk along K; each multiplies its slice by the rows of A,
// which it holds in registers, in tensor-core MMAs with the roles swapped (16 rows of W are the MMA's
// M, 8 rows of A its N; mma.sync m16n8k16, bfloat16 in, 32-bit accumulation), and leaves its partial
// sums in shared memory (two buffers, handed over through mbarriers).  A tenth warp adds the eight partial
// sums of a tile in a fixed order, applies the epilogue and stores, while the consumers are at the next
// tile: no consumer waits for the slowest one or pays for the sums (when every consumer warp joined in
// them, that was 430 clocks of a tile's 2,000).  A result does not depend on what else was in the batch.
//
// K is walked in blocks of 32.  Lane (g = lane / 4, t = lane % 4) takes the 8 consecutive elements
// 8t..8t+7 of rows g and g + 8 of the weight tile and of row g of A; the two MMAs of a block take
// elements {0,1 | 2,3} and {4,5 | 6,7} of those as their k-slices.  Even and odd blocks add into two
// accumulators (two chains of dependent MMAs instead of one; a warp's MMAs, not the memory, were what a tile
// of short rows waited for), which are added at the end.  A sum does not care in which
// order its terms are listed, and A and W list them alike.  Rows copied one by one lie 64 bytes (mod 128)
// apart in a stage, so that the 16-byte reads of a quarter warp fall into distinct banks; a tile copied whole
// keeps its rows back to back, and its reads meet two to a bank when the row length is a multiple of 64
// elements, which the consumers, idle most of the time, can afford.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets a block-wide flag, all roles
// leave their loops, the producer waits (bounded again) for its copies in flight, and the kernel
// reports error 5 through the error flag.
//
// The kernel may start while the kernel before it ends (see dep_wait in common.cuh): the producer of
// a dense product starts to fetch weights, which no kernel writes, before the activations are there.
#include <cstdlib>
#include <type_traits>

#include "api.h"
#include "common.cuh"
#include "mma_sync.cuh"
#include "gemm_internal.h"
#include "tcgen05.cuh"

namespace dlmk {

namespace {

using namespace tc5;      // mbarrier helpers with bounded waits

constexpr int CW = 8;                        // consumer warps
constexpr int THREADS = (CW + 2) * 32;       // + the producer warp + the warp that finishes tiles
constexpr int RT = 16;                       // rows of W per tile
constexpr int STAGES = 3;
constexpr int KC_MAX = 2048;                 // most elements of a row per stage
constexpr int MAX_ACTIVE = 1024;             // most experts with rows in one launch

struct StreamParams {
    const __nv_bfloat16* a; int lda; const int32_t* a_rows;
    const __nv_bfloat16* w; int ldw; long long w_expert_stride;
    const int32_t* expert_offsets; int num_experts;
    const float* bias;
    void* out; int ldo;
    int M, N, K;
    int tiles;            // ceil(N / RT)
    int n_chunks, kc;     // chunks of K per tile, elements per chunk (the last may be shorter)
    int slice;            // elements of a chunk per consumer warp: a multiple of 32, at most 256
    int pitch;            // bytes between the rows of a stage
    int whole_tile;       // a tile's rows are contiguous in memory and come as one copy
    int* err;
};

// One row piece: global -> shared, `bytes` a multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// The MMA without `volatile`: the compiler may interleave the two accumulator chains and move the loads of
// the next blocks of K between them (the mbarrier operations around a stage clobber memory, so nothing
// crosses them).
__device__ __forceinline__ void mma_free(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Work { int expert, row0, m_count, tile; };

// The experts that have rows, in ascending order, with their rows: filled once per block, so that a tile costs
// no load from global memory before its copy can be asked for.
struct ActiveExperts {
    int expert[MAX_ACTIVE];
    int row0[MAX_ACTIVE];
    int count[MAX_ACTIVE];
};

// Item `item` of the launch: dense, tile `item` for all rows of A; grouped, tile item % tiles of the
// (item / tiles)-th expert that has rows.
__device__ __forceinline__ Work get_work(const StreamParams& p, const ActiveExperts& act, int item) {
    Work wk{0, 0, p.M, item};
    if (p.expert_offsets != nullptr) {
        const int slot = item / p.tiles;
        wk.tile = item - slot * p.tiles;
        wk.expert = act.expert[slot];
        wk.row0 = act.row0[slot];
        wk.m_count = act.count[slot];
    }
    return wk;
}

template <int NT, int NCH, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS, 1) gemm_stream_kernel(StreamParams p) {
    constexpr int MP = 8 * NT;                       // rows of A per pass
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];     // a stage has arrived
    __shared__ __align__(8) uint64_t empty_bar[STAGES];    // all consumer warps have read a stage
    __shared__ __align__(8) uint64_t red_full[2];          // partial sums of a tile written by all consumer warps
    __shared__ __align__(8) uint64_t red_empty[2];         // ... and added up and stored: the buffer is free again
    __shared__ ActiveExperts s_active;
    __shared__ int s_n_active, s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t stage_bytes = (size_t)RT * p.pitch;
    float* red = reinterpret_cast<float*>(smem + STAGES * stage_bytes);      // [2][CW][16][MP + 1]
    const bool grouped = p.expert_offsets != nullptr;
    const bool early = !grouped;       // grouped: every thread has waited for the kernel before this one below
    volatile int* abort_flag = &s_abort;

    if (tid == 0) {
        s_abort = 0;
        s_n_active = 1;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], CW); }
        mbar_init(&red_full[0], CW);
        mbar_init(&red_full[1], CW);
        mbar_init(&red_empty[0], 1);
        mbar_init(&red_empty[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (grouped) {
        dep_wait();
        dep_launch_next();
        __syncthreads();
        // the experts that have rows, in ascending order
        if (warp == 0) {
            int seen = 0;
            for (int base = 0; base < p.num_experts; base += 32) {
                const int e = base + lane;
                const int first = e < p.num_experts ? p.expert_offsets[e] : 0;
                const int count = e < p.num_experts ? min(p.expert_offsets[e + 1], p.M) - first : 0;
                const bool has = count > 0;
                const unsigned mask = __ballot_sync(0xffffffffu, has);
                const int slot = seen + __popc(mask & ((1u << lane) - 1));
                if (has && slot < MAX_ACTIVE) {
                    s_active.expert[slot] = e;
                    s_active.row0[slot] = first;
                    s_active.count[slot] = count;
                }
                seen += __popc(mask);
            }
            if (lane == 0) s_n_active = min(seen, MAX_ACTIVE);
        }
    }
    __syncthreads();
    const long long total = (long long)s_n_active * p.tiles;
    const int item_begin = (int)(total * blockIdx.x / gridDim.x);
    const int item_end = (int)(total * (blockIdx.x + 1) / gridDim.x);

    if (warp == CW) {
        // ------------------------------------------------------------------ producer
        uint32_t it = 0;                                  // stages issued so far
        bool ok = true;
        for (int item = item_begin; item < item_end && ok; ++item) {
            const Work wk = get_work(p, s_active, item);
            const int passes = (wk.m_count + MP - 1) / MP;
            const int row = min(wk.tile * RT + (lane & (RT - 1)), p.N - 1);      // rows beyond N: a valid row again
            const __nv_bfloat16* src_row = p.w + (long long)wk.expert * p.w_expert_stride + (long long)row * p.ldw;
            for (int pc = 0; pc < passes * p.n_chunks; ++pc, ++it) {
                const int c = pc % p.n_chunks;
                const uint32_t s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                const int k0 = c * p.kc;
                const uint32_t len = (uint32_t)min(p.kc, p.K - k0);
                if (p.whole_tile) {
                    // the rows that exist (the last tile of a matrix may be short; what lies behind them in the
                    // stage is left over from earlier tiles and only meets outputs that are not stored)
                    if (lane == 0) {
                        const uint32_t bytes = (uint32_t)min(RT, p.N - wk.tile * RT) * (uint32_t)p.K * 2u;
                        mbar_expect_tx(&full_bar[s], bytes);
                        bulk_copy(smem + s * stage_bytes,
                                  p.w + (long long)wk.expert * p.w_expert_stride + (long long)wk.tile * RT * p.ldw, bytes,
                                  &full_bar[s]);
                    }
                    continue;
                }
                if (lane == 0) mbar_expect_tx(&full_bar[s], RT * len * 2);
                __syncwarp();
                if (lane < RT) bulk_copy(smem + s * stage_bytes + (size_t)lane * p.pitch, src_row + k0, len * 2, &full_bar[s]);
            }
        }
        if (!grouped) dep_wait();            // every thread waits for the kernel before this one before it ends
        if (!ok) {
            // copies in flight must land before the block's shared memory is given up
            const uint32_t first = it > STAGES ? it - STAGES : 0;
            for (uint32_t j = first; j < it; ++j) {
                for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                    if (mbar_try_wait(&full_bar[j % STAGES], (j / STAGES) & 1)) break;
            }
        }
    } else if (warp < CW) {
        // ----------------------------------------------------------------- consumers
        if (!grouped) {
            dep_wait();
            dep_launch_next();
        }
        // This lane's pieces of the rows of A of the current (expert, pass), for NCH chunks of K.  A tile of one
        // chunk, or of two with NCH = 2: they stay in registers from tile to tile.  More chunks than NCH: they are
        // fetched again at every chunk, and those loads queue in L2 behind the weights in flight (rows of 2,560
        // and 3,584 elements streamed at 2.8 TB/s that way; NCH = 2 with 8 rows a pass is for them).
        uint4 xb[NT][8 * NCH];
        const bool held_for_tile = p.n_chunks <= NCH;
        long long held = -1;                             // (first row, pass) whose rows of A are in xb
        const int g = lane >> 2, t = lane & 3;
        const int kw = warp * p.slice;                   // this warp's first element within a chunk
        const int nb = p.slice >> 5;                     // its blocks of 32 elements
        // fills xb[.][XO .. XO + 7] with the pieces of chunk c
        auto load_rows = [&](const Work& wk, int m0, int c, auto xo) {
            constexpr int XO = decltype(xo)::value;
            const int k0 = c * p.kc;
            const int len = min(p.kc, p.K - k0);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int m = m0 + nt * 8 + g;
                const __nv_bfloat16* arow = nullptr;
                if (m < wk.m_count) {
                    const int src = p.a_rows ? p.a_rows[wk.row0 + m] : wk.row0 + m;
                    arow = p.a + (long long)src * p.lda + k0 + kw + 8 * t;
                }
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    xb[nt][XO + b] = make_uint4(0, 0, 0, 0);
                    if (b < nb && arow != nullptr && kw + 32 * b + 8 * t < len)
                        xb[nt][XO + b] = __ldg(reinterpret_cast<const uint4*>(arow + 32 * b));
                }
            }
        };
        uint32_t it = 0, ep = 0;
        bool ok = true;
        float acc[NT][2][4];
        // one chunk of a tile: waits for its stage, multiplies, gives the stage back
        auto do_chunk = [&](int c, auto xo) -> bool {
            constexpr int XO = decltype(xo)::value;
            const int len = min(p.kc, p.K - c * p.kc);
            const uint32_t s = it % STAGES;
            if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag)) return false;
            const unsigned char* st = smem + s * stage_bytes + (size_t)(kw + 8 * t) * 2;
            // the weights of GB blocks of K are read before their MMAs are issued
            constexpr int GB = 4;
#pragma unroll
            for (int b0 = 0; b0 < 8; b0 += GB) {
                if (b0 < nb) {
                    uint4 wa[GB], wb[GB];
#pragma unroll
                    for (int j = 0; j < GB; ++j) {
                        const int b = b0 + j;
                        wa[j] = wb[j] = make_uint4(0, 0, 0, 0);
                        // K is a multiple of 8: a lane's 8 elements are all in or all out
                        if (b < nb && kw + 32 * b + 8 * t < len) {
                            wa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * p.pitch + 64 * b);
                            wb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * p.pitch + 64 * b);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < GB; ++j) {
                        const int b = b0 + j;
                        if (b < nb) {
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                mma_free(acc[nt][0], wa[j].x, wb[j].x, wa[j].y, wb[j].y, xb[nt][XO + b].x, xb[nt][XO + b].y);
                                mma_free(acc[nt][1], wa[j].z, wb[j].z, wa[j].w, wb[j].w, xb[nt][XO + b].z, xb[nt][XO + b].w);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
            ++it;
            return true;
        };
        using X0 = std::integral_constant<int, 0>;
        using X1 = std::integral_constant<int, NCH == 2 ? 8 : 0>;
        for (int item = item_begin; item < item_end && ok; ++item) {
            const Work wk = get_work(p, s_active, item);
            const int passes = (wk.m_count + MP - 1) / MP;
            for (int pass = 0; pass < passes && ok; ++pass) {
                const int m0 = pass * MP;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[nt][0][i] = acc[nt][1][i] = 0.f;
                const long long key = ((long long)wk.row0 << 20) | (long long)pass;
                if (held_for_tile) {
                    if (key != held) {
                        held = key;
                        load_rows(wk, m0, 0, X0{});
                        if (NCH == 2 && p.n_chunks == 2) load_rows(wk, m0, 1, X1{});
                    }
                    ok = do_chunk(0, X0{});
                    if (NCH == 2 && p.n_chunks == 2 && ok) ok = do_chunk(1, X1{});
                } else {
                    for (int c = 0; c < p.n_chunks && ok; ++c) {
                        load_rows(wk, m0, c, X0{});
                        ok = do_chunk(c, X0{});
                    }
                }
                if (!ok) break;
                // Partial sums to shared memory: red[ep % 2][warp][weight row][row of A], once the finishing warp
                // has read what tile ep - 2 left there (it has, as a rule, long ago).
                if (ep >= 2 && !mbar_wait(&red_empty[ep & 1], ((ep >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                float* mine = red + ((size_t)(ep & 1) * CW + warp) * 16 * (MP + 1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mine[g * (MP + 1) + nt * 8 + 2 * t] = acc[nt][0][0] + acc[nt][1][0];
                    mine[g * (MP + 1) + nt * 8 + 2 * t + 1] = acc[nt][0][1] + acc[nt][1][1];
                    mine[(g + 8) * (MP + 1) + nt * 8 + 2 * t] = acc[nt][0][2] + acc[nt][1][2];
                    mine[(g + 8) * (MP + 1) + nt * 8 + 2 * t + 1] = acc[nt][0][3] + acc[nt][1][3];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[ep & 1]);
                ++ep;
            }
        }
    } else {
        // ------------------------------------------------------- the warp that finishes tiles
        // It adds the eight partial sums of a tile in a fixed order, applies the epilogue and stores, while the
        // consumer warps are at the next tile: none of them waits for the slowest one.
        if (early) dep_wait();
        uint32_t e = 0;
        bool ok = true;
        for (int item = item_begin; item < item_end && ok; ++item) {
            const Work wk = get_work(p, s_active, item);
            const int passes = (wk.m_count + MP - 1) / MP;
            for (int pass = 0; pass < passes; ++pass, ++e) {
                const int out_row0 = wk.row0 + pass * MP, m_here = min(MP, wk.m_count - pass * MP), n_base = wk.tile * RT;
                if (!mbar_wait(&red_full[e & 1], (e >> 1) & 1, abort_flag)) { ok = false; break; }
                const float* rb = red + (size_t)(e & 1) * CW * 16 * (MP + 1);
                if (EPI == EPI_SWIGLU) {
                    // element = (row of A, pair of weight rows)
#pragma unroll
                    for (int i = lane; i < MP * 8; i += 32) {
                        const int pr = i & 7, m = i >> 3;
                        const int n = n_base + 2 * pr;
                        if (m >= m_here || n + 1 >= p.N) continue;
                        float gate = 0.f, up = 0.f;
#pragma unroll
                        for (int ww = 0; ww < CW; ++ww) {
                            gate += rb[((size_t)ww * 16 + 2 * pr) * (MP + 1) + m];
                            up += rb[((size_t)ww * 16 + 2 * pr + 1) * (MP + 1) + m];
                        }
                        static_cast<TOut*>(p.out)[(long long)(out_row0 + m) * p.ldo + (n >> 1)] =
                            from_f32<TOut>(silu_f(gate) * up);
                    }
                } else {
#pragma unroll
                    for (int i = lane; i < MP * 16; i += 32) {
                        const int row = i & 15, m = i >> 4;
                        const int n = n_base + row;
                        if (m >= m_here || n >= p.N) continue;
                        float v = 0.f;
#pragma unroll
                        for (int ww = 0; ww < CW; ++ww) v += rb[((size_t)ww * 16 + row) * (MP + 1) + m];
                        const long long o = (long long)(out_row0 + m) * p.ldo + n;
                        if (EPI == EPI_ADD) static_cast<float*>(p.out)[o] += v;
                        else static_cast<TOut*>(p.out)[o] = from_f32<TOut>(v + (p.bias ? p.bias[n] : 0.f));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_empty[e & 1]);
            }
        }
    }
    __syncthreads();
    if (tid == 0 && s_abort) *p.err = 5;
}

template <int NT, int NCH, int EPI, typename TOut>
void launch_one(const StreamParams& p, int grid, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * RT * p.pitch + 2 * sizeof(float) * CW * 16 * (8 * NT + 1);
    auto kern = gemm_stream_kernel<NT, NCH, EPI, TOut>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_dep(kern, grid, THREADS, smem, stream, p);
}

template <int NT, int NCH>
void launch_nt(const StreamParams& p, int grid, int out_dtype, int epilogue, cudaStream_t stream) {
    const bool f32 = out_dtype == F32;
    switch (epilogue) {
        case EPI_STORE: if (f32) launch_one<NT, NCH, EPI_STORE, float>(p, grid, stream);
                        else launch_one<NT, NCH, EPI_STORE, __nv_bfloat16>(p, grid, stream); break;
        case EPI_ADD: launch_one<NT, NCH, EPI_ADD, float>(p, grid, stream); break;
        default: if (f32) launch_one<NT, NCH, EPI_SWIGLU, float>(p, grid, stream);
                 else launch_one<NT, NCH, EPI_SWIGLU, __nv_bfloat16>(p, grid, stream); break;
    }
}

}  // namespace

bool gemm_stream_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* off = std::getenv("DLM_B200_NO_STREAM");
        on = (off != nullptr && off[0] != '\0' && off[0] != '0') ? 0 : 1;
    }
    return on == 1;
}

bool gemm_stream_ok(const void* a, int lda, const void* w, int ldw, long long w_expert_stride,
                    const int32_t* expert_offsets, int num_experts, int M, int N, int K, int in_dtype) {
    if (!(in_dtype == BF16 && M > 0 && N > 0 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
          w_expert_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
          (reinterpret_cast<uintptr_t>(w) & 15) == 0))
        return false;
    // the list of experts with rows lives in shared memory
    if (expert_offsets != nullptr && (num_experts < M ? num_experts : M) > MAX_ACTIVE) return false;
    return true;
}

void gemm_stream(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
                 const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N,
                 int K, int out_dtype, int epilogue, int rows_per_pass, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return;
    DLM_CHECK(epilogue != EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N");
    DLM_CHECK(epilogue != EPI_ADD || out_dtype == F32, "gemm: the accumulate epilogue needs a float32 output");
    StreamParams p;
    p.a = static_cast<const __nv_bfloat16*>(a); p.lda = lda; p.a_rows = a_rows;
    p.w = static_cast<const __nv_bfloat16*>(w); p.ldw = ldw; p.w_expert_stride = w_expert_stride;
    p.expert_offsets = expert_offsets; p.num_experts = num_experts; p.bias = bias; p.out = out; p.ldo = ldo;
    p.M = M; p.N = N; p.K = K;
    p.tiles = (N + RT - 1) / RT;
    // 8 or 16 rows of A a pass.  (32 rows a pass hold 128 registers of A alone; with 288 threads a block the
    // register file allows 168 a thread, the compiler spilled, and that variant ran at 40 % of this one's speed:
    // more rows take more passes instead.)
    p.n_chunks = (K + KC_MAX - 1) / KC_MAX;
    // Rows of two chunks: a lane holds its pieces of 8 rows of A for both chunks (as many registers as 16 rows
    // of one chunk); more rows take more passes, whose weights come from L2.
    const bool hold2 = p.n_chunks == 2 && rows_per_pass <= 8;
    const int nt = (rows_per_pass <= 8 || hold2) ? 1 : 2;
    p.kc = ((K + p.n_chunks - 1) / p.n_chunks + 31) / 32 * 32;
    if (p.kc > K) p.kc = K;
    p.slice = ((p.kc + CW - 1) / CW + 31) / 32 * 32;
    // rows of a stage 64 bytes (mod 128) apart; or, a tile in one copy, back to back as they lie in memory
    const int row_bytes = p.kc * 2;
    // (measured on rows of 512 / 1,024 / 1,408 / 1,536 / 2,048 elements: one copy per tile 3.1 / 5.7 / 6.2 / 6.2 /
    // 6.2 TB/s, one copy per row 2.3 / 4.5 / 5.7 / 6.1 / 6.3: the row copies' padding keeps the reads free of
    // bank conflicts, which shows once the rows are long enough for their issue not to matter)
    p.whole_tile = (p.n_chunks == 1 && ldw == K && K < 2048) ? 1 : 0;
    p.pitch = p.whole_tile ? row_bytes : row_bytes + ((64 - row_bytes % 128) + 128) % 128;
    p.err = error_flag_ptr();
    const int groups = expert_offsets ? (num_experts < M ? num_experts : M) : 1;
    const long long items = (long long)p.tiles * groups;
    const int grid = (int)(items < sm_count() ? items : sm_count());
    if (hold2) launch_nt<1, 2>(p, grid, out_dtype, epilogue, stream);
    else if (nt == 1) launch_nt<1, 1>(p, grid, out_dtype, epilogue, stream);
    else launch_nt<2, 1>(p, grid, out_dtype, epilogue, stream);
    check_launch("gemm_stream");
}

}  // namespace dlmk
