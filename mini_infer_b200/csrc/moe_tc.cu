// Grouped expert products for prefill-sized batches on the fifth-generation tensor cores:
// tcgen05.mma with both operands in shared memory (fed by TMA, 128-byte swizzle) and the
// accumulators in tensor memory, read back with tcgen05.ld for the epilogue.
//
// Rows are the (token, slot) pairs sorted by expert and gathered into a contiguous matrix, so
// an expert's rows are the contiguous range offsets[e] .. offsets[e+1].  The product is computed
// transposed: the expert's weights are the M operand (128 features per tile) and the rows are the
// N operand, whose size follows the expert's row count (a multiple of 16 up to the tile limit TN of
// 128 or 256 rows): an expert with 137 rows is one tile with N = 144 under TN = 256, or a tile of 128
// and one of 16 under TN = 128, where two blocks share an SM.  Two families of kernels: the first
// below computes one (expert, row tile, feature tile) per block; the persistent one further down
// (the default) walks one block per SM over all of them.  Either way a tile has two accumulators,
// gate and up of 128 features (mode 1), or one or two neighbouring tiles of 128 features that share
// the row tile (mode 0), and three roles:
//   warp 0    TMA producer: weight tile(s) (128 features x 64 k) and row tile (rows x 64 k)
//   warp 1    allocates tensor memory, issues the MMAs, commits stages back to the producer
//   warps 2-5 epilogue: accumulators -> registers -> SwiGLU / store, one TMEM lane quarter each
//             (a lane is a feature, a column is a row of the expert: for each row a warp stores 32
//             consecutive features)
// A row tile that crosses the end of its expert's range computes rows of the next expert too; they
// are simply not stored.  The k loop runs in ascending order whatever the number of rows.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets an error status that the host
// reads, lets all roles fall through to the common exit, and the tensor memory is freed there.
//
// The reference runs three cuBLAS products per used expert over all tokens and masks afterwards
// (src/layers/moe.cpp:246-270, src/layers/mlp.cpp:255-300); it has no grouped kernel.

#include "tcgen05.cuh"

namespace mi {
namespace tc {

constexpr int BF = 128;                        // features per tile (MMA M)
constexpr int W_TILE_BYTES = BF * BK * 2;      // one weight tile of one stage: 16 KiB
// instruction descriptor without N: D float32, A and B bfloat16, both K-major, M = 128
constexpr uint32_t IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BF >> 4) << 24);

// The row-tile maps differ in their box height only (16, 32, 64, 128, 256 rows): a row tile is fetched
// as the fewest boxes that cover its rows rounded up to 16, so that no bandwidth goes to rows that
// the MMA does not read.
struct RowMaps {
    CUtensorMap m[5];
};

// MODE 1: C[r, n] = silu(a_r . W[e, n]) * (a_r . W[e, Nout + n])  (bfloat16); MODE 0: C[r, n] = a_r . W[e, n] (float)
// TN: rows per tile at most (128 or 256); STAGES: pipeline depth; BLOCKS: blocks meant to share an SM
// (with TN = 128 two blocks fit: while one drains its accumulators the other keeps the loads going).
template <int MODE, int TN, int STAGES, int BLOCKS>
__global__ void __launch_bounds__(192, BLOCKS)
grouped_gemm_tc_kernel(const __grid_constant__ RowMaps maps_a, const __grid_constant__ CUtensorMap map_w,
                       const int* __restrict__ offsets, void* __restrict__ C, int E, int Nout, int Kd,
                       int* __restrict__ status, int skip_kb, uint32_t wait_limit) {
    // skip_kb >= 0 (tests of the bounded waits only): the producer stops before the loads of that k block, so
    // the wait for them runs out after `wait_limit` rounds, every role gives up and the status word says so.
    constexpr int NB = 2;                                 // weight tiles per stage: gate and up (MODE 1), or two
                                                          // neighbouring feature tiles sharing the row tile (MODE 0)
    constexpr int R_TILE_BYTES = TN * BK * 2;             // room for the row tile of one stage
    constexpr int FEATS = MODE == 1 ? BF : 2 * BF;        // output features per block
    constexpr int STAGE_BYTES = NB * W_TILE_BYTES + R_TILE_BYTES;
    constexpr uint32_t TMEM_COLS = NB * TN;               // 512 or 256: a power of two >= 32
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    // which expert and row tile does blockIdx.y stand for?
    int slot = blockIdx.y, e = 0, row0 = 0, rows = 0;
    bool found = false;
    for (e = 0; e < E; ++e) {
        const int b0 = offsets[e], cnt = offsets[e + 1] - b0;
        const int tiles = (cnt + TN - 1) / TN;
        if (slot < tiles) { row0 = b0 + slot * TN; rows = min(TN, cnt - slot * TN); found = true; break; }
        slot -= tiles;
    }
    if (!found) return;                                   // uniform for the whole block
    const int n0 = blockIdx.x * FEATS;
    const int wrows = MODE == 1 ? 2 * Nout : Nout;
    const int num_kb = Kd / BK;
    const int n_mma = (rows + 15) & ~15;                  // MMA N: a multiple of 16 for M = 128
    const uint32_t row_bytes = (uint32_t)n_mma * BK * 2;  // bytes the row-tile copies deliver
    const uint32_t idesc = IDESC_BASE | ((uint32_t)(n_mma >> 3) << 17);

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = ((kb / STAGES) & 1) ^ 1;
                if (!mbar_wait(&empty_bar[s], parity, abort_flag, 1, wait_limit)) break;
                if (kb == skip_kb) break;                  // (tests only) this block's data never arrives
                uint8_t* st = smem + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], NB * W_TILE_BYTES + row_bytes);
                tma_load_2d(st, &map_w, kb * BK, e * wrows + n0, &full_bar[s]);
                tma_load_2d(st + W_TILE_BYTES, &map_w, kb * BK, e * wrows + (MODE == 1 ? Nout + n0 : n0 + BF), &full_bar[s]);
                for (int done = 0; done < n_mma;) {
                    const int left = n_mma - done;
                    const int b = left >= 256 ? 4 : (left >= 128 ? 3 : (left >= 64 ? 2 : (left >= 32 ? 1 : 0)));
                    tma_load_2d(st + NB * W_TILE_BYTES + done * (BK * 2), &maps_a.m[b], kb * BK, row0 + done,
                                &full_bar[s]);
                    done += 16 << b;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = (kb / STAGES) & 1;
                ok = mbar_wait(&full_bar[s], parity, abort_flag, 2, wait_limit);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t w_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                const uint32_t r_addr = w_addr + NB * W_TILE_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                    const uint64_t rd = umma_desc(r_addr + k * 32);
                    umma_bf16(tmem_base, umma_desc(w_addr + k * 32), rd, idesc, acc);
                    umma_bf16(tmem_base + TN, umma_desc(w_addr + W_TILE_BYTES + k * 32), rd, idesc, acc);
                }
                umma_commit(&empty_bar[s]);               // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(&accum_bar);              // accumulators complete
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31; a lane is a feature of a 128-feature tile
        const int quarter = warp & 3;
        const int fl = quarter * 32 + lane;
        bool ok = mbar_wait(&accum_bar, 0, abort_flag, 3, wait_limit);
        ok = __all_sync(0xffffffffu, ok);                 // tcgen05.ld is warp-wide: all lanes or none
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // With whole 16-byte groups of features per row the tile is transposed through the (now
        // idle) pipeline memory and leaves in 16-byte stores; otherwise element by element.
        constexpr int OUT_BYTES = MODE == 1 ? 2 : 4;
        constexpr int PER16 = 16 / OUT_BYTES;                         // features per 16-byte group
        constexpr int HALVES = MODE == 1 ? 1 : 2;                     // accumulators that are outputs of their own
        const bool staged = (Nout % PER16) == 0 && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        uint8_t* stage = smem;                                        // [rows][BF] outputs, row pitch BF * OUT_BYTES
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
        for (int half = 0; half < HALVES; ++half) {
            const int fbase = n0 + half * BF;                         // first feature of this accumulator
            const int f = fbase + fl;
            if (ok && fbase < Nout) {
#pragma unroll 1
                for (int c0 = 0; c0 < rows; c0 += 32) {  // columns beyond n_mma hold nothing; they are not stored
                    uint32_t g[32];
                    tmem_ld32(lane_addr + half * TN + c0, g);
                    if (MODE == 1) {
                        uint32_t u[32];
                        tmem_ld32(lane_addr + TN + c0, u);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C) + (int64_t)(row0 + c0) * Nout + f;
                        __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage) + (size_t)c0 * BF + fl;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (c0 + i < rows) {
                                const float gv = __uint_as_float(g[i]);
                                // the result is rounded to bfloat16: the fast exponential and division are exact enough
                                const __nv_bfloat16 v =
                                    __float2bfloat16_rn(__fdividef(gv, 1.0f + __expf(-gv)) * __uint_as_float(u[i]));
                                if (staged) st[(size_t)i * BF] = v;
                                else if (f < Nout) out[(int64_t)i * Nout] = v;
                            }
                        }
                    } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        float* out = reinterpret_cast<float*>(C) + (int64_t)(row0 + c0) * Nout + f;
                        float* st = reinterpret_cast<float*>(stage) + (size_t)c0 * BF + fl;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (c0 + i < rows) {
                                if (staged) st[(size_t)i * BF] = __uint_as_float(g[i]);
                                else if (f < Nout) out[(int64_t)i * Nout] = __uint_as_float(g[i]);
                            }
                        }
                    }
                }
            }
            if (staged) {
                asm volatile("bar.sync 1, 128;" ::: "memory");        // the four epilogue warps, whatever `ok`
                if (ok && *abort_flag == 0 && fbase < Nout) {
                    constexpr int GROUPS = BF / PER16;                // 16-byte groups per row of the tile
                    const int et = threadIdx.x - 64;                  // 0..127 among the epilogue threads
                    const uint4* src = reinterpret_cast<const uint4*>(stage);
                    uint8_t* dst = reinterpret_cast<uint8_t*>(C);
                    for (int idx = et; idx < rows * GROUPS; idx += 128) {
                        const int r = idx / GROUPS, gq = idx - r * GROUPS;
                        const int feat = fbase + gq * PER16;
                        if (feat < Nout)
                            *reinterpret_cast<uint4*>(dst + ((int64_t)(row0 + r) * Nout + feat) * OUT_BYTES) = src[idx];
                    }
                }
                if (half + 1 < HALVES) asm volatile("bar.sync 1, 128;" ::: "memory");   // staging is reused
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_s != 0) atomicMax(status, abort_s);
}

// The same product as a persistent kernel: one block per SM walks over the (row tile, feature tile)
// pairs, feature tiles fastest.  The loads never stop at a tile's end: the producer runs on into the
// next tile's k blocks while the epilogue warps drain the accumulators.  A tile's accumulators lie at
// the low end of the tensor memory for even tiles and at the high end for odd ones, so the MMA warp
// starts the next tile at once when the two tiles fit side by side (2 x NW x N columns of 512), and
// after the epilogue otherwise.  An expert's rows are split evenly over its row tiles of up to TN
// rows, so an expert with 137 rows is one tile (N = 144) and its weights cross the memory system
// once.  The table of row tiles is built by every block for itself from the experts' offsets.
//   warp 0    builds the table; TMA producer
//   warp 1    tensor memory, MMAs
//   warps 2-5 epilogue, one TMEM lane quarter each; a warp turns its 32 features x 32 rows through its
//             own patch of shared memory so that rows leave in 16-byte stores
// NB: feature tiles of 128 per block in mode 0 (they share the row tile); mode 1 has gate and up.
template <int MODE, int TN, int STAGES, int NB>
__global__ void __launch_bounds__(192, 1)
grouped_gemm_tc_persistent_kernel(const __grid_constant__ RowMaps maps_a, const __grid_constant__ CUtensorMap map_w,
                                  const int* __restrict__ offsets, void* __restrict__ C, int E, int Nout, int Kd,
                                  int* __restrict__ status) {
    constexpr int NW = MODE == 1 ? 2 : NB;                // weight tiles per stage = accumulators per tile
    constexpr int STAGE_BYTES = NW * W_TILE_BYTES + TN * BK * 2;
    constexpr int FEATS = MODE == 1 ? BF : NB * BF;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int OUT_BYTES = MODE == 1 ? 2 : 4;
    constexpr int PER16 = 16 / OUT_BYTES;                 // features per 16-byte group
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_full[2], accum_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s, row_tiles_s;
    constexpr int TURN_ROWS = MODE == 1 ? 32 : 16;        // rows of a warp's patch: 2 KiB either way
    __shared__ __align__(16) uint8_t turn_s[4][TURN_ROWS * 32 * OUT_BYTES];   // per epilogue warp: [rows][32 features]

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    int2* table = reinterpret_cast<int2*>(smem + (size_t)STAGES * STAGE_BYTES);   // .x first row, .y expert << 16 | rows
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&accum_full[s], 1); mbar_init(&accum_empty[s], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        int base = 0;                                     // row tiles of the experts before this round of 32
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            int b0 = 0, cnt = 0;
            if (e < E) { b0 = offsets[e]; cnt = offsets[e + 1] - b0; }
            const int tiles = (cnt + TN - 1) / TN;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            if (tiles > 0) {
                const int per = ((cnt + tiles - 1) / tiles + 15) & ~15;          // an even split, whole MMA columns
                for (int j = 0; j < tiles; ++j)
                    table[base + incl - tiles + j] = make_int2(b0 + j * per, (e << 16) | max(0, min(per, cnt - j * per)));
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) row_tiles_s = base;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    const int n_feat = (Nout + FEATS - 1) / FEATS;
    const int total = row_tiles_s * n_feat;
    const int wrows = MODE == 1 ? 2 * Nout : Nout;
    const int num_kb = Kd / BK;
    // accumulator b of a tile with `n_mma` columns: tensor-memory columns col0 + b * pitch .. + n_mma, with
    // pitch = n_mma rounded up to 32 and col0 = 0 (even tiles of this block) or 512 - NW * pitch (odd)

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;                              // k blocks so far, over all tiles of this block
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                const int r = tile / n_feat, n0 = (tile - r * n_feat) * FEATS;
                const int2 ent = table[r];
                const int rows = ent.y & 0xffff, e = ent.y >> 16, row0 = ent.x;
                if (rows == 0) continue;
                const int n_mma = (rows + 15) & ~15;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t parity = ((it / STAGES) & 1) ^ 1;
                    ok = mbar_wait(&empty_bar[s], parity, abort_flag, 1);
                    if (!ok) break;
                    uint8_t* st = smem + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], NW * W_TILE_BYTES + (uint32_t)n_mma * BK * 2);
#pragma unroll
                    for (int b = 0; b < NW; ++b)
                        tma_load_2d(st + b * W_TILE_BYTES, &map_w, kb * BK,
                                    e * wrows + (MODE == 1 ? b * Nout + n0 : n0 + b * BF), &full_bar[s]);
                    for (int done = 0; done < n_mma;) {
                        const int left = n_mma - done;
                        const int b = left >= 256 ? 4 : (left >= 128 ? 3 : (left >= 64 ? 2 : (left >= 32 ? 1 : 0)));
                        tma_load_2d(st + NW * W_TILE_BYTES + done * (BK * 2), &maps_a.m[b], kb * BK, row0 + done,
                                    &full_bar[s]);
                        done += 16 << b;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, i = 0;                       // k blocks and tiles of this block so far
            int width_before = 0;                         // columns of the tile before
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                const int rows = table[tile / n_feat].y & 0xffff;
                if (rows == 0) continue;
                const int n_mma = (rows + 15) & ~15, pitch = (n_mma + 31) & ~31, width = NW * pitch;
                const uint32_t side = i & 1;
                const uint32_t col0 = tmem_base + (side ? 512 - width : 0);
                const uint32_t idesc = IDESC_BASE | ((uint32_t)(n_mma >> 3) << 17);
                // this side is free once the epilogue warps have read tile i - 2; the other side's tile
                // i - 1 must have been read too if the two tiles overlap
                ok = mbar_wait(&accum_empty[side], ((i >> 1) & 1) ^ 1, abort_flag, 4);
                if (ok && i > 0 && width_before + width > 512)
                    ok = mbar_wait(&accum_empty[side ^ 1], ((i - 1) >> 1) & 1, abort_flag, 5);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t w_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint32_t r_addr = w_addr + NW * W_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        const uint64_t rd = umma_desc(r_addr + k * 32);
#pragma unroll
                        for (int b = 0; b < NW; ++b)
                            umma_bf16(col0 + b * pitch, umma_desc(w_addr + b * W_TILE_BYTES + k * 32), rd, idesc, acc);
                    }
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&accum_full[side]);
                width_before = width;
                ++i;
            }
        }
    } else {
        const int quarter = warp & 3;
        const int fl = quarter * 32 + lane;
        const bool staged = (Nout % PER16) == 0 && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        uint8_t* turn = turn_s[quarter];
        uint32_t i = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
            const int r = tile / n_feat, n0 = (tile - r * n_feat) * FEATS;
            const int2 ent = table[r];
            const int rows = ent.y & 0xffff, row0 = ent.x;
            if (rows == 0) continue;
            const int n_mma = (rows + 15) & ~15, pitch = (n_mma + 31) & ~31, width = NW * pitch;
            const uint32_t side = i & 1;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (side ? 512 - width : 0);
            ok = mbar_wait(&accum_full[side], (i >> 1) & 1, abort_flag, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int half = 0; half < (MODE == 1 ? 1 : NB); ++half) {
                const int fbase = n0 + half * BF;
                if (fbase >= Nout) break;
                const int f = fbase + fl;
#pragma unroll 1
                for (int c0 = 0; c0 < rows; c0 += 32) {
                    uint32_t g[32];
                    tmem_ld32(lane_addr + half * pitch + c0, g);
                    if (MODE == 1) {
                        uint32_t u[32];
                        tmem_ld32(lane_addr + pitch + c0, u);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float gv = __uint_as_float(g[j]);
                            // the result is rounded to bfloat16: the fast exponential and division are exact enough
                            g[j] = (uint32_t)__bfloat16_as_ushort(
                                __float2bfloat16_rn(__fdividef(gv, 1.0f + __expf(-gv)) * __uint_as_float(u[j])));
                        }
                    } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    }
                    if (staged) {
                        constexpr int GROUPS = 32 / PER16;                // 16-byte groups per row of the patch
                        const uint4* src = reinterpret_cast<const uint4*>(turn);
                        uint8_t* dst = reinterpret_cast<uint8_t*>(C);
#pragma unroll
                        for (int h0 = 0; h0 < 32; h0 += TURN_ROWS) {
                            __syncwarp();                                 // the patch's readers of the round before
                            if (MODE == 1) {
                                __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(turn) + lane;
#pragma unroll
                                for (int j = 0; j < TURN_ROWS; ++j) st[j * 32] = __ushort_as_bfloat16((unsigned short)g[h0 + j]);
                            } else {
                                float* st = reinterpret_cast<float*>(turn) + lane;
#pragma unroll
                                for (int j = 0; j < TURN_ROWS; ++j) st[j * 32] = __uint_as_float(g[h0 + j]);
                            }
                            __syncwarp();
#pragma unroll
                            for (int q = 0; q < TURN_ROWS * GROUPS / 32; ++q) {
                                const int idx = q * 32 + lane;
                                const int rr = h0 + idx / GROUPS, gq = idx % GROUPS;
                                const int feat = fbase + quarter * 32 + gq * PER16;
                                if (c0 + rr < rows && feat < Nout)
                                    *reinterpret_cast<uint4*>(dst + ((int64_t)(row0 + c0 + rr) * Nout + feat) * OUT_BYTES) = src[idx];
                            }
                        }
                    } else if (f < Nout) {
                        if (MODE == 1) {
                            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C) + (int64_t)(row0 + c0) * Nout + f;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (c0 + j < rows) out[(int64_t)j * Nout] = __ushort_as_bfloat16((unsigned short)g[j]);
                        } else {
                            float* out = reinterpret_cast<float*>(C) + (int64_t)(row0 + c0) * Nout + f;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (c0 + j < rows) out[(int64_t)j * Nout] = __uint_as_float(g[j]);
                        }
                    }
                }
            }
            // this warp has read its quarter of the tile's accumulators
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&accum_empty[side]);
            ++i;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_s != 0) atomicMax(status, abort_s);
}

// out[r, :] = x[rows[r], :]  (bfloat16, 16 bytes per thread and step)
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ rows, uint4* __restrict__ out,
                                   int vec_per_row) {
    const int r = blockIdx.x;
    const uint4* src = x + (int64_t)rows[r] * vec_per_row;
    uint4* dst = out + (int64_t)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
}

}  // namespace tc
}  // namespace mi

using namespace mi;

extern "C" {

// 1 if the prefill-sized tensor-core grouped product takes these sizes.
int mi_grouped_gemm_tc_supported(int Kd) { return (Kd > 0 && Kd % tc::BK == 0) ? 1 : 0; }

int mi_gather_rows_bf16(const void* x, const int* rows, void* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return kOk;
    if (width % 8) {
        set_last_error("gather_rows: width %d is not a multiple of 8", width);
        return kBadShape;
    }
    tc::gather_rows_kernel<<<n_rows, 128, 0, stream>>>((const uint4*)x, rows, (uint4*)out, width / 8);
    return finish_launch("gather_rows");
}

// Shared memory a persistent form needs beside its static part: alignment slack, the pipeline and
// the table of row tiles (one entry per tile; n_rows / tn + E bounds their number).
static size_t persistent_smem(int tn, int stages, int nw, int n_rows, int E) {
    return 1024 + (size_t)stages * (nw * tc::W_TILE_BYTES + tn * tc::BK * 2) + ((size_t)n_rows / tn + E) * sizeof(int2);
}
constexpr size_t kPersistentSmemLimit = 232448 - 8704;    // 227 KiB less the kernel's static shared memory

// For the test of the bounded waits: the next launch of a one-block-per-tile form (form 0 or 1) stops loading
// at k block `skip_kb` and gives every wait `wait_limit` rounds, so that a wait runs out, the
// kernel returns by itself and the status word reports it.  Nothing else is changed; the launch after
// that is a normal one again.
static int g_test_skip_kb = -1;
static uint32_t g_test_wait_limit = 0;
void mi_grouped_gemm_tc_test_fault(int skip_kb, unsigned int wait_limit) {
    g_test_skip_kb = skip_kb;
    g_test_wait_limit = wait_limit;
}

// A: [n_rows, Kd] bfloat16, rows sorted by expert (offsets[E+1]); W: [E, wrows, Kd] bfloat16.
// mode 1: C bfloat16 [n_rows, Nout] = silu(gate) * up with W holding 2*Nout rows per expert;
// mode 0: C float [n_rows, Nout].  `status` (device int, zero before the first call) receives a
// non-zero code if a wait inside the kernel ran out.
// form: -1 chooses; 0 / 1 one block per tile with row tiles of 128 (two blocks per SM) / 256;
//       2 / 3 persistent with row tiles of 160 and four pipeline stages / 256 and three.
int mi_grouped_gemm_tc_form(const void* A, const void* W, const int* offsets, void* C, int* status, int n_rows,
                            int E, int Nout, int Kd, int mode, int form, cudaStream_t stream) {
    if (n_rows <= 0) return kOk;
    if (!mi_grouped_gemm_tc_supported(Kd)) {
        set_last_error("grouped product (tensor cores): inner size %d is not a multiple of %d", Kd, tc::BK);
        return kBadShape;
    }
    if (form < -1 || form > 3) {
        set_last_error("grouped product (tensor cores): no form %d", form);
        return kBadShape;
    }
    const int wrows = mode == 1 ? 2 * Nout : Nout;
    // Measured on B200 (60 experts, 2048 x 1408): the persistent forms win everywhere; four stages
    // win while an expert's rows make one or two row tiles of 160, the larger tile otherwise.
    // With few rows per expert the product is bound by reading the weights once, and single feature
    // tiles in mode 0 spread that more evenly over the SMs.
    const double per_expert = (double)n_rows / E;
    const int nb160 = per_expert <= 170.0 ? 1 : 2;        // feature tiles per block in mode 0, form 2
    const bool fits2 = E < 32768 && persistent_smem(160, 4, mode == 1 ? 2 : nb160, n_rows, E) <= kPersistentSmemLimit;
    const bool fits3 = E < 32768 && persistent_smem(256, 3, 2, n_rows, E) <= kPersistentSmemLimit;
    if (form == -1) {
        const bool want2 = per_expert <= 170.0 || (per_expert > 256.0 && per_expert <= 330.0);
        if (want2 && fits2) form = 2;
        else if (fits3) form = 3;
        else form = (int64_t)n_rows <= (int64_t)160 * E ? 0 : 1;
    }
    if ((form == 2 && !fits2) || (form == 3 && !fits3)) {
        set_last_error("grouped product (tensor cores): %d rows of %d experts exceed the persistent form's table",
                       n_rows, E);
        return kBadShape;
    }
    const int tn = form == 0 ? 128 : 256;
    const int max_tiles = (n_rows + tn - 1) / tn + E;
    if (form < 2 && max_tiles > 65535) {
        set_last_error("grouped product (tensor cores): %d row tiles exceed the grid limit", max_tiles);
        return kBadShape;
    }
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) {
        set_last_error("grouped product (tensor cores): operands must be 16-byte aligned");
        return kBadShape;
    }
    tc::RowMaps maps_a;
    CUtensorMap map_w;
    bool ok = tc::make_map(&map_w, W, (uint64_t)E * wrows, (uint64_t)Kd, tc::BF);
    for (int i = 0; i < 5 && ok; ++i) ok = tc::make_map(&maps_a.m[i], A, (uint64_t)n_rows, (uint64_t)Kd, 16u << i);
    if (!ok) {
        set_last_error("grouped product (tensor cores): cuTensorMapEncodeTiled failed");
        return kLaunchFailed;
    }
    if (form >= 2) {
        static int num_sms = 0;
        if (num_sms == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        }
        const int ptn = form == 2 ? 160 : 256, nb = form == 2 ? nb160 : 2;
        const int feats = mode == 1 ? tc::BF : nb * tc::BF;
        const int64_t tiles = ((int64_t)n_rows / ptn + E) * ((Nout + feats - 1) / feats);
        const size_t smem = persistent_smem(ptn, form == 2 ? 4 : 3, mode == 1 ? 2 : nb, n_rows, E);
        const int blocks = (int)(tiles < num_sms ? tiles : num_sms);
#define MI_TCP_LAUNCH(MODE, TN, ST, NB)                                                               \
    do {                                                                                              \
        auto kern = tc::grouped_gemm_tc_persistent_kernel<MODE, TN, ST, NB>;                          \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        kern<<<blocks, 192, smem, stream>>>(maps_a, map_w, offsets, C, E, Nout, Kd, status);          \
    } while (0)
        if (form == 3) { if (mode == 1) MI_TCP_LAUNCH(1, 256, 3, 2); else MI_TCP_LAUNCH(0, 256, 3, 2); }
        else if (mode == 1) MI_TCP_LAUNCH(1, 160, 4, 2);
        else if (nb == 1) MI_TCP_LAUNCH(0, 160, 4, 1);
        else MI_TCP_LAUNCH(0, 160, 4, 2);
#undef MI_TCP_LAUNCH
        return finish_launch("grouped_gemm_tc");
    }
    const int feats = mode == 1 ? tc::BF : 2 * tc::BF;
    const dim3 grid((Nout + feats - 1) / feats, max_tiles);
    const int skip_kb = g_test_skip_kb;
    const uint32_t wait_limit = g_test_wait_limit ? g_test_wait_limit : tc::WAIT_LIMIT;
    g_test_skip_kb = -1;                                  // a test's fault holds for one launch
    g_test_wait_limit = 0;
#define MI_TC_LAUNCH(MODE, TN, STAGES, BLOCKS)                                                         \
    do {                                                                                               \
        const size_t smem = STAGES * (size_t)(2 * tc::W_TILE_BYTES + TN * tc::BK * 2) + 1024;          \
        auto kern = tc::grouped_gemm_tc_kernel<MODE, TN, STAGES, BLOCKS>;                              \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
        kern<<<grid, 192, smem, stream>>>(maps_a, map_w, offsets, C, E, Nout, Kd, status, skip_kb,     \
                                          wait_limit);                                                 \
    } while (0)
    if (form == 0) {
        if (mode == 1) MI_TC_LAUNCH(1, 128, 2, 2); else MI_TC_LAUNCH(0, 128, 2, 2);
    } else {
        if (mode == 1) MI_TC_LAUNCH(1, 256, 3, 1); else MI_TC_LAUNCH(0, 256, 3, 1);
    }
#undef MI_TC_LAUNCH
    return finish_launch("grouped_gemm_tc");
}

int mi_grouped_gemm_tc(const void* A, const void* W, const int* offsets, void* C, int* status, int n_rows, int E,
                       int Nout, int Kd, int mode, cudaStream_t stream) {
    return mi_grouped_gemm_tc_form(A, W, offsets, C, status, n_rows, E, Nout, Kd, mode, -1, stream);
}

}  // extern "C"
