// Grouped expert products for prefill-sized batches on the fifth-generation tensor cores:
// tcgen05.mma with both operands in shared memory (fed by TMA, 128-byte swizzle) and the
// accumulators in tensor memory, read back with tcgen05.ld for the epilogue.
//
// Rows are the (token, slot) pairs sorted by expert and gathered into a contiguous matrix, so
// an expert's rows are the contiguous range offsets[e] .. offsets[e+1].  The product is computed
// transposed: the expert's weights are the M operand (128 features per tile) and the rows are the
// N operand, whose size follows the expert's row count (a multiple of 16 up to the tile limit TN of
// 128 or 256 rows): an expert with 137 rows is one tile with N = 144 under TN = 256, or a tile of 128
// and one of 16 under TN = 128, where two blocks share an SM.  One block computes one (expert, row
// tile, feature tile) with two accumulators: gate and up of 128 features (mode 1), or two neighbouring
// tiles of 128 features that share the row tile (mode 0):
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

// The four row-tile maps differ in their box height only (32, 64, 128, 256 rows).
struct RowMaps {
    CUtensorMap m[4];
};

// MODE 1: C[r, n] = silu(a_r . W[e, n]) * (a_r . W[e, Nout + n])  (bfloat16); MODE 0: C[r, n] = a_r . W[e, n] (float)
// TN: rows per tile at most (128 or 256); STAGES: pipeline depth; BLOCKS: blocks meant to share an SM
// (with TN = 128 two blocks fit: while one drains its accumulators the other keeps the loads going).
template <int MODE, int TN, int STAGES, int BLOCKS>
__global__ void __launch_bounds__(192, BLOCKS)
grouped_gemm_tc_kernel(const __grid_constant__ RowMaps maps_a, const __grid_constant__ CUtensorMap map_w,
                       const int* __restrict__ offsets, void* __restrict__ C, int E, int Nout, int Kd,
                       int* __restrict__ status) {
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
    const int box = rows <= 32 ? 0 : (rows <= 64 ? 1 : (rows <= 128 ? 2 : 3));
    const uint32_t row_bytes = (32u << box) * BK * 2;     // bytes the row-tile copy delivers
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
                if (!mbar_wait(&empty_bar[s], parity, abort_flag, 1)) break;
                uint8_t* st = smem + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], NB * W_TILE_BYTES + row_bytes);
                tma_load_2d(st, &map_w, kb * BK, e * wrows + n0, &full_bar[s]);
                tma_load_2d(st + W_TILE_BYTES, &map_w, kb * BK, e * wrows + (MODE == 1 ? Nout + n0 : n0 + BF), &full_bar[s]);
                tma_load_2d(st + NB * W_TILE_BYTES, &maps_a.m[box], kb * BK, row0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = (kb / STAGES) & 1;
                ok = mbar_wait(&full_bar[s], parity, abort_flag, 2);
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
        bool ok = mbar_wait(&accum_bar, 0, abort_flag, 3);
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

// A: [n_rows, Kd] bfloat16, rows sorted by expert (offsets[E+1]); W: [E, wrows, Kd] bfloat16.
// mode 1: C bfloat16 [n_rows, Nout] = silu(gate) * up with W holding 2*Nout rows per expert;
// mode 0: C float [n_rows, Nout].  `status` (device int, zero before the first call) receives a
// non-zero code if a wait inside the kernel ran out.
int mi_grouped_gemm_tc(const void* A, const void* W, const int* offsets, void* C, int* status, int n_rows, int E,
                       int Nout, int Kd, int mode, cudaStream_t stream) {
    if (n_rows <= 0) return kOk;
    if (!mi_grouped_gemm_tc_supported(Kd)) {
        set_last_error("grouped product (tensor cores): inner size %d is not a multiple of %d", Kd, tc::BK);
        return kBadShape;
    }
    const int wrows = mode == 1 ? 2 * Nout : Nout;
    // Row tiles of 128 let two blocks share an SM (one drains its accumulators while the other loads),
    // but an expert with more rows than that is read once per row tile; measured on B200 the small
    // tile wins while the experts hold about one tile's worth of rows on average.
    const int variant = (int64_t)n_rows <= (int64_t)160 * E ? 0 : 1;
    const int tn = variant == 0 ? 128 : 256;
    const int max_tiles = (n_rows + tn - 1) / tn + E;
    if (max_tiles > 65535) {
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
    for (int i = 0; i < 4 && ok; ++i) ok = tc::make_map(&maps_a.m[i], A, (uint64_t)n_rows, (uint64_t)Kd, 32u << i);
    if (!ok) {
        set_last_error("grouped product (tensor cores): cuTensorMapEncodeTiled failed");
        return kLaunchFailed;
    }
    const int feats = mode == 1 ? tc::BF : 2 * tc::BF;
    const dim3 grid((Nout + feats - 1) / feats, max_tiles);
#define MI_TC_LAUNCH(MODE, TN, STAGES, BLOCKS)                                                         \
    do {                                                                                               \
        const size_t smem = STAGES * (size_t)(2 * tc::W_TILE_BYTES + TN * tc::BK * 2) + 1024;          \
        auto kern = tc::grouped_gemm_tc_kernel<MODE, TN, STAGES, BLOCKS>;                              \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
        kern<<<grid, 192, smem, stream>>>(maps_a, map_w, offsets, C, E, Nout, Kd, status);             \
    } while (0)
    if (variant == 0) {
        if (mode == 1) MI_TC_LAUNCH(1, 128, 2, 2); else MI_TC_LAUNCH(0, 128, 2, 2);
    } else {
        if (mode == 1) MI_TC_LAUNCH(1, 256, 3, 1); else MI_TC_LAUNCH(0, 256, 3, 1);
    }
#undef MI_TC_LAUNCH
    return finish_launch("grouped_gemm_tc");
}

}  // extern "C"
