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

#include "common.cuh"

#include <cuda.h>

namespace mi {
namespace tc {

constexpr int BF = 128;                        // features per tile (MMA M)
constexpr int BK = 64;                         // k per pipeline stage (one 128-byte swizzle row)
constexpr int W_TILE_BYTES = BF * BK * 2;      // one weight tile of one stage: 16 KiB
constexpr uint32_t WAIT_LIMIT = 400000;        // try_wait rounds before a wait gives up
// instruction descriptor without N: D float32, A and B bfloat16, both K-major, M = 128
constexpr uint32_t IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BF >> 4) << 24);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if it gave up or another role already did.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (it > 2048) __nanosleep(128);
    }
    *abort_flag = code;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows at a pitch of 128 B,
// groups of 8 rows 1024 B apart (stride byte offset), leading byte offset unused (1), version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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
}

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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Row-major bfloat16 matrix [rows, cols], box of 64 columns x box_rows rows, 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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
