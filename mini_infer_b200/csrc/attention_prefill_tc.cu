// Prefill attention on the fifth-generation tensor cores (bfloat16, head size 64 or 128): portions
// of prompts of a ragged batch over the paged cache, flash-attention style, with both products on
// tcgen05.mma and their accumulators in tensor memory.
//
// Block = 128 queries of one head; two blocks share an SM, so that one's softmax runs beside the
// other's tensor-core work.  Key tiles of 64, aligned to absolute positions, arrive page by page
// through TMA (128-byte swizzle) into rings of three K and two V tiles.  Per key tile:
//   S = Q K^T    A = Q tile (K-major), B = K tile (K-major), accumulator S[buf] in tensor memory
//   softmax      one thread per query row (a row is a lane of tensor memory, so the row maximum and
//                sum need no exchange between threads): the row of S comes to registers with
//                tcgen05.ld, P = exp2(s - reference) is rounded to bfloat16 and written over S in
//                place with tcgen05.st (two keys per 32-bit column); the reference follows the
//                running maximum only when that moved by more than 8 (P stays below 2^8), and only
//                then O is scaled in place (tcgen05.ld / .st)
//   O += P V     A = P straight from tensor memory, B = V tile as it lies in the cache (keys x head,
//                i.e. MN-major), accumulator O in tensor memory
//   warp 0    TMA producer (Q once; K and V tiles of every key tile, one copy per page and 64 columns)
//   warp 1    allocates tensor memory, issues the MMAs
//   warps 2-5 softmax and epilogue, one lane quarter of tensor memory each
// S is double-buffered, so the next tile's S = Q K^T runs beside this tile's softmax.  Masking is positional: key j is visible from the
// query at position p iff j <= p and (window == 0 or j > p - window) and j < kv_len.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets an error status that the host
// reads, lets all roles fall through to the common exit, and the tensor memory is freed there.
//
// The reference computes prefill with one block per (request, head, query) and scalar dot
// products over every page of the request (src/kernels/paged_attn_kernel.cu:102-288).

#include "tcgen05.cuh"

namespace mi {
namespace pt {

using namespace mi::tc;

constexpr int BQ = 128;            // queries per block (MMA M)
constexpr int BN = 64;             // keys per tile
constexpr int NK = 3;              // stages of the K ring
constexpr int NV = 2;              // stages of the V ring
constexpr int HALF_BYTES = 128 * 64 * 2;   // a tile of 128 rows x 64 columns: 16 KiB (Q, P)
constexpr int KV_HALF = BN * 64 * 2;       // a tile of BN keys x 64 columns: 8 KiB

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Matrix descriptor of an MN-major operand with 128-byte swizzle: rows of 128 bytes are steps of the
// contraction index, 8 of them 1024 B apart (stride byte offset); the next 64 elements of the
// non-contracted index lie `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// tcgen05.mma with the A operand in tensor memory (lane = row, a 32-bit column holds two bfloat16 of
// consecutive k) and B in shared memory.
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mbar_arrive_after_tmem(uint64_t* bar) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    mbar_arrive(bar);
}

struct Maps {
    CUtensorMap q, k, v;
};

template <int D>
__global__ void __launch_bounds__(192, 2)
attn_prefill_tc_kernel(const __grid_constant__ Maps maps, const int* __restrict__ block_table,
                       const int* __restrict__ q_start, const int* __restrict__ kv_len,
                       __nv_bfloat16* __restrict__ out, int nh, int nkv, int page_size, int max_pages,
                       int window, float scale_log2, int* __restrict__ status) {
    constexpr int DH = D / 64;                            // 64-column halves of a head
    constexpr uint32_t TMEM_COLS = 256;                   // S[0], S[1] (BN columns each), O (D): two blocks share an SM
    constexpr uint32_t COL_S = 0, COL_O = 2 * BN;
    // instruction descriptors: D float32, A and B bfloat16, M = 128
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((128u >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) |
                                  ((128u >> 4) << 24);    // B (the V tile) MN-major
    extern __shared__ __align__(1024) uint8_t smem[];     // tiles first (the swizzle wants 1024-byte alignment)
    uint8_t* sQ = smem;                                   // DH halves of [128 queries][64]
    uint8_t* sK = sQ + DH * HALF_BYTES;                   // NK stages of DH halves of [BN keys][64]
    uint8_t* sV = sK + NK * DH * KV_HALF;                 // NV stages of the same for V
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NV * DH * KV_HALF);
    uint64_t* q_full = bars;                              // then the barriers and a few words
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = k_full + NK;
    uint64_t* k_empty = v_full + NV;
    uint64_t* v_empty = k_empty + NK;
    uint64_t* s_full = v_empty + NV;
    uint64_t* p_full = s_full + 2;                        // per S/P buffer: the softmax may be a tile ahead
    uint64_t* o_done = p_full + 2;
    uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(o_done + 1);
    int* abort_p = reinterpret_cast<int*>(tmem_base_p + 1);
    int* tile_pages = abort_p + 1;                        // BN / 8 entries

    // later query tiles see more keys: they are launched first, so that the short ones fill the tail
    const int b = blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;
    const int q0 = q_start[b], q_len = q_start[b + 1] - q0;
    if (qt * BQ >= q_len) return;                         // uniform for the whole block
    const int kvl = kv_len[b];
    const int hk = h / (nh / nkv);
    const int nq = min(BQ, q_len - qt * BQ);
    const int p_lo = kvl - q_len + qt * BQ;               // position of the tile's first query
    const int p_hi = p_lo + nq - 1;
    int k_begin = 0;
    if (window > 0) k_begin = max(0, p_lo - window + 1);
    k_begin = (k_begin / BN) * BN;
    const int k_end = min(kvl, p_hi + 1);
    const int n_tiles = (k_end - k_begin + BN - 1) / BN;  // >= 1: the query's own key is visible

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = abort_p;

    if (threadIdx.x == 0) {
        *abort_p = (smem_u32(smem) & 1023u) ? 10 : 0;     // misplaced tiles: nothing is issued
        mbar_init(q_full, 1);
        for (int s = 0; s < NK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < NV; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 128); }
        mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Key and value stages start as zeros: rows that no copy fills (pages a window has released, the
    // end of the last tile) are masked in S, and P = 0 times a finite stale value is 0.
    for (int i = threadIdx.x; i < (NK + NV) * DH * KV_HALF / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(sK)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_base_p)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_base_p;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, DH * HALF_BYTES);
            for (int hh = 0; hh < DH; ++hh)
                tma_load_2d(sQ + hh * HALF_BYTES, &maps.q, h * D + hh * 64, q0 + qt * BQ, q_full);
        }
        const int* table = block_table + (int64_t)b * max_pages;
        const int pages_per_tile = BN / page_size;
        const uint32_t page_bytes = (uint32_t)page_size * 128u;
        const int items = pages_per_tile * DH;            // page x 64-column half: one copy each
        // One tile of K or of V: wait for its stage, look its pages up, copy those that exist (inside the
        // request, not released by a window).  A K stage is free once S = Q K^T of two tiles before has
        // run, a V stage once O += P V of two tiles before has: K runs a tile ahead of V.
        auto load_tile = [&](int j, bool is_k) -> bool {
            const int ns = is_k ? NK : NV;
            const int s = j % ns;
            const uint32_t parity = ((j / ns) & 1) ^ 1;
            const int k0 = k_begin + j * BN;
            int my_page = -1;                             // looked up before the wait: the latencies overlap
            if (lane < pages_per_tile) {
                const int kpos = k0 + lane * page_size;
                if (kpos < kvl) my_page = table[kpos / page_size];
            }
            bool ok = true;
            if (lane == 0) ok = mbar_wait(is_k ? &k_empty[s] : &v_empty[s], parity, abort_flag, is_k ? 11 : 21);
            if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
            const unsigned have = __ballot_sync(0xffffffffu, my_page >= 0);
            if (lane < pages_per_tile) tile_pages[lane] = my_page;
            uint64_t* bar = is_k ? &k_full[s] : &v_full[s];
            if (lane == 0) mbar_expect_tx(bar, (uint32_t)__popc(have) * page_bytes * DH);
            __syncwarp();
            for (int it = lane; it < items; it += 32) {
                const int pg = it / DH, hh = it - pg * DH;
                const int page = tile_pages[pg];
                if (page < 0) continue;
                const int row = (page * nkv + hk) * page_size;
                uint8_t* dst = (is_k ? sK : sV) + (size_t)s * DH * KV_HALF + hh * KV_HALF + (size_t)pg * page_bytes;
                tma_load_2d(dst, is_k ? &maps.k : &maps.v, hh * 64, row, bar);
            }
            __syncwarp();                                 // tile_pages is rewritten by the next call
            return true;
        };
        for (int i = 0; i <= n_tiles + 1; ++i) {          // K runs two tiles ahead of V
            if (i < n_tiles && !load_tile(i, true)) break;
            if (i >= 2 && !load_tile(i - 2, false)) break;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = *abort_flag == 0 && mbar_wait(q_full, 0, abort_flag, 12);
            // descriptors of the tile origins; an offset of b bytes inside a tile adds b / 16 to the address field
            const uint64_t dq = umma_desc(smem_u32(sQ));
            // S of tile j goes to buffer j & 1.  P of tile j overwrites S of tile j in place (bfloat16, two
            // keys per 32-bit column) and is the A operand of O += P V straight from tensor memory; S of
            // tile j + 2 goes to the same buffer and is issued once O += P V of tile j is complete.
            auto issue_s = [&](int j) -> bool {
                const int s = j % NK, buf = j & 1;
                if (!mbar_wait(&k_full[s], (j / NK) & 1, abort_flag, 13)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dks = umma_desc(smem_u32(sK + (size_t)s * DH * KV_HALF));
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t sub = (uint32_t)(kk & 3) * 32;
                    umma_bf16(tmem_base + COL_S + buf * BN, dq + (((uint32_t)(kk >> 2) * HALF_BYTES + sub) >> 4),
                              dks + (((uint32_t)(kk >> 2) * KV_HALF + sub) >> 4), IDESC_S, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[buf]);
                umma_commit(&k_empty[s]);                 // the K stage is free once these MMAs have read it
                return true;
            };
            if (ok) ok = issue_s(0);
            if (ok && n_tiles > 1) ok = issue_s(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % NV, buf = j & 1;
                ok = mbar_wait(&p_full[buf], (j >> 1) & 1, abort_flag, 15) &&
                     mbar_wait(&v_full[s], (j / NV) & 1, abort_flag, 16);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dvs = umma_desc_mn(smem_u32(sV + (size_t)s * DH * KV_HALF), KV_HALF);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)     // 16 keys of P are 8 columns of tensor memory
                    umma_bf16_tmem_a(tmem_base + COL_O, tmem_base + COL_S + buf * BN + ks * 8,
                                     dvs + (((uint32_t)ks * 2048) >> 4), IDESC_PV, (j > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&v_empty[s]);                 // the V stage is free once these MMAs have read it
                umma_commit(o_done);                      // O holds tile j
                if (j + 2 < n_tiles) ok = mbar_wait(o_done, j & 1, abort_flag, 14) && issue_s(j + 2);
            }
        }
    } else {
        // softmax and epilogue: thread = query row = tensor-memory lane
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int p_row = p_lo + r;                       // position of this thread's query
        const int vis_hi = min(p_row, kvl - 1);           // last visible key
        const int vis_lo = window > 0 ? p_row - window + 1 : 0;   // first visible key
        float m_ref = -INFINITY;                          // reference of the exponentials, in log2 units
        float l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int buf = j & 1;
            const int k0 = k_begin + j * BN;
            ok = mbar_wait(&s_full[buf], (j >> 1) & 1, abort_flag, 17);
            ok = __all_sync(0xffffffffu, ok);             // tcgen05.ld and .st are warp-wide: all lanes or none
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the whole row of S to registers; the buffer is free for the tile after next at once
            uint32_t v[BN];
            const uint32_t s_addr = lane_addr + COL_S + buf * BN;
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32) tmem_ld32(s_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&v[c0]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // does any (row, key) of this tile need the mask?
            const bool masked = (k0 + BN - 1 > p_lo) || (k0 + BN > kvl) || (window > 0 && k0 < p_hi - window + 1);
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one of BN steps
            if (masked) {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const int kj = k0 + i;
                    if (kj > vis_hi || kj < vis_lo) v[i] = 0xff800000u;                 // -inf
                    mxs[i & 3] = fmaxf(mxs[i & 3], __uint_as_float(v[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < BN; ++i) mxs[i & 3] = fmaxf(mxs[i & 3], __uint_as_float(v[i]));
            }
            // the scale is positive: the maximum of the scaled scores is the scaled maximum
            const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * scale_log2;
            // the reference follows the maximum only when that moved by more than 8: exponentials stay
            // below 2^8, and O needs scaling only then
            float alpha = 1.f;
            if (mx > m_ref + 8.f || (m_ref == -INFINITY && mx > -INFINITY)) {
                alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx);
                m_ref = mx;
            }
            const float base = m_ref == -INFINITY ? 0.f : m_ref;
            float sums[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[BN / 2];
#pragma unroll
            for (int i = 0; i < BN; i += 2) {
                const float e0 = fast_exp2(fmaf(__uint_as_float(v[i]), scale_log2, -base));
                const float e1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), scale_log2, -base));
                sums[(i >> 1) & 3] += e0 + e1;
                pk[i >> 1] = pack_bf16(e0, e1);
            }
            l_run = l_run * alpha + ((sums[0] + sums[1]) + (sums[2] + sums[3]));
            // O is scaled only after the O += P V of tile j - 1 is complete
            const bool rescale = j > 0 && !__all_sync(0xffffffffu, alpha == 1.f);
            if (rescale) ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, 18);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (rescale) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(lane_addr + COL_O + c0, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_addr + COL_O + c0, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // Follow the O += P V barrier phase by phase, and do so BEFORE this tile's P is handed over:
            // O += P V of tile j cannot complete before every thread has arrived below, so the barrier
            // cannot run a second phase ahead of a thread that has not yet seen tile j - 1 complete (a
            // parity wait that falls two phases behind never returns).  The product of tile j - 1 was
            // issued a tile ago, so this seldom waits.
            if (j > 0) {
                ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, 19);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            // P over S in place: 64 keys are 32 columns of two bfloat16 each
            tmem_st32(s_addr, pk);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            mbar_arrive_after_tmem(&p_full[buf]);
        }
        if (ok) {
            ok = mbar_wait(o_done, (n_tiles - 1) & 1, abort_flag, 20);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* dst = out + ((int64_t)(q0 + qt * BQ + r) * nh + h) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(lane_addr + COL_O + c0, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < nq) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + i) = w;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_p != 0) atomicMax(status, *abort_p);
}

// Row-major bfloat16 matrix [rows, cols] with a row pitch of `pitch` elements, box of 64 columns x
// box_rows rows, 128-byte swizzle.
static bool make_map_pitched(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch,
                             uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pt
}  // namespace mi

using namespace mi;

extern "C" {

// 1 if the tcgen05 prefill attention takes this geometry: head size 64 or 128; pages of 8, 16, 32 or 64
// tokens (a page is one TMA box of whole 8-row swizzle groups, and pages tile a key tile).
int mi_attn_prefill_tc_supported(int d, int page_size) {
    const bool ps_ok = page_size >= 8 && page_size <= pt::BN && (page_size & (page_size - 1)) == 0;
    return ((d == 64 || d == 128) && ps_ok) ? 1 : 0;
}

// q [T, nh, d], out [T, nh, d] bfloat16; k_cache, v_cache one layer's [num_pages, nkv, page_size, d].
// `status` (device int, zero before the first call) receives a non-zero code if a wait inside the
// kernel ran out.
int mi_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                       const int* q_start, const int* kv_len, void* out, int* status, int T, int B, int max_q_len,
                       int nh, int nkv, int d, int page_size, int num_pages, int max_pages, int window, float scale,
                       cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0 || T <= 0) return kOk;
    if (!mi_attn_prefill_tc_supported(d, page_size)) {
        set_last_error("prefill attention (tcgen05): head_dim %d with pages of %d tokens is not taken", d, page_size);
        return kBadShape;
    }
    if (nkv < 1 || nh % nkv != 0) {
        set_last_error("attention: %d query heads are not a multiple of %d key/value heads", nh, nkv);
        return kBadShape;
    }
    if (B > 65535 || nh > 65535) {
        set_last_error("attention: batch %d or head count %d exceeds the grid limit 65535", B, nh);
        return kBadShape;
    }
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(out)) & 15) {
        set_last_error("prefill attention (tcgen05): operands must be 16-byte aligned");
        return kBadShape;
    }
    pt::Maps maps;
    const uint64_t cache_rows = (uint64_t)num_pages * nkv * page_size;
    bool ok = pt::make_map_pitched(&maps.q, q, (uint64_t)T, (uint64_t)nh * d, (uint64_t)nh * d, pt::BQ) &&
              pt::make_map_pitched(&maps.k, k_cache, cache_rows, (uint64_t)d, (uint64_t)d, (uint32_t)page_size) &&
              pt::make_map_pitched(&maps.v, v_cache, cache_rows, (uint64_t)d, (uint64_t)d, (uint32_t)page_size);
    if (!ok) {
        set_last_error("prefill attention (tcgen05): cuTensorMapEncodeTiled failed");
        return kLaunchFailed;
    }
    const dim3 grid((max_q_len + pt::BQ - 1) / pt::BQ, nh, B);
    const float scale_log2 = scale * 1.4426950408889634f;
    const int dh = d / 64;
    const size_t smem = (size_t)dh * pt::HALF_BYTES + (size_t)(pt::NK + pt::NV) * dh * pt::KV_HALF + 256;
#define MI_PT(DD)                                                                                         \
    do {                                                                                                  \
        auto kern = pt::attn_prefill_tc_kernel<DD>;                                                       \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
        kern<<<grid, 192, smem, stream>>>(maps, block_table, q_start, kv_len, (__nv_bfloat16*)out, nh,    \
                                          nkv, page_size, max_pages, window, scale_log2, status);         \
    } while (0)
    if (d == 64) MI_PT(64); else MI_PT(128);
#undef MI_PT
    return finish_launch("attn_prefill_tc");
}

}  // extern "C"
