// Prefill attention on tensor cores (bfloat16): portions of prompts of a ragged batch over the
// paged cache, flash-attention style.
//
// Block = 4 warps = 64 queries of one head (16 per warp, held as MMA fragments); key tiles of 64,
// aligned to absolute positions, are gathered page row by page row into shared memory with
// cp.async (three stages), S = Q K^T and O += P V run on mma.sync m16n8k16 with float
// accumulators, the softmax runs online in float on the accumulator fragments.  Masking is
// positional: key j is visible from the query at position p iff j <= p and (window == 0 or
// j > p - window); rows of keys that are masked for the whole tile are zero-filled.
//
// The reference computes prefill with one block per (request, head, query) and scalar dot
// products over every page of the request (src/kernels/paged_attn_kernel.cu:102-288).

#include "common.cuh"

namespace mi {
namespace pf {

constexpr int BQ = 64, BKEYS = 64, THREADS = 128, NSTAGE = 3;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Shared tiles are [rows][D] bfloat16 with the 16-byte chunks of a row XOR-swizzled by (row & 7).
template <int D>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                    const int* __restrict__ q_start, const int* __restrict__ kv_len, __nv_bfloat16* __restrict__ out,
                    int nh, int nkv, int page_size, int max_pages, int window, float scale_log2) {
    constexpr int CH = D / 8;          // 16-byte chunks per row
    constexpr int KS = D / 16;         // k-steps of S = Q K^T
    constexpr int DT = D / 8;          // n-tiles of O
    constexpr int TILE = BKEYS * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int64_t row_off[NSTAGE][BKEYS];

    // later query tiles see more keys: they are launched first, so that the short ones fill the tail
    const int b = blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;
    const int q0 = q_start[b], q_len = q_start[b + 1] - q0;
    if (qt * BQ >= q_len) return;
    const int kvl = kv_len[b];
    const int hk = h / (nh / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int nq = min(BQ, q_len - qt * BQ);
    const int p_lo = kvl - q_len + qt * BQ;            // position of the tile's first query
    const int p_hi = p_lo + nq - 1;

    // The Q tile borrows the last pipeline stage: it is turned into register fragments before the
    // first key tile that uses that stage is requested.
    static_assert(BQ * D * 2 <= 2 * TILE, "the Q tile must fit a pipeline stage");
    const uint32_t s0 = smem_u32(smem);
    auto sK = [&](int buf) { return s0 + (uint32_t)(2 * buf * TILE); };
    auto sV = [&](int buf) { return s0 + (uint32_t)(2 * buf * TILE + TILE); };
    const uint32_t sQ = sK(NSTAGE - 1);

    // ---- Q tile -> shared (rows beyond nq zero-filled) ---------------------------------------
    for (int idx = tid; idx < BQ * CH; idx += THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const bool valid = r < nq;
        const __nv_bfloat16* src = q + ((int64_t)(q0 + qt * BQ + (valid ? r : 0)) * nh + h) * D + c * 8;
        cp_async16(tile_addr<D>(sQ, r, c), src, valid);
    }
    cp_async_commit();

    int k_begin = 0;
    if (window > 0) k_begin = max(0, p_lo - window + 1);
    k_begin = (k_begin / BKEYS) * BKEYS;
    const int k_end = min(kvl, p_hi + 1);
    const int n_tiles = (k_end - k_begin + BKEYS - 1) / BKEYS;
    const int* table = block_table + (int64_t)b * max_pages;

    auto load_tile = [&](int ti, int buf) {
        const int kt = k_begin + ti * BKEYS;
        if (tid < BKEYS) {
            const int kj = kt + tid;
            int64_t off = -1;
            if (kj < k_end) {
                const int page = table[kj / page_size];
                if (page >= 0) off = ((int64_t)page * nkv + hk) * page_size * D + (int64_t)(kj % page_size) * D;
            }
            row_off[buf][tid] = off;
        }
        __syncthreads();
        for (int idx = tid; idx < BKEYS * CH; idx += THREADS) {
            const int r = idx / CH, c = idx - r * CH;
            const int64_t off = row_off[buf][r];
            const bool valid = off >= 0;
            const int64_t o = (valid ? off : 0) + c * 8;
            cp_async16(tile_addr<D>(sK(buf), r, c), k_cache + o, valid);
            cp_async16(tile_addr<D>(sV(buf), r, c), v_cache + o, valid);
        }
        cp_async_commit();
    };

    // prefetch distance NSTAGE - 1: one commit group per tile (empty when there is no such tile)
#pragma unroll
    for (int i = 0; i < NSTAGE - 1; ++i) {
        if (i < n_tiles) load_tile(i, i);
        else cp_async_commit();
    }
    cp_async_wait<NSTAGE - 1>();   // the Q tile has landed (key tiles may still be in flight)
    __syncthreads();

    // ---- Q fragments ---------------------------------------------------------------------------
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(qf[ks], tile_addr<D>(sQ, row, ks * 2 + (lane >> 4)));
    }

    __syncthreads();               // every warp holds its Q fragments: the borrowed stage is free

    float o_acc[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_a = warp * 16 + g, row_b = row_a + 8;          // rows of this thread inside the tile
    const int pos_a = p_lo + row_a, pos_b = p_lo + row_b;

    for (int ti = 0; ti < n_tiles; ++ti) {
        const int buf = ti % NSTAGE;
        if (ti + NSTAGE - 1 < n_tiles) load_tile(ti + NSTAGE - 1, (ti + NSTAGE - 1) % NSTAGE);
        else cp_async_commit();
        cp_async_wait<NSTAGE - 1>();   // all but the newest NSTAGE-1 groups are done: tile ti is here
        __syncthreads();
        const int kt = k_begin + ti * BKEYS;

        // S = Q K^T : 16 x 64 per warp
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s[nt][j] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ks += 2) {
                uint32_t kb[4];   // b0,b1 of k-step ks, b0,b1 of k-step ks+1
                ldmatrix_x4(kb, tile_addr<D>(sK(buf), nt * 8 + (lane & 7), ks * 2 + (lane >> 3)));
                mma16816(s[nt], qf[ks], kb[0], kb[1]);
                mma16816(s[nt], qf[ks + 1], kb[2], kb[3]);
            }
        }
        // mask, scale (log2 domain), running maximum; a tile wholly visible to every row of the
        // block (all keys at or below the first query, inside every window, all rows real) skips the tests
        float mx[2] = {-INFINITY, -INFINITY};
        const bool all_visible = nq == BQ && kt + BKEYS - 1 <= p_lo && kt + BKEYS <= k_end &&
                                 (window == 0 || kt > p_hi - window) && row_off[buf][BKEYS - 1] >= 0 &&
                                 row_off[buf][0] >= 0;
        if (all_visible) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float v = s[nt][j] * scale_log2;
                    s[nt][j] = v;
                    mx[j >> 1] = fmaxf(mx[j >> 1], v);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int kj = kt + nt * 8 + 2 * t + (j & 1);
                    const int pos = (j & 2) ? pos_b : pos_a;
                    const int row = (j & 2) ? row_b : row_a;
                    const bool vis = row < nq && kj <= pos && (window == 0 || kj > pos - window) &&
                                     row_off[buf][kj - kt] >= 0;
                    const float v = vis ? s[nt][j] * scale_log2 : -INFINITY;
                    s[nt][j] = v;
                    mx[j >> 1] = fmaxf(mx[j >> 1], v);
                }
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            alpha[r] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
        }
        float ps[2] = {0.f, 0.f};
        uint32_t pa[4][4];          // P as A fragments: k-step j covers keys 16j .. 16j+15
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float m = m_run[j >> 1];
                p[j] = (m == -INFINITY) ? 0.f : exp2f(s[nt][j] - m);
                ps[j >> 1] += p[j];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            ps[r] += __shfl_xor_sync(0xffffffffu, ps[r], 1);
            ps[r] += __shfl_xor_sync(0xffffffffu, ps[r], 2);
            l_run[r] = l_run[r] * alpha[r] + ps[r];
        }
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) {
            o_acc[dt][0] *= alpha[0]; o_acc[dt][1] *= alpha[0];
            o_acc[dt][2] *= alpha[1]; o_acc[dt][3] *= alpha[1];
        }
        // O += P V
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int dt = 0; dt < DT; dt += 2) {
                uint32_t vb[4];   // b0,b1 for d-tile dt, b0,b1 for d-tile dt+1
                const int row = 16 * j + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(vb, tile_addr<D>(sV(buf), row, dt + (lane >> 4)));
                mma16816(o_acc[dt], pa[j], vb[0], vb[1]);
                mma16816(o_acc[dt + 1], pa[j], vb[2], vb[3]);
            }
        }
        __syncthreads();   // all warps are done with this buffer before it is filled again
    }

    // ---- output ----------------------------------------------------------------------------------
    const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
    const float inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
        const int c = dt * 8 + 2 * t;
        if (row_a < nq) {
            __nv_bfloat16* o = out + ((int64_t)(q0 + qt * BQ + row_a) * nh + h) * D + c;
            *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(o_acc[dt][0] * inv_a, o_acc[dt][1] * inv_a);
        }
        if (row_b < nq) {
            __nv_bfloat16* o = out + ((int64_t)(q0 + qt * BQ + row_b) * nh + h) * D + c;
            *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(o_acc[dt][2] * inv_b, o_acc[dt][3] * inv_b);
        }
    }
}

}  // namespace pf
}  // namespace mi

using namespace mi;

extern "C" {

// 1 if the tensor-core prefill kernel is built for this head size (bfloat16 only).
int mi_attn_prefill_supported(int d) { return (d == 64 || d == 128) ? 1 : 0; }

int mi_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                    const int* q_start, const int* kv_len, void* out, int B, int max_q_len, int nh, int nkv, int d,
                    int page_size, int max_pages, int window, float scale, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return kOk;
    if (!mi_attn_prefill_supported(d)) {
        set_last_error("prefill attention (tensor cores): head_dim %d is not built (64, 128)", d);
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
    const dim3 grid((max_q_len + pf::BQ - 1) / pf::BQ, nh, B);
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = 2 * pf::NSTAGE * (size_t)pf::BKEYS * d * 2;
#define MI_PF(DD)                                                                                          \
    do {                                                                                                   \
        auto kern = pf::attn_prefill_kernel<DD>;                                                           \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
        kern<<<grid, pf::THREADS, smem, stream>>>(                                                         \
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,         \
            block_table, q_start, kv_len, (__nv_bfloat16*)out, nh, nkv, page_size, max_pages, window,      \
            scale_log2);                                                                                   \
    } while (0)
    if (d == 64) MI_PF(64); else MI_PF(128);
#undef MI_PF
    return finish_launch("attn_prefill");
}

}  // extern "C"
