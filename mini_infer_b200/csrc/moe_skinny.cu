// Grouped expert products for decode-sized batches (a few rows per expert), bfloat16.
//
// At decode every expert sees zero to a handful of tokens, so the product is
// bound by reading each used expert's weights once from HBM.  The weights are
// the M operand of the tensor-core instruction (16 output features per warp),
// the tokens are the N operand (8 per instruction), and weight fragments go
// from global memory straight into registers with 16-byte loads: every weight
// element is used exactly once, so shared memory would only add a copy.
//
// A thread's 16-byte load holds 8 consecutive k of one row; the two k-slots
// pairs of two instructions are fed from it, and the token operand is loaded
// with the same permutation of k, which leaves the dot product unchanged.
// The order of additions for a (row, feature) pair depends on K only, never on
// how many rows the expert has.
//
// The reference runs three cuBLAS products per used expert over ALL tokens and
// masks afterwards (src/layers/moe.cpp:246-270, src/layers/mlp.cpp:255-300).

#include "common.cuh"

namespace mi {

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// MODE 0: C[r, n] = a_r . W[e, n, :]                       (C float)
// MODE 1: C[r, n] = silu(a_r . W[e, n, :]) * (a_r . W[e, Nout + n, :])   (C bfloat16)
// Block = 4 warps x 16 features; grid = (ceil(Nout / 64), E).
// Rows r < rows of this pass: source row src[r] (row0 + r without src), result row dst[r] (row0 + r
// without dst).
template <int MODE, int NT>
__device__ __forceinline__ void skinny_pass(const __nv_bfloat16* __restrict__ A, const int* src, const int* dst,
                                            const __nv_bfloat16* __restrict__ We, void* __restrict__ C, int row0,
                                            int rows, int f0, int Nout, int Kd) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // weight rows of this thread (clamped so that a partial feature tile never reads outside)
    const int fa = min(f0 + g, Nout - 1), fb = min(f0 + g + 8, Nout - 1);
    const uint4* wa = reinterpret_cast<const uint4*>(We + (int64_t)fa * Kd) + t;
    const uint4* wb = reinterpret_cast<const uint4*>(We + (int64_t)fb * Kd) + t;
    const uint4* ua = nullptr;
    const uint4* ub = nullptr;
    if (MODE == 1) {
        ua = reinterpret_cast<const uint4*>(We + (int64_t)(Nout + fa) * Kd) + t;
        ub = reinterpret_cast<const uint4*>(We + (int64_t)(Nout + fb) * Kd) + t;
    }
    // token rows: tile j holds tokens 8j + g
    const uint4* xr[NT];
    bool xv[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int r = 8 * j + g;
        xv[j] = r < rows;
        const int from = xv[j] ? (src ? src[r] : row0 + r) : 0;
        xr[j] = reinterpret_cast<const uint4*>(A + (int64_t)from * Kd) + t;
    }
    float acc[NT][2][4];   // [tile][gate|up][fragment]
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][h][i] = 0.f;

    const int chunks = Kd >> 5;   // 32 k per chunk; 4 uint4 per row per chunk
#pragma unroll 4
    for (int c = 0; c < chunks; ++c) {
        const uint4 va = ld_stream(wa + 4 * c), vb = ld_stream(wb + 4 * c);
        uint4 pa, pb;
        if (MODE == 1) { pa = ld_stream(ua + 4 * c); pb = ld_stream(ub + 4 * c); }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            uint4 x = make_uint4(0u, 0u, 0u, 0u);
            if (xv[j]) x = __ldg(xr[j] + 4 * c);
            mma_bf16_16816(acc[j][0], va.x, vb.x, va.y, vb.y, x.x, x.y);
            mma_bf16_16816(acc[j][0], va.z, vb.z, va.w, vb.w, x.z, x.w);
            if (MODE == 1) {
                mma_bf16_16816(acc[j][1], pa.x, pb.x, pa.y, pb.y, x.x, x.y);
                mma_bf16_16816(acc[j][1], pa.z, pb.z, pa.w, pb.w, x.z, x.w);
            }
        }
    }
    // fragment: [0] (feature f0+g, token 2t) [1] (f0+g, 2t+1) [2] (f0+g+8, 2t) [3] (f0+g+8, 2t+1)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int f = f0 + g + ((i & 2) ? 8 : 0);
            const int r = 8 * j + 2 * t + (i & 1);
            if (f < Nout && r < rows) {
                const int64_t o = (int64_t)(dst ? dst[r] : row0 + r) * Nout + f;
                if (MODE == 1) {
                    const float gv = acc[j][0][i];
                    reinterpret_cast<__nv_bfloat16*>(C)[o] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * acc[j][1][i]);
                } else {
                    reinterpret_cast<float*>(C)[o] = acc[j][0][i];
                }
            }
        }
}

template <int MODE>
__global__ void __launch_bounds__(128)
grouped_gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, const int* __restrict__ gather,
                           const __nv_bfloat16* __restrict__ W, const int* __restrict__ offsets,
                           void* __restrict__ C, int Nout, int Kd) {
    const int e = blockIdx.y;
    const int b0 = offsets[e], cnt = offsets[e + 1] - b0;
    if (cnt <= 0) return;
    const int f0 = blockIdx.x * 64 + (threadIdx.x >> 5) * 16;
    if (f0 >= Nout) return;
    const int wrows = MODE == 1 ? 2 * Nout : Nout;
    const __nv_bfloat16* We = W + (int64_t)e * wrows * Kd;
    if (cnt <= 8) {
        skinny_pass<MODE, 1>(A, gather ? gather + b0 : nullptr, nullptr, We, C, b0, cnt, f0, Nout, Kd);
    } else {
        for (int r0 = 0; r0 < cnt; r0 += 16)
            skinny_pass<MODE, 2>(A, gather ? gather + b0 + r0 : nullptr, nullptr, We, C, b0 + r0,
                                 min(16, cnt - r0), f0, Nout, Kd);
    }
}

// The same product without a permutation, for a step of at most PAIR_MAX_TOKENS tokens: the rows of
// expert e are the (token, slot) pairs i = t * K + k with topk_idx[i] == e, found by one warp with
// ballots, in ascending i.  Result rows are indexed by pair.  src_is_token: the source row of pair i
// is token i / K (first product); otherwise it is row i (second product).
constexpr int PAIR_MAX_TOKENS = 128;
constexpr int PAIR_SPLITK_MAX_TOKENS = 8;   // steps up to this size use the split-inner-dimension kernel

template <int MODE>
__global__ void __launch_bounds__(128)
grouped_gemm_skinny_pairs_kernel(const __nv_bfloat16* __restrict__ A, const int* __restrict__ topk_idx,
                                 const __nv_bfloat16* __restrict__ W, void* __restrict__ C, int n_pairs, int K,
                                 int src_is_token, int Nout, int Kd) {
    __shared__ int pair_sh[PAIR_MAX_TOKENS], from_sh[PAIR_MAX_TOKENS];
    __shared__ int cnt_sh;
    const int e = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        int run = 0;
        for (int base = 0; base < n_pairs; base += 32) {
            const int i = base + lane;
            const bool mine = i < n_pairs && topk_idx[i] == e;
            const unsigned bal = __ballot_sync(0xffffffffu, mine);
            const int at = run + __popc(bal & ((1u << lane) - 1u));
            if (mine && at < PAIR_MAX_TOKENS) {
                pair_sh[at] = i;
                from_sh[at] = src_is_token ? i / K : i;
            }
            run += __popc(bal);
        }
        if (lane == 0) cnt_sh = min(run, PAIR_MAX_TOKENS);
    }
    __syncthreads();
    const int cnt = cnt_sh;
    if (cnt <= 0) return;
    const int f0 = blockIdx.x * 64 + warp * 16;
    if (f0 >= Nout) return;
    const int wrows = MODE == 1 ? 2 * Nout : Nout;
    const __nv_bfloat16* We = W + (int64_t)e * wrows * Kd;
    if (cnt <= 8) {
        skinny_pass<MODE, 1>(A, from_sh, pair_sh, We, C, 0, cnt, f0, Nout, Kd);
    } else {
        for (int r0 = 0; r0 < cnt; r0 += 16)
            skinny_pass<MODE, 2>(A, from_sh + r0, pair_sh + r0, We, C, 0, min(16, cnt - r0), f0, Nout, Kd);
    }
}


// Dense product for a step of a few tokens: C[r, n] = a_r . W[n, :] (+ bias[n]), all of W read once.
// A block owns 16 output features; its 8 warps split the inner dimension into 8 contiguous ranges
// (so a block keeps 8 x 2 KB x unroll of weight loads in flight) and their partial sums are added
// in warp order through shared memory: the order of additions depends on K only.
// MODE 0 writes float; MODE 1 holds gate and up rows (W has 2 * Nout rows) and writes
// silu(gate) * up as bfloat16.  Tile j of NT holds rows 8j .. 8j+7.
template <int MODE, int NT, int WARPS = 8>
__device__ __forceinline__ void splitk_tile(const __nv_bfloat16* __restrict__ A, const int* src, const int* dst,
                                            const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                                            void* __restrict__ C, int rows, int f0, int Nout, int Kd) {
    constexpr int H = MODE == 1 ? 2 : 1;
    __shared__ float red[WARPS][NT * H * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int fa = min(f0 + g, Nout - 1), fb = min(f0 + g + 8, Nout - 1);
    const uint4* wa = reinterpret_cast<const uint4*>(W + (int64_t)fa * Kd) + t;
    const uint4* wb = reinterpret_cast<const uint4*>(W + (int64_t)fb * Kd) + t;
    const uint4* ua = nullptr;
    const uint4* ub = nullptr;
    if (MODE == 1) {
        ua = reinterpret_cast<const uint4*>(W + (int64_t)(Nout + fa) * Kd) + t;
        ub = reinterpret_cast<const uint4*>(W + (int64_t)(Nout + fb) * Kd) + t;
    }
    const uint4* xr[NT];
    bool xv[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int r = 8 * j + g;
        xv[j] = r < rows;
        const int from = xv[j] ? (src ? src[r] : r) : 0;
        xr[j] = reinterpret_cast<const uint4*>(A + (int64_t)from * Kd) + t;
    }
    float acc[NT][H][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int h = 0; h < H; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][h][i] = 0.f;

    const int chunks = Kd >> 5;
    const int per = (chunks + WARPS - 1) / WARPS;
    const int c_begin = min(warp * per, chunks), c_end = min(c_begin + per, chunks);
#pragma unroll 4
    for (int c = c_begin; c < c_end; ++c) {
        const uint4 va = ld_stream(wa + 4 * c), vb = ld_stream(wb + 4 * c);
        uint4 pa, pb;
        if (MODE == 1) { pa = ld_stream(ua + 4 * c); pb = ld_stream(ub + 4 * c); }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            uint4 x = make_uint4(0u, 0u, 0u, 0u);
            if (xv[j]) x = __ldg(xr[j] + 4 * c);
            mma_bf16_16816(acc[j][0], va.x, vb.x, va.y, vb.y, x.x, x.y);
            mma_bf16_16816(acc[j][0], va.z, vb.z, va.w, vb.w, x.z, x.w);
            if (MODE == 1) {
                mma_bf16_16816(acc[j][H - 1], pa.x, pb.x, pa.y, pb.y, x.x, x.y);
                mma_bf16_16816(acc[j][H - 1], pa.z, pb.z, pa.w, pb.w, x.z, x.w);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int h = 0; h < H; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[warp][(j * H + h) * 4 + i][lane] = acc[j][h][i];
    __syncthreads();
    // one thread per (tile, fragment element, lane); fragment element i of lane (g, t) is
    // feature f0 + g + (i & 2 ? 8 : 0), row 8j + 2t + (i & 1)
    for (int o = threadIdx.x; o < NT * 4 * 32; o += blockDim.x) {
        const int l = o & 31, i = (o >> 5) & 3, j = o >> 7;
        const int f = f0 + (l >> 2) + ((i & 2) ? 8 : 0);
        const int r = 8 * j + 2 * (l & 3) + (i & 1);
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            s0 += red[w][(j * H) * 4 + i][l];
            if (MODE == 1) s1 += red[w][(j * H + H - 1) * 4 + i][l];
        }
        if (f < Nout && r < rows) {
            const int64_t at = (int64_t)(dst ? dst[r] : r) * Nout + f;
            if (MODE == 1) {
                if (bias) { s0 += bias[f]; s1 += bias[Nout + f]; }
                reinterpret_cast<__nv_bfloat16*>(C)[at] = __float2bfloat16_rn(s0 / (1.0f + expf(-s0)) * s1);
            } else {
                if (bias) s0 += bias[f];
                reinterpret_cast<float*>(C)[at] = s0;
            }
        }
    }
}

template <int MODE, int NT>
__global__ void __launch_bounds__(256)
dense_skinny_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                    const float* __restrict__ bias, void* __restrict__ C, int rows, int Nout, int Kd) {
    wait_for_earlier_kernels();
    splitk_tile<MODE, NT>(A, nullptr, nullptr, W, bias, C, rows, blockIdx.x * 16, Nout, Kd);
}

// The same with 32 warps to a block, for products with so few output features that their tiles do not
// even fill the SMs (an output projection, the second product of a shared expert; mode 0 only): the
// inner dimension is split 32 ways and a block keeps four times as many loads in flight.
template <int MODE, int NT>
__global__ void __launch_bounds__(1024)
dense_skinny_wide_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                         const float* __restrict__ bias, void* __restrict__ C, int rows, int Nout, int Kd) {
    wait_for_earlier_kernels();
    splitk_tile<MODE, NT, 32>(A, nullptr, nullptr, W, bias, C, rows, blockIdx.x * 16, Nout, Kd);
}

// The pair-indexed grouped product for the smallest steps (at most 8 tokens, so at most 8 rows per
// expert): with few experts in use, blocks of 64 features leave most of the device idle, so here a
// block owns 16 features and its 8 warps split the inner dimension, as in the dense kernel.
// grid = (ceil(Nout / 16), E), block row y serving expert y; or, with `compact` (few pairs beside many
// experts), grid = (ceil(Nout / 16), pairs) and block row y serving the y-th distinct expert of
// topk_idx in the order of first occurrence, so that no block is launched for an expert that nobody
// chose (at batch 1 that is 4 block rows instead of 60; finding the expert costs every block a little,
// which from a handful of tokens on is more than the empty blocks cost).
template <int MODE, bool COMPACT>
__global__ void __launch_bounds__(256)
grouped_gemm_skinny_pairs_splitk_kernel(const __nv_bfloat16* __restrict__ A, const int* __restrict__ topk_idx,
                                        const __nv_bfloat16* __restrict__ W, void* __restrict__ C, int n_pairs,
                                        int K, int src_is_token, int Nout, int Kd) {
    __shared__ int pair_sh[8], from_sh[8];
    __shared__ int cnt_sh, e_sh;
    wait_for_earlier_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        // the blockIdx.y-th distinct expert
        int e = COMPACT ? -1 : (int)blockIdx.y, distinct = 0;
        for (int base = 0; COMPACT && base < n_pairs && e < 0; base += 32) {
            const int i = base + lane;
            const int v = i < n_pairs ? topk_idx[i] : -1 - lane;     // lanes past the end match nobody
            bool seen = false;                                       // in a round before this one
            for (int j = 0; j < base; ++j) seen |= topk_idx[j] == v;
            const unsigned same = __match_any_sync(0xffffffffu, v);
            const bool first = i < n_pairs && !seen && lane == __ffs(same) - 1;
            const unsigned firsts = __ballot_sync(0xffffffffu, first);
            const int rank = distinct + __popc(firsts & ((1u << lane) - 1u));
            const unsigned hit = __ballot_sync(0xffffffffu, first && rank == (int)blockIdx.y);
            if (hit) e = __shfl_sync(0xffffffffu, v, __ffs(hit) - 1);
            distinct += __popc(firsts);
        }
        int run = 0;
        if (e >= 0) {
            for (int base = 0; base < n_pairs; base += 32) {
                const int i = base + lane;
                const bool mine = i < n_pairs && topk_idx[i] == e;
                const unsigned bal = __ballot_sync(0xffffffffu, mine);
                const int at = run + __popc(bal & ((1u << lane) - 1u));
                if (mine && at < 8) {
                    pair_sh[at] = i;
                    from_sh[at] = src_is_token ? i / K : i;
                }
                run += __popc(bal);
            }
        }
        if (lane == 0) {
            cnt_sh = min(run, 8);
            if (COMPACT) e_sh = e;
        }
    }
    __syncthreads();
    const int cnt = cnt_sh, e = COMPACT ? e_sh : (int)blockIdx.y;
    if (cnt <= 0) return;
    const int wrows = MODE == 1 ? 2 * Nout : Nout;
    splitk_tile<MODE, 1>(A, from_sh, pair_sh, W + (int64_t)e * wrows * Kd, nullptr, C, cnt, blockIdx.x * 16, Nout, Kd);
}

// Query/key/value projection of a step of a few tokens with its whole epilogue: bias, rotary
// position encoding of q and k (half-split pairing, angle = position * inv_freq in float), q
// written as bfloat16 and k, v written into their cache pages.  A block owns 8 rotation pairs
// (i, i + d/2) of one head: fragment rows g and g + 8 are the two members of pair g, so the thread
// that sums the warps' partial sums holds both.  Split of the inner dimension as in
// dense_skinny_kernel.  grid = (d / 16, nh + 2 * nkv).
template <int NT>
__global__ void __launch_bounds__(256)
qkv_skinny_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                  const float* __restrict__ bias, const int* __restrict__ positions,
                  const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                  __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                  __nv_bfloat16* __restrict__ v_cache, int rows, int Kd, int nh, int nkv, int d, int page_size) {
    __shared__ float red[8][NT * 4][32];
    wait_for_earlier_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y, half = d >> 1;
    const int p0 = blockIdx.x * 8;
    const int fa = head * d + p0 + g, fb = fa + half;
    const uint4* wa = reinterpret_cast<const uint4*>(W + (int64_t)fa * Kd) + t;
    const uint4* wb = reinterpret_cast<const uint4*>(W + (int64_t)fb * Kd) + t;
    const uint4* xr[NT];
    bool xv[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int r = 8 * j + g;
        xv[j] = r < rows;
        xr[j] = reinterpret_cast<const uint4*>(A + (int64_t)(xv[j] ? r : 0) * Kd) + t;
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const int chunks = Kd >> 5;
    const int per = (chunks + 7) >> 3;
    const int c_begin = min(warp * per, chunks), c_end = min(c_begin + per, chunks);
#pragma unroll 4
    for (int c = c_begin; c < c_end; ++c) {
        const uint4 va = ld_stream(wa + 4 * c), vb = ld_stream(wb + 4 * c);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            uint4 x = make_uint4(0u, 0u, 0u, 0u);
            if (xv[j]) x = __ldg(xr[j] + 4 * c);
            mma_bf16_16816(acc[j], va.x, vb.x, va.y, vb.y, x.x, x.y);
            mma_bf16_16816(acc[j], va.z, vb.z, va.w, vb.w, x.z, x.w);
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][j * 4 + i][lane] = acc[j][i];
    __syncthreads();
    // one thread per (tile j, token parity i, lane): pair p0 + (lane >> 2) of token 8j + 2(lane & 3) + i
    for (int o = threadIdx.x; o < NT * 2 * 32; o += blockDim.x) {
        const int l = o & 31, i = (o >> 5) & 1, j = o >> 6;
        const int r = 8 * j + 2 * (l & 3) + i;
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) { lo += red[w][j * 4 + i][l]; hi += red[w][j * 4 + i + 2][l]; }
        if (r >= rows) continue;
        const int pi = p0 + (l >> 2);
        const int c0 = head * d + pi, c1 = c0 + half;
        if (bias) { lo += bias[c0]; hi += bias[c1]; }
        __nv_bfloat16* dst = nullptr;
        if (head < nh) {
            dst = q_out + ((int64_t)r * nh + head) * d;
        } else {
            const int slot = slot_mapping[r];
            if (slot >= 0) {
                const int page = slot / page_size, off = slot - page * page_size;
                const int hk = head < nh + nkv ? head - nh : head - nh - nkv;
                dst = (head < nh + nkv ? k_cache : v_cache) + ((int64_t)page * nkv + hk) * page_size * d +
                      (int64_t)off * d;
            }
        }
        if (!dst) continue;
        float ylo = lo, yhi = hi;
        if (inv_freq && head < nh + nkv) {
            const float ang = (float)positions[r] * inv_freq[pi];
            const float ca = cosf(ang), sa = sinf(ang);
            ylo = lo * ca - hi * sa;
            yhi = hi * ca + lo * sa;
        }
        dst[pi] = __float2bfloat16_rn(ylo);
        dst[pi + half] = __float2bfloat16_rn(yhi);
    }
}

}  // namespace mi

using namespace mi;

extern "C" {

// 1 if the decode-sized grouped product takes these sizes (else use the plain kernel).
int mi_grouped_gemm_skinny_supported(int Kd) { return (Kd > 0 && Kd % 32 == 0) ? 1 : 0; }

// A, W bfloat16; C bfloat16 for mode 1 (SwiGLU pair, W holds 2*Nout rows per expert), float for mode 0.
int mi_grouped_gemm_skinny(const void* A, const int* gather, const void* W, const int* offsets, void* C,
                           int E, int Nout, int Kd, int mode, cudaStream_t stream) {
    if (!mi_grouped_gemm_skinny_supported(Kd)) {
        set_last_error("grouped product (decode): inner size %d is not a multiple of 32", Kd);
        return kBadShape;
    }
    if (E < 1 || E > 65535) {
        set_last_error("grouped product (decode): %d experts exceed the grid limit", E);
        return kBadShape;
    }
    const dim3 grid((Nout + 63) / 64, E);
    if (mode == 1)
        grouped_gemm_skinny_kernel<1><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)A, gather, (const __nv_bfloat16*)W, offsets, C, Nout, Kd);
    else
        grouped_gemm_skinny_kernel<0><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)A, gather, (const __nv_bfloat16*)W, offsets, C, Nout, Kd);
    return finish_launch("grouped_gemm_skinny");
}


// Largest step (in tokens) of the pair-indexed grouped product.
int mi_grouped_gemm_skinny_pairs_max_tokens() { return PAIR_MAX_TOKENS; }
// Steps of up to this many tokens take the form whose blocks split the inner dimension over their warps.
int mi_grouped_gemm_skinny_pairs_split_inner_max_tokens() { return PAIR_SPLITK_MAX_TOKENS; }

// The decode-sized grouped product without a permutation.  topk_idx [T*K]: expert of pair t*K+k (each
// token names an expert at most once).  mode 1: A [T, Kd], C bfloat16 [T*K, Nout] = SwiGLU pair of
// token t's row under the pair's expert; mode 0: A [T*K, Kd] indexed by pair, C float [T*K, Nout].
int mi_grouped_gemm_skinny_pairs(const void* A, const int* topk_idx, const void* W, void* C, int T, int K, int E,
                                 int Nout, int Kd, int mode, cudaStream_t stream) {
    if (!mi_grouped_gemm_skinny_supported(Kd)) {
        set_last_error("grouped product (decode): inner size %d is not a multiple of 32", Kd);
        return kBadShape;
    }
    if (T < 1 || T > PAIR_MAX_TOKENS || K < 1) {
        set_last_error("grouped product (decode, by pair): %d tokens, takes 1..%d", T, PAIR_MAX_TOKENS);
        return kBadShape;
    }
    if (E < 1 || E > 65535) {
        set_last_error("grouped product (decode): %d experts exceed the grid limit", E);
        return kBadShape;
    }
    if (T <= PAIR_SPLITK_MAX_TOKENS) {
        const bool compact = 4 * T * K <= E;
        const dim3 sgrid((Nout + 15) / 16, compact ? T * K : E);
#define MI_PAIRS_SPLITK(MODE, COMPACT)                                                                   \
    launch_dependent(grouped_gemm_skinny_pairs_splitk_kernel<MODE, COMPACT>, sgrid, dim3(256), 0, stream, \
        (const __nv_bfloat16*)A, topk_idx, (const __nv_bfloat16*)W, C, T * K, K, MODE, Nout, Kd)
        if (mode == 1) { if (compact) MI_PAIRS_SPLITK(1, true); else MI_PAIRS_SPLITK(1, false); }
        else { if (compact) MI_PAIRS_SPLITK(0, true); else MI_PAIRS_SPLITK(0, false); }
#undef MI_PAIRS_SPLITK
        return finish_launch("grouped_gemm_skinny_pairs");
    }
    const dim3 grid((Nout + 63) / 64, E);
    if (mode == 1)
        grouped_gemm_skinny_pairs_kernel<1><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)A, topk_idx, (const __nv_bfloat16*)W, C, T * K, K, 1, Nout, Kd);
    else
        grouped_gemm_skinny_pairs_kernel<0><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)A, topk_idx, (const __nv_bfloat16*)W, C, T * K, K, 0, Nout, Kd);
    return finish_launch("grouped_gemm_skinny_pairs");
}

// Largest step (in rows) that the dense decode-sized product takes.
int mi_dense_skinny_max_rows() { return 32; }

// C = A @ W^T (+ bias) for rows <= 32.  A [rows, Kd], W [Nout (mode 0) or 2*Nout (mode 1), Kd] bfloat16;
// bias float or null; C float [rows, Nout] (mode 0) or bfloat16 silu(gate)*up (mode 1).
int mi_dense_skinny(const void* A, const void* W, const float* bias, void* C, int rows, int Nout, int Kd,
                    int mode, cudaStream_t stream) {
    if (Kd <= 0 || Kd % 32 != 0) {
        set_last_error("dense product (decode): inner size %d is not a multiple of 32", Kd);
        return kBadShape;
    }
    if (rows < 1 || rows > mi_dense_skinny_max_rows()) {
        set_last_error("dense product (decode): %d rows, takes 1..%d", rows, mi_dense_skinny_max_rows());
        return kBadShape;
    }
    if (Nout < 1) {
        set_last_error("dense product (decode): %d output features", Nout);
        return kBadShape;
    }
    const dim3 grid((Nout + 15) / 16), block(256);
    const __nv_bfloat16* a = (const __nv_bfloat16*)A;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // the choice depends on the product's shape only, never on the number of rows (more than 16 rows
    // go in two launches: the partial sums of 32 rows x 32 warps would not fit the static shared memory)
    if (mode == 0 && (int)grid.x <= num_sms && Kd >= 1024) {
        float* c = (float*)C;
        if (rows <= 8) launch_dependent(dense_skinny_wide_kernel<0, 1>, grid, dim3(1024), 0, stream, a, w, bias, c, rows, Nout, Kd);
        else launch_dependent(dense_skinny_wide_kernel<0, 2>, grid, dim3(1024), 0, stream, a, w, bias, c, rows < 16 ? rows : 16, Nout, Kd);
        if (rows > 16)
            launch_dependent(dense_skinny_wide_kernel<0, 2>, grid, dim3(1024), 0, stream, a + (int64_t)16 * Kd, w, bias,
                             c + (int64_t)16 * Nout, rows - 16, Nout, Kd);
        return finish_launch("dense_skinny", rows > 16 ? 2 : 1);
    }
#define MI_DENSE_SKINNY(MODE, NT) launch_dependent(dense_skinny_kernel<MODE, NT>, grid, block, 0, stream, a, w, bias, C, rows, Nout, Kd)
    if (mode == 1) {
        if (rows <= 8) MI_DENSE_SKINNY(1, 1);
        else if (rows <= 16) MI_DENSE_SKINNY(1, 2);
        else MI_DENSE_SKINNY(1, 4);
    } else {
        if (rows <= 8) MI_DENSE_SKINNY(0, 1);
        else if (rows <= 16) MI_DENSE_SKINNY(0, 2);
        else MI_DENSE_SKINNY(0, 4);
    }
#undef MI_DENSE_SKINNY
    return finish_launch("dense_skinny");
}

// 1 if the fused projection takes this geometry: whole pairs tiles (d a multiple of 16), rotation
// over the whole head (or none), inner size a multiple of 32.
int mi_qkv_skinny_supported(int Kd, int d, int rot_dim) {
    return (Kd > 0 && Kd % 32 == 0 && d > 0 && d % 16 == 0 && (rot_dim == d || rot_dim == 0)) ? 1 : 0;
}

// q, k, v = A @ W^T + bias for rows <= mi_dense_skinny_max_rows(), rotated and stored:
// A [rows, Kd], W [(nh + 2*nkv) * d, Kd] bfloat16; bias float [(nh + 2*nkv) * d] or null;
// inv_freq float [d/2] or null (no rotation); q_out [rows, nh, d]; k_cache, v_cache one layer's
// [pages, nkv, page_size, d]; slot_mapping[r] = page * page_size + offset of row r (or < 0: not stored).
int mi_qkv_skinny(const void* A, const void* W, const float* bias, const int* positions, const float* inv_freq,
                  const int* slot_mapping, void* q_out, void* k_cache, void* v_cache, int rows, int Kd, int nh,
                  int nkv, int d, int page_size, cudaStream_t stream) {
    if (!mi_qkv_skinny_supported(Kd, d, inv_freq ? d : 0)) {
        set_last_error("fused q/k/v projection: inner size %d or head size %d not taken", Kd, d);
        return kBadShape;
    }
    if (rows < 1 || rows > mi_dense_skinny_max_rows()) {
        set_last_error("fused q/k/v projection: %d rows, takes 1..%d", rows, mi_dense_skinny_max_rows());
        return kBadShape;
    }
    if (nh < 1 || nkv < 1 || nh + 2 * nkv > 65535) {
        set_last_error("fused q/k/v projection: %d query and %d key/value heads", nh, nkv);
        return kBadShape;
    }
    const dim3 grid(d / 16, nh + 2 * nkv), block(256);
#define MI_QKV_SKINNY(NT)                                                                                  \
    launch_dependent(qkv_skinny_kernel<NT>, grid, block, 0, stream,                                        \
        (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, positions, inv_freq, slot_mapping,         \
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, rows, Kd, nh, nkv, d, page_size)
    if (rows <= 8) MI_QKV_SKINNY(1);
    else if (rows <= 16) MI_QKV_SKINNY(2);
    else MI_QKV_SKINNY(4);
#undef MI_QKV_SKINNY
    return finish_launch("qkv_skinny");
}

}  // extern "C"
