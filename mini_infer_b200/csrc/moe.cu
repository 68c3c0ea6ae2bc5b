// Mixture-of-experts kernels: router (logits, softmax, top-k, shared gate),
// token permutation, and the plain grouped expert products.
//
// The reference computes router logits with cuBLAS into FP16
// (src/layers/moe.cpp:215-220), selects with one thread per token
// (src/kernels/moe_kernel.cu:12-63), copies the indices to the host, runs every
// used expert on all tokens and masks (src/layers/moe.cpp:239-270).  Here the
// routing stays on the device: router logits are float sums in a fixed order per
// token (float dot products; for large bfloat16 steps tensor-core products with
// float accumulation), the (token, slot) pairs are sorted by expert with a stable
// counting sort, and each expert multiplies only its own rows.

#include <cooperative_groups.h>

#include "common.cuh"

namespace mi {

// ---------------------------------------------------------------------------
// Router, in two kernels.
//   logits:  z[t, e] = x[t] . Wr[e]   (and the shared-expert gate row as column E)
//            block = 8 tokens x 8 weight rows (one warp per row): a weight row is read once for
//            the block's tokens, the tokens' rows sit in shared memory as float.  Each lane
//            takes interleaved 16-byte chunks of the row, then a butterfly sum: the order of a
//            dot product's additions depends on H only.
//   select:  one warp per token: p = softmax(z) over all experts; K rounds of arg-max over p,
//            lowest index wins ties (moe_kernel.cu:28-47); w_k = p[idx_k] (divided by their sum
//            when norm_topk); gate = sigmoid(z[E]) (moe_kernel.cu:137-139)
// ---------------------------------------------------------------------------
constexpr int RT_TOK = 8;    // tokens per block
constexpr int RT_ROWS = 8;   // weight rows per block (warps)

template <typename WT> struct RowChunk;
template <> struct RowChunk<__nv_bfloat16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        const uint4 x = __ldg(reinterpret_cast<const uint4*>(p));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    }
};
template <> struct RowChunk<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(p));
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
};

// 16 bytes of activations -> floats in shared memory
__device__ __forceinline__ void stage_chunk(const __nv_bfloat16* src, float* dst) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(src));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); dst[2 * j] = f.x; dst[2 * j + 1] = f.y; }
}
__device__ __forceinline__ void stage_chunk(const float* src, float* dst) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(src));
    dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
}

// Block = 8 warps, RT_TOK tokens, `rows_per_block` weight rows (a warp takes every 8th of them).
template <typename AT, typename WT>
__global__ void __launch_bounds__(32 * RT_ROWS)
moe_router_logits_kernel(const AT* __restrict__ x, const WT* __restrict__ wr, const WT* __restrict__ wsg,
                         float* __restrict__ z, int T, int H, int E, int rows_per_block) {
    extern __shared__ __align__(16) float xs[];   // [RT_TOK][H]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * RT_TOK;
    const int nt = min(RT_TOK, T - t0);
    constexpr int AV = 16 / sizeof(AT);           // activations per 16-byte load
    if (H % AV == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const int per_row = H / AV;
        for (int idx = threadIdx.x; idx < RT_TOK * per_row; idx += 32 * RT_ROWS) {
            const int j = idx / per_row, c = idx - j * per_row;
            float* dst = xs + j * H + c * AV;
            if (j < nt) stage_chunk(x + (int64_t)(t0 + j) * H + c * AV, dst);
            else
#pragma unroll
                for (int u = 0; u < AV; ++u) dst[u] = 0.f;
        }
    } else {
        for (int idx = threadIdx.x; idx < RT_TOK * H; idx += 32 * RT_ROWS) {
            const int j = idx / H, i = idx - j * H;
            xs[idx] = j < nt ? to_float(x[(int64_t)(t0 + j) * H + i]) : 0.f;
        }
    }
    __syncthreads();
    const int ncols = E + (wsg ? 1 : 0);
    const int e_end = min(ncols, (int)(blockIdx.y + 1) * rows_per_block);
    constexpr int CN = RowChunk<WT>::N;
    constexpr int RR = 4;                          // weight rows per pass: a staged chunk of the tokens is
                                                   // read from shared memory once for RR rows
    const bool x_ok = H % 4 == 0;                  // rows of xs stay 16-byte aligned
    for (int e0 = blockIdx.y * rows_per_block + warp; e0 < e_end; e0 += RT_ROWS * RR) {
        const WT* w[RR];
        bool aligned = x_ok;
#pragma unroll
        for (int r = 0; r < RR; ++r) {
            const int e = min(e0 + r * RT_ROWS, e_end - 1);          // rows past the end repeat the last one
            w[r] = e < E ? wr + (int64_t)e * H : wsg;
            aligned = aligned && (reinterpret_cast<uintptr_t>(w[r]) & 15) == 0;
        }
        const int main = aligned ? (H / CN) * CN : 0;
        float acc[RR][RT_TOK];
#pragma unroll
        for (int r = 0; r < RR; ++r)
#pragma unroll
            for (int j = 0; j < RT_TOK; ++j) acc[r][j] = 0.f;
        for (int i = lane * CN; i < main; i += 32 * CN) {
            RowChunk<WT> c[RR];
#pragma unroll
            for (int r = 0; r < RR; ++r) c[r].load(w[r] + i);
#pragma unroll
            for (int j = 0; j < RT_TOK; ++j) {
                const float4* xr = reinterpret_cast<const float4*>(xs + j * H + i);
#pragma unroll
                for (int u = 0; u < CN / 4; ++u) {
                    const float4 xv = xr[u];
#pragma unroll
                    for (int r = 0; r < RR; ++r) {
                        acc[r][j] += xv.x * c[r].v[4 * u];
                        acc[r][j] += xv.y * c[r].v[4 * u + 1];
                        acc[r][j] += xv.z * c[r].v[4 * u + 2];
                        acc[r][j] += xv.w * c[r].v[4 * u + 3];
                    }
                }
            }
        }
        for (int i = main + lane; i < H; i += 32) {
#pragma unroll
            for (int r = 0; r < RR; ++r) {
                const float wv = to_float(w[r][i]);
#pragma unroll
                for (int j = 0; j < RT_TOK; ++j) acc[r][j] += xs[j * H + i] * wv;
            }
        }
#pragma unroll
        for (int r = 0; r < RR; ++r) {
            const int e = e0 + r * RT_ROWS;
#pragma unroll
            for (int j = 0; j < RT_TOK; ++j) {
                const float v = warp_sum(acc[r][j]);
                if (lane == 0 && j < nt && e < e_end) z[(int64_t)(t0 + j) * ncols + e] = v;
            }
        }
    }
}

// Many tokens, bfloat16 activations and weights: the same logits on the tensor cores (products of
// two bfloat16 are exact in float, the accumulator is float).  Block = 16 tokens x 64 columns, 8 warps
// that take the 32-wide k chunks in turn (warp w: chunks w, w + 8, ...); fragments are loaded straight
// from global memory with the k permutation of a 16-byte load on both operands, which leaves a dot
// product unchanged.  The warps' partial sums are added in warp order, so the order of a logit's
// additions depends on H only.
constexpr int RM_TOK = 16, RM_COLS = 64, RM_WARPS = 8, RM_PITCH = RM_COLS + 2;

__global__ void __launch_bounds__(32 * RM_WARPS)
moe_router_logits_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr,
                             const __nv_bfloat16* __restrict__ wsg, float* __restrict__ z, int T, int H, int E) {
    __shared__ float part[RM_WARPS][RM_TOK * RM_PITCH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int t0 = blockIdx.x * RM_TOK, c0 = blockIdx.y * RM_COLS;
    const int ncols = E + (wsg ? 1 : 0);
    // rows past the end repeat a valid one; their results are not stored
    const uint4* xa = reinterpret_cast<const uint4*>(x + (int64_t)min(t0 + g, T - 1) * H) + t;
    const uint4* xb = reinterpret_cast<const uint4*>(x + (int64_t)min(t0 + g + 8, T - 1) * H) + t;
    const uint4* wp[RM_COLS / 8];
#pragma unroll
    for (int j = 0; j < RM_COLS / 8; ++j) {
        const int c = c0 + 8 * j + g;
        const __nv_bfloat16* row = c < E ? wr + (int64_t)c * H : (c == E && wsg ? wsg : wr);
        wp[j] = reinterpret_cast<const uint4*>(row) + t;
    }
    float acc[RM_COLS / 8][4];
#pragma unroll
    for (int j = 0; j < RM_COLS / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const int chunks = H >> 5;
#pragma unroll 2
    for (int c = warp; c < chunks; c += RM_WARPS) {
        const uint4 va = __ldg(xa + 4 * c), vb = __ldg(xb + 4 * c);
        uint4 w[RM_COLS / 8];
#pragma unroll
        for (int j = 0; j < RM_COLS / 8; ++j) w[j] = __ldg(wp[j] + 4 * c);
#pragma unroll
        for (int j = 0; j < RM_COLS / 8; ++j) {
            mma_bf16_16816(acc[j], va.x, vb.x, va.y, vb.y, w[j].x, w[j].y);
            mma_bf16_16816(acc[j], va.z, vb.z, va.w, vb.w, w[j].z, w[j].w);
        }
    }
    // fragment: [0] (token g, column 8j+2t) [1] (g, 8j+2t+1) [2] (g+8, 8j+2t) [3] (g+8, 8j+2t+1)
    float* mine = part[warp];
#pragma unroll
    for (int j = 0; j < RM_COLS / 8; ++j) {
        mine[g * RM_PITCH + 8 * j + 2 * t] = acc[j][0];
        mine[g * RM_PITCH + 8 * j + 2 * t + 1] = acc[j][1];
        mine[(g + 8) * RM_PITCH + 8 * j + 2 * t] = acc[j][2];
        mine[(g + 8) * RM_PITCH + 8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    for (int o = threadIdx.x; o < RM_TOK * RM_COLS; o += 32 * RM_WARPS) {
        const int r = o / RM_COLS, c = o - r * RM_COLS;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < RM_WARPS; ++w) v += part[w][r * RM_PITCH + c];
        if (t0 + r < T && c0 + c < ncols) z[(int64_t)(t0 + r) * ncols + c0 + c] = v;
    }
}

// Few tokens (decode): one block per weight row and group of RT_TOK tokens; the 8 warps split the
// row, so every lane has a single round of loads in flight, and the warps' partial sums are added
// in warp order.  The order of a dot product's additions depends on H only.
template <typename AT, typename WT, int TOK>
__device__ __forceinline__ void router_logits_small_block(const AT* __restrict__ x, const WT* __restrict__ wr,
                                                          const WT* __restrict__ wsg, float* __restrict__ z,
                                                          int T, int H, int E, int e, int t0) {
    __shared__ float part[8][TOK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = min(TOK, T - t0);
    const int ncols = E + (wsg ? 1 : 0);
    const WT* w = e < E ? wr + (int64_t)e * H : wsg;
    constexpr int CN = RowChunk<WT>::N;
    constexpr int AV = 16 / sizeof(AT);
    constexpr int L = CN > AV ? CN : AV;          // elements per thread and round: whole 16-byte loads of both
    const bool vec = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     H % L == 0;
    const int main = vec ? H : 0;
    float acc[TOK];
#pragma unroll
    for (int j = 0; j < TOK; ++j) acc[j] = 0.f;
    for (int i = threadIdx.x * L; i < main; i += 256 * L) {
        float wv[L];
#pragma unroll
        for (int u = 0; u < L; u += CN) {
            RowChunk<WT> c;
            c.load(w + i + u);
#pragma unroll
            for (int k = 0; k < CN; ++k) wv[u + k] = c.v[k];
        }
#pragma unroll
        for (int j = 0; j < TOK; ++j) {
            if (j < nt) {
                float xv[L];
                const AT* xp = x + (int64_t)(t0 + j) * H + i;
#pragma unroll
                for (int u = 0; u < L; u += AV) stage_chunk(xp + u, xv + u);
#pragma unroll
                for (int u = 0; u < L; ++u) acc[j] += xv[u] * wv[u];
            }
        }
    }
    for (int i = main + threadIdx.x; i < H; i += 256) {
        const float wv = to_float(w[i]);
#pragma unroll
        for (int j = 0; j < TOK; ++j)
            if (j < nt) acc[j] += to_float(x[(int64_t)(t0 + j) * H + i]) * wv;
    }
#pragma unroll
    for (int j = 0; j < TOK; ++j) {
        const float v = warp_sum(acc[j]);
        if (lane == 0) part[warp][j] = v;
    }
    __syncthreads();
    if (threadIdx.x < nt) {
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) v += part[wv][threadIdx.x];
        z[(int64_t)(t0 + threadIdx.x) * ncols + e] = v;
    }
}

template <typename AT, typename WT>
__global__ void __launch_bounds__(256)
moe_router_logits_small_kernel(const AT* __restrict__ x, const WT* __restrict__ wr, const WT* __restrict__ wsg,
                               float* __restrict__ z, int T, int H, int E) {
    router_logits_small_block<AT, WT, RT_TOK>(x, wr, wsg, z, T, H, E, blockIdx.x, blockIdx.y * RT_TOK);
}

// Softmax over all experts, K rounds of arg-max (lowest index among equals), weights; one warp per
// token.  `p` is the warp's E floats of shared memory and holds the token's logits, `mx` the largest
// of the lane's own, `gate_logit` (lane 0) the shared expert's.
__device__ __forceinline__ void router_select_loaded(float mx, float gate_logit, int has_gate,
                                                     int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                     float* __restrict__ gate, float* __restrict__ probs_out,
                                                     float* p, int* idx_copy, int t, int E, int K, int norm_topk) {
    const int lane = threadIdx.x & 31;
    if (has_gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-gate_logit));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(p[e] - mx);
        p[e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        const float v = p[e] / sum;
        p[e] = v;
        if (probs_out) probs_out[(int64_t)t * E + e] = v;
    }
    __syncwarp();
    float wsum = 0.f;
    float my_w = 0.f;  // lane k keeps weight k (K <= 32 checked on the host)
    for (int k = 0; k < K; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = p[e];
            if (v > best) { best = v; bi = e; }  // ascending e within a lane: first maximum kept
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == k) my_w = best;
        wsum += best;
        if (lane == 0) {
            topk_idx[(int64_t)t * K + k] = bi;
            if (idx_copy) idx_copy[t * K + k] = bi;
            p[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane < K) topk_w[(int64_t)t * K + lane] = norm_topk ? my_w / wsum : my_w;
}

// the logits of token t in global memory, read around L1 (other blocks of the same launch may have written them)
__device__ __forceinline__ void router_select_token(const float* __restrict__ z, int has_gate,
                                                    int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                    float* __restrict__ gate, float* __restrict__ probs_out,
                                                    float* p, int* idx_copy, int t, int E, int K,
                                                    int norm_topk) {
    const int lane = threadIdx.x & 31;
    const int ncols = E + (has_gate ? 1 : 0);
    const float* zr = z + (int64_t)t * ncols;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = __ldcg(zr + e); p[e] = v; mx = fmaxf(mx, v); }
    const float gl = (has_gate && lane == 0) ? __ldcg(zr + E) : 0.f;
    router_select_loaded(mx, gl, has_gate, topk_idx, topk_w, gate, probs_out, p, idx_copy, t, E, K, norm_topk);
}

// the logits of ONE token in this block's shared memory
__device__ __forceinline__ void router_select_logits(const float* zs, int has_gate,
                                                     int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                     float* __restrict__ gate, float* __restrict__ probs_out,
                                                     float* p, int* idx_copy, int t, int E, int K,
                                                     int norm_topk) {
    const int lane = threadIdx.x & 31;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = zs[e]; p[e] = v; mx = fmaxf(mx, v); }
    const float gl = (has_gate && lane == 0) ? zs[E] : 0.f;
    router_select_loaded(mx, gl, has_gate, topk_idx, topk_w, gate, probs_out, p, idx_copy, t, E, K, norm_topk);
}

__global__ void __launch_bounds__(256)
moe_router_select_kernel(const float* __restrict__ z, int has_gate, int* __restrict__ topk_idx,
                         float* __restrict__ topk_w, float* __restrict__ gate, float* __restrict__ probs_out,
                         int T, int E, int K, int norm_topk) {
    extern __shared__ float smem[];  // [8][E]
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    router_select_token(z, has_gate, topk_idx, topk_w, gate, probs_out, smem + warp * E, nullptr, t, E, K,
                        norm_topk);
}

// ---------------------------------------------------------------------------
// Permutation (one block): counts per expert, exclusive scan, stable placement.
//   offsets[E+1]; sorted_token[N] = token of sorted row; inv_perm[t*K+k] = sorted row
// ---------------------------------------------------------------------------
__device__ __forceinline__ void permute_block(const int* __restrict__ topk_idx, int* __restrict__ offsets,
                                              int* __restrict__ sorted_token, int* __restrict__ inv_perm,
                                              int* sh, int N, int E, int K, int idx_in_smem) {
    int* sidx = sh + E + 1;
    const int tid = threadIdx.x;
    for (int e = tid; e <= E; e += blockDim.x) sh[e] = 0;
    __syncthreads();
    // idx_in_smem: 0 read the indices from global memory, 1 copy them to shared memory first,
    // 2 the caller has put them there already, 3 as 1 but other blocks of this launch wrote them
    // (read around L1)
    for (int i = tid; i < N; i += blockDim.x) {
        const int e = idx_in_smem == 2 ? sidx[i] : (idx_in_smem == 3 ? __ldcg(topk_idx + i) : topk_idx[i]);
        if (idx_in_smem == 1 || idx_in_smem == 3) sidx[i] = e;
        if (e >= 0 && e < E) atomicAdd(&sh[e + 1], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e <= E; ++e) { run += sh[e]; sh[e] = run; }  // sh[e] = start of expert e
    }
    __syncthreads();
    for (int e = tid; e <= E; e += blockDim.x) offsets[e] = sh[e];
    const int* src = idx_in_smem ? sidx : topk_idx;
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
        int run = sh[e];
        const int end = sh[e + 1];
        for (int base = 0; base < N && run < end; base += 32) {
            const int i = base + lane;
            const bool mine = (i < N) && (src[i] == e);
            const unsigned bal = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int pos = run + __popc(bal & ((1u << lane) - 1u));
                sorted_token[pos] = i / K;
                inv_perm[i] = pos;
            }
            run += __popc(bal);
        }
    }
}

__global__ void __launch_bounds__(1024)
moe_permute_kernel(const int* __restrict__ topk_idx, int* __restrict__ offsets, int* __restrict__ sorted_token,
                   int* __restrict__ inv_perm, int N, int E, int K, int idx_in_smem) {
    extern __shared__ int sh[];  // [E+1] starts, then (if it fits) a copy of topk_idx
    permute_block(topk_idx, offsets, sorted_token, inv_perm, sh, N, E, K, idx_in_smem);
}

// Routing of a decode-sized step in one launch: every block computes the logits of one weight row for
// a group of TOK tokens (one token for the smallest steps, where more blocks mean less latency).
// No block waits for another: the block that finishes a group's rows of logits last (a ticket
// counter per group) selects those tokens' experts, a warp per token, and, if `offsets` is given, the
// block that finishes the last group (one more counter) builds the permutation.  `tickets` holds
// 1 + T counters that are zero before the launch and zero again after.
template <typename AT, typename WT, int TOK>
__global__ void __launch_bounds__(256)
moe_route_small_kernel(const AT* __restrict__ x, const WT* __restrict__ wr, const WT* __restrict__ wsg,
                       float* __restrict__ z, unsigned* __restrict__ tickets, int* __restrict__ topk_idx,
                       float* __restrict__ topk_w, float* __restrict__ gate, float* __restrict__ probs_out,
                       int* __restrict__ offsets, int* __restrict__ sorted_token, int* __restrict__ inv_perm,
                       int T, int H, int E, int K, int norm_topk) {
    extern __shared__ int route_sh[];  // select: [TOK][E] floats; then permute: [E+1] + [T*K] ints
    __shared__ bool last;
    const int grp = blockIdx.y, t0 = grp * TOK;
    router_logits_small_block<AT, WT, TOK>(x, wr, wsg, z, T, H, E, blockIdx.x, t0);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&tickets[1 + grp], 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x == 0) tickets[1 + grp] = 0u;
    const int warp = threadIdx.x >> 5;
    if (warp < TOK && t0 + warp < T)
        router_select_token(z, wsg ? 1 : 0, topk_idx, topk_w, gate, probs_out,
                            reinterpret_cast<float*>(route_sh) + warp * E, nullptr, t0 + warp, E, K, norm_topk);
    if (!offsets) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&tickets[0], 1u) == gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x == 0) tickets[0] = 0u;
    permute_block(topk_idx, offsets, sorted_token, inv_perm, route_sh + TOK * E, T * K, E, K, 3);
}

// The residual addition and RMSNorm that precede the router and the routing itself in one launch, for the
// smallest steps: a CLUSTER of NR_CLUSTER blocks per token.  Every block first asks for its share of the
// router's rows (asynchronous copies into shared memory: all of them in flight at once), then forms
// v = hidden[t] + delta[t] and its RMS itself (thread i holds the float4s i, i + 256, ...: the additions run
// in the order of add_rmsnorm's vector kernel, so the normalised row has that kernel's bits), keeps the
// normalised row, rounded to the activation type, in shared memory, and takes its rows' logits from there;
// the logits go to the first block's shared memory over the cluster's network.  After one cluster barrier
// the first block writes hidden[t] (no block reads it any more) and selects the token's experts.  Nothing
// waits on a counter in memory.  H is a multiple of 4 of at most 4 * 8 * 256.
// four consecutive elements of a row, held as loaded and widened when used
template <typename T4> struct Row4;
template <> struct Row4<float> {
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = __ldg(reinterpret_cast<const float4*>(p)); }
    __device__ __forceinline__ void get(float (&o)[4]) const { o[0] = raw.x; o[1] = raw.y; o[2] = raw.z; o[3] = raw.w; }
};
template <> struct Row4<__nv_bfloat16> {
    uint2 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = __ldg(reinterpret_cast<const uint2*>(p)); }
    __device__ __forceinline__ void get(float (&o)[4]) const {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    }
};
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = o;
}

constexpr int NR_VMAX = 8;

constexpr int NR_CLUSTER = 8;

template <typename WT> struct AsyncRow4;
template <> struct AsyncRow4<float> {
    static __device__ __forceinline__ void copy(float* dst, const float* src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
    }
};
template <> struct AsyncRow4<__nv_bfloat16> {
    static __device__ __forceinline__ void copy(__nv_bfloat16* dst, const __nv_bfloat16* src) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
    }
};
__device__ __forceinline__ void load4_shared(const float* p, float (&o)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    o[0] = r.x; o[1] = r.y; o[2] = r.z; o[3] = r.w;
}
__device__ __forceinline__ void load4_shared(const __nv_bfloat16* p, float (&o)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

// shared memory of a block: the normalised row [H] floats, the block's router rows [rows][H] of WT, and (used
// by the cluster's first block) the token's logits [ncols] and the selection's scratch [E]
__host__ __device__ inline size_t norm_route_small_smem(int H, int E, int ncols, size_t wbytes) {
    const int rows = (ncols + NR_CLUSTER - 1) / NR_CLUSTER;
    return sizeof(float) * (size_t)H + wbytes * (size_t)rows * H + sizeof(float) * ((size_t)ncols + E + 4);
}

template <typename AT, typename WT, typename NT>
__global__ void __launch_bounds__(256)
moe_norm_route_small_kernel(float* __restrict__ hidden, const float* __restrict__ delta,
                            const NT* __restrict__ norm_w, float eps, AT* __restrict__ x_out,
                            const WT* __restrict__ wr, const WT* __restrict__ wsg,
                            int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ gate,
                            float* __restrict__ probs_out, int T, int H, int E, int K, int norm_topk) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(16) unsigned char nr_raw[];
    __shared__ float scratch[32];
    const int ncols = E + (wsg ? 1 : 0);
    const int rows = (ncols + NR_CLUSTER - 1) / NR_CLUSTER;
    float* xs = reinterpret_cast<float*>(nr_raw);
    WT* wrows = reinterpret_cast<WT*>(nr_raw + sizeof(float) * (size_t)H);
    float* zs = reinterpret_cast<float*>(nr_raw + sizeof(float) * (size_t)H + sizeof(WT) * (size_t)rows * H);
    float* sel = zs + ncols;
    const int rank = blockIdx.x;                              // the grid is (NR_CLUSTER, T): the rank in the cluster
    const int t = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nv = H >> 2;
    const int r0 = min(ncols, rank * rows), r1 = min(ncols, r0 + rows);
    wait_for_earlier_kernels();
    // first half of a barrier that is completed before the first write into another block's shared memory:
    // that block has to have started by then
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    for (int r = r0; r < r1; ++r) {
        const WT* src = r < E ? wr + (int64_t)r * H : wsg;
        WT* dst = wrows + (size_t)(r - r0) * H;
        for (int i = threadIdx.x; i < nv; i += 256) AsyncRow4<WT>::copy(dst + 4 * i, src + 4 * i);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    float4* h4 = reinterpret_cast<float4*>(hidden + (int64_t)t * H);
    const float4* d4 = delta ? reinterpret_cast<const float4*>(delta + (int64_t)t * H) : nullptr;
    float4 v[NR_VMAX];
    Row4<NT> nrow[NR_VMAX];                                  // fetched before the sum of squares is known
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NR_VMAX; ++j) {
        const int i = threadIdx.x + 256 * j;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nv) {
            nrow[j].load(norm_w + 4 * i);
            v[j] = h4[i];
            if (d4) {
                const float4 dv = d4[i];
                v[j].x += dv.x; v[j].y += dv.y; v[j].z += dv.z; v[j].w += dv.w;
            }
            ss += v[j].x * v[j].x;
            ss += v[j].y * v[j].y;
            ss += v[j].z * v[j].z;
            ss += v[j].w * v[j].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rrms = rsqrtf(ss / (float)H + eps);
    AT* xo = x_out + (int64_t)t * H;
#pragma unroll
    for (int j = 0; j < NR_VMAX; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < nv) {
            float nw[4];
            nrow[j].get(nw);
            const float xv[4] = {v[j].x * rrms * nw[0], v[j].y * rrms * nw[1], v[j].z * rrms * nw[2],
                                 v[j].w * rrms * nw[3]};
            if (rank == 0) store4(xo + 4 * i, xv);
            // the row as the following kernels will read it: rounded to the activation type
            *reinterpret_cast<float4*>(xs + 4 * i) =
                make_float4(to_float(from_float<AT>(xv[0])), to_float(from_float<AT>(xv[1])),
                            to_float(from_float<AT>(xv[2])), to_float(from_float<AT>(xv[3])));
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    float* zs0 = cluster.map_shared_rank(zs, 0);
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    for (int r = r0 + warp; r < r1; r += 8) {
        const WT* w = wrows + (size_t)(r - r0) * H;
        float acc = 0.f;
        for (int i = lane; i < nv; i += 32) {
            float ww[4];
            load4_shared(w + 4 * i, ww);
            const float4 x = *reinterpret_cast<const float4*>(xs + 4 * i);
            acc += x.x * ww[0];
            acc += x.y * ww[1];
            acc += x.z * ww[2];
            acc += x.w * ww[3];
        }
        acc = warp_sum(acc);
        if (lane == 0) zs0[r] = acc;
    }
    cluster.sync();                                           // the logits have arrived; nobody reads hidden[t] any more
    if (rank != 0) return;
    if (d4) {
#pragma unroll
        for (int j = 0; j < NR_VMAX; ++j) {
            const int i = threadIdx.x + 256 * j;
            if (i < nv) h4[i] = v[j];
        }
    }
    if (threadIdx.x < 32)
        router_select_logits(zs, wsg ? 1 : 0, topk_idx, topk_w, gate, probs_out, sel, nullptr, t, E, K, norm_topk);
}

// For many rows: one block per expert, no atomics and no scratch.  A warp owns a contiguous run of
// pairs.  Pass 1 counts, per warp, the block's own pairs and the pairs of lower experts (their total
// is the expert's first place); a scan over the warps gives every warp its first place; pass 2 places
// the pairs in token order.
__global__ void __launch_bounds__(1024)
moe_permute_expert_kernel(const int* __restrict__ topk_idx, int* __restrict__ offsets,
                          int* __restrict__ sorted_token, int* __restrict__ inv_perm, int N, int E, int K) {
    __shared__ int own_s[32], below_s[32];
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per = ((N + 1023) / 1024) * 32;                 // pairs per warp: whole rounds of 32
    const int lo = min(N, warp * per), hi = min(N, lo + per);
    int own = 0, below = 0;
#pragma unroll 4
    for (int i = lo; i < hi; i += 32) {
        const int v = i + lane < hi ? __ldg(topk_idx + i + lane) : E;
        own += __popc(__ballot_sync(0xffffffffu, v == e));
        below += __popc(__ballot_sync(0xffffffffu, v < e));
    }
    if (lane == 0) { own_s[warp] = own; below_s[warp] = below; }
    __syncthreads();
    int o = own_s[lane], b = below_s[lane], before = lane < warp ? o : 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        o += __shfl_xor_sync(0xffffffffu, o, d);
        b += __shfl_xor_sync(0xffffffffu, b, d);
        before += __shfl_xor_sync(0xffffffffu, before, d);
    }
    if (threadIdx.x == 0) {
        offsets[e] = b;
        if (e == E - 1) offsets[E] = b + o;
    }
    if (own == 0) return;                                     // uniform for the warp
    int pos = b + before;
    for (int i = lo; i < hi; i += 32) {
        const int v = i + lane < hi ? __ldg(topk_idx + i + lane) : E;
        const unsigned m = __ballot_sync(0xffffffffu, v == e);
        if (v == e) {
            const int p = pos + __popc(m & ((1u << lane) - 1u));
            sorted_token[p] = (i + lane) / K;
            inv_perm[i + lane] = p;
        }
        pos += __popc(m);
    }
}

// ---------------------------------------------------------------------------
// Plain grouped product (float arithmetic on CUDA cores; the 32-bit path and the
// reference for the tensor-core kernels):
//   rows r of expert e (offsets[e] <= r < offsets[e+1]), a_r = A[gather ? gather[r] : r, :]
//   mode 0: C[r, n] = a_r . W[e, n, :]
//   mode 1: C[r, n] = silu(a_r . W[e, n, :]) * (a_r . W[e, Nout + n, :])      (W is [E, 2*Nout, Kd])
// Tiles of 32 rows x 32 columns; the k loop runs in steps of 32 in ascending
// order whatever the number of rows, so a row's sum never depends on its neighbours.
// ---------------------------------------------------------------------------
constexpr int GB = 32;

template <typename AT, typename WT, typename CT, int MODE>
__global__ void __launch_bounds__(256)
grouped_gemm_plain_kernel(const AT* __restrict__ A, const int* __restrict__ gather, const WT* __restrict__ W,
                          const int* __restrict__ offsets, CT* __restrict__ C, int E, int Nout, int Kd) {
    __shared__ float As[GB][GB + 1];
    __shared__ float Ws[GB][GB + 1];
    __shared__ float Us[MODE == 1 ? GB : 1][GB + 1];
    // which expert and row tile does blockIdx.y stand for?
    int slot = blockIdx.y, e = 0, row0 = 0, rows = 0;
    bool found = false;
    for (e = 0; e < E; ++e) {
        const int b0 = offsets[e], cnt = offsets[e + 1] - b0;
        const int tiles = (cnt + GB - 1) / GB;
        if (slot < tiles) { row0 = b0 + slot * GB; rows = min(GB, cnt - slot * GB); found = true; break; }
        slot -= tiles;
    }
    if (!found) return;
    const int n0 = blockIdx.x * GB;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // ty 0..7, 4 rows each
    const int wrows = MODE == 1 ? 2 * Nout : Nout;
    const WT* We = W + (int64_t)e * wrows * Kd;
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acu[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < Kd; k0 += GB) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < GB * GB; idx += 256) {
            const int r = idx >> 5, c = idx & 31;
            float av = 0.f, wv = 0.f, uv = 0.f;
            if (k0 + c < Kd) {
                if (r < rows) {
                    const int src = gather ? gather[row0 + r] : row0 + r;
                    av = to_float(A[(int64_t)src * Kd + k0 + c]);
                }
                if (n0 + r < Nout) {
                    wv = to_float(We[(int64_t)(n0 + r) * Kd + k0 + c]);
                    if (MODE == 1) uv = to_float(We[(int64_t)(Nout + n0 + r) * Kd + k0 + c]);
                }
            }
            As[r][c] = av;
            Ws[r][c] = wv;
            if (MODE == 1) Us[r][c] = uv;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GB; ++kk) {
            const float wv = Ws[tx][kk];
            const float uv = MODE == 1 ? Us[tx][kk] : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float av = As[ty * 4 + i][kk];
                acc[i] += av * wv;
                if (MODE == 1) acu[i] += av * uv;
            }
        }
    }
    const int n = n0 + tx;
    if (n < Nout) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty * 4 + i;
            if (r < rows) {
                float v = acc[i];
                if (MODE == 1) v = v / (1.0f + expf(-v)) * acu[i];
                C[(int64_t)(row0 + r) * Nout + n] = from_float<CT>(v);
            }
        }
    }
}

}  // namespace mi

using namespace mi;

extern "C" {

// `z_scratch` holds T * (E + 1) floats (router logits and the shared gate's logit).
int mi_moe_router(const void* x, int adtype, const void* wr, const void* wsg, int wdtype, float* z_scratch,
                  int* topk_idx, float* topk_w, float* gate, float* probs_out, int T, int H, int E, int K,
                  int norm_topk, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (K < 1 || K > 32 || K > E) {
        set_last_error("router: experts per token %d must lie in [1, min(32, %d)]", K, E);
        return kBadShape;
    }
    const size_t smem_x = sizeof(float) * RT_TOK * (size_t)H;
    const size_t smem_p = sizeof(float) * 8 * (size_t)E;
    if (smem_x > 200 * 1024 || smem_p > 48 * 1024) {
        set_last_error("router: hidden size %d or %d experts exceed the shared memory of a block", H, E);
        return kBadShape;
    }
    const int ncols = E + (wsg ? 1 : 0);
    // few tokens: spread the weight rows over many blocks; many tokens: stage a token tile once
    // and run all rows over it
    const int token_tiles = (T + RT_TOK - 1) / RT_TOK;
    const int rows_per_block = token_tiles >= 64 ? ((ncols + RT_ROWS - 1) / RT_ROWS) * RT_ROWS : RT_ROWS;
    const dim3 grid(token_tiles, (ncols + rows_per_block - 1) / rows_per_block);
    if (grid.y > 65535) {
        set_last_error("router: %d experts exceed the grid limit", E);
        return kBadShape;
    }
    // Float activations (the true 32-bit path) take this form at every size: it adds a token's products in
    // one fixed order, so that a token's logits do not depend on how many tokens share its step.
    if (T <= 4 * RT_TOK || (adtype == kF32 && token_tiles <= 65535)) {
        const dim3 sgrid(ncols, token_tiles);
        MI_DISPATCH_2(adtype, AT, wdtype, WT,
            moe_router_logits_small_kernel<AT, WT><<<sgrid, 256, 0, stream>>>(
                (const AT*)x, (const WT*)wr, (const WT*)wsg, z_scratch, T, H, E));
        moe_router_select_kernel<<<(T + 7) / 8, 256, smem_p, stream>>>(z_scratch, wsg ? 1 : 0, topk_idx, topk_w,
                                                                        gate, probs_out, T, E, K, norm_topk);
        return finish_launch("moe_router", 2);
    }
    if (adtype == kBF16 && wdtype == kBF16 && H % 32 == 0 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wr) | reinterpret_cast<uintptr_t>(wsg)) & 15) == 0) {
        const dim3 mgrid((T + RM_TOK - 1) / RM_TOK, (ncols + RM_COLS - 1) / RM_COLS);
        if (mgrid.y <= 65535) {
            moe_router_logits_mma_kernel<<<mgrid, 32 * RM_WARPS, 0, stream>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)wr, (const __nv_bfloat16*)wsg, z_scratch, T, H, E);
            moe_router_select_kernel<<<(T + 7) / 8, 256, smem_p, stream>>>(z_scratch, wsg ? 1 : 0, topk_idx, topk_w,
                                                                            gate, probs_out, T, E, K, norm_topk);
            return finish_launch("moe_router", 2);
        }
    }
#define MI_ROUTER_ATTR(AT, WT)                                                                              \
    if (smem_x > 48 * 1024)                                                                                 \
        cudaFuncSetAttribute(moe_router_logits_kernel<AT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             (int)smem_x)
    MI_DISPATCH_2(adtype, AT, wdtype, WT,
        MI_ROUTER_ATTR(AT, WT);
        moe_router_logits_kernel<AT, WT><<<grid, 32 * RT_ROWS, smem_x, stream>>>(
            (const AT*)x, (const WT*)wr, (const WT*)wsg, z_scratch, T, H, E, rows_per_block));
    moe_router_select_kernel<<<(T + 7) / 8, 256, smem_p, stream>>>(z_scratch, wsg ? 1 : 0, topk_idx, topk_w, gate,
                                                                    probs_out, T, E, K, norm_topk);
    return finish_launch("moe_router", 2);
}

// Router and (unless `offsets` is null) permutation of a step of at most
// mi_moe_route_small_max_tokens() tokens in one launch.
// `tickets` holds 1 + T unsigned that are zero before the first call; the kernel leaves them zero.
int mi_moe_route_small_max_tokens() { return 128; }

int mi_moe_route_small(const void* x, int adtype, const void* wr, const void* wsg, int wdtype, float* z_scratch,
                       unsigned* tickets, int* topk_idx, float* topk_w, float* gate, float* probs_out,
                       int* offsets, int* sorted_token, int* inv_perm, int T, int H, int E, int K, int norm_topk,
                       cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (T > mi_moe_route_small_max_tokens()) {
        set_last_error("router (decode): %d tokens, takes at most %d", T, mi_moe_route_small_max_tokens());
        return kBadShape;
    }
    if (K < 1 || K > 32 || K > E) {
        set_last_error("router: experts per token %d must lie in [1, min(32, %d)]", K, E);
        return kBadShape;
    }
    // groups of four tokens from 33 tokens on: a weight row is then read once for four tokens
    const int tok = T > 32 ? 4 : 1;
    const size_t smem = sizeof(float) * (size_t)tok * E + sizeof(int) * ((size_t)E + 1 + (size_t)T * K);
    if (smem > 160 * 1024 || E + 1 > 65535) {
        set_last_error("router (decode): %d experts exceed the shared memory of a block", E);
        return kBadShape;
    }
    const int ncols = E + (wsg ? 1 : 0);
    const dim3 grid(ncols, (T + tok - 1) / tok);
#define MI_ROUTE_LAUNCH(AT, WT, TOK)                                                                           \
    do {                                                                                                       \
        if (smem > 48 * 1024)                                                                                  \
            cudaFuncSetAttribute(moe_route_small_kernel<AT, WT, TOK>,                                          \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
        moe_route_small_kernel<AT, WT, TOK><<<grid, 256, smem, stream>>>(                                      \
            (const AT*)x, (const WT*)wr, (const WT*)wsg, z_scratch, tickets, topk_idx, topk_w, gate, probs_out, \
            offsets, sorted_token, inv_perm, T, H, E, K, norm_topk);                                           \
    } while (0)
    if (tok == 1) {
        MI_DISPATCH_2(adtype, AT, wdtype, WT, MI_ROUTE_LAUNCH(AT, WT, 1));
    } else {
        MI_DISPATCH_2(adtype, AT, wdtype, WT, MI_ROUTE_LAUNCH(AT, WT, 4));
    }
#undef MI_ROUTE_LAUNCH
    return finish_launch("moe_route_small");
}

// mi_moe_route_small with the residual addition and RMSNorm before it in the same launch:
// hidden [T, H] float (+= delta if given), x_out [T, H] of type `adtype` receives the normalised rows.
// ndtype: type of the norm's weights.  Takes H % 4 == 0, H <= mi_moe_norm_route_small_max_width().
int mi_moe_norm_route_small_max_width() { return 4 * NR_VMAX * 256; }
// whether the launch below takes a router of E rows (one more with a shared-expert gate) of width H whose
// weights have `wbytes` bytes an element: its blocks keep their rows in shared memory
int mi_moe_norm_route_small_takes(int H, int E, int gated, int wbytes) {
    return H > 0 && H % 4 == 0 && H <= mi_moe_norm_route_small_max_width() && E > 0 &&
           norm_route_small_smem(H, E, E + (gated ? 1 : 0), (size_t)wbytes) <= 200 * 1024;
}

int mi_moe_norm_route_small(float* hidden, const float* delta, const void* norm_w, int ndtype, float eps,
                            void* x_out, int adtype, const void* wr, const void* wsg, int wdtype,
                            int* topk_idx, float* topk_w, float* gate, float* probs_out, int T, int H, int E, int K,
                            int norm_topk, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (T > mi_moe_route_small_max_tokens()) {
        set_last_error("router (decode): %d tokens, takes at most %d", T, mi_moe_route_small_max_tokens());
        return kBadShape;
    }
    if (K < 1 || K > 32 || K > E) {
        set_last_error("router: experts per token %d must lie in [1, min(32, %d)]", K, E);
        return kBadShape;
    }
    if (H % 4 != 0 || H > mi_moe_norm_route_small_max_width() ||
        ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(x_out) |
          reinterpret_cast<uintptr_t>(norm_w) | reinterpret_cast<uintptr_t>(wr) | reinterpret_cast<uintptr_t>(wsg)) & 15)) {
        set_last_error("router with norm: width %d must be a multiple of 4 of at most %d and all rows 16-byte aligned",
                       H, mi_moe_norm_route_small_max_width());
        return kBadShape;
    }
    const int ncols = E + (wsg ? 1 : 0);
    const size_t smem = norm_route_small_smem(H, E, ncols, wdtype == 1 ? 2 : 4);
    if (smem > 200 * 1024) {
        set_last_error("router with norm: %d experts of width %d exceed the shared memory of a block (%zu bytes); "
                       "ask mi_moe_norm_route_small_takes first", E, H, smem);
        return kBadShape;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(NR_CLUSTER, T);
    lc.blockDim = dim3(256);
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = NR_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = dependent_launch_enabled() ? 2 : 1;
#define MI_NR_LAUNCH(AT, WT, NT)                                                                                 \
    do {                                                                                                         \
        if (smem > 48 * 1024)                                                                                    \
            cudaFuncSetAttribute(moe_norm_route_small_kernel<AT, WT, NT>,                                        \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                        \
        (void)cudaLaunchKernelEx(&lc, moe_norm_route_small_kernel<AT, WT, NT>, hidden, delta,             \
                                 (const NT*)norm_w, eps, (AT*)x_out, (const WT*)wr, (const WT*)wsg,              \
                                 topk_idx, topk_w, gate, probs_out, T, H, E, K, norm_topk);                      \
    } while (0)
    const int combo = adtype * 4 + wdtype * 2 + ndtype;
    if (adtype < 0 || adtype > 1 || wdtype < 0 || wdtype > 1 || ndtype < 0 || ndtype > 1) {
        set_last_error("router with norm: unknown dtype code");
        return kBadDType;
    }
    switch (combo) {
        case 0: MI_NR_LAUNCH(float, float, float); break;
        case 4: MI_NR_LAUNCH(__nv_bfloat16, float, float); break;
        case 5: MI_NR_LAUNCH(__nv_bfloat16, float, __nv_bfloat16); break;
        case 6: MI_NR_LAUNCH(__nv_bfloat16, __nv_bfloat16, float); break;
        case 7: MI_NR_LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
        default:
            set_last_error("router with norm: float activations want float weights");
            return kBadDType;
    }
#undef MI_NR_LAUNCH
    return finish_launch("moe_norm_route_small");
}

// `counts_scratch` is not used any more (the signature is kept).
int mi_moe_permute(const int* topk_idx, int* offsets, int* sorted_token, int* inv_perm, int* counts_scratch, int T,
                   int E, int K, cudaStream_t stream) {
    if (E + 1 > 12000) {
        set_last_error("permute: %d experts exceed the shared-memory table", E);
        return kBadShape;
    }
    const int64_t N = (int64_t)T * K;
    // one block per expert whatever the number of rows: 2-3 us for 64 to 2,048 rows, where the single block
    // below takes 3-14 us (it remains for more experts than a grid's row of blocks is given here)
    if (E <= 65535) {
        (void)counts_scratch;
        moe_permute_expert_kernel<<<E, 1024, 0, stream>>>(topk_idx, offsets, sorted_token, inv_perm, (int)N, E, K);
        return finish_launch("moe_permute");
    }
    size_t smem = sizeof(int) * (E + 1);
    const int idx_in_smem = (smem + sizeof(int) * N <= 160 * 1024) ? 1 : 0;
    if (idx_in_smem) smem += sizeof(int) * N;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(moe_permute_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    moe_permute_kernel<<<1, 1024, smem, stream>>>(topk_idx, offsets, sorted_token, inv_perm, (int)N, E, K,
                                                  idx_in_smem);
    return finish_launch("moe_permute");
}

// Plain grouped product; `n_rows` is the total number of sorted rows (T*K), used for the grid only.
// cdtype: type of C (0 float, 1 bfloat16).  mode 1 = SwiGLU pair (W holds 2*Nout rows per expert).
int mi_grouped_gemm_plain(const void* A, int adtype, const int* gather, const void* W, int wdtype,
                          const int* offsets, void* C, int cdtype, int n_rows, int E, int Nout, int Kd,
                          int mode, cudaStream_t stream) {
    if (n_rows <= 0) return kOk;
    const int max_tiles = (n_rows + GB - 1) / GB + E;
    if (max_tiles > 65535) {
        set_last_error("grouped product: %d row tiles exceed the grid limit", max_tiles);
        return kBadShape;
    }
    const dim3 grid((Nout + GB - 1) / GB, max_tiles);
#define MI_GG(MODE)                                                                                     \
    MI_DISPATCH_2(adtype, AT, wdtype, WT, MI_DISPATCH_1(cdtype, CT,                                     \
        grouped_gemm_plain_kernel<AT, WT, CT, MODE><<<grid, 256, 0, stream>>>(                          \
            (const AT*)A, gather, (const WT*)W, offsets, (CT*)C, E, Nout, Kd)))
    if (mode == 0) MI_GG(0); else MI_GG(1);
#undef MI_GG
    return finish_launch("grouped_gemm_plain");
}

}  // extern "C"
