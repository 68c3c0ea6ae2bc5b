// Attention over the paged cache for a ragged batch: every request brings
// q_len new query tokens (a portion of a prompt, or one decoded token) that sit
// at the tail of its kv_len cached keys.
//
// The reference runs one block per (request, head, query token) and walks all
// pages of the request with scalar dot products, for prefill and decode alike
// (src/kernels/paged_attn_kernel.cu:102-288), accepts head sizes 64 and 128
// only (:313-315) and masks causally only in "prefill" mode (:228-231).
// Here: a tiled kernel for any head size up to 256 (float arithmetic, used by
// the 32-bit path and as the fallback of the bfloat16 path) and a split-KV
// decode kernel with a merge step.  Masking is positional in all cases:
// key j is visible from the query at absolute position p iff j <= p and
// (window == 0 or j > p - window)  (same rule as :228-236).
//
// Cache layout per layer: [page, kv_head, page_size, d]; block_table[b, i] is
// the page of keys [i*page_size, (i+1)*page_size) of request b, or -1 once a
// window has passed it.

#include "common.cuh"

namespace mi {

// ---------------------------------------------------------------------------
// Tiled kernel.  Block = 128 threads, 16 queries of one head, key tiles of 32
// aligned to absolute positions (so the order of a row's additions does not
// depend on where a portion starts, up to the first tile under a window).
// ---------------------------------------------------------------------------
constexpr int TQ = 16;   // queries per block
constexpr int TK = 32;   // keys per tile

template <typename AT, int ND>  // ND = ceil(d / 8) accumulators per thread
__global__ void __launch_bounds__(128)
attn_tiled_kernel(const AT* __restrict__ q, const AT* __restrict__ k_cache, const AT* __restrict__ v_cache,
                  const int* __restrict__ block_table, const int* __restrict__ q_start,
                  const int* __restrict__ kv_len, AT* __restrict__ out, int nh, int nkv, int d,
                  int page_size, int max_pages, int window, float scale) {
    extern __shared__ float smem[];
    const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
    const int q0 = q_start[b], q_len = q_start[b + 1] - q0;
    if (qt * TQ >= q_len) return;
    const int kvl = kv_len[b];
    const int hk = h / (nh / nkv);
    const int tid = threadIdx.x;
    const int dp = d + 1;
    float* Qs = smem;                       // [TQ][d+1]
    float* Ks = Qs + TQ * dp;               // [TK][d+1]
    float* Vs = Ks + TK * dp;               // [TK][d]
    float* Ss = Vs + TK * d;                // [TQ][TK+1]
    __shared__ int64_t row_off[TK];

    const int nq = min(TQ, q_len - qt * TQ);
    // absolute position of local query i of this tile
    const int p_lo = kvl - q_len + qt * TQ;
    const int p_hi = p_lo + nq - 1;

    for (int idx = tid; idx < TQ * d; idx += 128) {
        const int i = idx / d, c = idx - i * d;
        float v = 0.f;
        if (i < nq) v = to_float(q[((int64_t)(q0 + qt * TQ + i) * nh + h) * d + c]) * scale;
        Qs[i * dp + c] = v;
    }

    const int qi = tid >> 3;       // query row of this thread (0..15)
    const int sub = tid & 7;       // position among the 8 threads of the row
    const int my_pos = p_lo + qi;  // meaningful when qi < nq
    float m_run = -INFINITY, l_run = 0.f;
    float acc[ND];
#pragma unroll
    for (int j = 0; j < ND; ++j) acc[j] = 0.f;

    int k_begin = 0;
    if (window > 0) k_begin = max(0, p_lo - window + 1);
    k_begin = (k_begin / TK) * TK;
    const int k_end = min(kvl, p_hi + 1);
    const int* table = block_table + (int64_t)b * max_pages;

    for (int kt = k_begin; kt < k_end; kt += TK) {
        __syncthreads();  // previous tile fully consumed (and Qs written, first time)
        if (tid < TK) {
            const int kj = kt + tid;
            int64_t off = -1;
            if (kj < k_end) {
                const int page = table[kj / page_size];
                if (page >= 0)
                    off = ((int64_t)page * nkv + hk) * page_size * d + (int64_t)(kj % page_size) * d;
            }
            row_off[tid] = off;
        }
        __syncthreads();
        for (int idx = tid; idx < TK * d; idx += 128) {
            const int r = idx / d, c = idx - r * d;
            const int64_t off = row_off[r];
            float kv = 0.f, vv = 0.f;
            if (off >= 0) { kv = to_float(k_cache[off + c]); vv = to_float(v_cache[off + c]); }
            Ks[r * dp + c] = kv;
            Vs[r * d + c] = vv;
        }
        __syncthreads();
        // scores: this thread owns keys sub, sub+8, sub+16, sub+24 of row qi
        float s[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kr = sub + 8 * j;
            const int kj = kt + kr;
            float dot = 0.f;
            const float* qrow = Qs + qi * dp;
            const float* krow = Ks + kr * dp;
            for (int c = 0; c < d; ++c) dot += qrow[c] * krow[c];
            const bool vis = (qi < nq) && (kj <= my_pos) && (window == 0 || kj > my_pos - window) &&
                             (row_off[kr] >= 0);
            s[j] = vis ? dot : -INFINITY;
        }
        float tmax = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m_run, tmax);
        float alpha = 1.f, psum = 0.f;
        if (m_new == -INFINITY) {
#pragma unroll
            for (int j = 0; j < 4; ++j) Ss[qi * (TK + 1) + sub + 8 * j] = 0.f;
        } else {
            alpha = expf(m_run - m_new);  // m_run = -inf gives 0
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p = expf(s[j] - m_new);
                Ss[qi * (TK + 1) + sub + 8 * j] = p;
                psum += p;
            }
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l_run = l_run * alpha + psum;
        m_run = m_new;
        __syncwarp();  // the 8 threads of a row live in one warp: their Ss writes are visible
        const float* prow = Ss + qi * (TK + 1);
#pragma unroll
        for (int j = 0; j < ND; ++j) {
            const int c = sub + 8 * j;
            if (c < d) {
                float a = acc[j] * alpha;
                for (int kr = 0; kr < TK; ++kr) a += prow[kr] * Vs[kr * d + c];
                acc[j] = a;
            }
        }
    }
    if (qi < nq) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        AT* o = out + ((int64_t)(q0 + qt * TQ + qi) * nh + h) * d;
#pragma unroll
        for (int j = 0; j < ND; ++j) {
            const int c = sub + 8 * j;
            if (c < d) o[c] = from_float<AT>(acc[j] * inv);
        }
    }
}

// ---------------------------------------------------------------------------
// Split-KV decode: one query token per request (q_len == 1).  Block = (request,
// head, split of SPLIT keys); 16 groups of 8 threads, each group walks every
// 16th key of the split with its own running (m, l, acc); groups are merged in
// shared memory in group order, splits by the merge kernel in split order.
// The number of splits of a request depends on its own kv_len only.
// Partials: part_o [B, nh, max_splits, D], part_ml [B, nh, max_splits, 2].
// ---------------------------------------------------------------------------
// E consecutive elements (E a multiple of 8, 16-byte aligned) as floats, with 16-byte loads
template <typename AT, int E> __device__ __forceinline__ void load_vec(const AT* p, float (&out)[E]);
template <> __device__ __forceinline__ void load_vec<float, 8>(const float* p, float (&out)[8]) {
    const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) { const float4 x = __ldg(v + i); out[4*i] = x.x; out[4*i+1] = x.y; out[4*i+2] = x.z; out[4*i+3] = x.w; }
}
template <> __device__ __forceinline__ void load_vec<float, 16>(const float* p, float (&out)[16]) {
    const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float4 x = __ldg(v + i); out[4*i] = x.x; out[4*i+1] = x.y; out[4*i+2] = x.z; out[4*i+3] = x.w; }
}
template <> __device__ __forceinline__ void load_vec<float, 32>(const float* p, float (&out)[32]) {
    const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) { const float4 x = __ldg(v + i); out[4*i] = x.x; out[4*i+1] = x.y; out[4*i+2] = x.z; out[4*i+3] = x.w; }
}
__device__ __forceinline__ void unpack8(const uint4 x, float* out) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2*i] = f.x; out[2*i+1] = f.y; }
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* p, float (&out)[8]) {
    unpack8(__ldg(reinterpret_cast<const uint4*>(p)), out);
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16, 16>(const __nv_bfloat16* p, float (&out)[16]) {
    const uint4* v = reinterpret_cast<const uint4*>(p);
    unpack8(__ldg(v), out); unpack8(__ldg(v + 1), out + 8);
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16, 32>(const __nv_bfloat16* p, float (&out)[32]) {
    const uint4* v = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) unpack8(__ldg(v + i), out + 8 * i);
}

// E consecutive elements held as they were loaded (16-byte words), unpacked to float when used
template <typename AT, int E> struct RawVec;
template <int E> struct RawVec<float, E> {
    float4 w[E / 4];
    __device__ __forceinline__ void load(const float* p) {
#pragma unroll
        for (int i = 0; i < E / 4; ++i) w[i] = __ldg(reinterpret_cast<const float4*>(p) + i);
    }
    __device__ __forceinline__ void unpack(float (&out)[E]) const {
#pragma unroll
        for (int i = 0; i < E / 4; ++i) { out[4*i] = w[i].x; out[4*i+1] = w[i].y; out[4*i+2] = w[i].z; out[4*i+3] = w[i].w; }
    }
};
template <int E> struct RawVec<__nv_bfloat16, E> {
    uint4 w[E / 8];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
#pragma unroll
        for (int i = 0; i < E / 8; ++i) w[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
    }
    __device__ __forceinline__ void unpack(float (&out)[E]) const {
#pragma unroll
        for (int i = 0; i < E / 8; ++i) unpack8(w[i], &out[8 * i]);
    }
};

// Splits of a request with `kvl` keys: SPLIT keys each; a tail of up to a quarter of a split joins
// the split before it instead of making a block of its own.  A function of the request's own length only.
template <int SPLIT>
__device__ __forceinline__ int decode_splits(int kvl) {
    return max(1, (kvl + SPLIT - SPLIT / 4 - 1) / SPLIT);
}

constexpr int DEC_SPLIT = 512;      // keys per split by default; smaller splits spread one or two requests over the device
constexpr int DEC_GROUPS = 16;

template <typename AT, int D, int SPLIT>
__global__ void __launch_bounds__(128)
attn_decode_split_kernel(const AT* __restrict__ q, const AT* __restrict__ k_cache, const AT* __restrict__ v_cache,
                         const int* __restrict__ block_table, const int* __restrict__ q_start,
                         const int* __restrict__ kv_len, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int nh, int nkv, int page_size, int max_pages,
                         int max_splits, int window, float scale) {
    constexpr int E = D / 8;  // elements per thread
    wait_for_earlier_kernels();
    const int b = blockIdx.z, h = blockIdx.y, sp = blockIdx.x;
    const int kvl = kv_len[b];
    const int pos = kvl - 1;
    int k_first = 0;
    if (window > 0) k_first = max(0, pos - window + 1);
    // never more splits than the caller's scratch holds (a caller whose max_splits is too small for its
    // longest request gets a result over fewer keys, never an access outside the scratch)
    const int n_splits = min(decode_splits<SPLIT>(kvl), max_splits);
    const int first_split = min(k_first / SPLIT, n_splits - 1);
    if (sp < first_split || sp >= n_splits) return;
    const int hk = h / (nh / nkv);
    const int tid = threadIdx.x, grp = tid >> 3, sub = tid & 7;
    // the 8 threads of a group stay together; groups of one warp may diverge
    const unsigned gmask = 0xFFu << ((tid & 31) & ~7);
    const int t = q_start[b];
    float qr[E];
    load_vec<AT, E>(q + ((int64_t)t * nh + h) * D + sub * E, qr);
#pragma unroll
    for (int i = 0; i < E; ++i) qr[i] *= scale;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[E];
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] = 0.f;
    constexpr int SPAN = SPLIT + SPLIT / 4;                   // the last split may hold a short tail too
    const int k_lo = max(sp * SPLIT, k_first);
    const int k_hi = sp == n_splits - 1 ? min(kvl, sp * SPLIT + SPAN) : (sp + 1) * SPLIT;
    const int span = k_hi - sp * SPLIT;
    // the pages of this split, looked up once
    __shared__ int64_t key_off[SPAN];
    {
        const int* table = block_table + (int64_t)b * max_pages;
        for (int i = tid; i < span; i += 128) {
            const int kj = sp * SPLIT + i;
            int64_t off = -1;
            if (kj >= k_lo && kj < k_hi) {
                const int page = table[kj / page_size];
                if (page >= 0) off = ((int64_t)page * nkv + hk) * page_size * D + (int64_t)(kj % page_size) * D;
            }
            key_off[i] = off;
        }
    }
    __syncthreads();
    // KPR keys per round: all their loads are issued before any is used
    constexpr int KPR = (sizeof(AT) == 2 || E <= 16) ? 4 : 2;
    using Raw = RawVec<AT, E>;
    for (int i0 = grp; i0 < span; i0 += KPR * DEC_GROUPS) {
        int64_t off[KPR];
        Raw kr[KPR], vr[KPR];
#pragma unroll
        for (int u = 0; u < KPR; ++u) {
            const int i = i0 + u * DEC_GROUPS;
            off[u] = i < span ? key_off[i] : -1;
            if (off[u] >= 0) { kr[u].load(k_cache + off[u] + sub * E); vr[u].load(v_cache + off[u] + sub * E); }
        }
#pragma unroll
        for (int u = 0; u < KPR; ++u) {
            if (off[u] < 0) continue;
            float kf[E];
            kr[u].unpack(kf);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < E; ++i) dot += qr[i] * kf[i];
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) dot += __shfl_xor_sync(gmask, dot, o);
            const float m_new = fmaxf(m_run, dot);
            const float alpha = expf(m_run - m_new);
            const float p = expf(dot - m_new);
            l_run = l_run * alpha + p;
            vr[u].unpack(kf);
#pragma unroll
            for (int i = 0; i < E; ++i) acc[i] = acc[i] * alpha + p * kf[i];
            m_run = m_new;
        }
    }
    // merge the 16 groups in group order
    __shared__ float sm_m[DEC_GROUPS], sm_l[DEC_GROUPS];
    __shared__ float sm_o[DEC_GROUPS][D];
    if (sub == 0) { sm_m[grp] = m_run; sm_l[grp] = l_run; }
#pragma unroll
    for (int i = 0; i < E; ++i) sm_o[grp][sub * E + i] = acc[i];
    __syncthreads();
    float m_all = -INFINITY;
    for (int g = 0; g < DEC_GROUPS; ++g) m_all = fmaxf(m_all, sm_m[g]);
    const int64_t pidx = ((int64_t)b * nh + h) * max_splits + sp;
    for (int c = tid; c < D; c += 128) {
        float o = 0.f;
        for (int g = 0; g < DEC_GROUPS; ++g) {
            const float w = (sm_m[g] == -INFINITY) ? 0.f : expf(sm_m[g] - m_all);
            o += w * sm_o[g][c];
        }
        part_o[pidx * D + c] = o;
    }
    if (tid == 0) {
        float l = 0.f;
        for (int g = 0; g < DEC_GROUPS; ++g) {
            const float w = (sm_m[g] == -INFINITY) ? 0.f : expf(sm_m[g] - m_all);
            l += w * sm_l[g];
        }
        part_ml[pidx * 2] = m_all;
        part_ml[pidx * 2 + 1] = l;
    }
}

// Merge of a (request, head)'s splits in split order.  The splits' maxima and sums are fetched by all
// threads at once and their weights exp(m_s - m) kept in shared memory (up to MERGE_CAP splits; more
// are re-read from global memory), so the block waits for global memory twice, not once per split.
constexpr int MERGE_CAP = 512;

template <typename AT, int D, int SPLIT>
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int* __restrict__ q_start, const int* __restrict__ kv_len,
                                         AT* __restrict__ out, int nh, int max_splits, int window) {
    __shared__ float sm_w[MERGE_CAP], sm_l[MERGE_CAP], sm_red[4];
    wait_for_earlier_kernels();
    const int b = blockIdx.y, h = blockIdx.x;
    const int kvl = kv_len[b];
    const int pos = kvl - 1;
    int k_first = 0;
    if (window > 0) k_first = max(0, pos - window + 1);
    const int n_splits = min(decode_splits<SPLIT>(kvl), max_splits);
    const int first_split = min(k_first / SPLIT, n_splits - 1);
    const int64_t base = ((int64_t)b * nh + h) * max_splits;
    const int t = q_start[b];
    const int n = n_splits - first_split;
    if (n <= MERGE_CAP) {
        const float2* ml = reinterpret_cast<const float2*>(part_ml) + base + first_split;
        float mx = -INFINITY;
        for (int s = threadIdx.x; s < n; s += blockDim.x) {
            const float2 v = ml[s];
            sm_w[s] = v.x;
            sm_l[s] = v.y;
            mx = fmaxf(mx, v.x);
        }
        mx = warp_max(mx);
        if ((threadIdx.x & 31) == 0) sm_red[threadIdx.x >> 5] = mx;
        __syncthreads();
        float m_all = -INFINITY;
        for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w) m_all = fmaxf(m_all, sm_red[w]);
        for (int s = threadIdx.x; s < n; s += blockDim.x) {
            const float m = sm_w[s];
            sm_w[s] = m == -INFINITY ? 0.f : expf(m - m_all);
        }
        __syncthreads();
        float l = 0.f;
        for (int s = 0; s < n; ++s) l += sm_w[s] * sm_l[s];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const float* po = part_o + (base + first_split) * D;
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            float o = 0.f;
#pragma unroll 4
            for (int s = 0; s < n; ++s) o += sm_w[s] * po[(int64_t)s * D + c];
            out[((int64_t)t * nh + h) * D + c] = from_float<AT>(o * inv);
        }
        return;
    }
    float m_all = -INFINITY;
    for (int s = first_split; s < n_splits; ++s) m_all = fmaxf(m_all, part_ml[(base + s) * 2]);
    float l = 0.f;
    for (int s = first_split; s < n_splits; ++s) {
        const float m = part_ml[(base + s) * 2];
        l += (m == -INFINITY ? 0.f : expf(m - m_all)) * part_ml[(base + s) * 2 + 1];
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float o = 0.f;
        for (int s = first_split; s < n_splits; ++s) {
            const float m = part_ml[(base + s) * 2];
            o += (m == -INFINITY ? 0.f : expf(m - m_all)) * part_o[(base + s) * D + c];
        }
        out[((int64_t)t * nh + h) * D + c] = from_float<AT>(o * inv);
    }
}

template <typename AT>
static int launch_tiled(const void* q, const void* kc, const void* vc, const int* block_table,
                        const int* q_start, const int* kv_len, void* out, int B, int max_q_len, int nh,
                        int nkv, int d, int page_size, int max_pages, int window, float scale,
                        cudaStream_t stream) {
    const dim3 grid((max_q_len + TQ - 1) / TQ, nh, B);
    const size_t smem = sizeof(float) * ((size_t)TQ * (d + 1) + (size_t)TK * (d + 1) + (size_t)TK * d + TQ * (TK + 1));
#define MI_TILED(ND)                                                                                   \
    do {                                                                                               \
        auto kern = attn_tiled_kernel<AT, ND>;                                                         \
        if (smem > 48 * 1024)                                                                          \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        kern<<<grid, 128, smem, stream>>>((const AT*)q, (const AT*)kc, (const AT*)vc, block_table,     \
                                          q_start, kv_len, (AT*)out, nh, nkv, d, page_size, max_pages, \
                                          window, scale);                                              \
    } while (0)
    if (d <= 16) MI_TILED(2);
    else if (d <= 32) MI_TILED(4);
    else if (d <= 64) MI_TILED(8);
    else if (d <= 128) MI_TILED(16);
    else MI_TILED(32);
#undef MI_TILED
    return finish_launch("attn_tiled");
}

}  // namespace mi

using namespace mi;

extern "C" {

// Attention for any mix of portions and single tokens.  max_q_len bounds the
// longest portion in the batch (grid size).
int mi_attn_tiled(const void* q, const void* k_cache, const void* v_cache, int adtype, const int* block_table,
                  const int* q_start, const int* kv_len, void* out, int B, int max_q_len, int nh, int nkv,
                  int d, int page_size, int max_pages, int window, float scale, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return kOk;
    if (d < 1 || d > 256) {
        set_last_error("attention: head_dim %d is outside [1, 256]", d);
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
    MI_DISPATCH_1(adtype, AT,
        return launch_tiled<AT>(q, k_cache, v_cache, block_table, q_start, kv_len, out, B, max_q_len, nh,
                                nkv, d, page_size, max_pages, window, scale, stream));
    return kOk;
}

// 1 if the split-KV decode kernel is built for this head size.
int mi_attn_decode_supported(int d) { return (d == 64 || d == 128 || d == 256) ? 1 : 0; }

int mi_attn_decode_split_size() { return DEC_SPLIT; }

// 1 if `split` keys per split is built (128, 256, 512).
int mi_attn_decode_split_supported(int split) { return (split == 128 || split == 256 || split == 512) ? 1 : 0; }

// Decode attention: every request has exactly one query token.  `part_o` needs
// B*nh*max_splits*d floats, `part_ml` B*nh*max_splits*2, with max_splits >= ceil(max_kv_len / split).
int mi_attn_decode_split(const void* q, const void* k_cache, const void* v_cache, int adtype, const int* block_table,
                         const int* q_start, const int* kv_len, void* out, float* part_o, float* part_ml, int B,
                         int nh, int nkv, int d, int page_size, int max_pages, int max_splits, int split, int window,
                         float scale, cudaStream_t stream) {
    if (B <= 0) return kOk;
    if (!mi_attn_decode_supported(d)) {
        set_last_error("decode attention: head_dim %d is not built (64, 128, 256)", d);
        return kBadShape;
    }
    if (!mi_attn_decode_split_supported(split)) {
        set_last_error("decode attention: splits of %d keys are not built (128, 256, 512)", split);
        return kBadShape;
    }
    if (nkv < 1 || nh % nkv != 0) {
        set_last_error("attention: %d query heads are not a multiple of %d key/value heads", nh, nkv);
        return kBadShape;
    }
    if (B > 65535 || nh > 65535 || max_splits < 1) {
        set_last_error("decode attention: bad grid (B=%d, nh=%d, max_splits=%d)", B, nh, max_splits);
        return kBadShape;
    }
    const dim3 grid(max_splits, nh, B);
    const dim3 mgrid(nh, B);
#define MI_DEC(DD, SS)                                                                                    \
    do {                                                                                                  \
        launch_dependent(attn_decode_split_kernel<AT, DD, SS>, grid, dim3(128), 0, stream,                \
            (const AT*)q, (const AT*)k_cache, (const AT*)v_cache, block_table, q_start, kv_len, part_o,  \
            part_ml, nh, nkv, page_size, max_pages, max_splits, window, scale);                           \
        launch_dependent(attn_decode_merge_kernel<AT, DD, SS>, mgrid, dim3(DD <= 128 ? DD : 128), 0, stream, \
            part_o, part_ml, q_start, kv_len, (AT*)out, nh, max_splits, window);                          \
    } while (0)
#define MI_DEC_D(SS) do { if (d == 64) MI_DEC(64, SS); else if (d == 128) MI_DEC(128, SS); else MI_DEC(256, SS); } while (0)
    MI_DISPATCH_1(adtype, AT,
        if (split == 128) MI_DEC_D(128); else if (split == 256) MI_DEC_D(256); else MI_DEC_D(512));
#undef MI_DEC_D
#undef MI_DEC
    return finish_launch("attn_decode", 2);
}

// The same with the default split size.
int mi_attn_decode(const void* q, const void* k_cache, const void* v_cache, int adtype, const int* block_table,
                   const int* q_start, const int* kv_len, void* out, float* part_o, float* part_ml, int B,
                   int nh, int nkv, int d, int page_size, int max_pages, int max_splits, int window,
                   float scale, cudaStream_t stream) {
    return mi_attn_decode_split(q, k_cache, v_cache, adtype, block_table, q_start, kv_len, out, part_o, part_ml, B, nh,
                                nkv, d, page_size, max_pages, max_splits, DEC_SPLIT, window, scale, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate (see attention_noalloc.h): the
// split partials live in an array that is part of the library image instead of caller scratch.
// ---------------------------------------------------------------------------------------------
#include "attention_noalloc.h"

namespace mi {

static __device__ __align__(256) unsigned char g_noalloc_scratch[MI_ATTN_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// Device address of g_noalloc_scratch per device.  In host code the array's name is only a
// handle for cudaGetSymbolAddress, never a pointer a kernel could use.
static float* g_noalloc_ptr[kMaxDevices] = {nullptr};

// Looks the address up once per device, with that device current.  Returns nullptr on failure.
static float* noalloc_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_last_error("decode attention (no allocation): cannot identify the current device");
        return nullptr;
    }
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            set_last_error("decode attention (no allocation): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    return g_noalloc_ptr[dev];
}

}  // namespace mi

extern "C" {

unsigned int mi_attn_decode_noalloc_capacity(void) { return MI_ATTN_NOALLOC_SCRATCH_BYTES; }

int mi_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, int adtype,
                           const int* block_table, const int* q_start, const int* kv_len, void* out, int B,
                           int nh, int nkv, int d, int page_size, int max_pages, int max_splits, int window,
                           float scale, cudaStream_t stream) {
    if (B <= 0) return kOk;
    if (max_splits < 1 || nh < 1 || d < 1) {
        set_last_error("decode attention (no allocation): bad sizes (nh=%d, d=%d, max_splits=%d)", nh, d, max_splits);
        return kBadShape;
    }
    const unsigned long long n_part = (unsigned long long)B * nh * max_splits;
    const unsigned long long need = n_part * ((unsigned long long)d + 2ull) * sizeof(float);
    if (need > MI_ATTN_NOALLOC_SCRATCH_BYTES) {
        set_last_error("decode attention (no allocation): B=%d, heads=%d, splits=%d, head_dim=%d need %llu bytes of "
                       "scratch, the built-in array holds %u", B, nh, max_splits, d, need,
                       (unsigned)MI_ATTN_NOALLOC_SCRATCH_BYTES);
        return kBadShape;
    }
    float* scratch = noalloc_scratch_for_current_device();
    if (!scratch) return kLaunchFailed;
    float* part_o = scratch;                       // [B, nh, max_splits, d]
    float* part_ml = scratch + n_part * d;         // [B, nh, max_splits, 2]
    return mi_attn_decode(q, k_cache, v_cache, adtype, block_table, q_start, kv_len, out, part_o, part_ml, B, nh,
                          nkv, d, page_size, max_pages, max_splits, window, scale, stream);
}

}  // extern "C"
