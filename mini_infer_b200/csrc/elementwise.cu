// Row-wise kernels: embedding gather, residual add + RMSNorm, bias + rotary
// position encoding + cache write, SwiGLU, expert combine.
//
// Counterparts in the reference (all FP16, one op per kernel, default stream):
//   embedding gather      src/kernels/model_utils_kernel.cu:45-64
//   residual add          src/kernels/model_utils_kernel.cu:31-42
//   RMSNorm               src/kernels/rmsnorm_kernel.cu:30-67
//   bias add              src/kernels/model_utils_kernel.cu:11-28
//   rotary tables + apply src/kernels/rope_kernel.cu:27-77
//   cache scatter         src/kernels/model_utils_kernel.cu:108-164
//   SwiGLU                src/kernels/swiglu_kernel.cu:16-26
//   expert accumulate     src/kernels/moe_kernel.cu:65-146
// Here the residual stream is float in both precision paths, sums are float,
// and ops that follow one another on the same row are one kernel.

#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>

namespace mi {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

static std::atomic<long long> g_launches{0};
static std::atomic<int> g_dependent_launch{0};

bool dependent_launch_enabled() { return g_dependent_launch.load(std::memory_order_relaxed) != 0; }

int finish_launch(const char* what, int n_kernels) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("%s: %s", what, cudaGetErrorString(e));
        return kLaunchFailed;
    }
    g_launches.fetch_add(n_kernels, std::memory_order_relaxed);
    return kOk;
}

// ---------------------------------------------------------------------------
// embedding: hidden[t, :] = table[ids[t], :]
// ---------------------------------------------------------------------------
template <typename WT>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const WT* __restrict__ table,
                                    float* __restrict__ hidden, int H, int V) {
    wait_for_earlier_kernels();
    const int t = blockIdx.x;
    int id = ids[t];
    // ids are validated on the host; clamp so that a bad id can never read outside the table
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const WT* row = table + (int64_t)id * H;
    float* out = hidden + (int64_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_float(row[i]);
}

// ---------------------------------------------------------------------------
// hidden += delta (optional); out = hidden * rsqrt(mean(hidden^2) + eps) * w
// With `rows`, output row r is computed from hidden row rows[r] and hidden is
// left untouched (the same row may be asked for twice).
// ---------------------------------------------------------------------------
template <typename AT, typename WT>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const float* __restrict__ delta,
                                   const int* __restrict__ rows, const WT* __restrict__ weight,
                                   AT* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* h = hidden + (int64_t)src * H;
    const float* d = delta ? delta + (int64_t)src * H : nullptr;
    AT* o = out + (int64_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = h[i];
        if (d) {
            v += d[i];
            if (!rows) h[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rrms = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = h[i];
        if (d && rows) v += d[i];
        o[i] = from_float<AT>(v * rrms * to_float(weight[i]));
    }
}

// The same for rows of H = 4 * VPT * 256 floats at most: a thread keeps its float4s in registers
// between the two passes.  Threads take interleaved float4s, so the order of the additions of a
// row's sum of squares differs from the scalar kernel's but depends on H only.
template <typename AT, typename WT, int VPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ hidden, const float* __restrict__ delta,
                       const int* __restrict__ rows, const WT* __restrict__ weight,
                       AT* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float4* h = reinterpret_cast<float4*>(hidden + (int64_t)src * H);
    const float4* d = delta ? reinterpret_cast<const float4*>(delta + (int64_t)src * H) : nullptr;
    const int nv = H >> 2;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + 256 * j;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nv) {
            v[j] = h[i];
            if (d) {
                const float4 dv = d[i];
                v[j].x += dv.x; v[j].y += dv.y; v[j].z += dv.z; v[j].w += dv.w;
                if (!rows) h[i] = v[j];
            }
            ss += v[j].x * v[j].x;
            ss += v[j].y * v[j].y;
            ss += v[j].z * v[j].z;
            ss += v[j].w * v[j].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rrms = rsqrtf(ss / (float)H + eps);
    AT* o = out + (int64_t)r * H;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < nv) {
            const int c = 4 * i;
            o[c] = from_float<AT>(v[j].x * rrms * to_float(weight[c]));
            o[c + 1] = from_float<AT>(v[j].y * rrms * to_float(weight[c + 1]));
            o[c + 2] = from_float<AT>(v[j].z * rrms * to_float(weight[c + 2]));
            o[c + 3] = from_float<AT>(v[j].w * rrms * to_float(weight[c + 3]));
        }
    }
}

// ---------------------------------------------------------------------------
// q/k/v post-processing for one token per block:
//   add bias; rotate the first rot_dim dims of every q and k head by
//   angle = position * inv_freq[i] (pairs (i, i + rot_dim/2));
//   q -> q_out[t, head, :]; k, v -> cache slot slot_mapping[t]
// cache layout per layer: [page, kv_head, page_size, d]
// ---------------------------------------------------------------------------
constexpr int QKV_HEADS_PER_BLOCK = 8;

__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <typename AT, typename WT>
__global__ void __launch_bounds__(128)
qkv_post_kernel(const float* __restrict__ qkv, const WT* __restrict__ bias,
                const int* __restrict__ positions, const float* __restrict__ inv_freq,
                const int* __restrict__ slot_mapping, AT* __restrict__ q_out,
                AT* __restrict__ k_cache, AT* __restrict__ v_cache,
                int nh, int nkv, int d, int rot_dim, int page_size, int heads_per_block) {
    const int t = blockIdx.x;
    const int total_heads = nh + 2 * nkv;
    const int h_lo = blockIdx.y * heads_per_block;
    const int h_hi = min(total_heads, h_lo + heads_per_block);
    const float* row = qkv + (int64_t)t * total_heads * d;
    const float pos = (float)positions[t];
    const int half = rot_dim >> 1;
    const int rest = d - rot_dim;
    int64_t kbase = -1;
    if (nkv > 0) {
        const int slot = slot_mapping[t];
        if (slot >= 0) {
            const int page = slot / page_size, off = slot - page * page_size;
            kbase = (int64_t)page * nkv * page_size * d + (int64_t)off * d;
        }
    }
    // work items: (head of this block, two neighbouring pair indices i, i+1 < half); when the number
    // of items per head divides the block size a thread keeps the same i for all its heads and
    // computes the angles' cosines and sines once.  Values travel in pairs (8-byte loads, 4- or
    // 8-byte stores).
    const int n_heads = h_hi - h_lo;
    if ((half & 1) == 0 && half > 0) {
        const int hp = half >> 1;
        const bool same_i = (blockDim.x % hp) == 0;
        float c0k = 1.f, s0k = 0.f, c1k = 1.f, s1k = 0.f;
        if (same_i && inv_freq) {
            const int i = 2 * (threadIdx.x % hp);
            const float a0 = pos * inv_freq[i], a1 = pos * inv_freq[i + 1];
            c0k = cosf(a0); s0k = sinf(a0); c1k = cosf(a1); s1k = sinf(a1);
        }
        for (int idx = threadIdx.x; idx < n_heads * hp; idx += blockDim.x) {
            const int head = h_lo + idx / hp, i = 2 * (idx % hp);
            if (head >= nh + nkv) break;                     // v heads follow the q and k heads
            AT* dst = nullptr;
            if (head < nh) dst = q_out + ((int64_t)t * nh + head) * d;
            else if (kbase >= 0) dst = k_cache + kbase + (int64_t)(head - nh) * page_size * d;
            if (!dst) continue;
            const int c0 = head * d + i, c1 = c0 + half;
            float2 lo = *reinterpret_cast<const float2*>(row + c0);
            float2 hi = *reinterpret_cast<const float2*>(row + c1);
            if (bias) {
                lo.x += to_float(bias[c0]); lo.y += to_float(bias[c0 + 1]);
                hi.x += to_float(bias[c1]); hi.y += to_float(bias[c1 + 1]);
            }
            float2 ylo = lo, yhi = hi;
            if (inv_freq) {
                float ca = c0k, sa = s0k, cb = c1k, sb = s1k;
                if (!same_i) {
                    const float a0 = pos * inv_freq[i], a1 = pos * inv_freq[i + 1];
                    ca = cosf(a0); sa = sinf(a0); cb = cosf(a1); sb = sinf(a1);
                }
                ylo.x = lo.x * ca - hi.x * sa;  yhi.x = hi.x * ca + lo.x * sa;
                ylo.y = lo.y * cb - hi.y * sb;  yhi.y = hi.y * cb + lo.y * sb;
            }
            store_pair(dst + i, ylo.x, ylo.y);
            store_pair(dst + i + half, yhi.x, yhi.y);
        }
    } else {
        for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
            const int head = h_lo + idx / half, i = idx % half;
            if (head >= nh + nkv) break;
            AT* dst = nullptr;
            if (head < nh) dst = q_out + ((int64_t)t * nh + head) * d;
            else if (kbase >= 0) dst = k_cache + kbase + (int64_t)(head - nh) * page_size * d;
            if (!dst) continue;
            const int c0 = head * d + i, c1 = c0 + half;
            float x0 = row[c0], x1 = row[c1];
            if (bias) { x0 += to_float(bias[c0]); x1 += to_float(bias[c1]); }
            float y0 = x0, y1 = x1;
            if (inv_freq) {
                const float ang = pos * inv_freq[i];
                const float c = cosf(ang), sn = sinf(ang);
                y0 = x0 * c - x1 * sn;
                y1 = x1 * c + x0 * sn;
            }
            dst[i] = from_float<AT>(y0);
            dst[i + half] = from_float<AT>(y1);
        }
    }
    for (int head = h_lo; head < h_hi; ++head) {
        if (head < nh + nkv) {
            if (rest <= 0) continue;
            AT* dst = nullptr;
            if (head < nh) dst = q_out + ((int64_t)t * nh + head) * d;
            else if (kbase >= 0) dst = k_cache + kbase + (int64_t)(head - nh) * page_size * d;
            if (!dst) continue;
            for (int i = rot_dim + threadIdx.x; i < d; i += blockDim.x) {
                float x = row[head * d + i];
                if (bias) x += to_float(bias[head * d + i]);
                dst[i] = from_float<AT>(x);
            }
        } else if (kbase >= 0) {
            AT* dst = v_cache + kbase + (int64_t)(head - nh - nkv) * page_size * d;
            for (int i = threadIdx.x; i < d; i += blockDim.x) {
                float x = row[head * d + i];
                if (bias) x += to_float(bias[head * d + i]);
                dst[i] = from_float<AT>(x);
            }
        }
    }
}

// The same for many tokens in bfloat16 with the rotation over the whole head (or none) and
// d a multiple of 8: one block per token, four pairs per thread and step (16-byte loads of the
// float row, 8-byte stores), the angles' cosines and sines computed once when a thread keeps
// its pair index for all heads.
template <typename WT>
__global__ void __launch_bounds__(128)
qkv_post_rows_kernel(const float* __restrict__ qkv, const WT* __restrict__ bias,
                     const int* __restrict__ positions, const float* __restrict__ inv_freq,
                     const int* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ q_out,
                     __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                     int nh, int nkv, int d, int page_size) {
    const int t = blockIdx.x;
    const int total_heads = nh + 2 * nkv;
    const float* row = qkv + (int64_t)t * total_heads * d;
    const float pos = (float)positions[t];
    const int half = d >> 1, per_head = half >> 2;        // items of 4 pairs per head
    int64_t kbase = -1;
    if (nkv > 0) {
        const int slot = slot_mapping[t];
        if (slot >= 0) {
            const int page = slot / page_size, off = slot - page * page_size;
            kbase = (int64_t)page * nkv * page_size * d + (int64_t)off * d;
        }
    }
    const bool same_i = (blockDim.x % per_head) == 0;
    float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (same_i && inv_freq) {
        const int i = 4 * (threadIdx.x % per_head);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float a = pos * inv_freq[i + u];
            cs[u] = cosf(a); sn[u] = sinf(a);
        }
    }
    const int items = (nh + nkv) * per_head;
#pragma unroll 4
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
        const int head = idx / per_head, i = 4 * (idx - head * per_head);
        __nv_bfloat16* dst = nullptr;
        if (head < nh) dst = q_out + ((int64_t)t * nh + head) * d;
        else if (kbase >= 0) dst = k_cache + kbase + (int64_t)(head - nh) * page_size * d;
        if (!dst) continue;
        const int c0 = head * d + i, c1 = c0 + half;
        const float4 l4 = *reinterpret_cast<const float4*>(row + c0);
        const float4 h4 = *reinterpret_cast<const float4*>(row + c1);
        float lo[4] = {l4.x, l4.y, l4.z, l4.w}, hi[4] = {h4.x, h4.y, h4.z, h4.w};
        if (bias) {
#pragma unroll
            for (int u = 0; u < 4; ++u) { lo[u] += to_float(bias[c0 + u]); hi[u] += to_float(bias[c1 + u]); }
        }
        float ylo[4], yhi[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float ca = cs[u], sa = sn[u];
            if (!same_i && inv_freq) {
                const float a = pos * inv_freq[i + u];
                ca = cosf(a); sa = sinf(a);
            }
            ylo[u] = inv_freq ? lo[u] * ca - hi[u] * sa : lo[u];
            yhi[u] = inv_freq ? hi[u] * ca + lo[u] * sa : hi[u];
        }
        uint2 plo, phi;
        plo.x = pack2(ylo[0], ylo[1]); plo.y = pack2(ylo[2], ylo[3]);
        phi.x = pack2(yhi[0], yhi[1]); phi.y = pack2(yhi[2], yhi[3]);
        *reinterpret_cast<uint2*>(dst + i) = plo;
        *reinterpret_cast<uint2*>(dst + i + half) = phi;
    }
    if (kbase >= 0) {
        const int per_v = d >> 2;                             // float4 per head
#pragma unroll 4
        for (int idx = threadIdx.x; idx < nkv * per_v; idx += blockDim.x) {
            const int hv = idx / per_v, i = 4 * (idx - hv * per_v);
            const int c = (nh + nkv + hv) * d + i;
            float4 x = *reinterpret_cast<const float4*>(row + c);
            if (bias) {
                x.x += to_float(bias[c]); x.y += to_float(bias[c + 1]);
                x.z += to_float(bias[c + 2]); x.w += to_float(bias[c + 3]);
            }
            uint2 pk;
            pk.x = pack2(x.x, x.y); pk.y = pack2(x.z, x.w);
            *reinterpret_cast<uint2*>(v_cache + kbase + (int64_t)hv * page_size * d + i) = pk;
        }
    }
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, I + i]
// ---------------------------------------------------------------------------
template <typename AT>
__global__ void swiglu_kernel(const AT* __restrict__ gu, AT* __restrict__ out, int64_t total, int I) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = to_float(gu[t * 2 * I + i]);
        const float u = to_float(gu[t * 2 * I + I + i]);
        out[idx] = from_float<AT>(g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 rows with I a multiple of 8: 16 bytes per load and store
__global__ void swiglu_bf16x8_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, int64_t total_vec,
                                     int Iv) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vec;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / Iv;
        const int i = (int)(idx - t * Iv);
        const uint4 gv = __ldg(gu + t * 2 * Iv + i);
        const uint4 uv = __ldg(gu + t * 2 * Iv + Iv + i);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 r;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            r2[j] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        out[idx] = r;
    }
}

// ---------------------------------------------------------------------------
// out[t, :] = sum_k w[t, k] * y[inv_perm[t*K + k], :]   (k ascending: slot order)
//           + gate[t] * shared[t, :]                     (if shared)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ inv_perm,
                   const float* __restrict__ w, const float* __restrict__ shared,
                   const float* __restrict__ gate, float* __restrict__ out, int H, int K) {
    const int t = blockIdx.x;
    const int i0 = blockIdx.y * 512 + threadIdx.x;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < K; ++k) {
        const int r = inv_perm ? inv_perm[t * K + k] : t * K + k;
        const float wk = w[t * K + k];
        const float* yr = y + (int64_t)r * H;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + 128 * j;
            if (i < H) acc[j] += wk * yr[i];
        }
    }
    const float gt = shared ? gate[t] : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = i0 + 128 * j;
        if (i < H) {
            float v = acc[j];
            if (shared) v += gt * shared[(int64_t)t * H + i];
            out[(int64_t)t * H + i] = v;
        }
    }
}

// ---------------------------------------------------------------------------
// The expert combine and the residual addition and RMSNorm that follow it, in one pass over a row:
//   delta[t, :] = sum_k w[t, k] * y[inv_perm[t*K + k], :] + gate[t] * shared[t, :]   (as moe_combine)
//   hidden[t, :] += delta[t, :];  out = hidden * rsqrt(mean(hidden^2) + eps) * weight  (as add_rmsnorm)
// The additions run in the order of the two separate kernels, so the result is theirs bit for bit.
// ---------------------------------------------------------------------------
struct CombineArgs {
    const float* y;
    const int* inv_perm;
    const float* w;
    const float* shared;
    const float* gate;
    int K;
};

template <typename AT, typename WT>
__global__ void combine_add_rmsnorm_kernel(float* __restrict__ hidden, CombineArgs ca, const int* __restrict__ rows,
                                           const WT* __restrict__ weight, AT* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* h = hidden + (int64_t)src * H;
    AT* o = out + (int64_t)r * H;
    const float gt = ca.shared ? ca.gate[src] : 0.f;
    auto delta = [&](int i) {
        float acc = 0.f;
        for (int k = 0; k < ca.K; ++k) {
            const int yr = ca.inv_perm ? ca.inv_perm[src * ca.K + k] : src * ca.K + k;
            acc += ca.w[src * ca.K + k] * ca.y[(int64_t)yr * H + i];
        }
        if (ca.shared) acc += gt * ca.shared[(int64_t)src * H + i];
        return acc;
    };
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = h[i] + delta(i);
        if (!rows) h[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rrms = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = rows ? h[i] + delta(i) : h[i];
        o[i] = from_float<AT>(v * rrms * to_float(weight[i]));
    }
}

template <typename AT, typename WT, int VPT>
__global__ void __launch_bounds__(256)
combine_add_rmsnorm_vec_kernel(float* __restrict__ hidden, CombineArgs ca, const int* __restrict__ rows,
                               const WT* __restrict__ weight, AT* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float4* h = reinterpret_cast<float4*>(hidden + (int64_t)src * H);
    const int nv = H >> 2;
    float4 v[VPT], acc[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < ca.K; ++k) {
        const int yr = ca.inv_perm ? ca.inv_perm[src * ca.K + k] : src * ca.K + k;
        const float wk = ca.w[src * ca.K + k];
        const float4* yv = reinterpret_cast<const float4*>(ca.y + (int64_t)yr * H);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + 256 * j;
            if (i < nv) {
                const float4 t = yv[i];
                acc[j].x += wk * t.x; acc[j].y += wk * t.y; acc[j].z += wk * t.z; acc[j].w += wk * t.w;
            }
        }
    }
    if (ca.shared) {
        const float gt = ca.gate[src];
        const float4* sv = reinterpret_cast<const float4*>(ca.shared + (int64_t)src * H);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + 256 * j;
            if (i < nv) {
                const float4 t = sv[i];
                acc[j].x += gt * t.x; acc[j].y += gt * t.y; acc[j].z += gt * t.z; acc[j].w += gt * t.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + 256 * j;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nv) {
            v[j] = h[i];
            v[j].x += acc[j].x; v[j].y += acc[j].y; v[j].z += acc[j].z; v[j].w += acc[j].w;
            if (!rows) h[i] = v[j];
            ss += v[j].x * v[j].x;
            ss += v[j].y * v[j].y;
            ss += v[j].z * v[j].z;
            ss += v[j].w * v[j].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rrms = rsqrtf(ss / (float)H + eps);
    AT* o = out + (int64_t)r * H;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < nv) {
            const int c = 4 * i;
            o[c] = from_float<AT>(v[j].x * rrms * to_float(weight[c]));
            o[c + 1] = from_float<AT>(v[j].y * rrms * to_float(weight[c + 1]));
            o[c + 2] = from_float<AT>(v[j].z * rrms * to_float(weight[c + 2]));
            o[c + 3] = from_float<AT>(v[j].w * rrms * to_float(weight[c + 3]));
        }
    }
}

}  // namespace mi

using namespace mi;

extern "C" {

const char* mi_last_error() { return g_last_error; }

// Kernels of this library queued since it was loaded (all threads).
long long mi_launch_count() { return g_launches.load(std::memory_order_relaxed); }

// Switches programmatic dependent launch on (1) or off (0) for the kernels of decode-sized steps that
// are written for it (see common.cuh); returns the setting before.
int mi_set_dependent_launch(int on) { return g_dependent_launch.exchange(on ? 1 : 0, std::memory_order_relaxed); }

int mi_embed_gather(const int* ids, const void* table, int wdtype, float* hidden, int T, int H, int V,
                    cudaStream_t stream) {
    if (T <= 0) return kOk;
    MI_DISPATCH_1(wdtype, WT,
        launch_dependent(embed_gather_kernel<WT>, dim3(T), dim3(256), 0, stream, ids, (const WT*)table, hidden, H, V));
    return finish_launch("embed_gather");
}

int mi_add_rmsnorm(float* hidden, const float* delta, const int* rows, const void* weight, int wdtype,
                   void* out, int adtype, int n_rows, int H, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return kOk;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool aligned = ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(delta)) & 15) == 0;
    if (H % 4 == 0 && H >= 1024 && H <= 8192 && aligned) {
        if (H <= 2048) {
            MI_DISPATCH_2(adtype, AT, wdtype, WT,
                launch_dependent(add_rmsnorm_vec_kernel<AT, WT, 2>, dim3(n_rows), dim3(256), 0, stream,
                                 hidden, delta, rows, (const WT*)weight, (AT*)out, H, eps));
        } else if (H <= 4096) {
            MI_DISPATCH_2(adtype, AT, wdtype, WT,
                launch_dependent(add_rmsnorm_vec_kernel<AT, WT, 4>, dim3(n_rows), dim3(256), 0, stream,
                                 hidden, delta, rows, (const WT*)weight, (AT*)out, H, eps));
        } else {
            MI_DISPATCH_2(adtype, AT, wdtype, WT,
                launch_dependent(add_rmsnorm_vec_kernel<AT, WT, 8>, dim3(n_rows), dim3(256), 0, stream,
                                 hidden, delta, rows, (const WT*)weight, (AT*)out, H, eps));
        }
        return finish_launch("add_rmsnorm");
    }
    MI_DISPATCH_2(adtype, AT, wdtype, WT,
        add_rmsnorm_kernel<AT, WT><<<n_rows, threads, 0, stream>>>(
            hidden, delta, rows, (const WT*)weight, (AT*)out, H, eps));
    return finish_launch("add_rmsnorm");
}

// The expert combine (arguments as mi_moe_combine, rows of `y` indexed through `inv_perm` or by pair)
// fused with the residual addition and RMSNorm that follow (arguments as mi_add_rmsnorm).
int mi_combine_add_rmsnorm(float* hidden, const float* y, const int* inv_perm, const float* w, const float* shared,
                           const float* gate, int K, const int* rows, const void* weight, int wdtype, void* out,
                           int adtype, int n_rows, int H, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return kOk;
    const CombineArgs ca{y, inv_perm, w, shared, gate, K};
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool aligned = ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(y) |
                           reinterpret_cast<uintptr_t>(shared)) & 15) == 0;
    if (H % 4 == 0 && H >= 1024 && H <= 8192 && aligned) {
        if (H <= 2048) {
            MI_DISPATCH_2(adtype, AT, wdtype, WT,
                launch_dependent(combine_add_rmsnorm_vec_kernel<AT, WT, 2>, dim3(n_rows), dim3(256), 0, stream,
                                 hidden, ca, rows, (const WT*)weight, (AT*)out, H, eps));
        } else if (H <= 4096) {
            MI_DISPATCH_2(adtype, AT, wdtype, WT,
                launch_dependent(combine_add_rmsnorm_vec_kernel<AT, WT, 4>, dim3(n_rows), dim3(256), 0, stream,
                                 hidden, ca, rows, (const WT*)weight, (AT*)out, H, eps));
        } else {
            MI_DISPATCH_2(adtype, AT, wdtype, WT,
                launch_dependent(combine_add_rmsnorm_vec_kernel<AT, WT, 8>, dim3(n_rows), dim3(256), 0, stream,
                                 hidden, ca, rows, (const WT*)weight, (AT*)out, H, eps));
        }
        return finish_launch("combine_add_rmsnorm");
    }
    MI_DISPATCH_2(adtype, AT, wdtype, WT,
        combine_add_rmsnorm_kernel<AT, WT><<<n_rows, threads, 0, stream>>>(
            hidden, ca, rows, (const WT*)weight, (AT*)out, H, eps));
    return finish_launch("combine_add_rmsnorm");
}

int mi_qkv_post(const float* qkv, const void* bias, int wdtype, const int* positions, const float* inv_freq,
                const int* slot_mapping, void* q_out, void* k_cache, void* v_cache, int adtype,
                int T, int nh, int nkv, int d, int rot_dim, int page_size, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) {
        set_last_error("qkv_post: rot_dim %d must be even and within head_dim %d", rot_dim, d);
        return kBadShape;
    }
    if (!inv_freq) rot_dim = d;  // no rotation: treat all dims as "pairs" that are copied
    if (d & 1) {
        set_last_error("qkv_post: head_dim %d must be even", d);
        return kBadShape;
    }
    if (adtype == kBF16 && T >= 64 && d % 8 == 0 && (inv_freq == nullptr || rot_dim == d) &&
        (((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out)) & 15) == 0) &&
        (nkv == 0 || ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0)) {
        MI_DISPATCH_1(wdtype, WT,
            qkv_post_rows_kernel<WT><<<T, 128, 0, stream>>>(
                qkv, (const WT*)bias, positions, inv_freq, slot_mapping, (__nv_bfloat16*)q_out,
                (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, d, page_size));
        return finish_launch("qkv_post");
    }
    // few tokens: many blocks of a few heads; many tokens: a block per token, which looks up its
    // position and cache slot once and computes each angle once for all heads
    const int hpb = T >= 512 ? nh + 2 * nkv : QKV_HEADS_PER_BLOCK;
    const dim3 grid(T, (nh + 2 * nkv + hpb - 1) / hpb);
    MI_DISPATCH_2(adtype, AT, wdtype, WT,
        qkv_post_kernel<AT, WT><<<grid, 128, 0, stream>>>(
            qkv, (const WT*)bias, positions, inv_freq, slot_mapping, (AT*)q_out, (AT*)k_cache,
            (AT*)v_cache, nh, nkv, d, rot_dim, page_size, hpb));
    return finish_launch("qkv_post");
}

int mi_swiglu(const void* gu, void* out, int adtype, int64_t T, int I, cudaStream_t stream) {
    const int64_t total = T * I;
    if (total <= 0) return kOk;
    if (adtype == kBF16 && I % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int64_t total_vec = total / 8;
        int64_t vblocks = (total_vec + 255) / 256;
        if (vblocks > 148 * 16) vblocks = 148 * 16;
        swiglu_bf16x8_kernel<<<(int)vblocks, 256, 0, stream>>>((const uint4*)gu, (uint4*)out, total_vec, I / 8);
        return finish_launch("swiglu");
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    MI_DISPATCH_1(adtype, AT,
        swiglu_kernel<AT><<<(int)blocks, 256, 0, stream>>>((const AT*)gu, (AT*)out, total, I));
    return finish_launch("swiglu");
}

int mi_moe_combine(const float* y, const int* inv_perm, const float* w, const float* shared,
                   const float* gate, float* out, int T, int H, int K, cudaStream_t stream) {
    if (T <= 0) return kOk;
    moe_combine_kernel<<<dim3(T, (H + 511) / 512), 128, 0, stream>>>(y, inv_perm, w, shared, gate, out, H, K);
    return finish_launch("moe_combine");
}

}  // extern "C"
