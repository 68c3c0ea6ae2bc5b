// Sampling from float logits, one block per row: greedy, temperature, nucleus.
//
// The reference has an arg-max kernel whose tie order is an artefact of its
// tree reduction (src/kernels/sampling_kernel.cu:14-89) and a top-p kernel
// that falls back to greedy above 30000 vocabulary entries and picks uniformly
// inside the nucleus (:101-223).  The rules here are defined, not inherited:
//   greedy       lowest index among equal maxima
//   temperature  p = softmax(logits / T); token = first index whose cumulative
//                probability (index order) exceeds u
//   top-p        only tokens with p >= tau take part, tau being the largest
//                probability value whose at-or-above mass is >= top_p; u is
//                scaled by the nucleus mass
// u comes from the host (a counter-based generator keyed by seed, request and
// token number), so a request's tokens do not depend on its batch.

#include "common.cuh"

namespace mi {

constexpr int SAMP_THREADS = 1024;

struct ArgBest { float v; int i; };

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ ArgBest block_argmax(ArgBest x, ArgBest* scratch /*[32]*/) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    ArgBest r = (lane < (int)(blockDim.x >> 5)) ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest y;
        y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, y);
    }
    return r;
}

__global__ void __launch_bounds__(SAMP_THREADS)
sample_rows_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                   const float* __restrict__ top_p, const float* __restrict__ u, float* __restrict__ probs,
                   int* __restrict__ out, int V) {
    __shared__ float fscratch[32];
    __shared__ ArgBest ascratch[32];
    __shared__ float chunk_sum[SAMP_THREADS];
    __shared__ int chosen;
    wait_for_earlier_kernels();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (int64_t)r * V;
    const float T = temperature ? temperature[r] : 0.f;

    // arg-max (also the fallback of the sampling path)
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < V; i += SAMP_THREADS) {
        const float v = row[i];
        if (v > best.v) { best.v = v; best.i = i; }
    }
    best = block_argmax(best, ascratch);
    if (!(T > 0.f)) {
        if (tid == 0) out[r] = best.i;
        return;
    }

    float* p = probs + (int64_t)r * V;
    const float zmax = best.v / T;
    float s = 0.f;
    for (int i = tid; i < V; i += SAMP_THREADS) {
        const float e = expf(row[i] / T - zmax);
        p[i] = e;
        s += e;
    }
    s = block_sum(s, fscratch);
    float pmax = 0.f;
    for (int i = tid; i < V; i += SAMP_THREADS) {
        const float v = p[i] / s;
        p[i] = v;
        pmax = fmaxf(pmax, v);
    }
    pmax = block_max(pmax, fscratch);

    // nucleus threshold: largest bit pattern t with mass(p >= t) >= top_p
    float tau = 0.f;
    const float tp = top_p ? top_p[r] : 1.f;
    if (tp < 1.f) {
        unsigned lo = 0u, hi = __float_as_uint(pmax) + 1u;
        while (hi - lo > 1u) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            const float th = __uint_as_float(mid);
            float m = 0.f;
            for (int i = tid; i < V; i += SAMP_THREADS) {
                const float v = p[i];
                if (v >= th) m += v;
            }
            m = block_sum(m, fscratch);
            if (m >= tp) lo = mid; else hi = mid;
        }
        tau = __uint_as_float(lo);
    }

    // inverse CDF in index order over the kept tokens; thread c owns a contiguous chunk
    const int chunk = (V + SAMP_THREADS - 1) / SAMP_THREADS;
    const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);
    float cs = 0.f;
    for (int i = c0; i < c1; ++i) {
        const float v = p[i];
        if (v >= tau) cs += v;
    }
    chunk_sum[tid] = cs;
    if (tid == 0) chosen = -1;
    __syncthreads();
    // inclusive scan over the 1024 chunk sums (Hillis-Steele)
    for (int off = 1; off < SAMP_THREADS; off <<= 1) {
        const float add = tid >= off ? chunk_sum[tid - off] : 0.f;
        __syncthreads();
        chunk_sum[tid] += add;
        __syncthreads();
    }
    const float total = chunk_sum[SAMP_THREADS - 1];
    const float target = u[r] * total;
    const float incl = chunk_sum[tid];
    const float excl = tid ? chunk_sum[tid - 1] : 0.f;
    if (excl <= target && target < incl) {
        float run = excl;
        int pick = -1, last_kept = -1;
        for (int i = c0; i < c1; ++i) {
            const float v = p[i];
            if (v >= tau) {
                last_kept = i;
                run += v;
                if (run > target) { pick = i; break; }
            }
        }
        chosen = pick >= 0 ? pick : last_kept;
    }
    __syncthreads();
    if (tid == 0) out[r] = chosen >= 0 ? chosen : best.i;
}

}  // namespace mi

using namespace mi;

extern "C" {

// temperature/top_p/u may be null (all rows greedy); probs [R, V] is scratch for the sampled rows.
int mi_sample_rows(const float* logits, const float* temperature, const float* top_p, const float* u,
                   float* probs, int* out, int R, int V, cudaStream_t stream) {
    if (R <= 0) return kOk;
    if (temperature && (!u || !probs)) {
        set_last_error("sample_rows: temperature sampling needs the uniforms and a scratch row per request");
        return kBadShape;
    }
    launch_dependent(sample_rows_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits, temperature, top_p, u, probs, out, V);
    return finish_launch("sample_rows");
}

}  // extern "C"
