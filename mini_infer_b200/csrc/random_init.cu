// Counter-based random weights: element i of a tensor is a pure function of (key, i).
//
// value(i) = offset + scale * (h_0 + ... + h_7 - 262140), where h_0..h_7 are the eight 16-bit halves
// of Philox-4x32-10(counter = (i mod 2^32, i >> 32, 0, 0), key) and 262140 is the mean of their sum.
// The sum of eight uniform 16-bit integers is close to normal (variance 8 * (65536^2 - 1) / 12, bounded
// at 3.46 standard deviations); the arithmetic is one exact integer sum, one float multiplication and one
// float addition, each rounded once, so the host function of weights/random_init.py gives the same bits.
// The reference has no random-weight mode; its tests fill buffers with a counter generator on the host
// (tests/test_helpers.h:44-57).

#include <cuda_fp16.h>

#include "common.cuh"

namespace mi {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

template <typename T> __device__ __forceinline__ T store_as(float v);
template <> __device__ __forceinline__ float store_as<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 store_as<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half store_as<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
random_fill_kernel(T* __restrict__ out, int64_t n, uint32_t k0, uint32_t k1, float scale, float offset) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        uint32_t r[4];
        philox4x32_10((uint32_t)(i & 0xffffffffll), (uint32_t)(i >> 32), 0u, 0u, k0, k1, r);
        int s = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) s += (int)(r[j] & 0xffffu) + (int)(r[j] >> 16);
        // two roundings, never one fused multiply-add: the host does the same two steps
        const float v = __fadd_rn(__fmul_rn((float)(s - 262140), scale), offset);
        out[i] = store_as<T>(v);
    }
}

}  // namespace mi

// dtype codes: 0 float32, 1 bfloat16, 2 float16.
extern "C" int mi_random_fill(void* out, int dtype, long long n, unsigned int k0, unsigned int k1, float scale,
                              float offset, cudaStream_t stream) {
    using namespace mi;
    if (n < 0) { set_last_error("random_fill: negative element count"); return kBadShape; }
    if (n == 0) return kOk;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    if (dtype == 0) random_fill_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, n, k0, k1, scale, offset);
    else if (dtype == 1)
        random_fill_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, n, k0, k1, scale, offset);
    else if (dtype == 2) random_fill_kernel<__half><<<blocks, threads, 0, stream>>>((__half*)out, n, k0, k1, scale, offset);
    else { set_last_error("random_fill: unknown dtype code %d", dtype); return kBadDType; }
    return finish_launch("random_fill");
}
