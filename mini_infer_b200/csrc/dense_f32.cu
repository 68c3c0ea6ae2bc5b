// Dense product of the true 32-bit path: C[T, N] = A[T, K] . W[N, K]^T, float in, float out.
//
// Every output element is one chain of fused multiply-adds over k in ascending order, whatever the number
// of rows and wherever a row lies in its tile, so a token's result does not depend on how many other
// tokens share its step: the float32 path gives the same bits for every way of cutting and batching the
// work.  (A library product picks other kernels, and other orders of summation, for other row counts.)
// CUDA cores only, no reduced-precision mode: this path exists to show faults that bfloat16 hides, not to
// be fast.  The reference runs every dense product in FP16 through cuBLAS (src/layers/mlp.cpp:120-130).

#include "common.cuh"

namespace mi {

constexpr int DF_BM = 64, DF_BN = 64, DF_BK = 16;

template <bool VEC>
__global__ void __launch_bounds__(256)
dense_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int T, int N,
                 int K) {
    __shared__ float As[DF_BK][DF_BM + 4];
    __shared__ float Ws[DF_BK][DF_BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int row0 = blockIdx.y * DF_BM, n0 = blockIdx.x * DF_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += DF_BK) {
        if (VEC) {                                          // K % 4 == 0 and 16-byte aligned operands
            const int r = tid >> 2, c = (tid & 3) * 4;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), w = a;
            if (k0 + c < K) {
                if (row0 + r < T) a = __ldg(reinterpret_cast<const float4*>(A + (int64_t)(row0 + r) * K + k0 + c));
                if (n0 + r < N) w = __ldg(reinterpret_cast<const float4*>(W + (int64_t)(n0 + r) * K + k0 + c));
            }
            As[c][r] = a.x; As[c + 1][r] = a.y; As[c + 2][r] = a.z; As[c + 3][r] = a.w;
            Ws[c][r] = w.x; Ws[c + 1][r] = w.y; Ws[c + 2][r] = w.z; Ws[c + 3][r] = w.w;
        } else {
            for (int idx = tid; idx < DF_BM * DF_BK; idx += 256) {
                const int r = idx / DF_BK, c = idx % DF_BK;
                const bool kin = k0 + c < K;
                As[c][r] = (kin && row0 + r < T) ? A[(int64_t)(row0 + r) * K + k0 + c] : 0.f;
                Ws[c][r] = (kin && n0 + r < N) ? W[(int64_t)(n0 + r) * K + k0 + c] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < DF_BK; ++kk) {                // k beyond K holds zeros: fma(0, 0, acc) == acc
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(int64_t)r * N + n] = acc[i][j];
        }
    }
}

}  // namespace mi

extern "C" int mi_dense_f32(const float* A, const float* W, float* C, int T, int N, int K, cudaStream_t stream) {
    using namespace mi;
    if (T <= 0 || N <= 0) return kOk;
    if (K <= 0) { set_last_error("dense product (float32): inner size %d", K); return kBadShape; }
    const int64_t tiles_y = ((int64_t)T + DF_BM - 1) / DF_BM;
    if (tiles_y > 65535) { set_last_error("dense product (float32): %d rows exceed the grid limit", T); return kBadShape; }
    const dim3 grid((N + DF_BN - 1) / DF_BN, (unsigned)tiles_y);
    const bool vec = (K % 4 == 0) && (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) == 0);
    if (vec) dense_f32_kernel<true><<<grid, 256, 0, stream>>>(A, W, C, T, N, K);
    else dense_f32_kernel<false><<<grid, 256, 0, stream>>>(A, W, C, T, N, K);
    return finish_launch("dense_f32");
}
