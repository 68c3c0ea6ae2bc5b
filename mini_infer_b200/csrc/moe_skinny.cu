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

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// MODE 0: C[r, n] = a_r . W[e, n, :]                       (C float)
// MODE 1: C[r, n] = silu(a_r . W[e, n, :]) * (a_r . W[e, Nout + n, :])   (C bfloat16)
// Block = 4 warps x 16 features; grid = (ceil(Nout / 64), E).
template <int MODE, int NT>
__device__ __forceinline__ void skinny_pass(const __nv_bfloat16* __restrict__ A, const int* __restrict__ gather,
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
        const int src = xv[j] ? (gather ? gather[row0 + r] : row0 + r) : 0;
        xr[j] = reinterpret_cast<const uint4*>(A + (int64_t)src * Kd) + t;
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
                const int64_t o = (int64_t)(row0 + r) * Nout + f;
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
        skinny_pass<MODE, 1>(A, gather, We, C, b0, cnt, f0, Nout, Kd);
    } else {
        for (int r0 = 0; r0 < cnt; r0 += 16)
            skinny_pass<MODE, 2>(A, gather, We, C, b0 + r0, min(16, cnt - r0), f0, Nout, Kd);
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

}  // extern "C"
