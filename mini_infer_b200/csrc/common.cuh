// Shared device helpers for the sm_100a kernels of mini_infer_b200.
//
// Every kernel is a template over the storage type of its activations and of
// its weights (float or __nv_bfloat16); arithmetic is always float.  The
// reference has the same helpers for FP16 only (src/kernels/warp_reduce.cuh:10-62).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mi {

enum DType : int { kF32 = 0, kBF16 = 1 };

// Error codes returned by the extern "C" launchers (0 = launched).
enum Status : int {
    kOk = 0,
    kBadDType = -1,      // dtype code not 0/1 or a combination that is not built
    kBadShape = -2,      // a size the kernel refuses (message in mi_last_error)
    kLaunchFailed = -3,  // cudaGetLastError after the launch was not cudaSuccess
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// D += A * B on the tensor cores: A 16x16 (row-major fragments a0..a3), B 16x8 (b0, b1), bfloat16 in,
// float accumulate.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `scratch` holds at least 32 floats.  All threads get the sum.
// The order of additions depends only on blockDim, never on the data of other rows.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Programmatic dependent launch: a kernel launched through launch_dependent() may be placed on the SMs
// while the kernel before it in the stream is still running, so that its launch latency and the part of
// its prologue that reads nothing an earlier kernel wrote (index arithmetic, barrier set-up) overlap that
// kernel's tail.  Such a kernel calls wait_for_earlier_kernels() in every thread before its first read
// or write of memory that another kernel of the step touches, and before any return: the call returns
// once the kernel before it has completed and its writes are visible (and, since that kernel made the
// same call, so have all earlier ones).  Without the launch attribute the call returns at once.
__device__ __forceinline__ void wait_for_earlier_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel's blocks be placed from now on instead of from this block's exit (for kernels of
// at most one wave of blocks: a waiting block holds its SM's registers and shared memory).
__device__ __forceinline__ void allow_next_kernel() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Whether launch_dependent() sets the attribute (mi_set_dependent_launch; off by default).
bool dependent_launch_enabled();

template <typename... P, typename... A>
inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    A... args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = dependent_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&lc, kernel, static_cast<P>(args)...);
}

void set_last_error(const char* fmt, ...);

// Checks cudaGetLastError after a launcher queued `n_kernels` kernels and counts them.
int finish_launch(const char* what, int n_kernels = 1);

}  // namespace mi

// Dispatch helpers: run `BODY` with `AT`/`WT` bound to the C++ types of the codes.
#define MI_DISPATCH_1(code, T, ...)                                        \
    do {                                                                   \
        if ((code) == mi::kF32) { using T = float; __VA_ARGS__; }          \
        else if ((code) == mi::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else { mi::set_last_error("unknown dtype code %d", (int)(code)); return mi::kBadDType; } \
    } while (0)

#define MI_DISPATCH_2(acode, AT, wcode, WT, ...)                           \
    MI_DISPATCH_1(acode, AT, MI_DISPATCH_1(wcode, WT, __VA_ARGS__))
