// Bringing weights into L2 ahead of the kernel that streams them.
//
// A decode step is a chain of kernels, and some of them (the merge of the attention splits, the routing,
// the weighted sum of the experts' rows with the next norm) hardly touch HBM.  While such a kernel runs,
// a second stream asks L2 for the weights that the next weight-streaming kernel will read: the memory
// system is busy during the latency-bound kernel, and the streaming kernel starts on lines that are
// already on the chip.  The request is a hint (cp.async.bulk.prefetch.L2): nothing waits for it and a line
// that was evicted again is simply read from HBM.  The reference has no counterpart (it runs one library
// product after the other on one stream).

#include "common.cuh"

namespace mi {

constexpr uint32_t PF_CHUNK = 8192;     // bytes per prefetch request (a multiple of 16)

__global__ void __launch_bounds__(128)
l2_prefetch_kernel(const char* __restrict__ p, size_t bytes) {
    const size_t stride = (size_t)gridDim.x * blockDim.x * PF_CHUNK;
    for (size_t off = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * PF_CHUNK; off < bytes; off += stride) {
        const size_t left = bytes - off;
        const uint32_t n = (uint32_t)(left < PF_CHUNK ? (left & ~(size_t)15) : PF_CHUNK);
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"(n) : "memory");
    }
}

}  // namespace mi

// Ask L2 for `bytes` bytes from `p` (16-byte aligned).  Returns at once; the lines arrive on their own.
extern "C" int mi_l2_prefetch(const void* p, unsigned long long bytes, cudaStream_t stream) {
    using namespace mi;
    if (bytes == 0) return kOk;
    if (reinterpret_cast<uintptr_t>(p) & 15) {
        set_last_error("l2_prefetch: the address must be 16-byte aligned");
        return kBadShape;
    }
    const unsigned long long chunks = (bytes + PF_CHUNK - 1) / PF_CHUNK;
    const int blocks = (int)((chunks + 127) / 128 < 1184 ? (chunks + 127) / 128 : 1184);
    l2_prefetch_kernel<<<blocks, 128, 0, stream>>>((const char*)p, (size_t)bytes);
    return finish_launch("l2_prefetch");
}
