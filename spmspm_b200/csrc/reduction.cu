// Split-K reduction: C[e] = fp16_rn( sum_s float(W[s*M*N + e]) ), partials
// summed in fp32 in range order, the arithmetic of the reference's
// SplitK_Reduction (reference csrc/Reduction_Kernel.cuh:24-44).  HBM/L2-bound;
// each thread handles 8 consecutive outputs with 16-byte loads and stores.
#include "common.cuh"
#include <cuda_fp16.h>

namespace spb {
namespace {

__global__ void __launch_bounds__(256)
splitk_reduce_kernel(uint16_t* __restrict__ C, const uint16_t* __restrict__ W, size_t mn, int split_k)
{
    const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (e >= mn) return;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < split_k; ++s) {
        const uint4 v = *reinterpret_cast<const uint4*>(W + (size_t)s * mn + e);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
        }
    }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(C + e) = o;
}

}  // namespace

cudaError_t splitk_reduce(cudaStream_t s, uint16_t* C, const uint16_t* ws, int M, int N, int split_k)
{
    const size_t mn = (size_t)M * N;  // M % 64 == 0, so mn % 8 == 0
    const size_t threads = mn / 8;
    if (threads == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    splitk_reduce_kernel<<<blocks, 256, 0, s>>>(C, ws, mn, split_k);
    return cudaGetLastError();
}

}  // namespace spb
