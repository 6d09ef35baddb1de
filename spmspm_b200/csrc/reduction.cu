// Split-K reduction: C[e] = fp16_rn( sum_s float(W[s*M*N + e]) ), partials
// summed in fp32 in range order, the arithmetic of the reference's
// SplitK_Reduction (reference csrc/Reduction_Kernel.cuh:24-44).  HBM/L2-bound;
// each thread handles 8 consecutive outputs with 16-byte loads and stores.
#include "common.cuh"
#include "epilogue.cuh"
#include <cuda_fp16.h>

namespace spb {
namespace {

constexpr uint32_t kPollLimit = 1u << 21;  // about half a second with the sleep below

// kTail: with the element-wise tail of a linear layer and, when flags is given, a bounded wait for the sequence
// numbers of the n ranks whose stores filled W (flags[n] holds the number this rank's own SpMM gave the exchange).
template <bool kTail>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(uint16_t* __restrict__ C, const uint16_t* __restrict__ W, size_t mn, int split_k, int M,
                     Epilogue ep, uint32_t* flags, int n, int* status)
{
    if (kTail && flags) {
        if ((int)threadIdx.x < n) {
            const uint32_t want = *reinterpret_cast<volatile uint32_t*>(flags + n);
            bool ok = false;
            for (uint32_t i = 0; i < kPollLimit; ++i) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
                if ((int32_t)(v - want) >= 0) {
                    ok = true;
                    break;
                }
                __nanosleep(200);
            }
            if (!ok) atomicOr(status, (int)kStatusWaitTimeout);
            if (blockIdx.x == 0 && threadIdx.x == 0) flags[n + 1] = want;  // exchanges this rank has consumed
        }
        __syncthreads();
    }
    const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (e >= mn) return;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < split_k; ++s) {
        // partials written by other GPUs are read past the caches of this one
        const uint4 v = kTail ? __ldcg(reinterpret_cast<const uint4*>(W + (size_t)s * mn + e))
                              : *reinterpret_cast<const uint4*>(W + (size_t)s * mn + e);
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
    if (kTail) o = ep_apply8(o, ep.bias ? ep.bias + e % (size_t)M : nullptr, ep.residual ? ep.residual + e : nullptr, ep.activation);
    *reinterpret_cast<uint4*>(C + e) = o;
}

}  // namespace

cudaError_t splitk_reduce(cudaStream_t s, uint16_t* C, const uint16_t* ws, int M, int N, int split_k, const Epilogue& ep,
                          uint32_t* wait_flags, int wait_n, int* status)
{
    const size_t mn = (size_t)M * N;  // M % 64 == 0, so mn % 8 == 0
    const size_t threads = mn / 8;
    if (threads == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    count_launch();
    if (ep.any() || wait_flags)
        splitk_reduce_kernel<true><<<blocks, 256, 0, s>>>(C, ws, mn, split_k, M, ep, wait_flags, wait_n, status);
    else
        splitk_reduce_kernel<false><<<blocks, 256, 0, s>>>(C, ws, mn, split_k, M, ep, nullptr, 0, nullptr);
    return cudaGetLastError();
}

}  // namespace spb
