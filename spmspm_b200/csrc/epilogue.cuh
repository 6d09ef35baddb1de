// Element-wise tail of a linear layer, applied where the SpMM result is rounded to fp16:
//   y = fp16(sum)                       the SpMM result, as the plain entry points round it
//   y = fp16(y + bias[row])             when bias is given   (FasterTransformer adds the bias after the GEMM,
//   y = y <= 0 ? 0 : y                  activation 1 (ReLU)   third_party/ft_spinfer.patch:700-720 FFN,
//   y = fp16(residual + y)              when residual is given  1476-1490 attention output)
// Every step rounds to fp16 like the separate element-wise kernels it replaces, so the fused result has the same
// bits as SpMM followed by those kernels.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace spb {

__device__ __forceinline__ __half ep_one(__half y, bool has_bias, __half b, int act, bool has_res, __half r)
{
    if (has_bias) y = __float2half_rn(__half2float(y) + __half2float(b));
    if (act == 1) y = __half2float(y) <= 0.f ? __ushort_as_half((unsigned short)0) : y;   // NaN stays NaN
    if (has_res) y = __float2half_rn(__half2float(r) + __half2float(y));
    return y;
}

// 8 consecutive rows of one output column: sums already rounded to fp16 in o; bias8 / res8 point at the 8 bias values
// and the 8 residual values (16-byte aligned) or are null.
__device__ __forceinline__ uint4 ep_apply8(uint4 o, const uint16_t* bias8, const uint16_t* res8, int act)
{
    uint4 b = make_uint4(0, 0, 0, 0), r = make_uint4(0, 0, 0, 0);
    if (bias8) b = *reinterpret_cast<const uint4*>(bias8);
    if (res8) r = *reinterpret_cast<const uint4*>(res8);
    __half* oh = reinterpret_cast<__half*>(&o);
    const __half* bh = reinterpret_cast<const __half*>(&b);
    const __half* rh = reinterpret_cast<const __half*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) oh[j] = ep_one(oh[j], bias8 != nullptr, bh[j], act, res8 != nullptr, rh[j]);
    return o;
}

}  // namespace spb
