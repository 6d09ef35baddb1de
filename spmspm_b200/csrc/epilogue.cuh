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

// fp16 add with one rounding of the exact sum.  float(a) + float(b) rounded to fp16, which is what an element-wise
// fp16 kernel computing in fp32 does, gives the same bits: fp32 carries 24 >= 2 * 11 + 2 significand bits, so the
// intermediate rounding is innocuous.
__device__ __forceinline__ __half2 ep_pair(__half2 y, bool has_bias, __half2 b, int act, bool has_res, __half2 r)
{
    if (has_bias) y = __hadd2(y, b);
    if (act == 1) y = __hmax2_nan(y, __half2half2(__ushort_as_half((unsigned short)0)));   // NaN stays NaN, -0 becomes +0
    if (has_res) y = __hadd2(r, y);
    return y;
}
__device__ __forceinline__ __half ep_one(__half y, bool has_bias, __half b, int act, bool has_res, __half r)
{
    return __low2half(ep_pair(__half2half2(y), has_bias, __half2half2(b), act, has_res, __half2half2(r)));
}

// 8 consecutive rows of one output column: sums already rounded to fp16 in o; bias8 / res8 point at the 8 bias values
// and the 8 residual values (16-byte aligned) or are null.
__device__ __forceinline__ uint4 ep_apply8(uint4 o, const uint16_t* bias8, const uint16_t* res8, int act)
{
    uint4 b = make_uint4(0, 0, 0, 0), r = make_uint4(0, 0, 0, 0);
    if (bias8) b = *reinterpret_cast<const uint4*>(bias8);
    if (res8) r = *reinterpret_cast<const uint4*>(res8);
    __half2* oh = reinterpret_cast<__half2*>(&o);
    const __half2* bh = reinterpret_cast<const __half2*>(&b);
    const __half2* rh = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = ep_pair(oh[j], bias8 != nullptr, bh[j], act, res8 != nullptr, rh[j]);
    return o;
}

}  // namespace spb
