// float -> FP8 conversion shared by the FP8 kernels.
#ifndef ITEXB_CSRC_FP8_CAST_H_
#define ITEXB_CSRC_FP8_CAST_H_

#include <cuda_fp8.h>

#include <cstdint>

namespace itexb {

// Round to nearest even; a finite value beyond the largest finite code saturates to it; NaN stays NaN.  An infinite
// input gives the target type's numeric_limits::infinity(), which is NaN for e4m3fn (the format has no infinity) and
// +-infinity for e5m2: the reference's conversion tests for infinity before its saturating overflow branch
// (itex/core/utils/float8.h:665-668 before :713-718; infinity() at :313-315 and :400).  The hardware conversion with
// saturation would clamp an infinity to the largest finite code instead, hence the explicit case.
__device__ __forceinline__ uint8_t FloatToFp8Bits(float f, bool e4m3) {
  uint8_t r = (uint8_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, e4m3 ? __NV_E4M3 : __NV_E5M2);
  const uint32_t bits = __float_as_uint(f);
  if ((bits & 0x7fffffffu) == 0x7f800000u) r = uint8_t((bits >> 24) & 0x80u) | (e4m3 ? 0x7Fu : 0x7Cu);
  return r;
}

}  // namespace itexb

#endif  // ITEXB_CSRC_FP8_CAST_H_
