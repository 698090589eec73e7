// Host-side scalar math of the quantized ops: ranges, scales, output min/max.
// fp32 throughout, with the operator order of the reference lines each function cites,
// because re-associating changes the last bit of a scale and hence integer outputs at
// rounding ties.  Compiled with -ffp-contract=off.
#ifndef ITEXB_CSRC_HOSTMATH_H_
#define ITEXB_CSRC_HOSTMATH_H_

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "itexb200.h"

namespace itexb {
namespace hostmath {

inline float MaxIntOf(int dt) { return (dt == ITEXB_DT_QUINT8 || dt == ITEXB_DT_UINT8) ? 255.0f : 127.0f; }
inline float MinIntOf(int dt) { return (dt == ITEXB_DT_QUINT8 || dt == ITEXB_DT_UINT8) ? 0.0f : -128.0f; }

// QuantizeV2Op::AdjustInputMinMaxRange, itex/core/kernels/common/quantize_op.h:130-152.
// Returns false when max < min (the op fails with InvalidArgument).
inline bool AdjustInputMinMaxRange(float in_min, float in_max, float ensure_minimum_range, float* adj_min, float* adj_max) {
  if (!(in_max >= in_min)) return false;
  *adj_min = std::min(0.0f, in_min);
  const float epsilon = std::max(1.0f, std::max(fabsf(in_min), fabsf(in_max))) * ensure_minimum_range;
  *adj_max = std::max(0.0f, std::max(in_max, *adj_min + epsilon));
  return true;
}

// GetScaleAndZeropointAndAlignMinMax<T>, SCALED branch, itex/core/utils/quantization_util.h:61-71.
// Aligns min/max to +-abs_range and returns the quantize (max_int/abs) or dequantize (abs/max_int) scale.
inline float ScaledScale(float* min_v, float* max_v, int dt, bool quantize) {
  const float max_int = MaxIntOf(dt);
  const float abs_range = std::max(std::abs(*min_v), std::abs(*max_v));
  *max_v = abs_range;
  *min_v = -abs_range;
  return quantize ? (max_int / abs_range) : (abs_range / max_int);
}

// MIN_FIRST branch of the same function, :72-83.
inline void MinFirstScaleZp(float min_v, float max_v, int dt, bool quantize, float* scale, int32_t* zp) {
  const float max_int = MaxIntOf(dt), min_int = MinIntOf(dt);
  if (quantize) {
    *scale = (max_int - min_int) / (max_v - min_v);
    *zp = static_cast<int32_t>(std::round(max_int - max_v * *scale));
  } else {
    *scale = (max_v - min_v) / (max_int - min_int);
    *zp = static_cast<int32_t>(std::round(max_int - max_v / *scale));
  }
}

// OneDnnFloatForOneQuantizedLevel<T>, itex/core/kernels/onednn/block/quantized_ops.h:24-36.
inline float FloatForOneQuantizedLevel(float range_min, float range_max, int dt) {
  int64_t highest, lowest;
  if (dt == ITEXB_DT_QUINT8) { highest = 255; lowest = 0; }
  else if (dt == ITEXB_DT_QINT8) { highest = 127; lowest = -128; }
  else { highest = 2147483647ll; lowest = -2147483648ll; }
  if (lowest < -highest) ++lowest;
  return (range_max - range_min) / (highest - lowest);
}

// OneDnnQuantizationRangeForMultiplication<T1,T2,qint32>, quantized_ops.h:38-54.
inline void QuantizationRangeForMultiplication(float min_a, float max_a, float min_b, float max_b, int t1, int t2, float* min_c,
                                               float* max_c) {
  const float a_level = FloatForOneQuantizedLevel(min_a, max_a, t1);
  const float b_level = FloatForOneQuantizedLevel(min_b, max_b, t2);
  const int64_t c_highest = 2147483647ll, c_lowest = -2147483648ll;
  const float c_level = a_level * b_level;
  *min_c = c_level * c_lowest;
  *max_c = c_level * c_highest;
}

// QuantizedMatMulOp::ExtendInt8PostOps, itex/core/kernels/common/quantized_matmul_common.h:1472-1508.
// toutput: QUINT8 | QINT8 | FLOAT | BFLOAT16 | HALF.  Only element 0 of min_b/max_b is used.
inline float MatMulOutputScale(float min_a, float max_a, float min_b0, float max_b0, int toutput, float min_freezed,
                               float max_freezed) {
  float min_out, max_out;
  QuantizationRangeForMultiplication(min_a, max_a, min_b0, max_b0, ITEXB_DT_QUINT8, ITEXB_DT_QINT8, &min_out, &max_out);
  const float scale_int32 = std::max(std::abs(min_out), std::abs(max_out));
  if (toutput == ITEXB_DT_FLOAT || toutput == ITEXB_DT_BFLOAT16 || toutput == ITEXB_DT_HALF)
    return scale_int32 / static_cast<float>(1u << 31);
  const float scale_eightbit = std::max(std::abs(min_freezed), std::abs(max_freezed));
  if (toutput == ITEXB_DT_QUINT8) return scale_int32 / scale_eightbit / static_cast<float>(1u << 23);
  return scale_int32 / scale_eightbit / static_cast<float>(1u << 24);
}

// QuantizedFusedMatMulOp::ExtendInt8PostOps / QuantizedFusedMatMulV2Op::ExtendInt8PostOps,
// itex/core/kernels/common/quantized_matmul_common.h:1610-1650, 1817-1842: the dequantize scale of every
// weight range, range_input * range_weight[i] / (max_int8_input * 127).
inline void FusedMatMulOutputScales(float min_a, float max_a, const float* min_b, const float* max_b, size_t count, bool min_first,
                                    int t1, std::vector<float>* scales) {
  const float max_int8_input = MaxIntOf(t1), max_int8_weight = 127.0f;
  const float range_input = min_first ? max_a - min_a : std::max(std::abs(min_a), std::abs(max_a));
  scales->resize(count);
  for (size_t i = 0; i < count; ++i) {
    const float range_weight = std::max(std::abs(min_b[i]), std::abs(max_b[i]));
    (*scales)[i] = (range_input * range_weight) / (max_int8_input * max_int8_weight);
  }
}

// LegacyQuantizedConvOpBase::ExtendInt8PostOps, itex/core/kernels/common/quantized_conv_ops.h:329-395.
inline void ConvOutputScales(float min_input, float max_input, const float* min_filter, const float* max_filter, size_t depth,
                             int tinput, int toutput, float min_freezed, float max_freezed, std::vector<float>* scales) {
  scales->assign(depth, 1.f);
  if (toutput == ITEXB_DT_QINT32) return;
  if (toutput == ITEXB_DT_FLOAT || toutput == ITEXB_DT_BFLOAT16 || toutput == ITEXB_DT_HALF) {
    const float int_input_limit = (tinput == ITEXB_DT_QUINT8) ? 255.0 : 127.0;
    const float int_filter_limit = 127.0;
    const float src_qscale_f32 = std::max(std::abs(min_input), std::abs(max_input)) / int_input_limit;
    for (size_t i = 0; i < depth; ++i) {
      const float wei_qscale_f32 = std::max(std::abs(min_filter[i]), std::abs(max_filter[i])) / int_filter_limit;
      (*scales)[i] = src_qscale_f32 * wei_qscale_f32;
    }
    return;
  }
  const float int_output_limit = toutput == ITEXB_DT_QUINT8 ? 255.0f : 127.0f;
  const float float_input_range = std::max(std::abs(min_input), std::abs(max_input));
  const float float_output_range = std::max(std::abs(min_freezed), std::abs(max_freezed));
  const float int_const_scale_limit = (tinput == ITEXB_DT_QUINT8) ? 255.0 * 127.0 : 127.0 * 127.0;
  for (size_t i = 0; i < depth; ++i) {
    const float float_filter_range = std::max(std::abs(min_filter[i]), std::abs(max_filter[i]));
    (*scales)[i] = int_output_limit * float_input_range * float_filter_range / (int_const_scale_limit * float_output_range);
  }
}

// Per-channel factor the float conv bias is multiplied by, GetBiasHandle, quantized_conv_ops.h:542-568.
inline void ConvFloatBiasFactors(float min_input, float max_input, const float* min_filter, const float* max_filter, size_t depth,
                                 int tinput, const std::vector<float>& scales, std::vector<float>* factors) {
  const float int_const_scale_limit = (tinput == ITEXB_DT_QUINT8) ? 255.0 * 127.0 : 127.0 * 127.0;
  factors->resize(depth);
  for (size_t i = 0; i < depth; ++i) {
    const float tmp_scale = int_const_scale_limit / (std::max(std::abs(max_input), std::abs(min_input)) *
                                                     std::max(std::abs(max_filter[i]), std::abs(min_filter[i])));
    (*factors)[i] = tmp_scale * scales[i];
  }
}

// Factor for a qint32 conv bias with a float-typed output, quantized_conv_ops.h:473-504.
inline void ConvInt32BiasDequantFactors(float min_input, float max_input, const float* min_filter, const float* max_filter,
                                        size_t depth, int tinput, std::vector<float>* factors) {
  const float int_const_scale_limit = (tinput == ITEXB_DT_QUINT8) ? 255.0 * 127.0 : 127.0 * 127.0;
  factors->resize(depth);
  for (size_t i = 0; i < depth; ++i)
    (*factors)[i] = (std::max(std::abs(max_input), std::abs(min_input)) * std::max(std::abs(max_filter[i]), std::abs(min_filter[i]))) /
                    int_const_scale_limit;
}

// Sum post-op scale of the Sum-fused conv variants, quantized_conv_ops.h:398-434.
inline float ConvSumScale(float min_out, float max_out, float min_sum, float max_sum, int toutput, int summand_dtype) {
  const float scale_output = std::max(std::abs(min_out), std::abs(max_out));
  const float scale_summand = std::max(std::abs(min_sum), std::abs(max_sum));
  if (toutput == ITEXB_DT_QUINT8 && summand_dtype == ITEXB_DT_QINT8) return 255.0f * scale_summand / (scale_output * 127.0f);
  return scale_summand / scale_output;
}

// GetWindowedOutputSizeVerboseV2, itex/core/utils/common_shape_fns.cc:42-81.
// padding: 0 VALID, 1 SAME, 2 EXPLICIT (pad_before/pad_after given).  Returns false on a bad window.
inline bool WindowedOutputSize(int64_t input, int64_t filter, int64_t dilation, int64_t stride, int padding, int64_t* out,
                               int64_t* pad_before, int64_t* pad_after) {
  if (stride <= 0 || dilation < 1) return false;
  const int64_t eff = (filter - 1) * dilation + 1;
  if (padding == 0) {
    *out = (input - eff + stride) / stride;
    *pad_before = *pad_after = 0;
  } else if (padding == 2) {
    *out = (input + *pad_before + *pad_after - eff + stride) / stride;
  } else {
    *out = (input + stride - 1) / stride;
    const int64_t needed = std::max(int64_t(0), (*out - 1) * stride + eff - input);
    *pad_before = needed / 2;
    *pad_after = needed - *pad_before;
  }
  return *out >= 0;
}

}  // namespace hostmath
}  // namespace itexb

#endif  // ITEXB_CSRC_HOSTMATH_H_
