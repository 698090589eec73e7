// _ITEXQuantizeV2 / QuantizeV2 and _ITEXDequantize / Dequantize.
// Attr names, input/output order, HostMemory arguments and error texts follow
// QuantizeV2Op (itex/core/kernels/common/quantize_op.h:67-434) and DequantizeOp
// (itex/core/kernels/common/dequantize_op.h:43-190); registrations follow
// itex/core/kernels/gpu/quantize_op.cc:24-51 and gpu/dequantize_op.cc:24-47 (stock and
// _ITEX names, min_range/max_range and output_min/output_max in host memory).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hostmath.h"
#include "op_kernel.h"

namespace itexb {
namespace {

enum class QuantizeMode { MIN_COMBINED, MIN_FIRST, SCALED };

int ParseMode(const AttrMap& attrs, const char* default_mode, QuantizeMode* mode, std::string* mode_string) {
  *mode_string = default_mode;
  if (attrs.Has("mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("mode", mode_string));
  if (*mode_string == "MIN_COMBINED") *mode = QuantizeMode::MIN_COMBINED;
  else if (*mode_string == "MIN_FIRST") *mode = QuantizeMode::MIN_FIRST;
  else if (*mode_string == "SCALED") *mode = QuantizeMode::SCALED;
  else
    return SetError(ITEXB_INVALID_ARGUMENT, "Mode string must be 'MIN_COMBINED', 'MIN_FIRST', or 'SCALED', is '%s'",
                    mode_string->c_str());
  return ITEXB_OK;
}

// Value of -min rounded to the input element type (the reference casts the shift vector
// to the type of the data tensor, quantize_op.h:238-247).
float RoundToInputType(float v, int dtype) {
  if (dtype == ITEXB_DT_BFLOAT16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dtype == ITEXB_DT_HALF) return __half2float(__float2half_rn(v));
  return v;
}

class QuantizeV2Op : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    ITEXB_RETURN_IF_ERROR(attrs.GetType("T", &t_));
    ITEXB_REQUIRE(t_ == ITEXB_DT_QINT8 || t_ == ITEXB_DT_QUINT8, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for T=%s (qint8 and quint8 are)", name().c_str(), DtypeName(t_));
    std::string mode_string;
    ITEXB_RETURN_IF_ERROR(ParseMode(attrs, "SCALED", &mode_, &mode_string));
    classic_ = false;
    if (attrs.Has("classic_asymmetric_algorithm")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("classic_asymmetric_algorithm", &classic_));
    ITEXB_REQUIRE(mode_ == QuantizeMode::SCALED || mode_ == QuantizeMode::MIN_FIRST, ITEXB_INVALID_ARGUMENT,
                  "_ITEXQuantizeV2 only supports SCALED and MIN_FIRST MODE");
    std::string round_mode = "HALF_AWAY_FROM_ZERO";
    if (attrs.Has("round_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("round_mode", &round_mode));
    ITEXB_REQUIRE(round_mode == "HALF_AWAY_FROM_ZERO" || round_mode == "HALF_TO_EVEN", ITEXB_INVALID_ARGUMENT,
                  "Round mode string must be 'HALF_AWAY_FROM_ZERO' or 'HALF_TO_EVEN', is '%s'", round_mode.c_str());
    if (round_mode == "HALF_TO_EVEN")
      ITEXB_REQUIRE(mode_ == QuantizeMode::SCALED, ITEXB_INVALID_ARGUMENT,
                    "Round mode 'HALF_TO_EVEN' only supported for mode 'SCALED', but mode is '%s'.", mode_string.c_str());
    // round_mode is validated and then unused: the kernel always rounds to nearest even,
    // like the oneDNN reorder behind the reference op.  narrow_range is read and ignored.
    bool narrow_range = false;
    if (attrs.Has("narrow_range")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("narrow_range", &narrow_range));
    int64_t axis = -1;
    if (attrs.Has("axis")) ITEXB_RETURN_IF_ERROR(attrs.GetInt("axis", &axis));
    axis_ = int(axis);
    ensure_minimum_range_ = 0.01f;
    if (attrs.Has("ensure_minimum_range")) ITEXB_RETURN_IF_ERROR(attrs.GetFloat("ensure_minimum_range", &ensure_minimum_range_));
    dtype_ = ITEXB_DT_FLOAT;
    if (attrs.Has("dtype")) ITEXB_RETURN_IF_ERROR(attrs.GetType("dtype", &dtype_));
    return ITEXB_OK;
  }

  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 3, op));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "input"));
    const itexb_tensor_t& src = ctx->inputs[0];
    ITEXB_REQUIRE(src.dtype == ITEXB_DT_FLOAT || src.dtype == ITEXB_DT_BFLOAT16 || src.dtype == ITEXB_DT_HALF,
                  ITEXB_INVALID_ARGUMENT, "%s: input must be float, bfloat16 or half, is %s", op, DtypeName(src.dtype));
    const float *in_min, *in_max;
    int64_t n_min, n_max;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 1, op, "min_range", &in_min, &n_min));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 2, op, "max_range", &in_max, &n_max));
    int64_t num_slices = 1;
    if (axis_ > -1) num_slices = n_min;
    ITEXB_REQUIRE(n_max >= num_slices, ITEXB_INVALID_ARGUMENT, "%s: max_range has fewer elements than min_range", op);
    int64_t inner = 1;
    if (num_slices > 1) {
      ITEXB_REQUIRE(axis_ < src.rank && src.dims[axis_] == num_slices, ITEXB_INVALID_ARGUMENT,
                    "%s: min_range has %lld elements but dimension %d of the input has size %lld", op, (long long)num_slices, axis_,
                    (long long)(axis_ < src.rank ? src.dims[axis_] : -1));
      for (int d = axis_ + 1; d < src.rank; ++d) inner *= src.dims[d];
    }
    std::vector<float> min_range(num_slices), max_range(num_slices), scale(num_slices), shift(num_slices, 0.f);
    for (int64_t i = 0; i < num_slices; ++i)
      ITEXB_REQUIRE(hostmath::AdjustInputMinMaxRange(in_min[i], in_max[i], ensure_minimum_range_, &min_range[i], &max_range[i]),
                    ITEXB_INVALID_ARGUMENT, "input_max_range must be larger than input_min_range.");
    int kind = ITEXB_QUANT_SCALED;
    if (mode_ == QuantizeMode::SCALED) {
      for (int64_t i = 0; i < num_slices; ++i) scale[i] = hostmath::ScaledScale(&min_range[i], &max_range[i], t_, true);
    } else if (classic_) {
      kind = ITEXB_QUANT_MIN_FIRST_CLASSIC;
      for (int64_t i = 0; i < num_slices; ++i) {
        int32_t zp;
        hostmath::MinFirstScaleZp(min_range[i], max_range[i], t_, true, &scale[i], &zp);
        shift[i] = float(zp);
      }
    } else {
      kind = ITEXB_QUANT_MIN_FIRST_LEGACY;
      const int64_t number_of_steps = int64_t(1) << 8;
      for (int64_t i = 0; i < num_slices; ++i) {
        scale[i] = (number_of_steps - 1.0) / (max_range[i] - min_range[i]);
        shift[i] = RoundToInputType(-min_range[i], src.dtype);
      }
    }
    itexb_tensor_t dst, omin, omax;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, t_, src.dims, src.rank, false, &dst));
    const int mm_rank = num_slices == 1 ? 0 : ctx->inputs[1].rank;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, ctx->inputs[1].dims, mm_rank, true, &omin));
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, ctx->inputs[1].dims, mm_rank, true, &omax));
    const int64_t n = NumElements(src);
    cudaStream_t st = AsCuda(ctx->stream);
    if (n > 0) {
      const float *dscale = nullptr, *dshift = nullptr;
      if (num_slices > 1) {
        ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ctx->device_ordinal, st, scale.data(), scale.size(), &dscale));
        if (kind != ITEXB_QUANT_SCALED)
          ITEXB_RETURN_IF_ERROR(shift_cache_.Get(ctx->device_ordinal, st, shift.data(), shift.size(), &dshift));
      }
      ITEXB_RETURN_IF_ERROR(itexb_quantize(src.data, src.dtype, dst.data, t_, n, inner, num_slices, kind, dscale, dshift, scale[0],
                                           shift[0], ctx->stream));
    }
    float* pmin = static_cast<float*>(omin.data);
    float* pmax = static_cast<float*>(omax.data);
    for (int64_t i = 0; i < num_slices; ++i) {
      pmin[i] = (t_ == ITEXB_DT_QUINT8 && mode_ == QuantizeMode::SCALED) ? 0.f : min_range[i];
      pmax[i] = max_range[i];
    }
    return ITEXB_OK;
  }

 private:
  int t_ = ITEXB_DT_QINT8;
  QuantizeMode mode_ = QuantizeMode::SCALED;
  bool classic_ = false;
  int axis_ = -1;
  float ensure_minimum_range_ = 0.01f;
  int dtype_ = ITEXB_DT_FLOAT;
  DeviceVectorCache scale_cache_, shift_cache_;
};

class DequantizeOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    std::string mode_string;
    ITEXB_RETURN_IF_ERROR(ParseMode(attrs, "MIN_COMBINED", &mode_, &mode_string));
    ITEXB_REQUIRE(mode_ != QuantizeMode::MIN_COMBINED, ITEXB_UNIMPLEMENTED,
                  "%s: mode MIN_COMBINED is not supported (SCALED and MIN_FIRST are)", name().c_str());
    bool narrow_range = false;
    if (attrs.Has("narrow_range")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("narrow_range", &narrow_range));
    int64_t axis = -1;
    if (attrs.Has("axis")) ITEXB_RETURN_IF_ERROR(attrs.GetInt("axis", &axis));
    axis_ = int(axis);
    dtype_ = ITEXB_DT_FLOAT;
    if (attrs.Has("dtype")) ITEXB_RETURN_IF_ERROR(attrs.GetType("dtype", &dtype_));
    ITEXB_REQUIRE(dtype_ == ITEXB_DT_FLOAT || dtype_ == ITEXB_DT_BFLOAT16 || dtype_ == ITEXB_DT_HALF, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for dtype=%s", name().c_str(), DtypeName(dtype_));
    if (attrs.Has("T")) {
      int t;
      ITEXB_RETURN_IF_ERROR(attrs.GetType("T", &t));
      ITEXB_REQUIRE(t == ITEXB_DT_QINT8 || t == ITEXB_DT_QUINT8, ITEXB_INVALID_ARGUMENT,
                    "%s: no kernel registered for T=%s (qint8 and quint8 are)", name().c_str(), DtypeName(t));
    }
    return ITEXB_OK;
  }

  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 3, op));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "input"));
    const itexb_tensor_t& src = ctx->inputs[0];
    ITEXB_REQUIRE(src.dtype == ITEXB_DT_QINT8 || src.dtype == ITEXB_DT_QUINT8, ITEXB_INVALID_ARGUMENT,
                  "%s: input must be qint8 or quint8, is %s", op, DtypeName(src.dtype));
    const float *in_min, *in_max;
    int64_t n_min, n_max;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 1, op, "min_range", &in_min, &n_min));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 2, op, "max_range", &in_max, &n_max));
    int64_t num_slices = 1;
    if (axis_ > -1) num_slices = n_min;
    ITEXB_REQUIRE(n_max >= num_slices, ITEXB_INVALID_ARGUMENT, "%s: max_range has fewer elements than min_range", op);
    int64_t inner = 1;
    if (num_slices > 1) {
      ITEXB_REQUIRE(axis_ < src.rank && src.dims[axis_] == num_slices, ITEXB_INVALID_ARGUMENT,
                    "%s: min_range has %lld elements but dimension %d of the input has size %lld", op, (long long)num_slices, axis_,
                    (long long)(axis_ < src.rank ? src.dims[axis_] : -1));
      for (int d = axis_ + 1; d < src.rank; ++d) inner *= src.dims[d];
    }
    std::vector<float> scale(num_slices), zp(num_slices, 0.f);
    for (int64_t i = 0; i < num_slices; ++i) {
      float mn = in_min[i], mx = in_max[i];
      if (mode_ == QuantizeMode::SCALED) {
        scale[i] = hostmath::ScaledScale(&mn, &mx, src.dtype, false);
      } else {
        int32_t z;
        hostmath::MinFirstScaleZp(mn, mx, src.dtype, false, &scale[i], &z);
        zp[i] = float(z);
      }
    }
    itexb_tensor_t dst;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, dtype_, src.dims, src.rank, false, &dst));
    const int64_t n = NumElements(src);
    if (n == 0) return ITEXB_OK;
    cudaStream_t st = AsCuda(ctx->stream);
    const float *dscale = nullptr, *dzp = nullptr;
    if (num_slices > 1) {
      ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ctx->device_ordinal, st, scale.data(), scale.size(), &dscale));
      if (mode_ == QuantizeMode::MIN_FIRST) ITEXB_RETURN_IF_ERROR(zp_cache_.Get(ctx->device_ordinal, st, zp.data(), zp.size(), &dzp));
    }
    return itexb_dequantize(src.data, src.dtype, dst.data, dtype_, n, inner, num_slices, dscale, dzp, scale[0], zp[0], ctx->stream);
  }

 private:
  QuantizeMode mode_ = QuantizeMode::SCALED;
  int axis_ = -1;
  int dtype_ = ITEXB_DT_FLOAT;
  DeviceVectorCache scale_cache_, zp_cache_;
};

// inputs: input, min_range*, max_range*; outputs: output, output_min*, output_max*   (* = HostMemory)
ITEXB_REGISTER_OP("_ITEXQuantizeV2", QuantizeV2Op, 3, 3, 0x6u, 0x6u);
ITEXB_REGISTER_OP("QuantizeV2", QuantizeV2Op, 3, 3, 0x6u, 0x6u);
ITEXB_REGISTER_OP("_ITEXDequantize", DequantizeOp, 3, 1, 0x6u, 0x0u);
ITEXB_REGISTER_OP("Dequantize", DequantizeOp, 3, 1, 0x6u, 0x0u);

}  // namespace
}  // namespace itexb
