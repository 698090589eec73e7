// The old-API quantized Conv2D ops, NHWC: [_ITEX]QuantizedConv2D, ...PerChannel, ...WithBias, ...WithBiasAndRelu
// (qint32 outputs), ...AndRequantize, ...AndReluAndRequantize, ...WithBias[AndRelu]AndRequantize and the Sum-fused
// variants (8-bit outputs); and two fusions around them the remapper makes: _ITEXQuantizedConv2DWithDequantize /
// ...WithCast (a ...WithBiasAndRequantize whose Dequantize or Cast consumer is folded in: real-valued output,
// itex/core/graph/remapper/remapper.cc:2178-2240, scale rule kernels/onednn/block/conv_ops_impl.h:1928-1963) and
// _ITEXQuantizeV2WithQuantizedConv2D (a QuantizeV2 folded into the ...WithBiasAndReluAndRequantize it feeds: fp32
// input, remapper.cc:2099-2123, kernels/onednn/block/conv_ops_impl.h:1238-1420).
//
// Attrs, input order (input, filter, [bias,] min_input, max_input, min_filter, max_filter
// [, min_freezed_output, max_freezed_output][, summand, min_summand, max_summand]), the
// HostMemory lists and the checks follow LegacyQuantizedConvOpBase
// (itex/core/kernels/common/quantized_conv_ops.h:71-729) over ConvOpBase
// (itex/core/kernels/common/conv_ops.h:612-1133), registrations
// itex/core/kernels/gpu/quantized_conv_ops.cc:72-160.  Where the reference builds a
// dnnl::convolution_forward with per-channel scales on the weights argument, this op
// packs the filter once to [co][kh*kw*c], prepares the scaled bias on the device and
// launches the implicit-GEMM convolution with the fused epilogue.
#include "hostmath.h"
#include "op_kernel.h"

namespace itexb {
namespace {

enum class ConvFusion { kNone, kDequantizeTail, kQuantizeHead };

class QuantizedConv2DOp : public OpKernel {
 public:
  QuantizedConv2DOp(bool relu, bool sum, bool signed_sum, bool has_bias = true, bool requantize = true, bool new_api = false,
                    ConvFusion fusion = ConvFusion::kNone)
      : relu_(relu), sum_(sum), signed_sum_(signed_sum), has_bias_(has_bias), requantize_(requantize), new_api_(new_api),
        fusion_(fusion) {
    if (fusion == ConvFusion::kDequantizeTail) { requantize_ = false; dequantize_ = true; }
  }

  // New API (_QuantizedConv2D / _ITEXQuantizedConv2DV2): the fusion comes from the fused_ops attr
  // (LegacyQuantizedConvOpBase constructor, itex/core/kernels/common/quantized_conv_ops.h:76-312).
  int InitFusedOps(const AttrMap& attrs) {
    const char* op = name().c_str();
    std::vector<std::string> fused;
    if (attrs.Has("fused_ops")) ITEXB_RETURN_IF_ERROR(attrs.GetStringList("fused_ops", &fused));
    float alpha = 0.f;
    if (attrs.Has("alpha")) ITEXB_RETURN_IF_ERROR(attrs.GetFloat("alpha", &alpha));
    has_bias_ = relu_ = sum_ = requantize_ = dequantize_ = false;
    int pos = 0, act_at = -1, sum_at = -1;
    for (const std::string& f : fused) {
      if (f == "BiasAdd") has_bias_ = true;
      else if (f == "Requantize") requantize_ = true;
      else if (f == "Dequantize") dequantize_ = true;
      else if (f == "Sum") { sum_ = true; sum_at = pos++; }
      else if (f == "Relu") { relu_ = true; act_at = pos++; }
      else if (f == "LeakyRelu") { act_ = ITEXB_ACT_RELU; act_alpha_ = alpha; act_at = pos++; }
      else if (f == "Elu") { act_ = ITEXB_ACT_ELU; act_alpha_ = 1.f; act_at = pos++; }
      else if (f == "Sigmoid") { act_ = ITEXB_ACT_SIGMOID; act_at = pos++; }
      else if (f == "_FusedSwish") { act_ = ITEXB_ACT_SWISH; act_alpha_ = 1.f; act_at = pos++; }
      else return SetError(ITEXB_INVALID_ARGUMENT, "%s: unsupported fusion %s", op, f.c_str());
    }
    ITEXB_REQUIRE(!(requantize_ && dequantize_), ITEXB_INVALID_ARGUMENT, "%s: Requantize and Dequantize cannot both be fused", op);
    ITEXB_REQUIRE(!(sum_ && act_at >= 0 && act_at < sum_at), ITEXB_UNIMPLEMENTED,
                  "%s: an activation before Sum is not implemented (Sum, then activation is)", op);
    ITEXB_REQUIRE(!sum_ || requantize_, ITEXB_UNIMPLEMENTED, "%s: Sum is implemented with Requantize (8-bit summand) only", op);
    return ITEXB_OK;
  }

  int Init(const AttrMap& attrs) override {
    const char* op = name().c_str();
    std::vector<int64_t> strides, dilations = {1, 1, 1, 1};
    ITEXB_RETURN_IF_ERROR(attrs.GetIntList("strides", &strides));
    if (attrs.Has("dilations")) ITEXB_RETURN_IF_ERROR(attrs.GetIntList("dilations", &dilations));
    std::string data_format = "NHWC";
    if (attrs.Has("data_format")) ITEXB_RETURN_IF_ERROR(attrs.GetString("data_format", &data_format));
    ITEXB_REQUIRE(data_format == "NHWC" || data_format == "NCHW", ITEXB_INVALID_ARGUMENT, "Invalid data format");
    ITEXB_REQUIRE(data_format == "NHWC", ITEXB_UNIMPLEMENTED, "%s: only data_format NHWC is implemented", op);
    ITEXB_REQUIRE(strides.size() == 4, ITEXB_INVALID_ARGUMENT, "Sliding window strides field must specify 4 dimensions");
    ITEXB_REQUIRE(dilations.size() == 4, ITEXB_INVALID_ARGUMENT, "Sliding window dilations field must specify 4 dimensions");
    ITEXB_REQUIRE(strides[0] == 1 && strides[3] == 1, ITEXB_UNIMPLEMENTED,
                  "Current implementation does not yet support strides in the batch and depth dimensions.");
    ITEXB_REQUIRE(dilations[0] == 1 && dilations[3] == 1, ITEXB_INVALID_ARGUMENT,
                  "Current implementation does not yet support dilations in the batch and depth dimensions.");
    ITEXB_REQUIRE(strides[1] > 0 && strides[2] > 0, ITEXB_INVALID_ARGUMENT, "Row and column strides should be larger than 0.");
    ITEXB_REQUIRE(dilations[1] > 0 && dilations[2] > 0, ITEXB_INVALID_ARGUMENT, "Dilated rates should be larger than 0.");
    stride_h_ = int(strides[1]); stride_w_ = int(strides[2]);
    dil_h_ = int(dilations[1]); dil_w_ = int(dilations[2]);
    std::string padding;
    ITEXB_RETURN_IF_ERROR(attrs.GetString("padding", &padding));
    if (padding == "VALID") padding_ = 0;
    else if (padding == "SAME") padding_ = 1;
    else if (padding == "EXPLICIT") padding_ = 2;
    else return SetError(ITEXB_INVALID_ARGUMENT, "%s: unknown padding '%s'", op, padding.c_str());
    if (attrs.Has("explicit_paddings")) ITEXB_RETURN_IF_ERROR(attrs.GetIntList("explicit_paddings", &explicit_paddings_));
    // legacy int8 graphs carry the pads in padding_list (quantized_conv_ops.h:122-126)
    if (attrs.Has("padding_list")) {
      std::vector<int64_t> pl;
      ITEXB_RETURN_IF_ERROR(attrs.GetIntList("padding_list", &pl));
      if (!pl.empty()) explicit_paddings_ = pl;
    }
    if (padding_ == 2)
      ITEXB_REQUIRE(explicit_paddings_.size() == 8, ITEXB_INVALID_ARGUMENT, "%s: EXPLICIT padding needs 8 explicit_paddings values", op);
    is_filter_const_ = true;
    is_bias_const_ = true;
    if (attrs.Has("is_filter_const")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("is_filter_const", &is_filter_const_));
    if (attrs.Has("is_bias_const")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("is_bias_const", &is_bias_const_));
    tinput_ = ITEXB_DT_QUINT8;
    if (fusion_ == ConvFusion::kQuantizeHead) {
      // Tinput is the type of the real-valued data; what the convolution reads is quint8 (the only registration,
      // itex/core/kernels/onednn/block/conv_ops_impl_gpu.cc:716-773)
      treal_ = ITEXB_DT_FLOAT;
      if (attrs.Has("Tinput")) ITEXB_RETURN_IF_ERROR(attrs.GetType("Tinput", &treal_));
      ITEXB_REQUIRE(treal_ == ITEXB_DT_FLOAT || treal_ == ITEXB_DT_BFLOAT16, ITEXB_INVALID_ARGUMENT,
                    "%s: no kernel registered for Tinput=%s (float and bfloat16 are)", op, DtypeName(treal_));
      std::string mode = "SCALED";
      if (attrs.Has("mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("mode", &mode));
      ITEXB_REQUIRE(mode == "MIN_COMBINED" || mode == "MIN_FIRST" || mode == "SCALED", ITEXB_INVALID_ARGUMENT,
                    "Mode string must be 'MIN_COMBINED', 'MIN_FIRST', or 'SCALED', is '%s'", mode.c_str());
      ITEXB_REQUIRE(mode == "SCALED", ITEXB_UNIMPLEMENTED, "%s: only mode SCALED is implemented", op);
      std::string round_mode = "HALF_AWAY_FROM_ZERO";
      if (attrs.Has("round_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("round_mode", &round_mode));
      ITEXB_REQUIRE(round_mode == "HALF_AWAY_FROM_ZERO" || round_mode == "HALF_TO_EVEN", ITEXB_INVALID_ARGUMENT,
                    "Round mode string must be 'HALF_AWAY_FROM_ZERO' or 'HALF_TO_EVEN', is '%s'", round_mode.c_str());
      ensure_minimum_range_ = 0.01f;
      if (attrs.Has("ensure_minimum_range")) ITEXB_RETURN_IF_ERROR(attrs.GetFloat("ensure_minimum_range", &ensure_minimum_range_));
    } else {
      if (attrs.Has("Tinput")) ITEXB_RETURN_IF_ERROR(attrs.GetType("Tinput", &tinput_));
      ITEXB_REQUIRE(tinput_ == ITEXB_DT_QUINT8 || tinput_ == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT,
                    "%s: no kernel registered for Tinput=%s", op, DtypeName(tinput_));
    }
    int tfilter = ITEXB_DT_QINT8;
    if (attrs.Has("Tfilter")) ITEXB_RETURN_IF_ERROR(attrs.GetType("Tfilter", &tfilter));
    ITEXB_REQUIRE(tfilter == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT, "%s: no kernel registered for Tfilter=%s", op, DtypeName(tfilter));
    tbias_ = ITEXB_DT_FLOAT;
    if (attrs.Has("Tbias")) ITEXB_RETURN_IF_ERROR(attrs.GetType("Tbias", &tbias_));
    ITEXB_REQUIRE(tbias_ == ITEXB_DT_FLOAT || tbias_ == ITEXB_DT_QINT32, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for Tbias=%s", op, DtypeName(tbias_));
    if (new_api_) ITEXB_RETURN_IF_ERROR(InitFusedOps(attrs));
    out_type_ = requantize_ ? ITEXB_DT_QUINT8 : (dequantize_ ? ITEXB_DT_FLOAT : ITEXB_DT_QINT32);
    if (attrs.Has("out_type")) ITEXB_RETURN_IF_ERROR(attrs.GetType("out_type", &out_type_));
    if (new_api_) {
      if (requantize_)
        ITEXB_REQUIRE(out_type_ == ITEXB_DT_QINT8 || out_type_ == ITEXB_DT_QUINT8, ITEXB_INVALID_ARGUMENT,
                      "QuantizedConv: unsupported output type when Requantize is fused.");
      else if (dequantize_)
        ITEXB_REQUIRE(out_type_ == ITEXB_DT_FLOAT || out_type_ == ITEXB_DT_BFLOAT16, ITEXB_INVALID_ARGUMENT,
                      "QuantizedConv: unsupported output type when Dequantize is fused.");
      else
        ITEXB_REQUIRE(out_type_ == ITEXB_DT_QINT32, ITEXB_INVALID_ARGUMENT, "%s: out_type must be qint32 without Requantize / Dequantize", op);
    } else if (fusion_ == ConvFusion::kDequantizeTail)
      ITEXB_REQUIRE(out_type_ == ITEXB_DT_FLOAT || out_type_ == ITEXB_DT_BFLOAT16 || out_type_ == ITEXB_DT_HALF, ITEXB_INVALID_ARGUMENT,
                    "%s: no kernel registered for out_type=%s (float, bfloat16 and half are)", op, DtypeName(out_type_));
    else if (!requantize_)
      ITEXB_REQUIRE(out_type_ == ITEXB_DT_QINT32, ITEXB_INVALID_ARGUMENT, "%s: no kernel registered for out_type=%s (qint32 is)", op,
                    DtypeName(out_type_));
    else if (relu_)
      ITEXB_REQUIRE(out_type_ == ITEXB_DT_QUINT8, ITEXB_INVALID_ARGUMENT,
                    "%s: no kernel registered for out_type=%s (quint8 is)", op, DtypeName(out_type_));
    else
      ITEXB_REQUIRE(out_type_ == ITEXB_DT_QINT8 || out_type_ == ITEXB_DT_QUINT8, ITEXB_INVALID_ARGUMENT,
                    "%s: no kernel registered for out_type=%s (qint8 and quint8 are)", op, DtypeName(out_type_));
    return ITEXB_OK;
  }

  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    // Old API: input, filter, [bias], 4 ranges, [2 frozen output ranges], [summand, 2 summand ranges].
    // New API: input, filter, [bias], [summand], 4 ranges, [2 summand ranges], [2 frozen output ranges].
    const int i_rng = 2 + (has_bias_ ? 1 : 0) + (new_api_ && sum_ ? 1 : 0);  // first of min_input, max_input, min_filter, max_filter
    const int i_sum = new_api_ ? 2 + (has_bias_ ? 1 : 0) : i_rng + 4 + (requantize_ ? 2 : 0);   // summand
    const int i_sum_rng = new_api_ ? i_rng + 4 : i_sum + 1;                    // min_summand, max_summand
    const int i_frz = new_api_ ? i_rng + 4 + (sum_ ? 2 : 0) : i_rng + 4;       // min/max_freezed_output
    // (the Dequantize / Cast fusions keep the frozen output range of the op they replaced as two unused inputs)
    const bool frozen_inputs = requantize_ || fusion_ == ConvFusion::kDequantizeTail;
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, i_rng + 4 + (frozen_inputs ? 2 : 0) + (sum_ ? (new_api_ ? 2 : 3) : 0), op));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "input"));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 1, op, "filter"));
    if (has_bias_) ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 2, op, "bias"));
    const itexb_tensor_t& x = ctx->inputs[0];
    const itexb_tensor_t& f = ctx->inputs[1];
    static const itexb_tensor_t kNoTensor{};
    const itexb_tensor_t& bias = has_bias_ ? ctx->inputs[2] : kNoTensor;
    ITEXB_REQUIRE(x.rank == 4, ITEXB_INVALID_ARGUMENT, "input must be 4-dimensional");
    ITEXB_REQUIRE(f.rank == 4, ITEXB_INVALID_ARGUMENT, "filter must be 4-dimensional");
    const int want_x = fusion_ == ConvFusion::kQuantizeHead ? treal_ : tinput_;
    ITEXB_REQUIRE(x.dtype == want_x, ITEXB_INVALID_ARGUMENT, "%s: input has type %s, Tinput is %s", op, DtypeName(x.dtype),
                  DtypeName(want_x));
    ITEXB_REQUIRE(f.dtype == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT, "%s: filter must be qint8", op);
    ITEXB_REQUIRE(!has_bias_ || bias.dtype == tbias_, ITEXB_INVALID_ARGUMENT, "%s: bias has type %s, Tbias is %s", op,
                  DtypeName(bias.dtype), DtypeName(tbias_));
    const int64_t n = x.dims[0], h = x.dims[1], w = x.dims[2], c = x.dims[3];
    const int64_t kh = f.dims[0], kw = f.dims[1], co = f.dims[3];
    ITEXB_REQUIRE(f.dims[2] == c, ITEXB_INVALID_ARGUMENT, "input and filter must have the same depth: %lld vs %lld", (long long)c,
                  (long long)f.dims[2]);
    ITEXB_REQUIRE(!has_bias_ || (bias.rank == 1 && bias.dims[0] == co), ITEXB_INVALID_ARGUMENT,
                  "%s: bias must be a vector of %lld elements", op, (long long)co);
    int64_t oh, ow, pt = 0, pb = 0, pl = 0, pr = 0;
    if (padding_ == 2) { pt = explicit_paddings_[2]; pb = explicit_paddings_[3]; pl = explicit_paddings_[4]; pr = explicit_paddings_[5]; }
    ITEXB_REQUIRE(hostmath::WindowedOutputSize(h, kh, dil_h_, stride_h_, padding_, &oh, &pt, &pb) &&
                      hostmath::WindowedOutputSize(w, kw, dil_w_, stride_w_, padding_, &ow, &pl, &pr),
                  ITEXB_INVALID_ARGUMENT, "%s: computed output size would be negative", op);
    const float *pmin_in, *pmax_in, *pmin_f, *pmax_f, *pmin_o, *pmax_o;
    int64_t c1, c2, nf1, nf2;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng, op, "min_input", &pmin_in, &c1));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 1, op, "max_input", &pmax_in, &c2));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 2, op, "min_filter", &pmin_f, &nf1));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 3, op, "max_filter", &pmax_f, &nf2));
    static const float kZero = 0.f;
    pmin_o = pmax_o = &kZero;
    if (requantize_) {
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_frz, op, "min_freezed_output", &pmin_o, &c1));
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_frz + 1, op, "max_freezed_output", &pmax_o, &c2));
    }
    ITEXB_REQUIRE(nf1 == nf2 && (nf1 == 1 || nf1 == co), ITEXB_INVALID_ARGUMENT,
                  "%s: min_filter/max_filter must be scalars or vectors of %lld elements", op, (long long)co);
    float min_in = pmin_in[0], max_in = pmax_in[0];
    const float min_o = pmin_o[0], max_o = pmax_o[0];
    float quantize_scale = 1.f;
    if (fusion_ == ConvFusion::kQuantizeHead) {
      // QuantizeV2 SCALED to quint8 (quantize_op.h:130-152, 397-408): the convolution then sees the range [0, max]
      float qmin, qmax;
      ITEXB_REQUIRE(hostmath::AdjustInputMinMaxRange(min_in, max_in, ensure_minimum_range_, &qmin, &qmax), ITEXB_INVALID_ARGUMENT,
                    "input_max_range must be larger than input_min_range.");
      quantize_scale = hostmath::ScaledScale(&qmin, &qmax, ITEXB_DT_QUINT8, true);
      min_in = 0.f;
      max_in = qmax;
    }
    float sum_scale = 1.f;
    const itexb_tensor_t* summand = nullptr;
    if (sum_) {
      ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, i_sum, op, "summand"));
      summand = &ctx->inputs[i_sum];
      ITEXB_REQUIRE(summand->dtype == ITEXB_DT_QUINT8 || summand->dtype == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT,
                    "%s: summand must be quint8 or qint8", op);
      ITEXB_REQUIRE(summand->rank == 4 && summand->dims[0] == n && summand->dims[1] == oh && summand->dims[2] == ow &&
                        summand->dims[3] == co,
                    ITEXB_INVALID_ARGUMENT, "%s: summand must have the shape of the output", op);
      const float *ps1, *ps2;
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_sum_rng, op, "min_summand", &ps1, &c1));
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_sum_rng + 1, op, "max_summand", &ps2, &c2));
      sum_scale = hostmath::ConvSumScale(min_o, max_o, ps1[0], ps2[0], out_type_, summand->dtype);
    }

    itexb_tensor_t dst, omin, omax;
    const int64_t out_dims[4] = {n, oh, ow, co};
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, out_type_, out_dims, 4, false, &dst));
    if (dequantize_) {
      // a real-valued output carries no range
    } else if (requantize_) {
      ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, nullptr, 0, true, &omin));
      ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, nullptr, 0, true, &omax));
      *static_cast<float*>(omin.data) = min_o;
      *static_cast<float*>(omax.data) = max_o;
    } else {
      // qint32 output: the range one accumulator level spans, per filter range
      // (AllocateNativeOutputMinMax, itex/core/kernels/onednn/block/quantized_ops.h:166-195)
      const bool per_channel = ctx->inputs[i_rng + 2].rank != 0;
      const int64_t vec_dims[1] = {nf1};
      ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, vec_dims, per_channel ? 1 : 0, true, &omin));
      ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, vec_dims, per_channel ? 1 : 0, true, &omax));
      for (int64_t i = 0; i < (per_channel ? nf1 : 1); ++i)
        hostmath::QuantizationRangeForMultiplication(min_in, max_in, pmin_f[i], pmax_f[i], tinput_, ITEXB_DT_QINT8,
                                                     &static_cast<float*>(omin.data)[i], &static_cast<float*>(omax.data)[i]);
    }
    if (n == 0 || oh == 0 || ow == 0) return ITEXB_OK;

    cudaStream_t st = AsCuda(ctx->stream);
    const int ord = ctx->device_ordinal;
    itexb_conv_params_t p{};
    p.n = int(n); p.h = int(h); p.w = int(w); p.c = int(c);
    p.kh = int(kh); p.kw = int(kw); p.co = int(co);
    p.stride_h = stride_h_; p.stride_w = stride_w_; p.dil_h = dil_h_; p.dil_w = dil_w_;
    p.pad_top = int(pt); p.pad_left = int(pl);
    p.oh = int(oh); p.ow = int(ow);
    const int c_pad = itexb_conv2d_filter_c_pad(&p);       // channels per tap of the packed filter: c, or c rounded up to 128 ...
    const int64_t kp = (kh * kw * c_pad + 15) / 16 * 16;   // ... rows padded to the 16-byte pitch TMA needs

    // ---- filter: [co][kh*kw][c_pad], packed once when constant
    const bool hit = is_filter_const_ && packed_from_ == f.data && packed_.data() != nullptr && packed_bytes_ == size_t(co) * kp;
    if (!hit) {
      ITEXB_RETURN_IF_ERROR(packed_.Ensure(ord, size_t(co) * kp, st));
      ITEXB_RETURN_IF_ERROR(itexb_pack_filter_hwio(f.data, packed_.data(), int(kh), int(kw), int(c), int(co), c_pad, ctx->stream));
      packed_from_ = f.data;
      packed_bytes_ = size_t(co) * kp;
      bias_valid_ = false;
    }

    // ---- per-output-channel scale (ExtendInt8PostOps) and scaled bias (GetBiasHandle)
    std::vector<float> scales, factors;
    hostmath::ConvOutputScales(min_in, max_in, pmin_f, pmax_f, size_t(nf1), tinput_, out_type_, min_o, max_o, &scales);
    const float* d_scale = nullptr;
    ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ord, st, scales.data(), scales.size(), &d_scale));
    if (tbias_ == ITEXB_DT_QINT32 && dequantize_)
      hostmath::ConvInt32BiasDequantFactors(min_in, max_in, pmin_f, pmax_f, size_t(nf1), tinput_, &factors);
    else if (tbias_ == ITEXB_DT_QINT32) factors = scales;  // float(b32) * scale[o]
    else hostmath::ConvFloatBiasFactors(min_in, max_in, pmin_f, pmax_f, size_t(nf1), tinput_, scales, &factors);
    const bool reuse_bias = bias_valid_ && is_bias_const_ && bias_from_ == bias.data && factors == saved_factors_;
    if (has_bias_ && !reuse_bias) {
      ITEXB_RETURN_IF_ERROR(scaled_bias_.Ensure(ord, size_t(co) * sizeof(float), st));
      const float* d_f = nullptr;
      ITEXB_RETURN_IF_ERROR(factor_cache_.Get(ord, st, factors.data(), factors.size(), &d_f));
      ITEXB_RETURN_IF_ERROR(LaunchBiasPrep(kBiasMul, bias.data, tbias_, nullptr, d_f, int(factors.size()), nullptr, 0, 0.f,
                                           static_cast<float*>(scaled_bias_.data()), int(co), st));
      bias_valid_ = true;
      bias_from_ = bias.data;
      saved_factors_ = factors;
    }

    const void* x_data = x.data;
    if (fusion_ == ConvFusion::kQuantizeHead) {
      void* q = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(n) * h * w * c, false, &q));
      ITEXB_RETURN_IF_ERROR(itexb_quantize(x.data, x.dtype, q, ITEXB_DT_QUINT8, n * h * w * c, 1, 1, ITEXB_QUANT_SCALED, nullptr, nullptr,
                                           quantize_scale, 0.f, ctx->stream));
      x_data = q;
    }
    p.c_pad = c_pad;
    p.x_dtype = tinput_; p.out_dtype = out_type_;
    p.x = x_data; p.filter_packed = packed_.data(); p.out = dst.data;
    if (out_type_ != ITEXB_DT_QINT32) {
      p.ep.scale = d_scale;
      p.ep.scale_count = int(scales.size());
    }
    p.ep.bias = has_bias_ ? static_cast<const float*>(scaled_bias_.data()) : nullptr;
    p.ep.relu = relu_ ? 1 : 0;
    p.ep.raw_acc = (out_type_ == ITEXB_DT_QINT32 && !has_bias_ && !relu_ && summand == nullptr && act_ == ITEXB_ACT_NONE) ? 1 : 0;  // the exact accumulators
    // Element-wise post-ops run on the scaled value with post-op scale 1 (quantized_conv_ops.h:437-445)
    p.ep.activation = act_;
    p.ep.act_alpha = act_alpha_;
    if (summand != nullptr) {
      p.ep.summand = summand->data;
      p.ep.summand_dtype = summand->dtype;
      p.ep.ld_summand = co;
      p.ep.sum_scale = sum_scale;
    }
    const size_t ws = itexb_conv2d_workspace_bytes(&p);
    if (ws > 0) ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, ws, false, &p.workspace));
    p.status_word = StatusWord(ord, st);
    return itexb_conv2d(&p, ctx->stream);
  }

 private:
  bool relu_, sum_, signed_sum_, has_bias_, requantize_;
  const bool new_api_;
  const ConvFusion fusion_;
  bool dequantize_ = false;
  int treal_ = ITEXB_DT_FLOAT;           // kQuantizeHead: type of the real-valued input
  float ensure_minimum_range_ = 0.01f;   // kQuantizeHead: QuantizeV2's attr
  int act_ = ITEXB_ACT_NONE;
  float act_alpha_ = 0.f;
  int stride_h_ = 1, stride_w_ = 1, dil_h_ = 1, dil_w_ = 1, padding_ = 1;
  std::vector<int64_t> explicit_paddings_;
  bool is_filter_const_ = true, is_bias_const_ = true;
  int tinput_ = ITEXB_DT_QUINT8, tbias_ = ITEXB_DT_FLOAT, out_type_ = ITEXB_DT_QUINT8;
  DeviceBuffer packed_, scaled_bias_;
  const void* packed_from_ = nullptr;
  size_t packed_bytes_ = 0;
  bool bias_valid_ = false;
  const void* bias_from_ = nullptr;
  std::vector<float> saved_factors_;
  DeviceVectorCache scale_cache_, factor_cache_;
};

struct ConvBiasReluReq : QuantizedConv2DOp { ConvBiasReluReq() : QuantizedConv2DOp(true, false, false) {} };
struct ConvBiasReq : QuantizedConv2DOp { ConvBiasReq() : QuantizedConv2DOp(false, false, false) {} };
struct ConvBiasSumReluReq : QuantizedConv2DOp { ConvBiasSumReluReq() : QuantizedConv2DOp(true, true, false) {} };
struct ConvBiasSignedSumReluReq : QuantizedConv2DOp { ConvBiasSignedSumReluReq() : QuantizedConv2DOp(true, true, true) {} };

struct ConvS32 : QuantizedConv2DOp { ConvS32() : QuantizedConv2DOp(false, false, false, false, false) {} };
struct ConvReluS32 : QuantizedConv2DOp { ConvReluS32() : QuantizedConv2DOp(true, false, false, false, false) {} };
struct ConvBiasS32 : QuantizedConv2DOp { ConvBiasS32() : QuantizedConv2DOp(false, false, false, true, false) {} };
struct ConvBiasReluS32 : QuantizedConv2DOp { ConvBiasReluS32() : QuantizedConv2DOp(true, false, false, true, false) {} };
struct ConvReq : QuantizedConv2DOp { ConvReq() : QuantizedConv2DOp(false, false, false, false, true) {} };
struct ConvReluReq : QuantizedConv2DOp { ConvReluReq() : QuantizedConv2DOp(true, false, false, false, true) {} };

// qint32-output members (itex/core/kernels/gpu/quantized_conv_ops.cc:72-100): HostMemory inputs 2..5 (3..6 with a bias)
ITEXB_REGISTER_OP("QuantizedConv2D", ConvS32, 6, 3, 0x3cu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2D", ConvS32, 6, 3, 0x3cu, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DPerChannel", ConvS32, 6, 3, 0x3cu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DPerChannel", ConvS32, 6, 3, 0x3cu, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DAndRelu", ConvReluS32, 6, 3, 0x3cu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DAndRelu", ConvReluS32, 6, 3, 0x3cu, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DWithBias", ConvBiasS32, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithBias", ConvBiasS32, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DWithBiasAndRelu", ConvBiasReluS32, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithBiasAndRelu", ConvBiasReluS32, 7, 3, 0x78u, 0x6u);
// requantizing members without a bias (:104-110): HostMemory inputs 2..7
ITEXB_REGISTER_OP("QuantizedConv2DAndRequantize", ConvReq, 8, 3, 0xfcu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DAndRequantize", ConvReq, 8, 3, 0xfcu, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DAndReluAndRequantize", ConvReluReq, 8, 3, 0xfcu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DAndReluAndRequantize", ConvReluReq, 8, 3, 0xfcu, 0x6u);
struct ConvBiasDeq : QuantizedConv2DOp { ConvBiasDeq() : QuantizedConv2DOp(false, false, false, true, false, false, ConvFusion::kDequantizeTail) {} };
struct QuantConvBiasReluReq : QuantizedConv2DOp {
  QuantConvBiasReluReq() : QuantizedConv2DOp(true, false, false, true, true, false, ConvFusion::kQuantizeHead) {}
};
// HostMemory: the six ranges, inputs 3..8 (conv_ops_impl_gpu.cc:716-1000); outputs 1, 2 of the quantizing op.
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithDequantize", ConvBiasDeq, 9, 1, 0x1f8u, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithCast", ConvBiasDeq, 9, 1, 0x1f8u, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizeV2WithQuantizedConv2D", QuantConvBiasReluReq, 9, 3, 0x1f8u, 0x6u);
struct ConvV2 : QuantizedConv2DOp { ConvV2() : QuantizedConv2DOp(false, false, false, false, false, true) {} };
// New API: list-typed arguments (counts depend on fused_ops), every range in host memory
// (HostMemoryList2("host_inputs", "host_outputs"), itex/core/kernels/gpu/quantized_conv_ops.cc:171-200)
ITEXB_REGISTER_OP("_QuantizedConv2D", ConvV2, -1, -1, 0u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DV2", ConvV2, -1, -1, 0u, 0x6u);
// HostMemory: inputs 3..8 (and 10, 11), outputs 1, 2.
ITEXB_REGISTER_OP("QuantizedConv2DWithBiasAndReluAndRequantize", ConvBiasReluReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithBiasAndReluAndRequantize", ConvBiasReluReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DWithBiasAndRequantize", ConvBiasReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithBiasAndRequantize", ConvBiasReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DWithBiasSumAndReluAndRequantize", ConvBiasSumReluReq, 12, 3, 0xdf8u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize", ConvBiasSumReluReq, 12, 3, 0xdf8u, 0x6u);
ITEXB_REGISTER_OP("QuantizedConv2DWithBiasSignedSumAndReluAndRequantize", ConvBiasSignedSumReluReq, 12, 3, 0xdf8u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConv2DWithBiasSignedSumAndReluAndRequantize", ConvBiasSignedSumReluReq, 12, 3, 0xdf8u, 0x6u);

}  // namespace
}  // namespace itexb
