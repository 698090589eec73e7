// The fused int8 matmul family, three generations of the same kernel in the reference:
//
//   WithBias  [_ITEX]QuantizedMatMulWithBias, ...AndRelu, ...AndRequantize, ...AndReluAndRequantize,
//             ...AndDequantize.  Inputs a, b, bias, min_a, max_a, min_b, max_b[, min_freezed_output,
//             max_freezed_output]; one output scale from element 0 of min_b/max_b; quint8 activations only.
//             QuantizedMatMulOp / QuantizedMatMulReluOp, quantized_matmul_common.h:1414-1531.
//   FusedV1   _[ITEX]QuantizedFusedMatMul, ...AndRequantize, ...AndDequantize.  Inputs a, b,
//             args[num_args] (bias, then the addend of an "Add" post-op), the four ranges[, the frozen output
//             range]; fused_ops = [] | [BiasAdd] | [BiasAdd, <activation or Add>]; per-output-channel
//             scale; qint8 or quint8 activations.  QuantizedFusedMatMulOp, :1534-1710.
//   V2        _[ITEX]QuantizedMatMul.  device_inputs (a, b, bias[, addend]) and host_inputs (the ranges)
//             flattened in that order; fused_ops lists BiasAdd, an activation and/or Add, and Dequantize or
//             Requantize; output types from Tout.  QuantizedFusedMatMulV2Op, :1712-1908.
//
// All three run LegacyQuantizedMatMulOpBase::Compute (:61-336): HostMemory arguments, bias scaling
// (GetScaledBias :466-660, qint32 bias :1153-1334) and output ranges (AllocateNativeOutputMinMax,
// onednn/block/quantized_ops.h:142-203) are shared.  Registrations: itex/core/kernels/gpu/quantized_matmul.cc:35-260.
// Where the reference builds a oneDNN inner-product primitive, this op packs the weight once to K-major,
// prepares the scaled bias on the device and launches one tcgen05 GEMM with the fused epilogue.
//
// One behaviour of the reference is reproduced only on request: for "requantize after an activation" it
// computes a post-op scale (255|127 / output range) but oneDNN 3 eltwise post-ops take no scale, so the value
// is dropped and the stored integers are the activation's real-valued result.  Attr `_postop_scale_mode` or env
// ITEXB_POSTOP_SCALE_MODE = "literal" reproduces that; the default "intended" applies the scale.
#include <cstdlib>

#include "hostmath.h"
#include "op_kernel.h"

namespace itexb {
namespace {

enum class Tail { kNone, kRequantize, kDequantize };
enum class Flavor { kWithBias, kFusedV1, kV2 };

// Maps a fused_ops entry to an epilogue activation; false when it is not an element-wise post-op
// this library implements.  Names and alpha/beta as in PostOpUtil::GetAllPostOpInfo
// (itex/core/utils/onednn/onednn_post_op_util.cc:22-71).
bool ActivationByName(const std::string& name, float leakyrelu_alpha, int* kind, float* alpha, float* beta) {
  *alpha = 0.f;
  *beta = 0.f;
  if (name == "Relu") *kind = ITEXB_ACT_RELU;
  else if (name == "LeakyRelu") { *kind = ITEXB_ACT_RELU; *alpha = leakyrelu_alpha; }
  else if (name == "Relu6") { *kind = ITEXB_ACT_CLIP; *beta = 6.f; }
  else if (name == "GeluExact") *kind = ITEXB_ACT_GELU_ERF;
  else if (name == "GeluApproximate") *kind = ITEXB_ACT_GELU_TANH;
  else if (name == "Sigmoid") *kind = ITEXB_ACT_SIGMOID;
  else if (name == "Tanh") *kind = ITEXB_ACT_TANH;
  else if (name == "Elu") { *kind = ITEXB_ACT_ELU; *alpha = 1.f; }
  else if (name == "_ITEXSwish") { *kind = ITEXB_ACT_SWISH; *alpha = 1.f; }
  else return false;
  return true;
}

class QuantizedMatMulOp : public OpKernel {
 public:
  QuantizedMatMulOp(bool relu, Tail tail, Flavor flavor = Flavor::kWithBias) : relu_(relu), tail_(tail), flavor_(flavor) {}

  int InitFused(const AttrMap& attrs) {
    const char* op = name().c_str();
    std::vector<std::string> fused;
    if (attrs.Has("fused_ops")) ITEXB_RETURN_IF_ERROR(attrs.GetStringList("fused_ops", &fused));
    float leaky = 0.2f;
    if (attrs.Has("leakyrelu_alpha")) ITEXB_RETURN_IF_ERROR(attrs.GetFloat("leakyrelu_alpha", &leaky));
    if (flavor_ == Flavor::kFusedV1) {
      ITEXB_REQUIRE(fused.size() <= 2, ITEXB_INVALID_ARGUMENT, "_QuantizedFusedMatMul supports maximum 2 post ops");
      ITEXB_REQUIRE(fused.empty() || fused[0] == "BiasAdd", ITEXB_INVALID_ARGUMENT, "_QuantizedFusedMatMul first post op must be BiasAdd");
    }
    has_bias_ = false;
    bool saw_tail = false;
    int order = 0, act_at = -1, add_at = -1;
    for (const std::string& f : fused) {
      if (f == "BiasAdd") has_bias_ = true;
      else if (f == "Add") { has_add_ = true; add_at = order++; }
      else if (f == "Dequantize" || f == "Requantize" || f == "Quantized") {
        ITEXB_REQUIRE(flavor_ == Flavor::kV2, ITEXB_INVALID_ARGUMENT, "Found unsupported fusion in %s.", op);
        saw_tail = true;
        if (f == "Requantize") tail_ = Tail::kRequantize;
        if (f == "Dequantize") tail_ = Tail::kDequantize;
      } else {
        ITEXB_REQUIRE(ActivationByName(f, leaky, &act_, &act_alpha_, &act_beta_), ITEXB_INVALID_ARGUMENT,
                      "Found unsupported fusion in %s: %s", op, f.c_str());
        ITEXB_REQUIRE(act_at < 0, ITEXB_INVALID_ARGUMENT, "%s: more than one activation in fused_ops", op);
        act_at = order++;
      }
    }
    (void)saw_tail;
    ITEXB_REQUIRE(!(act_at >= 0 && add_at >= 0 && act_at < add_at), ITEXB_UNIMPLEMENTED,
                  "%s: an Add after the activation is not implemented (Add, then activation is)", op);
    if (flavor_ == Flavor::kV2) {
      ITEXB_REQUIRE(has_bias_, ITEXB_INVALID_ARGUMENT, "%s: fused_ops must contain BiasAdd (the input positions assume a bias)", op);
      std::string oq = "SCALED";
      if (attrs.Has("output_quant_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("output_quant_mode", &oq));
      ITEXB_REQUIRE(!(tail_ == Tail::kRequantize && oq == "MIN_FIRST"), ITEXB_UNIMPLEMENTED,
                    "%s: output_quant_mode=MIN_FIRST with Requantize is not implemented", op);
    }
    intended_postop_scale_ = true;
    std::string psm;
    const char* env = std::getenv("ITEXB_POSTOP_SCALE_MODE");
    if (env != nullptr) psm = env;
    if (attrs.Has("_postop_scale_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("_postop_scale_mode", &psm));
    if (!psm.empty()) {
      ITEXB_REQUIRE(psm == "literal" || psm == "intended", ITEXB_INVALID_ARGUMENT,
                    "post-op scale mode must be 'literal' or 'intended', is '%s'", psm.c_str());
      intended_postop_scale_ = psm == "intended";
    }
    return ITEXB_OK;
  }

  int Init(const AttrMap& attrs) override {
    const char* op = name().c_str();
    t1_ = ITEXB_DT_QUINT8;
    t2_ = ITEXB_DT_QINT8;
    if (attrs.Has("T1")) ITEXB_RETURN_IF_ERROR(attrs.GetType("T1", &t1_));
    if (attrs.Has("T2")) ITEXB_RETURN_IF_ERROR(attrs.GetType("T2", &t2_));
    const bool fused = flavor_ != Flavor::kWithBias;
    if (fused) ITEXB_RETURN_IF_ERROR(InitFused(attrs));
    ITEXB_REQUIRE((t1_ == ITEXB_DT_QUINT8 || (fused && t1_ == ITEXB_DT_QINT8)) && t2_ == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for T1=%s, T2=%s (only quint8 x qint8 is)", op, DtypeName(t1_), DtypeName(t2_));
    tbias_ = ITEXB_DT_FLOAT;
    const char* bias_attr = flavor_ == Flavor::kFusedV1 ? "Targs" : "Tbias";
    if (attrs.Has(bias_attr)) ITEXB_RETURN_IF_ERROR(attrs.GetType(bias_attr, &tbias_));
    ITEXB_REQUIRE(tbias_ == ITEXB_DT_FLOAT || tbias_ == ITEXB_DT_QINT32 || ((tail_ == Tail::kDequantize || fused) && tbias_ == ITEXB_DT_BFLOAT16),
                  ITEXB_INVALID_ARGUMENT, "%s: no kernel registered for %s=%s", op, bias_attr, DtypeName(tbias_));
    toutput_ = tail_ == Tail::kNone ? ITEXB_DT_QINT32 : (tail_ == Tail::kRequantize ? ITEXB_DT_QUINT8 : ITEXB_DT_FLOAT);
    const char* out_attr = flavor_ == Flavor::kV2 ? "Tout" : "Toutput";
    if (attrs.Has(out_attr)) ITEXB_RETURN_IF_ERROR(attrs.GetType(out_attr, &toutput_));
    if (flavor_ == Flavor::kV2 && tail_ == Tail::kNone && toutput_ != ITEXB_DT_QINT32)
      tail_ = (toutput_ == ITEXB_DT_QUINT8 || toutput_ == ITEXB_DT_QINT8) ? Tail::kRequantize : Tail::kDequantize;
    ITEXB_REQUIRE(!has_add_ || toutput_ == ITEXB_DT_FLOAT || toutput_ == ITEXB_DT_BFLOAT16 || toutput_ == ITEXB_DT_HALF, ITEXB_UNIMPLEMENTED,
                  "Quantized addend tensor is not implemented yet.");
    bool ok = false;
    if (tail_ == Tail::kNone) ok = toutput_ == ITEXB_DT_QINT32;
    if (tail_ == Tail::kRequantize) ok = toutput_ == ITEXB_DT_QUINT8 || toutput_ == ITEXB_DT_QINT8;
    if (tail_ == Tail::kDequantize) ok = toutput_ == ITEXB_DT_FLOAT || toutput_ == ITEXB_DT_BFLOAT16 || toutput_ == ITEXB_DT_HALF;
    ITEXB_REQUIRE(ok, ITEXB_INVALID_ARGUMENT, "%s: no kernel registered for Toutput=%s", op, DtypeName(toutput_));
    std::string mode = fused ? "SCALED" : "MIN_FIRST";  // the defaults of the respective op definitions
    if (attrs.Has("input_quant_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("input_quant_mode", &mode));
    if (mode == "MIN_FIRST") min_first_ = true;
    else if (mode == "SCALED") min_first_ = false;
    else return SetError(ITEXB_INVALID_ARGUMENT, "Quantization mode must be either MIN_FIRST or SCALED, but received %s", mode.c_str());
    is_weight_const_ = true;
    const char* wconst = flavor_ == Flavor::kFusedV1 ? "is_filter_const" : "is_weight_const";
    if (attrs.Has(wconst)) ITEXB_RETURN_IF_ERROR(attrs.GetBool(wconst, &is_weight_const_));
    // The scaled bias is cached only for a constant bias AND a constant weight (quantized_matmul_common.h:459,637,1146).
    is_bias_const_ = true;
    if (attrs.Has("is_bias_const")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("is_bias_const", &is_bias_const_));
    transpose_a_ = transpose_b_ = false;
    if (attrs.Has("transpose_a")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("transpose_a", &transpose_a_));
    if (attrs.Has("transpose_b")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("transpose_b", &transpose_b_));
    // How the SCALED-mode float bias is treated.  "literal" multiplies it by
    // 255*127/(range_input*range_weight) exactly as the reference lines 602-634 do;
    // "intended" expresses it in the units of the value it is added to (what y = scale*acc + bias needs):
    // unchanged for float outputs, times the requantize factor for 8-bit ones.
    literal_scaled_bias_ = true;
    std::string sbm;
    const char* env = std::getenv("ITEXB_SCALED_BIAS_MODE");
    if (env != nullptr) sbm = env;
    if (attrs.Has("_scaled_bias_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("_scaled_bias_mode", &sbm));
    if (!sbm.empty()) {
      ITEXB_REQUIRE(sbm == "literal" || sbm == "intended", ITEXB_INVALID_ARGUMENT,
                    "scaled bias mode must be 'literal' or 'intended', is '%s'", sbm.c_str());
      literal_scaled_bias_ = sbm == "literal";
    }
    return ITEXB_OK;
  }

  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    // Input positions: a, b, [bias], [addend], min_a, max_a, min_b, max_b, [min_freezed_output, max_freezed_output]
    const int i_bias = has_bias_ ? 2 : -1;
    const int i_add = has_add_ ? 2 + (has_bias_ ? 1 : 0) : -1;
    const int i_rng = 2 + (has_bias_ ? 1 : 0) + (has_add_ ? 1 : 0);
    const bool has_freezed = flavor_ == Flavor::kV2 ? tail_ == Tail::kRequantize : tail_ != Tail::kNone && !(flavor_ == Flavor::kFusedV1 && tail_ == Tail::kDequantize);
    const int nin = i_rng + 4 + (has_freezed ? 2 : 0);
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, nin, op));
    for (int i = 0; i < i_rng; ++i)
      ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, i, op, i == 0 ? "a" : (i == 1 ? "b" : (i == i_bias ? "bias" : "addend"))));
    const itexb_tensor_t& a = ctx->inputs[0];
    const itexb_tensor_t& b = ctx->inputs[1];
    static const itexb_tensor_t kNoTensor{};
    const itexb_tensor_t& bias = has_bias_ ? ctx->inputs[i_bias] : kNoTensor;
    ITEXB_REQUIRE(a.dtype == t1_ && b.dtype == t2_, ITEXB_INVALID_ARGUMENT, "%s: a/b have types %s/%s, attrs say %s/%s", op,
                  DtypeName(a.dtype), DtypeName(b.dtype), DtypeName(t1_), DtypeName(t2_));
    ITEXB_REQUIRE(!has_bias_ || bias.dtype == tbias_, ITEXB_INVALID_ARGUMENT, "%s: bias has type %s, Tbias is %s", op, DtypeName(bias.dtype),
                  DtypeName(tbias_));
    ITEXB_REQUIRE(a.rank == 2 && b.rank == 2, ITEXB_INVALID_ARGUMENT, "%s: a and b must be matrices", op);
    const int64_t m = transpose_a_ ? a.dims[1] : a.dims[0];
    const int64_t k = transpose_a_ ? a.dims[0] : a.dims[1];
    const int64_t kb = transpose_b_ ? b.dims[1] : b.dims[0];
    const int64_t n = transpose_b_ ? b.dims[0] : b.dims[1];
    ITEXB_REQUIRE(k == kb, ITEXB_INVALID_ARGUMENT, "Matrix size-incompatible: In[0]: [%lld,%lld], In[1]: [%lld,%lld]",
                  (long long)a.dims[0], (long long)a.dims[1], (long long)b.dims[0], (long long)b.dims[1]);
    ITEXB_REQUIRE(!has_bias_ || (bias.rank == 1 && bias.dims[0] == n), ITEXB_INVALID_ARGUMENT, "%s: bias must be a vector of %lld elements", op,
                  (long long)n);
    if (has_add_) {
      const itexb_tensor_t& z = ctx->inputs[i_add];
      ITEXB_REQUIRE(z.dtype == toutput_ && z.rank == 2 && z.dims[0] == m && z.dims[1] == n, ITEXB_INVALID_ARGUMENT,
                    "%s: the addend must have the type and shape of the output", op);
    }
    ITEXB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31) && k > 0, ITEXB_INVALID_ARGUMENT, "%s: dimension out of range", op);
    const float *pmin_a, *pmax_a, *pmin_b, *pmax_b;
    int64_t c1, c2, nb_min, nb_max;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng, op, "min_a", &pmin_a, &c1));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 1, op, "max_a", &pmax_a, &c2));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 2, op, "min_b", &pmin_b, &nb_min));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 3, op, "max_b", &pmax_b, &nb_max));
    ITEXB_REQUIRE(nb_min == nb_max && (nb_min == 1 || nb_min == n), ITEXB_INVALID_ARGUMENT,
                  "%s: min_b/max_b must be scalars or vectors of %lld elements", op, (long long)n);
    const float min_a = pmin_a[0], max_a = pmax_a[0];
    float min_freezed = 0.f, max_freezed = 0.f;
    if (has_freezed) {
      const float *p7, *p8;
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 4, op, "min_freezed_output", &p7, &c1));
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i_rng + 5, op, "max_freezed_output", &p8, &c2));
      min_freezed = p7[0];
      max_freezed = p8[0];
    }

    // ---- outputs
    itexb_tensor_t dst;
    const int64_t out_dims[2] = {m, n};
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, toutput_, out_dims, 2, false, &dst));
    if (tail_ != Tail::kDequantize) {
      itexb_tensor_t omin, omax;
      const bool per_channel = toutput_ == ITEXB_DT_QINT32 && ctx->inputs[i_rng + 2].rank != 0;
      const int64_t vec_dims[1] = {nb_min};
      ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, vec_dims, per_channel ? 1 : 0, true, &omin));
      ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, vec_dims, per_channel ? 1 : 0, true, &omax));
      float* o1 = static_cast<float*>(omin.data);
      float* o2 = static_cast<float*>(omax.data);
      if (toutput_ == ITEXB_DT_QINT32) {
        // AllocateNativeOutputMinMax, itex/core/kernels/onednn/block/quantized_ops.h:166-195.
        for (int64_t i = 0; i < (per_channel ? nb_min : 1); ++i)
          hostmath::QuantizationRangeForMultiplication(min_a, max_a, pmin_b[i], pmax_b[i], t1_, ITEXB_DT_QINT8, &o1[i], &o2[i]);
      } else {
        o1[0] = min_freezed;
        o2[0] = max_freezed;
      }
    }
    if (m == 0 || n == 0) return ITEXB_OK;

    cudaStream_t st = AsCuda(ctx->stream);
    const int ord = ctx->device_ordinal;
    const int64_t k_pad = (k + 15) / 16 * 16;

    // ---- weights: K-major [n, k_pad], packed once when constant
    const void* w_ptr = nullptr;
    int64_t ldb = k_pad;
    const bool cache_hit = is_weight_const_ && packed_from_ == b.data && packed_k_ == k && packed_n_ == n && packed_.data() != nullptr;
    if (transpose_b_ && k % 16 == 0 && (reinterpret_cast<uintptr_t>(b.data) & 15) == 0) {
      w_ptr = b.data;  // already [n, k] with a TMA-legal pitch
      ldb = k;
      if (packed_from_ != b.data || !is_weight_const_) {
        packed_from_ = b.data;
        colsum_valid_ = false;
        bias_valid_ = false;
      }
    } else if (cache_hit) {
      w_ptr = packed_.data();
    } else {
      ITEXB_RETURN_IF_ERROR(packed_.Ensure(ord, size_t(n) * k_pad, st));
      if (transpose_b_) {
        ITEXB_CUDA(cudaMemsetAsync(packed_.data(), 0, size_t(n) * k_pad, st));
        ITEXB_CUDA(cudaMemcpy2DAsync(packed_.data(), k_pad, b.data, k, k, n, cudaMemcpyDeviceToDevice, st));
      } else {
        ITEXB_RETURN_IF_ERROR(itexb_pack_weights_kn(b.data, packed_.data(), k, n, k_pad, ctx->stream));
      }
      packed_from_ = b.data;
      packed_k_ = k;
      packed_n_ = n;
      colsum_valid_ = false;
      bias_valid_ = false;
      w_ptr = packed_.data();
    }

    // ---- activations: [m, k] row-major with a TMA-legal pitch
    const void* a_ptr = a.data;
    int64_t lda = k;
    if (transpose_a_) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(m) * k_pad, false, &tmp));
      ITEXB_RETURN_IF_ERROR(itexb_pack_weights_kn(a.data, tmp, k, m, k_pad, ctx->stream));  // [k,m] -> [m,k_pad]
      a_ptr = tmp;
      lda = k_pad;
    } else if (k % 16 != 0 || (reinterpret_cast<uintptr_t>(a.data) & 15) != 0) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(m) * k_pad, false, &tmp));
      ITEXB_CUDA(cudaMemcpy2DAsync(tmp, k_pad, a.data, k, k, m, cudaMemcpyDeviceToDevice, st));
      a_ptr = tmp;
      lda = k_pad;
    }

    // ---- output scale (ExtendInt8PostOps).  WithBias ops: one scalar, from element 0 of min_b/max_b.
    //      Fused ops: one per weight range, folded with the requantize factor unless an activation
    //      sits in between (then that factor is the activation's post scale).
    const float* d_scale = nullptr;
    int scale_count = 0;
    float out_scale = 1.f, post_scale = 1.f;
    std::vector<float> scale_key;  // every value the scaled bias depends on besides the bias itself: all output scales
    const float max_in = hostmath::MaxIntOf(t1_);
    if (toutput_ != ITEXB_DT_QINT32) {
      if (flavor_ == Flavor::kWithBias) {
        out_scale = hostmath::MatMulOutputScale(min_a, max_a, pmin_b[0], pmax_b[0], toutput_, min_freezed, max_freezed);
        ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ord, st, &out_scale, 1, &d_scale));
        scale_count = 1;
        scale_key.assign(1, out_scale);
      } else {
        std::vector<float> sc;
        hostmath::FusedMatMulOutputScales(min_a, max_a, pmin_b, pmax_b, size_t(nb_min), min_first_, t1_, &sc);
        if (tail_ == Tail::kRequantize) {
          const float range_output = std::max(std::abs(min_freezed), std::abs(max_freezed));
          const float factor = hostmath::MaxIntOf(toutput_) / range_output;
          if (act_ == ITEXB_ACT_NONE) for (float& v : sc) v = v * factor;
          else if (intended_postop_scale_) post_scale = factor;
        }
        ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ord, st, sc.data(), sc.size(), &d_scale));
        scale_count = int(sc.size());
        scale_key = sc;
      }
    }

    // ---- scaled bias (GetScaledBias), cached like the reference: constant bias and weight,
    //      and an input range within 1e-5 of the one it was computed for
    // The weight ranges enter through scale_key (per channel) and, for qint32 outputs, through the bias factors, which
    // are functions of the same ranges and of (min_a, max_a).
    for (int64_t i = 0; i < nb_min; ++i) { scale_key.push_back(pmin_b[i]); scale_key.push_back(pmax_b[i]); }
    const bool reuse_bias = bias_valid_ && is_weight_const_ && is_bias_const_ && bias_from_ == bias.data &&
                            std::abs(min_a - saved_min_a_) < 1e-5f && std::abs(max_a - saved_max_a_) < 1e-5f && saved_scale_key_ == scale_key;
    if (has_bias_ && !reuse_bias) {
      ITEXB_RETURN_IF_ERROR(scaled_bias_.Ensure(ord, size_t(n) * sizeof(float), st));
      const float range_input = min_first_ ? max_a - min_a : std::max(std::abs(min_a), std::abs(max_a));
      std::vector<float> s(nb_min);
      for (int64_t i = 0; i < nb_min; ++i) {
        const float range_weight = std::max(std::abs(pmin_b[i]), std::abs(pmax_b[i]));
        s[i] = tbias_ == ITEXB_DT_QINT32 ? (range_input * range_weight) / (max_in * 127.0f)
                                          : (max_in * 127.0f) / (range_input * range_weight);
      }
      const float* d_s = nullptr;
      ITEXB_RETURN_IF_ERROR(bias_scale_cache_.Get(ord, st, s.data(), s.size(), &d_s));
      const bool out_float = tail_ == Tail::kDequantize;
      const bool out_int8 = tail_ == Tail::kRequantize;
      int mode = kBiasCopy;
      const float* f = nullptr;
      int f_count = 0;
      const float* g = nullptr;
      int g_count = 0;
      const int32_t* colsum = nullptr;
      float qmin = 0.f;
      if (tbias_ == ITEXB_DT_QINT32) {
        if (min_first_) {
          if (out_float) { mode = kBiasMul; f = d_s; f_count = int(nb_min); }
          else if (out_int8) { mode = kBiasMul; f = d_scale; f_count = scale_count; }
          else mode = kBiasCopy;
        } else {
          mode = kBiasMul; f = d_s; f_count = int(nb_min);
        }
      } else if (min_first_) {
        if (!colsum_valid_) {
          ITEXB_RETURN_IF_ERROR(colsum_.Ensure(ord, size_t(n) * sizeof(int32_t), st));
          if (transpose_b_) {
            // column sums of the [k,n] view = row sums of the [n,k] tensor: transpose first
            void* tmp = nullptr;
            ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(n) * k, false, &tmp));
            ITEXB_RETURN_IF_ERROR(itexb_pack_weights_kn(b.data, tmp, n, k, n, ctx->stream));  // [n,k] -> [k,n]
            ITEXB_RETURN_IF_ERROR(itexb_colsum_s8(static_cast<const int8_t*>(tmp), static_cast<int32_t*>(colsum_.data()), k, n, ctx->stream));
          } else {
            ITEXB_RETURN_IF_ERROR(itexb_colsum_s8(static_cast<const int8_t*>(b.data), static_cast<int32_t*>(colsum_.data()), k, n, ctx->stream));
          }
          colsum_valid_ = is_weight_const_;
        }
        colsum = static_cast<const int32_t*>(colsum_.data());
        qmin = max_in * min_a / range_input;
        f = d_s; f_count = int(nb_min);
        if (out_float) mode = kBiasMinFirstFloat;
        else if (out_int8) { mode = kBiasMinFirstInt8; g = d_scale; g_count = scale_count; }
        else mode = kBiasMinFirstS32;
      } else if (literal_scaled_bias_) {
        mode = kBiasMul; f = d_s; f_count = int(nb_min);
      } else {
        // "intended": the bias in the units of the value it is added to = the MIN_FIRST formulas without compensation
        f = d_s; f_count = int(nb_min);
        if (out_float) { mode = kBiasCopy; f = nullptr; f_count = 0; }
        else if (out_int8) { mode = kBiasMinFirstInt8; g = d_scale; g_count = scale_count; }
        else mode = kBiasMinFirstS32;
      }
      ITEXB_RETURN_IF_ERROR(LaunchBiasPrep(mode, bias.data, tbias_, colsum, f, f_count, g, g_count, qmin,
                                           static_cast<float*>(scaled_bias_.data()), int(n), st));
      bias_valid_ = true;
      bias_from_ = bias.data;
      saved_min_a_ = min_a;
      saved_max_a_ = max_a;
      saved_scale_key_ = scale_key;
    }

    // ---- the GEMM
    itexb_gemm_params_t p{};
    p.m = int(m); p.n = int(n); p.k = int(k);
    p.a_dtype = t1_; p.b_dtype = t2_; p.out_dtype = toutput_;
    p.a = a_ptr; p.lda = lda;
    p.b = w_ptr; p.ldb = ldb;
    p.out = dst.data; p.ldo = n;
    p.ep.scale = d_scale;
    p.ep.scale_count = scale_count;
    p.ep.bias = has_bias_ ? static_cast<const float*>(scaled_bias_.data()) : nullptr;
    p.ep.relu = relu_ ? 1 : 0;
    if (has_add_) {
      // oneDNN sum post-op with scale 1 (SetPostOpScale("Add", 1.0f)); the reference writes in place into the addend
      p.ep.summand = ctx->inputs[i_add].data;
      p.ep.summand_dtype = toutput_;
      p.ep.ld_summand = n;
      p.ep.sum_scale = 1.f;
    }
    p.ep.activation = act_;
    p.ep.act_alpha = act_alpha_;
    p.ep.act_beta = act_beta_;
    p.ep.post_scale = post_scale;
    p.status_word = StatusWord(ord, st);
    return itexb_gemm(&p, ctx->stream);
  }

 private:
  const bool relu_;
  Tail tail_;
  const Flavor flavor_;
  bool has_bias_ = true, has_add_ = false, intended_postop_scale_ = true;
  int act_ = ITEXB_ACT_NONE;
  float act_alpha_ = 0.f, act_beta_ = 0.f;
  int t1_ = ITEXB_DT_QUINT8, t2_ = ITEXB_DT_QINT8, tbias_ = ITEXB_DT_FLOAT, toutput_ = ITEXB_DT_QINT32;
  bool min_first_ = true, is_weight_const_ = true, is_bias_const_ = true, transpose_a_ = false, transpose_b_ = false, literal_scaled_bias_ = true;
  // weight cache (plays WeightCacheManager's role) and derived per-weight data
  DeviceBuffer packed_, colsum_, scaled_bias_;
  const void* packed_from_ = nullptr;
  int64_t packed_k_ = 0, packed_n_ = 0;
  bool colsum_valid_ = false, bias_valid_ = false;
  const void* bias_from_ = nullptr;
  float saved_min_a_ = 0.f, saved_max_a_ = 0.f;
  std::vector<float> saved_scale_key_;
  DeviceVectorCache scale_cache_, bias_scale_cache_;
};

struct WithBias : QuantizedMatMulOp { WithBias() : QuantizedMatMulOp(false, Tail::kNone) {} };
struct WithBiasRelu : QuantizedMatMulOp { WithBiasRelu() : QuantizedMatMulOp(true, Tail::kNone) {} };
struct WithBiasReq : QuantizedMatMulOp { WithBiasReq() : QuantizedMatMulOp(false, Tail::kRequantize) {} };
struct WithBiasReluReq : QuantizedMatMulOp { WithBiasReluReq() : QuantizedMatMulOp(true, Tail::kRequantize) {} };
struct WithBiasDeq : QuantizedMatMulOp { WithBiasDeq() : QuantizedMatMulOp(false, Tail::kDequantize) {} };

// HostMemory: inputs 3..6 (and 7, 8), outputs 1, 2.
ITEXB_REGISTER_OP("QuantizedMatMulWithBias", WithBias, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedMatMulWithBias", WithBias, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("QuantizedMatMulWithBiasAndRelu", WithBiasRelu, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedMatMulWithBiasAndRelu", WithBiasRelu, 7, 3, 0x78u, 0x6u);
ITEXB_REGISTER_OP("QuantizedMatMulWithBiasAndRequantize", WithBiasReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedMatMulWithBiasAndRequantize", WithBiasReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("QuantizedMatMulWithBiasAndReluAndRequantize", WithBiasReluReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedMatMulWithBiasAndReluAndRequantize", WithBiasReluReq, 9, 3, 0x1f8u, 0x6u);
ITEXB_REGISTER_OP("QuantizedMatMulWithBiasAndDequantize", WithBiasDeq, 9, 1, 0x1f8u, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizedMatMulWithBiasAndDequantize", WithBiasDeq, 9, 1, 0x1f8u, 0x0u);

struct FusedV1 : QuantizedMatMulOp { FusedV1() : QuantizedMatMulOp(false, Tail::kNone, Flavor::kFusedV1) {} };
struct FusedV1Req : QuantizedMatMulOp { FusedV1Req() : QuantizedMatMulOp(false, Tail::kRequantize, Flavor::kFusedV1) {} };
struct FusedV1Deq : QuantizedMatMulOp { FusedV1Deq() : QuantizedMatMulOp(false, Tail::kDequantize, Flavor::kFusedV1) {} };
struct MatMulV2 : QuantizedMatMulOp { MatMulV2() : QuantizedMatMulOp(false, Tail::kNone, Flavor::kV2) {} };

// The fused ops take a variable number of inputs (bias and addend are optional), so the registered
// count is the maximum and the host masks cover every position a range can occupy: the op checks,
// per call, that the tensors it reads as ranges are in host memory.
ITEXB_REGISTER_OP("_QuantizedFusedMatMul", FusedV1, -1, 3, 0u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedFusedMatMul", FusedV1, -1, 3, 0u, 0x6u);
ITEXB_REGISTER_OP("_QuantizedFusedMatMulAndRequantize", FusedV1Req, -1, 3, 0u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedFusedMatMulAndRequantize", FusedV1Req, -1, 3, 0u, 0x6u);
ITEXB_REGISTER_OP("_QuantizedFusedMatMulAndDequantize", FusedV1Deq, -1, 1, 0u, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizedFusedMatMulAndDequantize", FusedV1Deq, -1, 1, 0u, 0x0u);
ITEXB_REGISTER_OP("_QuantizedMatMul", MatMulV2, -1, -1, 0u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedMatMul", MatMulV2, -1, -1, 0u, 0x6u);

}  // namespace
}  // namespace itexb
