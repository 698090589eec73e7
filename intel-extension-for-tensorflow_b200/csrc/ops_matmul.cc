// The fused int8 matmul family: [_ITEX]QuantizedMatMulWithBias, ...AndRelu,
// ...AndRequantize, ...AndReluAndRequantize, ...AndDequantize.
//
// Attrs, input order (a, b, bias, min_a, max_a, min_b, max_b[, min_freezed_output,
// max_freezed_output]), HostMemory arguments and the type matrix follow QuantizedMatMulOp /
// QuantizedMatMulReluOp over LegacyQuantizedMatMulOpBase
// (itex/core/kernels/common/quantized_matmul_common.h:36-336, 1414-1531) and their
// registrations (itex/core/kernels/gpu/quantized_matmul.cc:35-102,
// itex/core/kernels/cpu/quantized_matmul.cc:23-62).  Where the reference builds a oneDNN
// inner-product primitive, this op packs the weight once to K-major, prepares the scaled
// bias on the device and launches one tcgen05 GEMM with the fused epilogue.
#include <cstdlib>

#include "hostmath.h"
#include "op_kernel.h"

namespace itexb {
namespace {

enum class Tail { kNone, kRequantize, kDequantize };

class QuantizedMatMulOp : public OpKernel {
 public:
  QuantizedMatMulOp(bool relu, Tail tail) : relu_(relu), tail_(tail) {}

  int Init(const AttrMap& attrs) override {
    const char* op = name().c_str();
    t1_ = ITEXB_DT_QUINT8;
    t2_ = ITEXB_DT_QINT8;
    if (attrs.Has("T1")) ITEXB_RETURN_IF_ERROR(attrs.GetType("T1", &t1_));
    if (attrs.Has("T2")) ITEXB_RETURN_IF_ERROR(attrs.GetType("T2", &t2_));
    ITEXB_REQUIRE(t1_ == ITEXB_DT_QUINT8 && t2_ == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for T1=%s, T2=%s (only quint8 x qint8 is)", op, DtypeName(t1_), DtypeName(t2_));
    tbias_ = ITEXB_DT_FLOAT;
    if (attrs.Has("Tbias")) ITEXB_RETURN_IF_ERROR(attrs.GetType("Tbias", &tbias_));
    ITEXB_REQUIRE(tbias_ == ITEXB_DT_FLOAT || tbias_ == ITEXB_DT_QINT32 || (tail_ == Tail::kDequantize && tbias_ == ITEXB_DT_BFLOAT16),
                  ITEXB_INVALID_ARGUMENT, "%s: no kernel registered for Tbias=%s", op, DtypeName(tbias_));
    toutput_ = tail_ == Tail::kNone ? ITEXB_DT_QINT32 : (tail_ == Tail::kRequantize ? ITEXB_DT_QUINT8 : ITEXB_DT_FLOAT);
    if (attrs.Has("Toutput")) ITEXB_RETURN_IF_ERROR(attrs.GetType("Toutput", &toutput_));
    bool ok = false;
    if (tail_ == Tail::kNone) ok = toutput_ == ITEXB_DT_QINT32;
    if (tail_ == Tail::kRequantize) ok = toutput_ == ITEXB_DT_QUINT8 || toutput_ == ITEXB_DT_QINT8;
    if (tail_ == Tail::kDequantize) ok = toutput_ == ITEXB_DT_FLOAT || toutput_ == ITEXB_DT_BFLOAT16 || toutput_ == ITEXB_DT_HALF;
    ITEXB_REQUIRE(ok, ITEXB_INVALID_ARGUMENT, "%s: no kernel registered for Toutput=%s", op, DtypeName(toutput_));
    std::string mode = "MIN_FIRST";
    if (attrs.Has("input_quant_mode")) ITEXB_RETURN_IF_ERROR(attrs.GetString("input_quant_mode", &mode));
    if (mode == "MIN_FIRST") min_first_ = true;
    else if (mode == "SCALED") min_first_ = false;
    else return SetError(ITEXB_INVALID_ARGUMENT, "Quantization mode must be either MIN_FIRST or SCALED, but received %s", mode.c_str());
    is_weight_const_ = true;
    if (attrs.Has("is_weight_const")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("is_weight_const", &is_weight_const_));
    transpose_a_ = transpose_b_ = false;
    if (attrs.Has("transpose_a")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("transpose_a", &transpose_a_));
    if (attrs.Has("transpose_b")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("transpose_b", &transpose_b_));
    // How the SCALED-mode float bias is treated.  "literal" multiplies it by
    // 255*127/(range_input*range_weight) exactly as the reference lines 602-634 do;
    // "intended" leaves it in real units (what y = scale*acc + bias needs).
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
    const int nin = tail_ == Tail::kNone ? 7 : 9;
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, nin, op));
    for (int i = 0; i < 3; ++i) ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, i, op, i == 0 ? "a" : (i == 1 ? "b" : "bias")));
    const itexb_tensor_t& a = ctx->inputs[0];
    const itexb_tensor_t& b = ctx->inputs[1];
    const itexb_tensor_t& bias = ctx->inputs[2];
    ITEXB_REQUIRE(a.dtype == t1_ && b.dtype == t2_, ITEXB_INVALID_ARGUMENT, "%s: a/b have types %s/%s, attrs say %s/%s", op,
                  DtypeName(a.dtype), DtypeName(b.dtype), DtypeName(t1_), DtypeName(t2_));
    ITEXB_REQUIRE(bias.dtype == tbias_, ITEXB_INVALID_ARGUMENT, "%s: bias has type %s, Tbias is %s", op, DtypeName(bias.dtype),
                  DtypeName(tbias_));
    ITEXB_REQUIRE(a.rank == 2 && b.rank == 2, ITEXB_INVALID_ARGUMENT, "%s: a and b must be matrices", op);
    const int64_t m = transpose_a_ ? a.dims[1] : a.dims[0];
    const int64_t k = transpose_a_ ? a.dims[0] : a.dims[1];
    const int64_t kb = transpose_b_ ? b.dims[1] : b.dims[0];
    const int64_t n = transpose_b_ ? b.dims[0] : b.dims[1];
    ITEXB_REQUIRE(k == kb, ITEXB_INVALID_ARGUMENT, "Matrix size-incompatible: In[0]: [%lld,%lld], In[1]: [%lld,%lld]",
                  (long long)a.dims[0], (long long)a.dims[1], (long long)b.dims[0], (long long)b.dims[1]);
    ITEXB_REQUIRE(bias.rank == 1 && bias.dims[0] == n, ITEXB_INVALID_ARGUMENT, "%s: bias must be a vector of %lld elements", op,
                  (long long)n);
    ITEXB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31) && k > 0, ITEXB_INVALID_ARGUMENT, "%s: dimension out of range", op);
    const float *pmin_a, *pmax_a, *pmin_b, *pmax_b;
    int64_t c1, c2, nb_min, nb_max;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 3, op, "min_a", &pmin_a, &c1));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 4, op, "max_a", &pmax_a, &c2));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 5, op, "min_b", &pmin_b, &nb_min));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 6, op, "max_b", &pmax_b, &nb_max));
    ITEXB_REQUIRE(nb_min == nb_max && (nb_min == 1 || nb_min == n), ITEXB_INVALID_ARGUMENT,
                  "%s: min_b/max_b must be scalars or vectors of %lld elements", op, (long long)n);
    const float min_a = pmin_a[0], max_a = pmax_a[0];
    float min_freezed = 0.f, max_freezed = 0.f;
    if (tail_ != Tail::kNone) {
      const float *p7, *p8;
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 7, op, "min_freezed_output", &p7, &c1));
      ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 8, op, "max_freezed_output", &p8, &c2));
      min_freezed = p7[0];
      max_freezed = p8[0];
    }

    // ---- outputs
    itexb_tensor_t dst;
    const int64_t out_dims[2] = {m, n};
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, toutput_, out_dims, 2, false, &dst));
    if (tail_ != Tail::kDequantize) {
      itexb_tensor_t omin, omax;
      const bool per_channel = toutput_ == ITEXB_DT_QINT32 && ctx->inputs[5].rank != 0;
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
      ITEXB_RETURN_IF_ERROR(packed_.Ensure(ord, size_t(n) * k_pad));
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

    // ---- output scale (ExtendInt8PostOps): one scalar, from element 0 of min_b/max_b
    const float* d_scale = nullptr;
    float out_scale = 1.f;
    if (toutput_ != ITEXB_DT_QINT32) {
      out_scale = hostmath::MatMulOutputScale(min_a, max_a, pmin_b[0], pmax_b[0], toutput_, min_freezed, max_freezed);
      ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ord, st, &out_scale, 1, &d_scale));
    }

    // ---- scaled bias (GetScaledBias), cached like the reference: constant bias and weight,
    //      and an input range within 1e-5 of the one it was computed for
    const bool reuse_bias = bias_valid_ && is_weight_const_ && bias_from_ == bias.data && std::abs(min_a - saved_min_a_) < 1e-5f &&
                            std::abs(max_a - saved_max_a_) < 1e-5f && saved_out_scale_ == out_scale;
    if (!reuse_bias) {
      ITEXB_RETURN_IF_ERROR(scaled_bias_.Ensure(ord, size_t(n) * sizeof(float)));
      const float range_input = min_first_ ? max_a - min_a : std::max(std::abs(min_a), std::abs(max_a));
      std::vector<float> s(nb_min);
      for (int64_t i = 0; i < nb_min; ++i) {
        const float range_weight = std::max(std::abs(pmin_b[i]), std::abs(pmax_b[i]));
        s[i] = tbias_ == ITEXB_DT_QINT32 ? (range_input * range_weight) / (255.0f * 127.0f)
                                          : (255.0f * 127.0f) / (range_input * range_weight);
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
          else if (out_int8) { mode = kBiasMul; f = d_scale; f_count = 1; }
          else mode = kBiasCopy;
        } else {
          mode = kBiasMul; f = d_s; f_count = int(nb_min);
        }
      } else if (min_first_) {
        if (!colsum_valid_) {
          ITEXB_RETURN_IF_ERROR(colsum_.Ensure(ord, size_t(n) * sizeof(int32_t)));
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
        qmin = 255.0f * min_a / range_input;
        f = d_s; f_count = int(nb_min);
        if (out_float) mode = kBiasMinFirstFloat;
        else if (out_int8) { mode = kBiasMinFirstInt8; g = d_scale; g_count = 1; }
        else mode = kBiasMinFirstS32;
      } else if (literal_scaled_bias_) {
        mode = kBiasMul; f = d_s; f_count = int(nb_min);
      } else {
        mode = kBiasCopy;
      }
      ITEXB_RETURN_IF_ERROR(LaunchBiasPrep(mode, bias.data, tbias_, colsum, f, f_count, g, g_count, qmin,
                                           static_cast<float*>(scaled_bias_.data()), int(n), st));
      bias_valid_ = true;
      bias_from_ = bias.data;
      saved_min_a_ = min_a;
      saved_max_a_ = max_a;
      saved_out_scale_ = out_scale;
    }

    // ---- the GEMM
    itexb_gemm_params_t p{};
    p.m = int(m); p.n = int(n); p.k = int(k);
    p.a_dtype = t1_; p.b_dtype = t2_; p.out_dtype = toutput_;
    p.a = a_ptr; p.lda = lda;
    p.b = w_ptr; p.ldb = ldb;
    p.out = dst.data; p.ldo = n;
    p.ep.scale = d_scale;
    p.ep.scale_count = d_scale != nullptr ? 1 : 0;
    p.ep.bias = static_cast<const float*>(scaled_bias_.data());
    p.ep.relu = relu_ ? 1 : 0;
    return itexb_gemm(&p, ctx->stream);
  }

 private:
  const bool relu_;
  const Tail tail_;
  int t1_ = ITEXB_DT_QUINT8, t2_ = ITEXB_DT_QINT8, tbias_ = ITEXB_DT_FLOAT, toutput_ = ITEXB_DT_QINT32;
  bool min_first_ = true, is_weight_const_ = true, transpose_a_ = false, transpose_b_ = false, literal_scaled_bias_ = true;
  // weight cache (plays WeightCacheManager's role) and derived per-weight data
  DeviceBuffer packed_, colsum_, scaled_bias_;
  const void* packed_from_ = nullptr;
  int64_t packed_k_ = 0, packed_n_ = 0;
  bool colsum_valid_ = false, bias_valid_ = false;
  const void* bias_from_ = nullptr;
  float saved_min_a_ = 0.f, saved_max_a_ = 0.f, saved_out_scale_ = 0.f;
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

}  // namespace
}  // namespace itexb
