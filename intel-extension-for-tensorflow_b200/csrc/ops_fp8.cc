// Fp8Quantize, Fp8Dequantize, Fp8Matmul, Fp8Gelu, Fp8LayerNorm (forward), Fp8QuantizeDbias and Fp8QuantizeDbiasDgelu.
//
// Op signatures follow itex/core/ops/fp8_ops.cc:22-61,192-226; kernels follow
// Fp8QuantizeOp / Fp8DequantizeOp (itex/core/kernels/gpu/fp8/fp8_quantize_op.cc:24-83)
// and Fp8MatmulOp (itex/core/kernels/gpu/fp8/fp8_matmul_op.cc:24-110).  FP8 bytes travel in
// int8 tensors; amax / scale / scale_inv are device tensors indexed by fp8_meta_index.
//
// The reference matmul dequantizes both operands into temporaries and runs a bf16/f32
// library GEMM (fp8_matmul_gpu.h:34-162).  Here the e4m3/e5m2 operands feed the tensor
// cores directly (tcgen05 kind::f8f6f4, fp32 accumulation) and the two inverse scales are
// applied once per output element in the epilogue: the same real-number sum, accumulated
// in a different order.
#include "op_kernel.h"

namespace itexb {
namespace {

int ParseFp8Dtype(const AttrMap& attrs, const char* attr, bool allow_empty, int* out) {
  std::string s;
  ITEXB_RETURN_IF_ERROR(attrs.GetString(attr, &s));
  if (s == "E4M3") *out = ITEXB_DT_FP8_E4M3;
  else if (s == "E5M2") *out = ITEXB_DT_FP8_E5M2;
  else if (s.empty() && allow_empty) *out = ITEXB_DT_INVALID;
  else return SetError(ITEXB_INVALID_ARGUMENT, "Unsupported fp8_dtype: %s", s.c_str());
  return ITEXB_OK;
}

bool IsFloatType(int dt) { return dt == ITEXB_DT_FLOAT || dt == ITEXB_DT_BFLOAT16 || dt == ITEXB_DT_HALF; }

int MetaPointer(const itexb_op_context_t* ctx, int input, int index, const char* op, const char* arg, float** p) {
  const itexb_tensor_t& t = ctx->inputs[input];
  ITEXB_REQUIRE(!t.on_host && t.dtype == ITEXB_DT_FLOAT, ITEXB_INVALID_ARGUMENT, "%s: '%s' must be a float tensor in device memory", op, arg);
  ITEXB_REQUIRE(index >= 0 && index < NumElements(t), ITEXB_INVALID_ARGUMENT, "%s: fp8_meta_index %d is out of range for '%s' (%lld elements)",
                op, index, arg, (long long)NumElements(t));
  *p = static_cast<float*>(t.data) + index;
  return ITEXB_OK;
}

class Fp8QuantizeOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    int64_t idx;
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index", &idx));
    index_ = int(idx);
    return ParseFp8Dtype(attrs, "fp8_dtype", false, &fp8_dtype_);
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 3, op));
    const itexb_tensor_t& x = ctx->inputs[0];
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "x"));
    ITEXB_REQUIRE(IsFloatType(x.dtype), ITEXB_INVALID_ARGUMENT, "%s: x must be float, bfloat16 or half", op);
    float *amax, *scale;
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 1, index_, op, "x_amax", &amax));
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 2, index_, op, "x_scale", &scale));
    itexb_tensor_t y;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, ITEXB_DT_INT8, x.dims, x.rank, false, &y));
    return itexb_fp8_quantize(x.data, x.dtype, y.data, fp8_dtype_, NumElements(x), scale, amax, ctx->stream);
  }

 private:
  int index_ = 0, fp8_dtype_ = ITEXB_DT_FP8_E4M3;
};

// Fp8Gelu(inp, amax, scale) -> gelu_out: GELU fused with the FP8 cast (itex/core/kernels/gpu/fp8/fp8_gelu_op.cc:25-64,
// op definition itex/core/ops/fp8_ops.cc:124-141).
class Fp8GeluOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    int64_t idx;
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index", &idx));
    index_ = int(idx);
    return ParseFp8Dtype(attrs, "fp8_dtype", false, &fp8_dtype_);
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 3, op));
    const itexb_tensor_t& x = ctx->inputs[0];
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "inp"));
    ITEXB_REQUIRE(IsFloatType(x.dtype), ITEXB_INVALID_ARGUMENT, "%s: inp must be float, bfloat16 or half", op);
    float *amax, *scale;
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 1, index_, op, "amax", &amax));
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 2, index_, op, "scale", &scale));
    itexb_tensor_t y;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, ITEXB_DT_INT8, x.dims, x.rank, false, &y));
    return itexb_fp8_gelu(x.data, x.dtype, y.data, fp8_dtype_, NumElements(x), scale, amax, ctx->stream);
  }

 private:
  int index_ = 0, fp8_dtype_ = ITEXB_DT_FP8_E4M3;
};

// Fp8LayerNorm(x, gamma, beta, z_amax, z_scale) -> z, mu, rsigma (itex/core/kernels/gpu/fp8/fp8_layernorm_op.cc:24-83,
// op definition itex/core/ops/fp8_ops.cc:63-88).  out_dtype int8 = FP8 bytes in the fp8_dtype format; a real out_dtype
// gives the plain normalisation and ignores z_amax / z_scale.
class Fp8LayerNormOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    int64_t idx;
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index", &idx));
    index_ = int(idx);
    epsilon_ = 1e-4f;
    if (attrs.Has("epsilon")) ITEXB_RETURN_IF_ERROR(attrs.GetFloat("epsilon", &epsilon_));
    out_dtype_ = ITEXB_DT_INT8;
    if (attrs.Has("out_dtype")) ITEXB_RETURN_IF_ERROR(attrs.GetType("out_dtype", &out_dtype_));
    ITEXB_REQUIRE(out_dtype_ == ITEXB_DT_INT8 || IsFloatType(out_dtype_), ITEXB_INVALID_ARGUMENT,
                  "%s: out_dtype must be int8 (FP8 bytes), float, bfloat16 or half", name().c_str());
    return ParseFp8Dtype(attrs, "fp8_dtype", false, &fp8_dtype_);
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 5, op));
    for (int i = 0; i < 3; ++i) ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, i, op, i == 0 ? "x" : (i == 1 ? "gamma" : "beta")));
    const itexb_tensor_t& x = ctx->inputs[0];
    const itexb_tensor_t& gamma = ctx->inputs[1];
    const itexb_tensor_t& beta = ctx->inputs[2];
    ITEXB_REQUIRE(x.rank == 2 && IsFloatType(x.dtype), ITEXB_INVALID_ARGUMENT, "%s: x must be a float, bfloat16 or half matrix", op);
    ITEXB_REQUIRE(gamma.dtype == beta.dtype && IsFloatType(gamma.dtype) && NumElements(gamma) == x.dims[1] && NumElements(beta) == x.dims[1],
                  ITEXB_INVALID_ARGUMENT, "%s: gamma and beta must be vectors of %lld elements of one real type", op, (long long)x.dims[1]);
    float *amax = nullptr, *scale = nullptr;
    if (out_dtype_ == ITEXB_DT_INT8) {
      ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 3, index_, op, "z_amax", &amax));
      ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 4, index_, op, "z_scale", &scale));
    }
    itexb_tensor_t z, mu, rs;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, out_dtype_, x.dims, 2, false, &z));
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, x.dims, 1, false, &mu));
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, x.dims, 1, false, &rs));
    return itexb_fp8_layernorm(x.data, x.dtype, gamma.data, beta.data, gamma.dtype, z.data,
                               out_dtype_ == ITEXB_DT_INT8 ? fp8_dtype_ : out_dtype_, static_cast<float*>(mu.data),
                               static_cast<float*>(rs.data), x.dims[0], x.dims[1], epsilon_, scale, amax, ctx->stream);
  }

 private:
  int index_ = 0, fp8_dtype_ = ITEXB_DT_FP8_E4M3, out_dtype_ = ITEXB_DT_INT8;
  float epsilon_ = 1e-4f;
};

class Fp8DequantizeOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    int64_t idx;
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index", &idx));
    index_ = int(idx);
    out_dtype_ = ITEXB_DT_FLOAT;
    if (attrs.Has("out_dtype")) ITEXB_RETURN_IF_ERROR(attrs.GetType("out_dtype", &out_dtype_));
    ITEXB_REQUIRE(IsFloatType(out_dtype_), ITEXB_INVALID_ARGUMENT, "%s: out_dtype must be float, bfloat16 or half", name().c_str());
    return ParseFp8Dtype(attrs, "fp8_dtype", false, &fp8_dtype_);
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 2, op));
    const itexb_tensor_t& x = ctx->inputs[0];
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "x"));
    ITEXB_REQUIRE(x.dtype == ITEXB_DT_INT8, ITEXB_INVALID_ARGUMENT, "%s: x must be int8 (fp8 bytes)", op);
    float* scale_inv;
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 1, index_, op, "x_scale_inv", &scale_inv));
    itexb_tensor_t y;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, out_dtype_, x.dims, x.rank, false, &y));
    return itexb_fp8_dequantize(x.data, fp8_dtype_, y.data, out_dtype_, NumElements(x), scale_inv, ctx->stream);
  }

 private:
  int index_ = 0, fp8_dtype_ = ITEXB_DT_FP8_E4M3, out_dtype_ = ITEXB_DT_FLOAT;
};

class Fp8MatmulOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    const char* op = name().c_str();
    int64_t ia, ib, ic = -1;
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index_a", &ia));
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index_b", &ib));
    if (attrs.Has("fp8_meta_index_c")) ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index_c", &ic));
    ia_ = int(ia); ib_ = int(ib); ic_ = int(ic);
    ITEXB_RETURN_IF_ERROR(ParseFp8Dtype(attrs, "fp8_dtype_a", false, &dt_a_));
    ITEXB_RETURN_IF_ERROR(ParseFp8Dtype(attrs, "fp8_dtype_b", false, &dt_b_));
    dt_c_ = ITEXB_DT_INVALID;
    if (attrs.Has("fp8_dtype_c")) ITEXB_RETURN_IF_ERROR(ParseFp8Dtype(attrs, "fp8_dtype_c", true, &dt_c_));
    if (attrs.Has("transpose_a")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("transpose_a", &transpose_a_));
    if (attrs.Has("transpose_b")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("transpose_b", &transpose_b_));
    ITEXB_RETURN_IF_ERROR(attrs.GetBool("use_bias", &use_bias_));
    if (attrs.Has("has_post_add")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("has_post_add", &has_post_add_));
    sum_dtype_ = ITEXB_DT_FLOAT;
    if (attrs.Has("sum_dtype")) ITEXB_RETURN_IF_ERROR(attrs.GetType("sum_dtype", &sum_dtype_));
    out_dtype_ = sum_dtype_;
    if (attrs.Has("out_dtype")) ITEXB_RETURN_IF_ERROR(attrs.GetType("out_dtype", &out_dtype_));
    // registered combinations: (sum, out) in {(f32,int8),(f32,f32),(bf16,int8),(bf16,bf16)}, fp8_matmul_op.cc:100-110
    ITEXB_REQUIRE(sum_dtype_ == ITEXB_DT_FLOAT || sum_dtype_ == ITEXB_DT_BFLOAT16, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for sum_dtype=%s", op, DtypeName(sum_dtype_));
    ITEXB_REQUIRE(out_dtype_ == sum_dtype_ || out_dtype_ == ITEXB_DT_INT8, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for sum_dtype=%s, out_dtype=%s", op, DtypeName(sum_dtype_), DtypeName(out_dtype_));
    if (out_dtype_ == ITEXB_DT_INT8)
      ITEXB_REQUIRE(dt_c_ != ITEXB_DT_INVALID && ic_ >= 0, ITEXB_INVALID_ARGUMENT,
                    "%s: an fp8 output needs fp8_dtype_c and fp8_meta_index_c", op);
    return ITEXB_OK;
  }

  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 8, op));
    const itexb_tensor_t& src = ctx->inputs[0];
    const itexb_tensor_t& weight = ctx->inputs[1];
    const itexb_tensor_t& bias = ctx->inputs[2];
    const itexb_tensor_t& post_add = ctx->inputs[3];
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "src"));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 1, op, "weight"));
    ITEXB_REQUIRE(src.dtype == ITEXB_DT_INT8 && weight.dtype == ITEXB_DT_INT8, ITEXB_INVALID_ARGUMENT,
                  "%s: src and weight must be int8 (fp8 bytes)", op);
    ITEXB_REQUIRE(src.rank == 2 && weight.rank == 2, ITEXB_INVALID_ARGUMENT, "%s: src and weight must be matrices", op);
    const int64_t m = transpose_a_ ? src.dims[1] : src.dims[0];
    const int64_t k = transpose_a_ ? src.dims[0] : src.dims[1];
    const int64_t kb = transpose_b_ ? weight.dims[1] : weight.dims[0];
    const int64_t n = transpose_b_ ? weight.dims[0] : weight.dims[1];
    ITEXB_REQUIRE(k == kb, ITEXB_INVALID_ARGUMENT, "Matrix size-incompatible: In[0]: [%lld,%lld], In[1]: [%lld,%lld]",
                  (long long)src.dims[0], (long long)src.dims[1], (long long)weight.dims[0], (long long)weight.dims[1]);
    ITEXB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31) && k > 0, ITEXB_INVALID_ARGUMENT, "%s: dimension out of range", op);
    float *a_inv, *b_inv, *c_amax = nullptr, *c_scale = nullptr;
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 4, ia_, op, "a_scale_inv", &a_inv));
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 5, ib_, op, "b_scale_inv", &b_inv));
    const bool fp8_out = out_dtype_ == ITEXB_DT_INT8;
    if (fp8_out) {
      ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 6, ic_, op, "c_amax", &c_amax));
      ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 7, ic_, op, "c_scale", &c_scale));
    }
    itexb_tensor_t dst;
    const int64_t out_dims[2] = {m, n};
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, out_dtype_, out_dims, 2, false, &dst));
    if (m == 0 || n == 0) return ITEXB_OK;
    cudaStream_t st = AsCuda(ctx->stream);
    const int64_t k_pad = (k + 15) / 16 * 16;

    const void* a_ptr = src.data;
    int64_t lda = k;
    if (transpose_a_) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(m) * k_pad, false, &tmp));
      ITEXB_RETURN_IF_ERROR(itexb_pack_weights_kn(src.data, tmp, k, m, k_pad, ctx->stream));
      a_ptr = tmp; lda = k_pad;
    } else if (k % 16 != 0 || (reinterpret_cast<uintptr_t>(src.data) & 15) != 0) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(m) * k_pad, false, &tmp));
      ITEXB_CUDA(cudaMemcpy2DAsync(tmp, k_pad, src.data, k, k, m, cudaMemcpyDeviceToDevice, st));
      a_ptr = tmp; lda = k_pad;
    }
    const void* b_ptr = weight.data;
    int64_t ldb = k;
    if (!transpose_b_) {
      // [k,n] -> K-major [n,k_pad]; weights are re-quantized every step, so nothing is cached
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(n) * k_pad, false, &tmp));
      ITEXB_RETURN_IF_ERROR(itexb_pack_weights_kn(weight.data, tmp, k, n, k_pad, ctx->stream));
      b_ptr = tmp; ldb = k_pad;
    } else if (k % 16 != 0 || (reinterpret_cast<uintptr_t>(weight.data) & 15) != 0) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(n) * k_pad, false, &tmp));
      ITEXB_CUDA(cudaMemcpy2DAsync(tmp, k_pad, weight.data, k, k, n, cudaMemcpyDeviceToDevice, st));
      b_ptr = tmp; ldb = k_pad;
    }

    itexb_gemm_params_t p{};
    p.m = int(m); p.n = int(n); p.k = int(k);
    p.a_dtype = dt_a_; p.b_dtype = dt_b_;
    p.out_dtype = fp8_out ? dt_c_ : out_dtype_;
    p.a = a_ptr; p.lda = lda;
    p.b = b_ptr; p.ldb = ldb;
    p.out = dst.data; p.ldo = n;
    p.ep.alpha_a = a_inv;
    p.ep.alpha_b = b_inv;
    if (use_bias_) {
      ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 2, op, "bias"));
      ITEXB_REQUIRE(bias.dtype == sum_dtype_ && NumElements(bias) == n, ITEXB_INVALID_ARGUMENT,
                    "%s: bias must be %s with %lld elements", op, DtypeName(sum_dtype_), (long long)n);
      if (bias.dtype == ITEXB_DT_FLOAT) {
        p.ep.bias = static_cast<const float*>(bias.data);
      } else {
        void* tmp = nullptr;
        ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(n) * sizeof(float), false, &tmp));
        ITEXB_RETURN_IF_ERROR(LaunchBiasPrep(kBiasCopy, bias.data, bias.dtype, nullptr, nullptr, 0, nullptr, 0, 0.f,
                                             static_cast<float*>(tmp), int(n), st));
        p.ep.bias = static_cast<const float*>(tmp);
      }
    }
    if (has_post_add_) {
      ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 3, op, "post_add"));
      ITEXB_REQUIRE(post_add.dtype == sum_dtype_ && post_add.rank == 2 && post_add.dims[0] == m && post_add.dims[1] == n,
                    ITEXB_INVALID_ARGUMENT, "%s: post_add must be a %s [%lld,%lld] tensor", op, DtypeName(sum_dtype_), (long long)m,
                    (long long)n);
      p.ep.summand = post_add.data;
      p.ep.summand_dtype = post_add.dtype;
      p.ep.ld_summand = n;
      p.ep.sum_scale = 1.f;
    }
    if (fp8_out) {
      p.ep.out_scale = c_scale;
      p.ep.amax = c_amax;
      p.ep.mid_dtype = sum_dtype_ == ITEXB_DT_FLOAT ? 0 : sum_dtype_;
    }
    p.status_word = StatusWord(ctx->device_ordinal, st);
    return itexb_gemm(&p, ctx->stream);
  }

 private:
  int ia_ = 0, ib_ = 1, ic_ = -1;
  int dt_a_ = ITEXB_DT_FP8_E4M3, dt_b_ = ITEXB_DT_FP8_E4M3, dt_c_ = ITEXB_DT_INVALID;
  bool transpose_a_ = false, transpose_b_ = false, use_bias_ = false, has_post_add_ = false;
  int sum_dtype_ = ITEXB_DT_FLOAT, out_dtype_ = ITEXB_DT_FLOAT;
};

ITEXB_REGISTER_OP("Fp8Quantize", Fp8QuantizeOp, 3, 1, 0x0u, 0x0u);
ITEXB_REGISTER_OP("Fp8Dequantize", Fp8DequantizeOp, 2, 1, 0x0u, 0x0u);
ITEXB_REGISTER_OP("Fp8Matmul", Fp8MatmulOp, 8, 1, 0x0u, 0x0u);
ITEXB_REGISTER_OP("Fp8Gelu", Fp8GeluOp, 3, 1, 0x0u, 0x0u);

// Fp8QuantizeDbias(grad, amax, scale) -> quantize_out, dbias and Fp8QuantizeDbiasDgelu(grad, gelu_inp, amax, scale) ->
// dgelu, dbias (itex/core/kernels/gpu/fp8/fp8_quantize_fusion_op.cc:24-116; op definitions itex/core/ops/fp8_ops.cc:145-190).
// The reference registers them for float and bfloat16 gradients; half is accepted here as well.
class Fp8QuantizeDbiasOp : public OpKernel {
 public:
  explicit Fp8QuantizeDbiasOp(bool dgelu) : dgelu_(dgelu) {}
  int Init(const AttrMap& attrs) override {
    int64_t idx;
    ITEXB_RETURN_IF_ERROR(attrs.GetInt("fp8_meta_index", &idx));
    index_ = int(idx);
    return ParseFp8Dtype(attrs, "fp8_dtype", false, &fp8_dtype_);
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    const int base = dgelu_ ? 1 : 0;
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 3 + base, op));
    const itexb_tensor_t& grad = ctx->inputs[0];
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "grad"));
    ITEXB_REQUIRE(grad.rank == 2 && IsFloatType(grad.dtype), ITEXB_INVALID_ARGUMENT, "%s: grad must be a float, bfloat16 or half matrix", op);
    const void* gelu_inp = nullptr;
    if (dgelu_) {
      const itexb_tensor_t& x = ctx->inputs[1];
      ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 1, op, "gelu_inp"));
      ITEXB_REQUIRE(x.dtype == grad.dtype && x.rank == 2 && x.dims[0] == grad.dims[0] && x.dims[1] == grad.dims[1], ITEXB_INVALID_ARGUMENT,
                    "%s: gelu_inp must have the type and shape of grad", op);
      gelu_inp = x.data;
    }
    float *amax, *scale;
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 1 + base, index_, op, "amax", &amax));
    ITEXB_RETURN_IF_ERROR(MetaPointer(ctx, 2 + base, index_, op, "scale", &scale));
    itexb_tensor_t out, dbias;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, ITEXB_DT_INT8, grad.dims, 2, false, &out));
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, grad.dtype, &grad.dims[1], 1, false, &dbias));
    void* ws = nullptr;
    const size_t ws_bytes = itexb_fp8_quantize_dbias_workspace_bytes(grad.dims[0], grad.dims[1]);
    if (ws_bytes > 0) ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, ws_bytes, false, &ws));
    return itexb_fp8_quantize_dbias(grad.data, gelu_inp, grad.dtype, out.data, fp8_dtype_, dbias.data, grad.dims[0], grad.dims[1], scale, amax, ws,
                                    ctx->stream);
  }

 private:
  const bool dgelu_;
  int index_ = 0, fp8_dtype_ = ITEXB_DT_FP8_E5M2;
};
struct Fp8QuantizeDbias : Fp8QuantizeDbiasOp { Fp8QuantizeDbias() : Fp8QuantizeDbiasOp(false) {} };
struct Fp8QuantizeDbiasDgelu : Fp8QuantizeDbiasOp { Fp8QuantizeDbiasDgelu() : Fp8QuantizeDbiasOp(true) {} };
ITEXB_REGISTER_OP("Fp8QuantizeDbias", Fp8QuantizeDbias, 3, 2, 0x0u, 0x0u);
ITEXB_REGISTER_OP("Fp8QuantizeDbiasDgelu", Fp8QuantizeDbiasDgelu, 4, 2, 0x0u, 0x0u);
ITEXB_REGISTER_OP("Fp8LayerNorm", Fp8LayerNormOp, 5, 3, 0x0u, 0x0u);

}  // namespace
}  // namespace itexb
