// Batched int8 matmul with dequantized output: the attention products of a quantized transformer
// (scores = Q x K^T scaled and masked, context = probabilities x V).
//
//   _[ITEX]QuantizedBatchMatMulV2AndDequantize       x, y, min_x, max_x, min_y, max_y
//   _[ITEX]QuantizedFusedBatchMatMulV2AndDequantize  x, y, args[num_args], min_x, max_x, min_y, max_y;
//                                                    fused_ops = [] | [Mul] | [Add] | [Mul, Add]
//   _[ITEX]QuantizedBatchMatMul                      device_inputs (x, y, args...), host_inputs (the ranges);
//                                                    fused_ops = [Mul][, Add], Dequantize
//
// QuantizedBatchMatMulV2Op (itex/core/kernels/common/batch_matmul_op.h:441-522) on BatchMatMulOp (:40-438); GPU
// registrations qint8 x qint8 -> float | bfloat16 | half, ranges in host memory
// (itex/core/kernels/gpu/matmul_op.cc:612-654).  Output = acc * range_x*range_y/(127*127), then the fused
// binary ops in order: Mul by a scalar tensor, Add of a tensor that broadcasts to the output.
//
// Lowering: one batched tcgen05 GEMM launch.  x is used in place when its rows are K-contiguous with a
// TMA-legal pitch (adj_x = false, K % 16 == 0); y likewise when adj_y = true.  Otherwise the operand is
// transposed / re-pitched per batch into a temporary by one batched pack launch.  The Mul scalar stays on the
// device: the kernel multiplies it with the dequantize scale (alpha_a * alpha_b), so the op never waits for it.
// The scalar product is formed first, i.e. acc * (scale * mul) where the reference's post-op chain computes
// (acc * scale) * mul: the two differ by at most one rounding of the scale product.
// An addend of the output's shape is read by the GEMM epilogue directly; any other broadcastable shape is
// expanded to the output's shape first.
#include <algorithm>
#include <cmath>

#include "hostmath.h"
#include "op_kernel.h"

namespace itexb {
namespace {

class QuantizedBatchMatMulOp : public OpKernel {
 public:
  explicit QuantizedBatchMatMulOp(bool v2) : v2_(v2) {}

  int Init(const AttrMap& attrs) override {
    const char* op = name().c_str();
    t1_ = t2_ = ITEXB_DT_QINT8;
    if (attrs.Has("T1")) ITEXB_RETURN_IF_ERROR(attrs.GetType("T1", &t1_));
    if (attrs.Has("T2")) ITEXB_RETURN_IF_ERROR(attrs.GetType("T2", &t2_));
    ITEXB_REQUIRE(t1_ == ITEXB_DT_QINT8 && t2_ == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for T1=%s, T2=%s (only qint8 x qint8 is)", op, DtypeName(t1_), DtypeName(t2_));
    toutput_ = ITEXB_DT_FLOAT;
    const char* out_attr = v2_ ? "Tout" : "Toutput";
    if (attrs.Has(out_attr)) ITEXB_RETURN_IF_ERROR(attrs.GetType(out_attr, &toutput_));
    ITEXB_REQUIRE(toutput_ == ITEXB_DT_FLOAT || toutput_ == ITEXB_DT_BFLOAT16 || toutput_ == ITEXB_DT_HALF, ITEXB_INVALID_ARGUMENT,
                  "%s: no kernel registered for %s=%s", op, out_attr, DtypeName(toutput_));
    adj_x_ = adj_y_ = false;
    if (attrs.Has("adj_x")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("adj_x", &adj_x_));
    if (attrs.Has("adj_y")) ITEXB_RETURN_IF_ERROR(attrs.GetBool("adj_y", &adj_y_));
    std::vector<std::string> fused;
    if (attrs.Has("fused_ops")) ITEXB_RETURN_IF_ERROR(attrs.GetStringList("fused_ops", &fused));
    int64_t num_args = -1;
    if (!v2_ && attrs.Has("num_args")) ITEXB_RETURN_IF_ERROR(attrs.GetInt("num_args", &num_args));
    has_mul_ = has_add_ = false;
    bool dequantize = false;
    int binaries = 0;
    for (const std::string& f : fused) {
      if (f == "Mul") {
        ITEXB_REQUIRE(!has_mul_ && !has_add_, ITEXB_UNIMPLEMENTED, "%s: fused_ops supports one Mul, before the Add", op);
        has_mul_ = true;
        ++binaries;
      } else if (f == "Add") {
        ITEXB_REQUIRE(!has_add_, ITEXB_UNIMPLEMENTED, "%s: fused_ops supports one Add", op);
        has_add_ = true;
        ++binaries;
      } else if (v2_ && f == "Dequantize") {
        dequantize = true;
      } else {
        return SetError(ITEXB_UNIMPLEMENTED, "Fusion is not implemented for QuantizedBatchMatMul: [%s]", f.c_str());
      }
    }
    if (v2_) {
      ITEXB_REQUIRE(dequantize, ITEXB_UNIMPLEMENTED, "%s: fused_ops must end in Dequantize (quantized outputs are not registered)", op);
      // the reference counts every fused_ops entry (Dequantize included) when it locates the ranges
      first_range_ = int(fused.size()) + 1;
    } else {
      ITEXB_REQUIRE(num_args < 0 || num_args == binaries, ITEXB_INVALID_ARGUMENT,
                    "_QuantizedFusedBatchMatMulV2AndDequantize should have same number of additional inputs as the number of fusions");
      first_range_ = 2 + binaries;
    }
    ITEXB_REQUIRE(first_range_ == 2 + binaries, ITEXB_INVALID_ARGUMENT, "%s: fused_ops and the input list disagree", op);
    return ITEXB_OK;
  }

  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    const int nin = first_range_ + 4;
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, nin, op));
    for (int i = 0; i < first_range_; ++i) ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, i, op, i == 0 ? "x" : (i == 1 ? "y" : "args")));
    const itexb_tensor_t& x = ctx->inputs[0];
    const itexb_tensor_t& y = ctx->inputs[1];
    ITEXB_REQUIRE(x.dtype == t1_ && y.dtype == t2_, ITEXB_INVALID_ARGUMENT, "%s: x/y have types %s/%s, attrs say %s/%s", op,
                  DtypeName(x.dtype), DtypeName(y.dtype), DtypeName(t1_), DtypeName(t2_));
    ITEXB_REQUIRE(x.rank >= 2 && y.rank >= 2, ITEXB_INVALID_ARGUMENT, "%s: x and y must have rank >= 2", op);
    int64_t d0 = x.dims[x.rank - 2], d1 = x.dims[x.rank - 1], d2 = y.dims[y.rank - 2], d3 = y.dims[y.rank - 1];
    if (adj_x_) std::swap(d0, d1);
    if (adj_y_) std::swap(d2, d3);
    ITEXB_REQUIRE(d1 == d2, ITEXB_INVALID_ARGUMENT, "Input[0] mismatch Input[1] shape :%lld vs. %lld", (long long)d1, (long long)d2);
    const int64_t m = d0, k = d1, n = d3;

    // ---- batch dims: numpy broadcast of the leading dims (MatMulBCast)
    const int xb = x.rank - 2, yb = y.rank - 2, ob = std::max(xb, yb);
    ITEXB_REQUIRE(ob + 2 <= ITEXB_MAX_DIMS, ITEXB_INVALID_ARGUMENT, "%s: rank out of range", op);
    int64_t out_dims[ITEXB_MAX_DIMS];
    int64_t x_batch = 1, y_batch = 1, o_batch = 1;
    for (int d = 0; d < ob; ++d) {
      const int64_t ex = d - (ob - xb) >= 0 ? x.dims[d - (ob - xb)] : 1;
      const int64_t ey = d - (ob - yb) >= 0 ? y.dims[d - (ob - yb)] : 1;
      ITEXB_REQUIRE(ex == ey || ex == 1 || ey == 1, ITEXB_INVALID_ARGUMENT, "Input tensors must have compatible batch dimensions");
      out_dims[d] = std::max(ex, ey) == 1 ? 1 : (ex == 1 ? ey : ex);
      if (ex == 0 || ey == 0) out_dims[d] = 0;
      x_batch *= ex;
      y_batch *= ey;
      o_batch *= out_dims[d];
    }
    out_dims[ob] = m;
    out_dims[ob + 1] = n;
    ITEXB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31) && o_batch < (1ll << 31), ITEXB_INVALID_ARGUMENT,
                  "%s: dimension out of range", op);

    const float *pmin_x, *pmax_x, *pmin_y, *pmax_y;
    int64_t c;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, first_range_, op, "min_x", &pmin_x, &c));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, first_range_ + 1, op, "max_x", &pmax_x, &c));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, first_range_ + 2, op, "min_y", &pmin_y, &c));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, first_range_ + 3, op, "max_y", &pmax_y, &c));

    itexb_tensor_t dst;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, toutput_, out_dims, ob + 2, false, &dst));
    if (o_batch == 0 || m == 0 || n == 0) return ITEXB_OK;
    ITEXB_REQUIRE(k > 0, ITEXB_UNIMPLEMENTED, "%s: an empty inner dimension is not implemented", op);

    // How batch i of the output picks its operands.  Uniform cases need no index table:
    // both operands advance with the output, or the right one is shared by every batch.
    const bool x_full = x_batch == o_batch, y_full = y_batch == o_batch;
    ITEXB_REQUIRE((x_full && (y_full || y_batch == 1)) || (x_batch == 1 && y_full), ITEXB_UNIMPLEMENTED,
                  "%s: batch dimensions that broadcast on both operands are not implemented", op);

    cudaStream_t st = AsCuda(ctx->stream);
    const int ord = ctx->device_ordinal;
    const int64_t k_pad = (k + 15) / 16 * 16;

    // ---- left operand as [x_batch][m][lda], K contiguous
    const void* a_ptr = x.data;
    int64_t lda = k;
    if (adj_x_) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(x_batch) * m * k_pad, false, &tmp));
      ITEXB_RETURN_IF_ERROR(PackBatched(x.data, tmp, k, m, k_pad, x_batch, ctx->stream));  // [k,m] -> [m,k_pad]
      a_ptr = tmp;
      lda = k_pad;
    } else if (k % 16 != 0 || (reinterpret_cast<uintptr_t>(x.data) & 15) != 0) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(x_batch) * m * k_pad, false, &tmp));
      if (k_pad != k) ITEXB_CUDA(cudaMemsetAsync(tmp, 0, size_t(x_batch) * m * k_pad, st));
      ITEXB_CUDA(cudaMemcpy2DAsync(tmp, k_pad, x.data, k, k, size_t(x_batch) * m, cudaMemcpyDeviceToDevice, st));
      a_ptr = tmp;
      lda = k_pad;
    }

    // ---- right operand as [y_batch][n][ldb], K contiguous
    const void* b_ptr = y.data;
    int64_t ldb = k;
    if (!adj_y_) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(y_batch) * n * k_pad, false, &tmp));
      ITEXB_RETURN_IF_ERROR(PackBatched(y.data, tmp, k, n, k_pad, y_batch, ctx->stream));  // [k,n] -> [n,k_pad]
      b_ptr = tmp;
      ldb = k_pad;
    } else if (k % 16 != 0 || (reinterpret_cast<uintptr_t>(y.data) & 15) != 0) {
      void* tmp = nullptr;
      ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(y_batch) * n * k_pad, false, &tmp));
      if (k_pad != k) ITEXB_CUDA(cudaMemsetAsync(tmp, 0, size_t(y_batch) * n * k_pad, st));
      ITEXB_CUDA(cudaMemcpy2DAsync(tmp, k_pad, y.data, k, k, size_t(y_batch) * n, cudaMemcpyDeviceToDevice, st));
      b_ptr = tmp;
      ldb = k_pad;
    }

    // ---- output scale, AccumulateMulAndInt8Scale (batch_matmul_op.h:497-514)
    const float range_lhs = std::max(std::abs(pmin_x[0]), std::abs(pmax_x[0]));
    const float range_rhs = std::max(std::abs(pmin_y[0]), std::abs(pmax_y[0]));
    const float scale_output = range_lhs * range_rhs / (127.0f * 127.0f);
    const float* d_scale = nullptr;
    ITEXB_RETURN_IF_ERROR(scale_cache_.Get(ord, st, &scale_output, 1, &d_scale));

    // ---- fused binaries
    int arg = 2;
    const float* d_mul = nullptr;
    if (has_mul_) {
      const itexb_tensor_t& t = ctx->inputs[arg++];
      ITEXB_REQUIRE(NumElements(t) == 1, ITEXB_UNIMPLEMENTED, "%s: the Mul operand must be a scalar tensor", op);
      ITEXB_REQUIRE(t.dtype == ITEXB_DT_FLOAT || t.dtype == ITEXB_DT_BFLOAT16 || t.dtype == ITEXB_DT_HALF, ITEXB_INVALID_ARGUMENT,
                    "%s: the Mul operand has type %s", op, DtypeName(t.dtype));
      if (t.dtype == ITEXB_DT_FLOAT) {
        d_mul = static_cast<const float*>(t.data);
      } else {
        ITEXB_RETURN_IF_ERROR(mul_f32_.Ensure(ord, sizeof(float), st));
        ITEXB_RETURN_IF_ERROR(LaunchBiasPrep(kBiasCopy, t.data, t.dtype, nullptr, nullptr, 0, nullptr, 0, 0.f,
                                             static_cast<float*>(mul_f32_.data()), 1, st));
        d_mul = static_cast<const float*>(mul_f32_.data());
      }
    }
    const void* addend = nullptr;
    if (has_add_) {
      const itexb_tensor_t& t = ctx->inputs[arg++];
      ITEXB_REQUIRE(t.dtype == toutput_, ITEXB_INVALID_ARGUMENT, "%s: the Add operand has type %s, the output %s", op, DtypeName(t.dtype),
                    DtypeName(toutput_));
      ITEXB_REQUIRE(NumElements(t) == 1 || t.rank >= 3, ITEXB_INVALID_ARGUMENT,
                    "Binary input of FusedBatchMatMul must be scalar or have 3 dims at least, but got %d", t.rank);
      ITEXB_REQUIRE(t.rank <= ob + 2, ITEXB_INVALID_ARGUMENT, "%s: the Add operand has more dims than the output", op);
      bool same = t.rank == ob + 2;
      for (int d = 0; same && d < t.rank; ++d) same = t.dims[d] == out_dims[d];
      if (same) {
        addend = t.data;
      } else {
        const int eb = toutput_ == ITEXB_DT_FLOAT ? 4 : 2;
        void* tmp = nullptr;
        ITEXB_RETURN_IF_ERROR(AllocateTemp(ctx, size_t(o_batch) * m * n * eb, false, &tmp));
        ITEXB_RETURN_IF_ERROR(LaunchBroadcast(t.data, t.dims, NumElements(t) == 1 ? 0 : t.rank, tmp, out_dims, ob + 2, eb, st));
        addend = tmp;
      }
    }

    // ---- one GEMM launch.  A right operand shared by all batches folds the batch into the rows.
    itexb_gemm_params_t p{};
    p.status_word = StatusWord(ord, st);
    p.a_dtype = t1_; p.b_dtype = t2_; p.out_dtype = toutput_;
    p.k = int(k); p.n = int(n);
    p.a = a_ptr; p.lda = lda;
    p.b = b_ptr; p.ldb = ldb;
    p.out = dst.data; p.ldo = n;
    if (has_mul_) { p.ep.alpha_a = d_scale; p.ep.alpha_b = d_mul; }
    else { p.ep.scale = d_scale; p.ep.scale_count = 1; }
    if (addend != nullptr) {
      p.ep.summand = addend;
      p.ep.summand_dtype = toutput_;
      p.ep.ld_summand = n;
      p.ep.sum_scale = 1.f;
    }
    if (x_full && y_batch == 1) {
      ITEXB_REQUIRE(o_batch * m < (1ll << 31), ITEXB_INVALID_ARGUMENT, "%s: dimension out of range", op);
      p.m = int(o_batch * m);
      return itexb_gemm(&p, ctx->stream);
    }
    p.m = int(m);
    if (x_full && y_full) {
      if (o_batch > 1) {
        p.batch = int(o_batch);
        p.stride_a = m * lda;
        p.stride_b = n * ldb;
        p.stride_out = m * n;
      }
      return itexb_gemm(&p, ctx->stream);
    }
    // the left operand is shared: one launch per batch of the right operand
    const int es = toutput_ == ITEXB_DT_FLOAT ? 4 : 2;
    for (int64_t i = 0; i < o_batch; ++i) {
      itexb_gemm_params_t q = p;
      q.b = static_cast<const uint8_t*>(b_ptr) + i * n * ldb;
      q.out = static_cast<uint8_t*>(dst.data) + i * m * n * es;
      if (addend != nullptr) q.ep.summand = static_cast<const uint8_t*>(addend) + i * m * n * es;
      ITEXB_RETURN_IF_ERROR(itexb_gemm(&q, ctx->stream));
    }
    return ITEXB_OK;
  }

 private:
  // [batch][rows_in = k][cols_in = n] -> [batch][n][k_pad]; grid.z carries the batch in chunks of 65535
  static int PackBatched(const void* src, void* dst, int64_t k, int64_t n, int64_t k_pad, int64_t batch, itexb_stream_t stream) {
    for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
      const int64_t nb = std::min<int64_t>(65535, batch - b0);
      ITEXB_RETURN_IF_ERROR(itexb_pack_weights_kn_batched(static_cast<const uint8_t*>(src) + b0 * k * n,
                                                          static_cast<uint8_t*>(dst) + b0 * n * k_pad, k, n, k_pad, nb, k * n, n * k_pad,
                                                          stream));
    }
    return ITEXB_OK;
  }

  const bool v2_;
  int t1_ = ITEXB_DT_QINT8, t2_ = ITEXB_DT_QINT8, toutput_ = ITEXB_DT_FLOAT;
  bool adj_x_ = false, adj_y_ = false, has_mul_ = false, has_add_ = false;
  int first_range_ = 2;
  DeviceVectorCache scale_cache_;
  DeviceBuffer mul_f32_;
};

struct BatchMatMulV1 : QuantizedBatchMatMulOp { BatchMatMulV1() : QuantizedBatchMatMulOp(false) {} };
struct BatchMatMulV2 : QuantizedBatchMatMulOp { BatchMatMulV2() : QuantizedBatchMatMulOp(true) {} };

// HostMemory: min_x, max_x, min_y, max_y (inputs 2..5 of the unfused op; the fused ops check per call).
ITEXB_REGISTER_OP("_QuantizedBatchMatMulV2AndDequantize", BatchMatMulV1, 6, 1, 0x3cu, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizedBatchMatMulV2AndDequantize", BatchMatMulV1, 6, 1, 0x3cu, 0x0u);
ITEXB_REGISTER_OP("_QuantizedFusedBatchMatMulV2AndDequantize", BatchMatMulV1, -1, 1, 0u, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizedFusedBatchMatMulV2AndDequantize", BatchMatMulV1, -1, 1, 0u, 0x0u);
ITEXB_REGISTER_OP("_QuantizedBatchMatMul", BatchMatMulV2, -1, 1, 0u, 0x0u);
ITEXB_REGISTER_OP("_ITEXQuantizedBatchMatMul", BatchMatMulV2, -1, 1, 0u, 0x0u);

}  // namespace
}  // namespace itexb
