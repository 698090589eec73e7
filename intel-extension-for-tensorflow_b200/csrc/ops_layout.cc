// The data-movement ops that sit between the quantized matmuls and convolutions of an int8 graph; each passes
// its range tensors through unchanged.
//   [_ITEX]QuantizedReshape   (tensor, shape*, input_min*, input_max*) -> (output, output_min*, output_max*)
//       itex/core/kernels/common/quantized_reshape_op.h:33-200 (op definition itex/core/ops/nn_ops.cc:3266-3289)
//   _QuantizedTranspose / _ITEXQuantizedTranspose   (x, perm*, min_x*, max_x*) -> (y, min_y*, max_y*)
//       itex/core/kernels/common/transpose_op.h:197-236, gpu/transpose_op.cc:48-56 (nn_ops.cc:562-585, 3291-3314)
//   QuantizedConcatV2 / _ITEXQuantizedConcatV2   (values x N, axis*, input_mins* x N, input_maxes* x N) -> (output,
//       output_min*, output_max*)   itex/core/kernels/common/quantized_concat_op.cc:30-276 (nn_ops.cc:734-758)
// (* = HostMemory).  A TensorFlow reshape aliases its input; an output here is memory of its own, so the bytes are
// copied device to device on the op's stream.
#include <cmath>
#include <string>

#include "op_kernel.h"

namespace itexb {
namespace {

int ScalarRange(const itexb_op_context_t* ctx, int i, const char* op, const char* arg, float* v) {
  const float* p;
  int64_t n;
  ITEXB_RETURN_IF_ERROR(HostFloats(ctx, i, op, arg, &p, &n));
  ITEXB_REQUIRE(ctx->inputs[i].rank <= 1 && n == 1, ITEXB_INVALID_ARGUMENT, "%s must be a scalar or a vector of 1 element", arg);
  *v = p[0];
  return ITEXB_OK;
}

int EmitRange(itexb_op_context_t* ctx, float mn, float mx) {
  itexb_tensor_t omin, omax;
  ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, nullptr, 0, true, &omin));
  ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, nullptr, 0, true, &omax));
  *static_cast<float*>(omin.data) = mn;
  *static_cast<float*>(omax.data) = mx;
  return ITEXB_OK;
}

class QuantizedReshapeOp : public OpKernel {
 public:
  int Init(const AttrMap&) override { return ITEXB_OK; }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 4, op));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "tensor"));
    const itexb_tensor_t& x = ctx->inputs[0];
    ITEXB_REQUIRE(ctx->inputs[1].rank <= 1, ITEXB_INVALID_ARGUMENT, "sizes input must be 1-D, not rank %d", ctx->inputs[1].rank);
    std::vector<int64_t> sizes;
    ITEXB_RETURN_IF_ERROR(HostInts(ctx, 1, op, "shape", &sizes));
    ITEXB_REQUIRE(int(sizes.size()) <= ITEXB_MAX_DIMS, ITEXB_INVALID_ARGUMENT, "%s: requested rank %d exceeds %d", op, int(sizes.size()), ITEXB_MAX_DIMS);
    // the rules of the reference's ValidateSizes / Compute: one -1 is inferred, zero-sized dimensions stay out of the
    // product so that the others can still be inferred
    int64_t product = 1, dims[ITEXB_MAX_DIMS];
    int unknown = -1;
    bool sizes_has_zero = false;
    for (size_t d = 0; d < sizes.size(); ++d) {
      const int64_t sz = sizes[d];
      if (sz == -1) {
        ITEXB_REQUIRE(unknown == -1, ITEXB_INVALID_ARGUMENT, "Only one input size may be -1, not both %d and %d", unknown, int(d));
        unknown = int(d);
        dims[d] = 1;
      } else {
        ITEXB_REQUIRE(sz >= 0, ITEXB_INVALID_ARGUMENT, "Size %d must be non-negative, not %lld", int(d), (long long)sz);
        dims[d] = sz;
        if (sz == 0) sizes_has_zero = true;
        else {
          ITEXB_REQUIRE(product <= (int64_t(1) << 62) / sz, ITEXB_INVALID_ARGUMENT, "%s: the requested shape has too many elements", op);
          product *= sz;
        }
      }
    }
    const int64_t count = NumElements(x);
    if (unknown != -1) {
      int64_t input_elems = 1;
      bool input_has_zero = false;
      for (int d = 0; d < x.rank; ++d) {
        if (x.dims[d] > 0 || !sizes_has_zero) input_elems *= x.dims[d];
        else input_has_zero = true;
      }
      const int64_t missing = input_elems / product;
      if (!input_has_zero)
        ITEXB_REQUIRE(product * missing == input_elems, ITEXB_INVALID_ARGUMENT,
                      "Input to reshape is a tensor with %lld values, but the requested shape requires a multiple of %lld",
                      (long long)input_elems, (long long)product);
      dims[unknown] = missing;
    }
    int64_t out_elems = 1;
    for (size_t d = 0; d < sizes.size(); ++d) out_elems *= dims[d];
    ITEXB_REQUIRE(out_elems == count, ITEXB_INVALID_ARGUMENT,
                  "Input to reshape is a tensor with %lld values, but the requested shape has %lld", (long long)count, (long long)out_elems);
    float mn, mx;
    ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, 2, op, "input_min", &mn));
    ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, 3, op, "input_max", &mx));
    itexb_tensor_t dst;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, x.dtype, dims, int(sizes.size()), false, &dst));
    if (count > 0)
      ITEXB_CUDA(cudaMemcpyAsync(dst.data, x.data, size_t(count) * size_t(DtypeSize(x.dtype)), cudaMemcpyDeviceToDevice, AsCuda(ctx->stream)));
    return EmitRange(ctx, mn, mx);
  }
};

class QuantizedTransposeOp : public OpKernel {
 public:
  int Init(const AttrMap&) override { return ITEXB_OK; }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 4, op));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "x"));
    const itexb_tensor_t& x = ctx->inputs[0];
    ITEXB_REQUIRE(DtypeSize(x.dtype) == 1 || x.dtype == ITEXB_DT_QINT32, ITEXB_INVALID_ARGUMENT, "%s: x must be a quantized type, is %s", op,
                  DtypeName(x.dtype));
    ITEXB_REQUIRE(ctx->inputs[1].rank == 1, ITEXB_INVALID_ARGUMENT, "perm must be a vector, not rank %d", ctx->inputs[1].rank);
    std::vector<int64_t> perm;
    ITEXB_RETURN_IF_ERROR(HostInts(ctx, 1, op, "perm", &perm));
    ITEXB_REQUIRE(int(perm.size()) == x.rank, ITEXB_INVALID_ARGUMENT, "transpose expects a vector of size %d. But input(1) is a vector of size %d",
                  x.rank, int(perm.size()));
    ITEXB_REQUIRE(x.rank <= ITEXB_TRANSPOSE_MAX_RANK, ITEXB_UNIMPLEMENTED, "%s: rank %d exceeds %d", op, x.rank, ITEXB_TRANSPOSE_MAX_RANK);
    itexb_transpose_params_t p{};
    p.rank = x.rank;
    p.elem_size = DtypeSize(x.dtype);
    int64_t od[ITEXB_MAX_DIMS];
    bool seen[ITEXB_MAX_DIMS] = {};
    for (int d = 0; d < x.rank; ++d) {
      const int64_t a = perm[size_t(d)];
      ITEXB_REQUIRE(a >= 0 && a < x.rank, ITEXB_INVALID_ARGUMENT, "%lld is out of range [0 .. %d)", (long long)a, x.rank);
      seen[a] = true;
      p.dims[d] = x.dims[d];
      p.perm[d] = int32_t(a);
      od[d] = x.dims[a];
    }
    for (int d = 0; d < x.rank; ++d) {
      if (seen[d]) continue;
      std::string list;
      for (int e = 0; e < x.rank; ++e) list += (e ? "," : "") + std::to_string(perm[size_t(e)]);
      return SetError(ITEXB_INVALID_ARGUMENT, "%d is missing from {%s}.", d, list.c_str());
    }
    float mn, mx;
    ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, 2, op, "min_x", &mn));
    ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, 3, op, "max_x", &mx));
    itexb_tensor_t dst;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, x.dtype, od, x.rank, false, &dst));
    p.x = x.data;
    p.y = dst.data;
    ITEXB_RETURN_IF_ERROR(itexb_transpose(&p, ctx->stream));
    return EmitRange(ctx, mn, mx);
  }
};

class QuantizedConcatOp : public OpKernel {
 public:
  int Init(const AttrMap& attrs) override {
    if (attrs.Has("N")) {
      ITEXB_RETURN_IF_ERROR(attrs.GetInt("N", &n_attr_));
      ITEXB_REQUIRE(n_attr_ >= 2, ITEXB_INVALID_ARGUMENT, "%s: N must be at least 2", name().c_str());
    }
    return ITEXB_OK;
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    const int num_inputs = ctx->num_inputs;
    ITEXB_REQUIRE(num_inputs > 3 && (num_inputs - 1) % 3 == 0, ITEXB_INVALID_ARGUMENT,
                  "Number of values must larger than 1, but got %d", num_inputs - 1);
    const int n = (num_inputs - 1) / 3;
    ITEXB_REQUIRE(n_attr_ == 0 || n_attr_ == n, ITEXB_INVALID_ARGUMENT, "%s: %d values were passed, attr N says %lld", op, n, (long long)n_attr_);
    ITEXB_REQUIRE(ctx->inputs[n].rank == 0 || (ctx->inputs[n].rank == 1 && ctx->inputs[n].dims[0] == 1), ITEXB_INVALID_ARGUMENT,
                  "axis tensor should be a scalar integer");
    std::vector<int64_t> axis_v;
    ITEXB_RETURN_IF_ERROR(HostInts(ctx, n, op, "axis", &axis_v));
    ITEXB_REQUIRE(axis_v.size() == 1, ITEXB_INVALID_ARGUMENT, "axis tensor should be a scalar integer");
    const int64_t concat_dim = axis_v[0];
    const itexb_tensor_t& x0 = ctx->inputs[0];
    const int rank = x0.rank;
    const int axis = int(concat_dim < 0 ? concat_dim + rank : concat_dim);
    ITEXB_REQUIRE(axis >= 0 && axis < rank, ITEXB_INVALID_ARGUMENT,
                  "ConcatOp : Expected concatenating dimensions in the range [%d, %d), but got %lld", -rank, rank, (long long)concat_dim);
    ITEXB_REQUIRE(x0.dtype == ITEXB_DT_QUINT8 || x0.dtype == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT, "%s: values must be quint8 or qint8", op);
    int64_t out_axis = 0;
    bool all_empty = true;
    for (int i = 0; i < n; ++i) {
      ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, i, op, "values"));
      const itexb_tensor_t& xi = ctx->inputs[i];
      ITEXB_REQUIRE(xi.rank == rank, ITEXB_INVALID_ARGUMENT, "ConcatOp : Ranks of all input tensors should match: rank %d vs. rank %d of input %d",
                    rank, xi.rank, i);
      ITEXB_REQUIRE(xi.dtype == x0.dtype, ITEXB_INVALID_ARGUMENT, "%s: values must share one type", op);
      for (int d = 0; d < rank; ++d)
        ITEXB_REQUIRE(d == axis || xi.dims[d] == x0.dims[d], ITEXB_INVALID_ARGUMENT,
                      "ConcatOp : Dimensions of inputs should match: dimension %d is %lld in input 0 and %lld in input %d", d,
                      (long long)x0.dims[d], (long long)xi.dims[d], i);
      all_empty = all_empty && NumElements(xi) == 0;
      out_axis += xi.dims[axis];
    }
    // the reference's GPU kernel serves equal input ranges only
    float mn0, mx0;
    ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, n + 1, op, "input_mins", &mn0));
    ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, 2 * n + 1, op, "input_maxes", &mx0));
    for (int i = 1; i < n; ++i) {
      float mn, mx;
      ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, n + 1 + i, op, "input_mins", &mn));
      ITEXB_RETURN_IF_ERROR(ScalarRange(ctx, 2 * n + 1 + i, op, "input_maxes", &mx));
      ITEXB_REQUIRE(std::fabs(mn0 - mn) <= 1.0e-6f && std::fabs(mx0 - mx) <= 1.0e-6f, ITEXB_ABORTED,
                    "TODO: Not implemented the case unequal input_mins / input_maxes.");
    }
    int64_t od[ITEXB_MAX_DIMS];
    int64_t outer = 1, inner = 1;
    for (int d = 0; d < rank; ++d) {
      od[d] = d == axis ? out_axis : x0.dims[d];
      if (d < axis) outer *= x0.dims[d];
      if (d > axis) inner *= x0.dims[d];
    }
    itexb_tensor_t dst;
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, x0.dtype, od, rank, false, &dst));
    if (!all_empty && outer > 0) {
      // every input is `outer` rows of dims[axis] * inner bytes: one strided copy each
      const size_t dpitch = size_t(out_axis * inner);
      size_t col = 0;
      for (int i = 0; i < n; ++i) {
        const size_t width = size_t(ctx->inputs[i].dims[axis] * inner);
        if (width == 0) continue;
        ITEXB_RETURN_IF_ERROR(itexb_copy_rows(ctx->inputs[i].data, dst.data, outer, int64_t(width), int64_t(dpitch), int64_t(col), ctx->stream));
        col += width;
      }
    }
    return EmitRange(ctx, mn0, mx0);
  }

 private:
  int64_t n_attr_ = 0;
};

ITEXB_REGISTER_OP("QuantizedReshape", QuantizedReshapeOp, 4, 3, 0xEu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedReshape", QuantizedReshapeOp, 4, 3, 0xEu, 0x6u);
ITEXB_REGISTER_OP("_QuantizedTranspose", QuantizedTransposeOp, 4, 3, 0xEu, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedTranspose", QuantizedTransposeOp, 4, 3, 0xEu, 0x6u);
// values x N, axis, input_mins x N, input_maxes x N: the count depends on N; every input after the values is HostMemory
ITEXB_REGISTER_OP("QuantizedConcatV2", QuantizedConcatOp, -1, 3, 0u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedConcatV2", QuantizedConcatOp, -1, 3, 0u, 0x6u);

}  // namespace
}  // namespace itexb
