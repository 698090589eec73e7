// [_ITEX]QuantizedMaxPool and [_ITEX|ITEX]QuantizedAvgPool: inputs (input, min_input*, max_input*),
// outputs (output, min_output*, max_output*), * = HostMemory; the range passes through.
// Op definition itex/core/ops/nn_ops.cc:4163-4186; kernels itex/core/kernels/cpu/maxpooling_op.cc:43-52,
// cpu/avgpooling_op.cc:50-58 (PoolingOp over oneDNN pooling_max / pooling_avg_exclude_padding).
#include "hostmath.h"
#include "op_kernel.h"

namespace itexb {
namespace {

class QuantizedPoolOp : public OpKernel {
 public:
  explicit QuantizedPoolOp(bool avg) : avg_(avg) {}
  int Init(const AttrMap& attrs) override {
    std::vector<int64_t> ksize, strides;
    ITEXB_RETURN_IF_ERROR(attrs.GetIntList("ksize", &ksize));
    ITEXB_RETURN_IF_ERROR(attrs.GetIntList("strides", &strides));
    ITEXB_REQUIRE(ksize.size() == 4, ITEXB_INVALID_ARGUMENT, "Sliding window ksize field must specify 4 dimensions");
    ITEXB_REQUIRE(strides.size() == 4, ITEXB_INVALID_ARGUMENT, "Sliding window stride field must specify 4 dimensions");
    ITEXB_REQUIRE(ksize[0] == 1 && strides[0] == 1, ITEXB_UNIMPLEMENTED, "Pooling is not yet supported on the batch dimension.");
    ITEXB_REQUIRE(ksize[3] == 1 && strides[3] == 1, ITEXB_UNIMPLEMENTED, "Pooling is not yet supported on the depth dimension.");
    ITEXB_REQUIRE(ksize[1] > 0 && ksize[2] > 0 && strides[1] > 0 && strides[2] > 0, ITEXB_INVALID_ARGUMENT,
                  "ksize and strides must be positive");
    kh_ = int(ksize[1]); kw_ = int(ksize[2]); sh_ = int(strides[1]); sw_ = int(strides[2]);
    std::string padding;
    ITEXB_RETURN_IF_ERROR(attrs.GetString("padding", &padding));
    if (padding == "VALID") padding_ = 0;
    else if (padding == "SAME") padding_ = 1;
    else return SetError(ITEXB_UNIMPLEMENTED, "%s: padding '%s' is not implemented (VALID and SAME are)", name().c_str(), padding.c_str());
    std::string fmt = "NHWC";
    if (attrs.Has("data_format")) ITEXB_RETURN_IF_ERROR(attrs.GetString("data_format", &fmt));
    ITEXB_REQUIRE(fmt == "NHWC", ITEXB_UNIMPLEMENTED, "%s: only data_format NHWC is implemented", name().c_str());
    return ITEXB_OK;
  }
  int Compute(itexb_op_context_t* ctx) override {
    const char* op = name().c_str();
    ITEXB_RETURN_IF_ERROR(RequireInputs(ctx, 3, op));
    ITEXB_RETURN_IF_ERROR(RequireDevice(ctx, 0, op, "input"));
    const itexb_tensor_t& x = ctx->inputs[0];
    ITEXB_REQUIRE(x.rank == 4, ITEXB_INVALID_ARGUMENT, "tensor_in must be 4-dimensional");
    ITEXB_REQUIRE(x.dtype == ITEXB_DT_QUINT8 || x.dtype == ITEXB_DT_QINT8, ITEXB_INVALID_ARGUMENT, "%s: input must be quint8 or qint8", op);
    const float *pmin, *pmax;
    int64_t c1, c2;
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 1, op, "min_input", &pmin, &c1));
    ITEXB_RETURN_IF_ERROR(HostFloats(ctx, 2, op, "max_input", &pmax, &c2));
    int64_t oh, ow, pt = 0, pb = 0, pl = 0, pr = 0;
    ITEXB_REQUIRE(hostmath::WindowedOutputSize(x.dims[1], kh_, 1, sh_, padding_, &oh, &pt, &pb) &&
                      hostmath::WindowedOutputSize(x.dims[2], kw_, 1, sw_, padding_, &ow, &pl, &pr) && oh > 0 && ow > 0,
                  ITEXB_INVALID_ARGUMENT, "%s: computed output size would be non-positive", op);
    itexb_tensor_t dst, omin, omax;
    const int64_t od[4] = {x.dims[0], oh, ow, x.dims[3]};
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 0, x.dtype, od, 4, false, &dst));
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 1, ITEXB_DT_FLOAT, nullptr, 0, true, &omin));
    ITEXB_RETURN_IF_ERROR(AllocateOutput(ctx, 2, ITEXB_DT_FLOAT, nullptr, 0, true, &omax));
    *static_cast<float*>(omin.data) = pmin[0];
    *static_cast<float*>(omax.data) = pmax[0];
    itexb_pool_params_t p{};
    p.n = int(x.dims[0]); p.h = int(x.dims[1]); p.w = int(x.dims[2]); p.c = int(x.dims[3]);
    p.kh = kh_; p.kw = kw_; p.stride_h = sh_; p.stride_w = sw_; p.pad_top = int(pt); p.pad_left = int(pl);
    p.oh = int(oh); p.ow = int(ow);
    p.dtype = x.dtype; p.is_avg = avg_ ? 1 : 0;
    p.x = x.data; p.out = dst.data;
    return itexb_pool2d(&p, ctx->stream);
  }

 private:
  const bool avg_;
  int kh_ = 1, kw_ = 1, sh_ = 1, sw_ = 1, padding_ = 0;
};

struct MaxPool : QuantizedPoolOp { MaxPool() : QuantizedPoolOp(false) {} };
struct AvgPool : QuantizedPoolOp { AvgPool() : QuantizedPoolOp(true) {} };

ITEXB_REGISTER_OP("QuantizedMaxPool", MaxPool, 3, 3, 0x6u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedMaxPool", MaxPool, 3, 3, 0x6u, 0x6u);
ITEXB_REGISTER_OP("QuantizedAvgPool", AvgPool, 3, 3, 0x6u, 0x6u);
ITEXB_REGISTER_OP("_ITEXQuantizedAvgPool", AvgPool, 3, 3, 0x6u, 0x6u);
ITEXB_REGISTER_OP("ITEXQuantizedAvgPool", AvgPool, 3, 3, 0x6u, 0x6u);

}  // namespace
}  // namespace itexb
