// Device-side preparation of the bias vector the int8 GEMM / conv epilogue adds:
// the arithmetic of GetScaledBias (itex/core/kernels/common/quantized_matmul_common.h:466-660,
// 1153-1334) and GetBiasHandle (itex/core/kernels/common/quantized_conv_ops.h:448-597) with
// their operator order, run on the op's stream so no device->host copy of bias or weights
// is needed (the reference copies both to the host and waits, :521-543).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "op_kernel.h"

namespace itexb {
namespace {

__device__ __forceinline__ float LoadBias(const void* b, int dt, int j) {
  switch (dt) {
    case ITEXB_DT_QINT32: case ITEXB_DT_INT32: return float(static_cast<const int*>(b)[j]);
    case ITEXB_DT_BFLOAT16: return __bfloat162float(static_cast<const __nv_bfloat16*>(b)[j]);
    case ITEXB_DT_HALF: return __half2float(static_cast<const __half*>(b)[j]);
    default: return static_cast<const float*>(b)[j];
  }
}

__global__ void BiasPrepKernel(int mode, const void* __restrict__ bias, int bias_dtype, const int32_t* __restrict__ colsum,
                               const float* __restrict__ f, int f_count, const float* __restrict__ g, int g_count, float qmin,
                               float* __restrict__ out, int n) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const float b = LoadBias(bias, bias_dtype, j);
  const float fj = f != nullptr ? f[f_count > 1 ? j : 0] : 1.f;
  const float gj = g != nullptr ? g[g_count > 1 ? j : 0] : 1.f;
  const float cs = colsum != nullptr ? float(colsum[j]) : 0.f;
  float r;
  switch (mode) {
    case kBiasMul: r = __fmul_rn(b, fj); break;
    case kBiasMinFirstFloat: r = __fadd_rn(b, __fdiv_rn(__fmul_rn(cs, qmin), fj)); break;
    case kBiasMinFirstInt8: r = __fadd_rn(__fmul_rn(__fmul_rn(b, fj), gj), __fmul_rn(__fmul_rn(cs, qmin), gj)); break;
    case kBiasMinFirstS32: r = __fadd_rn(__fmul_rn(b, fj), __fmul_rn(cs, qmin)); break;
    default: r = b; break;
  }
  out[j] = r;
}

}  // namespace

int LaunchBiasPrep(int mode, const void* bias, int bias_dtype, const int32_t* colsum, const float* f, int f_count, const float* g,
                   int g_count, float qmin, float* out, int n, cudaStream_t stream) {
  ITEXB_REQUIRE(bias != nullptr && out != nullptr && n > 0, ITEXB_INVALID_ARGUMENT, "bias_prep: bad arguments");
  BiasPrepKernel<<<(n + 127) / 128, 128, 0, stream>>>(mode, bias, bias_dtype, colsum, f, f_count, g, g_count, qmin, out, n);
  return CheckLaunch("BiasPrepKernel");
}

}  // namespace itexb
