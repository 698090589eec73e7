// Fp8LayerNorm forward: z = gamma * (x - mean) * rsigma + beta over the columns of a [rows, cols] matrix,
// written either as FP8 (times z_scale, with amax of the unscaled z) or as a real type; per-row mean and
// reciprocal standard deviation are returned for the backward pass.
// Arithmetic of Fp8LayerNormFwdKernel (itex/core/kernels/gpu/fp8/fp8_layernorm_gpu.h:108-257): fp32 throughout,
// two-pass variance (sum of squared differences from the mean), rsqrt(var + epsilon), amax before scaling.
// One CTA per row keeps the row in shared memory as fp32, so the input is read from HBM once (bound:
// 2-4 B read + 1-4 B written per element); the sums are reduced in a different order than the reference's
// sub-group tree, which moves results by rounding error only.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.h"
#include "fp8_cast.h"

namespace itexb {
namespace {

constexpr int kLnThreads = 256;

template <typename T> __device__ __forceinline__ float LnToFloat(T v);
template <> __device__ __forceinline__ float LnToFloat<float>(float v) { return v; }
template <> __device__ __forceinline__ float LnToFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float LnToFloat<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ void LnStore(float* p, float v) { *p = v; }
__device__ __forceinline__ void LnStore(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void LnStore(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float BlockSum(float v, float* s_red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kLnThreads / 32; ++w) t += s_red[w];
  __syncthreads();
  return t;
}

// TZ = uint8_t selects the FP8 output (E4M3 says which format), any other TZ a real-valued output.
template <typename TX, typename TW, typename TZ, bool E4M3>
__global__ void __launch_bounds__(kLnThreads) Fp8LayerNormKernel(const TX* __restrict__ x, const TW* __restrict__ gamma,
                                                                 const TW* __restrict__ beta, TZ* __restrict__ z,
                                                                 float* __restrict__ mu_out, float* __restrict__ rs_out, int cols,
                                                                 float epsilon, const float* __restrict__ z_scale,
                                                                 float* __restrict__ z_amax) {
  extern __shared__ float s_row[];
  __shared__ float s_red[kLnThreads / 32];
  const long long row = blockIdx.x;
  const TX* xr = x + row * cols;
  float sum = 0.f;
  for (int c = threadIdx.x; c < cols; c += kLnThreads) {
    const float v = LnToFloat<TX>(xr[c]);
    s_row[c] = v;
    sum += v;
  }
  const float rn = 1.f / float(cols);
  const float mu = BlockSum(sum, s_red) * rn;
  float sq = 0.f;
  for (int c = threadIdx.x; c < cols; c += kLnThreads) {
    const float d = s_row[c] - mu;
    sq += d * d;
  }
  const float rs = rsqrtf(BlockSum(sq, s_red) * rn + epsilon);
  if (threadIdx.x == 0) {
    mu_out[row] = mu;
    rs_out[row] = rs;
  }
  constexpr bool kFp8 = sizeof(TZ) == 1;
  const float scale = kFp8 ? __ldg(z_scale) : 1.f;
  float amax = 0.f;
  TZ* zr = z + row * cols;
  for (int c = threadIdx.x; c < cols; c += kLnThreads) {
    const float y = rs * (s_row[c] - mu);
    const float v = LnToFloat<TW>(gamma[c]) * y + LnToFloat<TW>(beta[c]);
    if constexpr (kFp8) {
      amax = fmaxf(amax, fabsf(v));
      zr[c] = (TZ)FloatToFp8Bits(v * scale, E4M3);
    } else {
      LnStore(zr + c, v);
    }
  }
  if constexpr (kFp8) {
    if (z_amax != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
      __syncthreads();
      if (threadIdx.x == 0) {
        float m = 0.f;
        for (int w = 0; w < kLnThreads / 32; ++w) m = fmaxf(m, s_red[w]);
        atomicMax(reinterpret_cast<int*>(z_amax), __float_as_int(m));  // m >= 0: integer order is float order
      }
    }
  }
}

template <typename TX, typename TW>
int LaunchLn(const void* x, const void* gamma, const void* beta, void* z, int z_dtype, float* mu, float* rs, int rows, int cols,
             float epsilon, const float* z_scale, float* z_amax, cudaStream_t st) {
  const size_t smem = size_t(cols) * sizeof(float);
  auto xp = static_cast<const TX*>(x);
  auto gp = static_cast<const TW*>(gamma);
  auto bp = static_cast<const TW*>(beta);
#define ITEXB_LN(TZ, E4)                                                                                                   \
  do {                                                                                                                     \
    if (smem > 48 * 1024)                                                                                                  \
      ITEXB_CUDA(cudaFuncSetAttribute(Fp8LayerNormKernel<TX, TW, TZ, E4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
    Fp8LayerNormKernel<TX, TW, TZ, E4><<<rows, kLnThreads, smem, st>>>(xp, gp, bp, static_cast<TZ*>(z), mu, rs, cols, epsilon,    \
                                                                       z_scale, z_amax);                                  \
  } while (0)
  switch (z_dtype) {
    case ITEXB_DT_FP8_E4M3: ITEXB_LN(uint8_t, true); break;
    case ITEXB_DT_FP8_E5M2: ITEXB_LN(uint8_t, false); break;
    case ITEXB_DT_FLOAT: ITEXB_LN(float, true); break;
    case ITEXB_DT_BFLOAT16: ITEXB_LN(__nv_bfloat16, true); break;
    case ITEXB_DT_HALF: ITEXB_LN(__half, true); break;
    default: return SetError(ITEXB_INVALID_ARGUMENT, "fp8_layernorm: unsupported output type %s", DtypeName(z_dtype));
  }
#undef ITEXB_LN
  return CheckLaunch("Fp8LayerNormKernel");
}

}  // namespace
}  // namespace itexb

using namespace itexb;

extern "C" int itexb_fp8_layernorm(const void* x, int x_dtype, const void* gamma, const void* beta, int w_dtype, void* z, int z_dtype,
                                   float* mu, float* rsigma, int64_t rows, int64_t cols, float epsilon, const float* z_scale,
                                   float* z_amax, itexb_stream_t stream) {
  ITEXB_REQUIRE(x && gamma && beta && z && mu && rsigma, ITEXB_INVALID_ARGUMENT, "fp8_layernorm: NULL tensor");
  ITEXB_REQUIRE(rows >= 0 && cols > 0 && rows < (1ll << 31), ITEXB_INVALID_ARGUMENT, "fp8_layernorm: bad shape");
  ITEXB_REQUIRE(cols <= 56 * 1024, ITEXB_UNIMPLEMENTED, "fp8_layernorm: rows of more than 57344 elements are not implemented");
  ITEXB_REQUIRE(!IsFp8(z_dtype) || z_scale != nullptr, ITEXB_INVALID_ARGUMENT, "fp8_layernorm: an FP8 output needs z_scale");
  if (rows == 0) return ITEXB_OK;
  cudaStream_t st = AsCuda(stream);
  const int r = int(rows), c = int(cols);
#define ITEXB_LN_W(TX)                                                                                                      \
  do {                                                                                                                      \
    if (w_dtype == ITEXB_DT_FLOAT) return LaunchLn<TX, float>(x, gamma, beta, z, z_dtype, mu, rsigma, r, c, epsilon, z_scale, z_amax, st); \
    if (w_dtype == ITEXB_DT_BFLOAT16)                                                                                       \
      return LaunchLn<TX, __nv_bfloat16>(x, gamma, beta, z, z_dtype, mu, rsigma, r, c, epsilon, z_scale, z_amax, st);       \
    if (w_dtype == ITEXB_DT_HALF) return LaunchLn<TX, __half>(x, gamma, beta, z, z_dtype, mu, rsigma, r, c, epsilon, z_scale, z_amax, st); \
  } while (0)
  if (x_dtype == ITEXB_DT_FLOAT) ITEXB_LN_W(float);
  else if (x_dtype == ITEXB_DT_BFLOAT16) ITEXB_LN_W(__nv_bfloat16);
  else if (x_dtype == ITEXB_DT_HALF) ITEXB_LN_W(__half);
#undef ITEXB_LN_W
  return SetError(ITEXB_INVALID_ARGUMENT, "fp8_layernorm: unsupported input / weight types %s / %s", DtypeName(x_dtype), DtypeName(w_dtype));
}
