// Fp8QuantizeDbias and Fp8QuantizeDbiasDgelu: the backward-side FP8 cast of a gradient fused with the bias gradient
// (column sums) and, in the second op, with the derivative of GELU.
//
//   t[r][c]      = grad[r][c]                                   (Dbias)
//                = dgelu(gelu_inp[r][c]) * grad[r][c]           (DbiasDgelu)
//   out[r][c]    = fp8(t * scale[0])        dbias[c] = sum_r t[r][c]  (fp32, cast to the gradient's type)
//   amax[0]      = max(amax[0], max |t|)
//
// Arithmetic of functor::Fp8QuantizeDbiasFused / Fp8QuantizeDbiasDgeluFused and ReduceDbiasKernel
// (itex/core/kernels/gpu/fp8/fp8_quantize_fusion_gpu.h:33-300); the GELU derivative is its dgelu() (:33-43).
//
// HBM-bound streaming work (read 2-4 B, write 1 B per element, twice the read for Dgelu).  A block of 32 x 8 threads
// owns a band of 128 columns and kRowsPerBlock rows: every thread reads four consecutive columns of one row per step
// (16-byte loads for fp32, 8-byte for 16-bit types; a warp covers 512 or 256 contiguous bytes of a row), keeps its four
// running column sums in registers, and the eight row groups meet in shared memory at the end.  The per-block partial
// sums go to a [row_blocks, cols] fp32 scratch matrix that a second small kernel adds up in a fixed order, so the
// result does not depend on scheduling (no float atomics).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "fp8_cast.h"

namespace itexb {
namespace {

constexpr int kRowsPerBlock = 256;
constexpr int kColsPerBlock = 128;

template <typename T> __device__ __forceinline__ float AsFloat(T v);
template <> __device__ __forceinline__ float AsFloat<float>(float v) { return v; }
template <> __device__ __forceinline__ float AsFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float AsFloat<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T OfFloat(float v);
template <> __device__ __forceinline__ float OfFloat<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 OfFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half OfFloat<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float DGelu(float x) {
  const float th = tanhf(__fmul_rn(__fmul_rn(0.79788456f, x), __fadd_rn(1.f, __fmul_rn(__fmul_rn(0.044715f, x), x))));
  const float a = __fmul_rn(__fmul_rn(0.5f, x),
                            __fmul_rn(__fsub_rn(1.f, __fmul_rn(th, th)), __fadd_rn(0.79788456f, __fmul_rn(__fmul_rn(0.1070322243f, x), x))));
  return __fadd_rn(a, __fmul_rn(0.5f, __fadd_rn(1.f, th)));
}

// Four consecutive elements of a row (vector load when VEC, element loads with a bound otherwise).
template <typename T, bool VEC> __device__ __forceinline__ void Load4(const T* p, int valid, float (&v)[4]) {
  if (VEC) {
    if (sizeof(T) == 4) {
      const float4 t = *reinterpret_cast<const float4*>(p);
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
      const uint2 t = *reinterpret_cast<const uint2*>(p);
      const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = AsFloat<T>(e[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = j < valid ? AsFloat<T>(p[j]) : 0.f;
  }
}

template <typename T, bool E4M3, bool DGELU, bool VEC>
__global__ void __launch_bounds__(256) Fp8QuantizeDbiasKernel(const T* __restrict__ grad, const T* __restrict__ gelu_inp, uint8_t* __restrict__ out,
                                                              float* __restrict__ partial, int rows, int cols, const float* __restrict__ scale,
                                                              float* __restrict__ amax) {
  __shared__ float s_sum[8][kColsPerBlock];
  __shared__ float s_max[8];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = blockIdx.x * kColsPerBlock + tx * 4;
  const int row_begin = blockIdx.y * kRowsPerBlock;
  const int row_end = min(rows, row_begin + kRowsPerBlock);
  const int valid = max(0, min(4, cols - col));
  const float s = __ldg(scale);
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  float m = 0.f;
  if (valid > 0) {
    for (int r = row_begin + ty; r < row_end; r += 8) {
      const long long at = (long long)r * cols + col;
      float t[4];
      Load4<T, VEC>(grad + at, valid, t);
      if (DGELU) {
        float x[4];
        Load4<T, VEC>(gelu_inp + at, valid, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = __fmul_rn(DGelu(x[j]), t[j]);
      }
      uint32_t packed = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sum[j] = __fadd_rn(sum[j], t[j]);
        m = fmaxf(m, fabsf(t[j]));
        packed |= uint32_t(FloatToFp8Bits(__fmul_rn(s, t[j]), E4M3)) << (8 * j);
      }
      if (VEC) {
        *reinterpret_cast<uint32_t*>(out + at) = packed;
      } else {
        for (int j = 0; j < valid; ++j) out[at + j] = uint8_t(packed >> (8 * j));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) s_sum[ty][tx * 4 + j] = sum[j];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (tx == 0) s_max[ty] = m;
  __syncthreads();
  if (ty == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = s_sum[0][tx * 4 + j];
#pragma unroll
      for (int g = 1; g < 8; ++g) a = __fadd_rn(a, s_sum[g][tx * 4 + j]);  // fixed order
      if (j < valid) partial[(long long)blockIdx.y * cols + col + j] = a;
    }
    if (tx == 0 && amax != nullptr) {
      float bm = s_max[0];
#pragma unroll
      for (int g = 1; g < 8; ++g) bm = fmaxf(bm, s_max[g]);
      atomicMax(reinterpret_cast<int*>(amax), __float_as_int(bm));  // bm >= 0: integer order is float order
    }
  }
}

template <typename T>
__global__ void DbiasReduceKernel(const float* __restrict__ partial, T* __restrict__ dbias, int row_blocks, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float a = 0.f;
  for (int b = 0; b < row_blocks; ++b) a = __fadd_rn(a, partial[(long long)b * cols + c]);
  dbias[c] = OfFloat<T>(a);
}

template <typename T>
int Launch(const void* grad, const void* gelu_inp, void* out, void* dbias, float* workspace, int rows, int cols, bool e4m3, const float* scale,
           float* amax, cudaStream_t st) {
  const dim3 block(32, 8);
  const int row_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  const dim3 grid((cols + kColsPerBlock - 1) / kColsPerBlock, row_blocks);
  const bool dgelu = gelu_inp != nullptr;
  const size_t align = sizeof(T) * 4;
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(grad) % align) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0 &&
                   (!dgelu || (reinterpret_cast<uintptr_t>(gelu_inp) % align) == 0);
  const T* g = static_cast<const T*>(grad);
  const T* x = static_cast<const T*>(gelu_inp);
  uint8_t* o = static_cast<uint8_t*>(out);
#define ITEXB_DBIAS(E4, DG, VE) Fp8QuantizeDbiasKernel<T, E4, DG, VE><<<grid, block, 0, st>>>(g, x, o, workspace, rows, cols, scale, amax)
  if (e4m3) {
    if (dgelu) { if (vec) ITEXB_DBIAS(true, true, true); else ITEXB_DBIAS(true, true, false); }
    else { if (vec) ITEXB_DBIAS(true, false, true); else ITEXB_DBIAS(true, false, false); }
  } else {
    if (dgelu) { if (vec) ITEXB_DBIAS(false, true, true); else ITEXB_DBIAS(false, true, false); }
    else { if (vec) ITEXB_DBIAS(false, false, true); else ITEXB_DBIAS(false, false, false); }
  }
#undef ITEXB_DBIAS
  ITEXB_RETURN_IF_ERROR(CheckLaunch("Fp8QuantizeDbiasKernel"));
  DbiasReduceKernel<T><<<(cols + 255) / 256, 256, 0, st>>>(workspace, static_cast<T*>(dbias), row_blocks, cols);
  return CheckLaunch("DbiasReduceKernel");
}

}  // namespace
}  // namespace itexb

using namespace itexb;

extern "C" size_t itexb_fp8_quantize_dbias_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return size_t((rows + kRowsPerBlock - 1) / kRowsPerBlock) * size_t(cols) * sizeof(float);
}

extern "C" int itexb_fp8_quantize_dbias(const void* grad, const void* gelu_inp, int dtype, void* out, int fp8_dtype, void* dbias, int64_t rows,
                                        int64_t cols, const float* scale, float* amax, void* workspace, itexb_stream_t stream) {
  ITEXB_REQUIRE(IsFp8(fp8_dtype), ITEXB_INVALID_ARGUMENT, "fp8_quantize_dbias: fp8_dtype must be E4M3 or E5M2");
  ITEXB_REQUIRE(rows >= 0 && cols >= 0 && rows < (1ll << 31) && cols < (1ll << 31), ITEXB_INVALID_ARGUMENT, "fp8_quantize_dbias: bad shape");
  if (cols == 0) return ITEXB_OK;
  ITEXB_REQUIRE(dbias != nullptr && scale != nullptr, ITEXB_INVALID_ARGUMENT, "fp8_quantize_dbias: NULL argument");
  if (rows == 0) {
    ITEXB_CUDA(cudaMemsetAsync(dbias, 0, size_t(cols) * DtypeSize(dtype), AsCuda(stream)));  // an empty sum
    return ITEXB_OK;
  }
  ITEXB_REQUIRE(grad != nullptr && out != nullptr && workspace != nullptr, ITEXB_INVALID_ARGUMENT, "fp8_quantize_dbias: NULL argument");
  const bool e4 = fp8_dtype == ITEXB_DT_FP8_E4M3;
  float* ws = static_cast<float*>(workspace);
  if (dtype == ITEXB_DT_FLOAT) return Launch<float>(grad, gelu_inp, out, dbias, ws, int(rows), int(cols), e4, scale, amax, AsCuda(stream));
  if (dtype == ITEXB_DT_BFLOAT16) return Launch<__nv_bfloat16>(grad, gelu_inp, out, dbias, ws, int(rows), int(cols), e4, scale, amax, AsCuda(stream));
  if (dtype == ITEXB_DT_HALF) return Launch<__half>(grad, gelu_inp, out, dbias, ws, int(rows), int(cols), e4, scale, amax, AsCuda(stream));
  return SetError(ITEXB_INVALID_ARGUMENT, "fp8_quantize_dbias: type %s is not float/bfloat16/half", DtypeName(dtype));
}
