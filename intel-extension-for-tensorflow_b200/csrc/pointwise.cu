// HBM-bound element-wise kernels of libitexb200 for sm_100a: QuantizeV2, Dequantize,
// FP8 quantize / dequantize, device-side range reduction, delayed-scaling update and
// the one-time weight / filter packers.
//
// Layout rule shared by the streaming kernels: a thread owns 16 consecutive elements,
// so the 1-byte side moves as one 16-byte vector and the wide side as 2-4 of them;
// a warp therefore touches 512 contiguous bytes of int8 and 1-2 KiB of fp16/fp32 per
// instruction group.  fp32 multiply and add are kept separate (the library is built
// with -fmad=false) so results match a CPU that does not contract.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <cfloat>

#include "common.h"
#include "fp8_cast.h"

namespace itexb {
namespace {

constexpr int kVec = 16;        // elements per thread
constexpr int kThreads = 256;

// ---- scalar conversions -----------------------------------------------------------
template <typename T> __device__ __forceinline__ float ToFloat(T v);
template <> __device__ __forceinline__ float ToFloat<float>(float v) { return v; }
template <> __device__ __forceinline__ float ToFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float ToFloat<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T FromFloat(float v);
template <> __device__ __forceinline__ float FromFloat<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 FromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half FromFloat<__half>(float v) { return __float2half_rn(v); }

// Saturate to [lo, hi] then round to nearest even; NaN converts to 0.  The rounding is done
// on the fp32 adder (x + 1.5*2^23 rounds to nearest even at integer granularity) because
// the conversion instructions run on the slow multi-function unit.  Only the low byte of
// the result is meaningful.
template <bool SIGNED> __device__ __forceinline__ int SatRne8(float f) {
  constexpr float lo = SIGNED ? -128.f : 0.f;
  constexpr float hi = SIGNED ? 127.f : 255.f;
  f = f < lo ? lo : (f > hi ? hi : f);
  f = (f != f) ? 0.f : f;
  return __float_as_int(__fadd_rn(f, 12582912.f)) & 0xff;
}

// float(v) for -2^22 <= v <= 2^22, exact, without a conversion instruction.
__device__ __forceinline__ float SmallIntToFloat(int v) { return __fsub_rn(__int_as_float(v + 0x4B400000), 12582912.f); }

// ---- 16-element vector load / store -----------------------------------------------
template <typename T> struct Vec16 { float v[kVec]; };

template <typename T> __device__ __forceinline__ void Load16(const T* p, float (&out)[kVec]);
template <> __device__ __forceinline__ void Load16<float>(const float* p, float (&out)[kVec]) {
  const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 t = __ldcs(p4 + i);
    out[4 * i + 0] = t.x; out[4 * i + 1] = t.y; out[4 * i + 2] = t.z; out[4 * i + 3] = t.w;
  }
}
template <> __device__ __forceinline__ void Load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[kVec]) {
  const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 t = __ldcs(p4 + i);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[8 * i + 2 * j + 0] = __uint_as_float(w[j] << 16);
      out[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
}
template <> __device__ __forceinline__ void Load16<__half>(const __half* p, float (&out)[kVec]) {
  const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 t = __ldcs(p4 + i);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
      float2 f = __half22float2(h);
      out[8 * i + 2 * j + 0] = f.x;
      out[8 * i + 2 * j + 1] = f.y;
    }
  }
}

__device__ __forceinline__ void StoreBytes16(void* p, const int (&q)[kVec]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    w[j] = uint32_t(q[4 * j] & 0xff) | (uint32_t(q[4 * j + 1] & 0xff) << 8) | (uint32_t(q[4 * j + 2] & 0xff) << 16) |
           (uint32_t(q[4 * j + 3] & 0xff) << 24);
  __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
}

template <bool SIGNED> __device__ __forceinline__ void LoadBytes16(const void* p, float (&out)[kVec]) {
  uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (w[j] >> (8 * b)) & 0xff;
      out[4 * j + b] = SmallIntToFloat(SIGNED ? int(int8_t(byte)) : int(byte));
    }
}

struct SliceArgs {
  const float* scale;
  const float* shift;
  float scale_host;
  float shift_host;
  long long inner;
  long long nslice;
};

__device__ __forceinline__ void SliceConsts(const SliceArgs& a, long long i, float* s, float* sh) {
  if (a.nslice <= 1) {
    *s = a.scale ? __ldg(a.scale) : a.scale_host;
    *sh = a.shift ? __ldg(a.shift) : a.shift_host;
  } else {
    const long long c = (i / a.inner) % a.nslice;
    *s = __ldg(a.scale + c);
    *sh = a.shift ? __ldg(a.shift + c) : a.shift_host;
  }
}

template <int KIND> __device__ __forceinline__ float QuantAffine(float x, float s, float sh) {
  float f = __fmul_rn(x, s);
  if (KIND == ITEXB_QUANT_MIN_FIRST_LEGACY) f = __fadd_rn(f, __fmul_rn(sh, s));
  if (KIND == ITEXB_QUANT_MIN_FIRST_CLASSIC) f = __fadd_rn(f, sh);
  return f;
}

// q = sat(rne(affine(x)))
// VEC: pointers 16-byte aligned; a 16-element group shares one slice when UNIFORM.
// A thread converts kGroups<TX> groups of 16 consecutive elements: one for fp32 inputs, two for 16-bit ones, so that
// either way it has 64 bytes of loads in flight before the first conversion (with 32 the 16-bit variant ran at 0.85 of
// the copy bandwidth).
template <typename TX> constexpr int kGroups = sizeof(TX) == 2 ? 2 : 1;

template <typename TX, bool SIGNED, int KIND, bool UNIFORM>
__global__ void __launch_bounds__(kThreads) QuantizeKernel(const TX* __restrict__ x, uint8_t* __restrict__ q, long long n,
                                                           SliceArgs a) {
  constexpr int G = kGroups<TX>;
  const long long g = (long long)blockIdx.x * kThreads + threadIdx.x;
  const long long i0 = g * (kVec * G);
  if (i0 >= n) return;
  float v[G][kVec];
#pragma unroll
  for (int h = 0; h < G; ++h)
    if (i0 + (h + 1) * kVec <= n) Load16<TX>(x + i0 + h * kVec, v[h]);
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const long long ih = i0 + h * kVec;
    if (ih >= n) break;
    if (ih + kVec <= n) {
      int r[kVec];
      if (UNIFORM) {
        float s, sh;
        SliceConsts(a, ih, &s, &sh);
#pragma unroll
        for (int j = 0; j < kVec; ++j) r[j] = SatRne8<SIGNED>(QuantAffine<KIND>(v[h][j], s, sh));
      } else {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          float s, sh;
          SliceConsts(a, ih + j, &s, &sh);
          r[j] = SatRne8<SIGNED>(QuantAffine<KIND>(v[h][j], s, sh));
        }
      }
      StoreBytes16(q + ih, r);
    } else {
      for (long long i = ih; i < n; ++i) {
        float s, sh;
        SliceConsts(a, i, &s, &sh);
        q[i] = uint8_t(SatRne8<SIGNED>(QuantAffine<KIND>(ToFloat<TX>(x[i]), s, sh)));
      }
    }
  }
}

// Same arithmetic, one element per thread: used when a pointer is not 16-byte aligned.
template <typename TX, bool SIGNED, int KIND>
__global__ void __launch_bounds__(kThreads) QuantizeScalarKernel(const TX* __restrict__ x, uint8_t* __restrict__ q, long long n,
                                                                 SliceArgs a) {
  long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
  const long long stride = (long long)gridDim.x * kThreads;
  for (; i < n; i += stride) {
    float s, sh;
    SliceConsts(a, i, &s, &sh);
    q[i] = uint8_t(SatRne8<SIGNED>(QuantAffine<KIND>(ToFloat<TX>(x[i]), s, sh)));
  }
}

// Four consecutive outputs of one thread -> one store (16 bytes of fp32, 8 bytes of a 16-bit type).
// Elements a thread converts per round of the two dequantize kernels: as many as make its store 16 bytes wide.
template <typename TY> constexpr int kPerRound = 16 / int(sizeof(TY));
constexpr int kRounds = 4;

template <int PER> struct Words;
template <> struct Words<4> {
  uint32_t w[1];
  __device__ __forceinline__ void Load(const uint8_t* p) { w[0] = __ldcs(reinterpret_cast<const uint32_t*>(p)); }
};
template <> struct Words<8> {
  uint32_t w[2];
  __device__ __forceinline__ void Load(const uint8_t* p) {
    const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    w[0] = t.x;
    w[1] = t.y;
  }
};

template <typename T> __device__ __forceinline__ void StoreRound(T* p, const float (&in)[kPerRound<T>]);
template <> __device__ __forceinline__ void StoreRound<float>(float* p, const float (&in)[4]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(in[0], in[1], in[2], in[3]));
}
template <> __device__ __forceinline__ void StoreRound<__nv_bfloat16>(__nv_bfloat16* p, const float (&in)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * j], in[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
}
template <> __device__ __forceinline__ void StoreRound<__half>(__half* p, const float (&in)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __half2 h = __floats2half2_rn(in[2 * j], in[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
}

// y = T((float(q) - zp) * s).  A block covers kThreads * PER * 4 consecutive elements in four rounds (PER = 4 for fp32
// results, 8 for 16-bit ones); in a round thread t converts elements PER*t .. PER*t + PER-1 of a run of kThreads * PER,
// so every load instruction of a warp reads 128 or 256 consecutive bytes and every store instruction writes 512
// consecutive bytes, 16 per thread - whole 32-byte sectors, which the write-dominated traffic of this kernel needs (a
// thread writing its own 64 consecutive bytes in four stores half-fills every sector it touches: 0.71 of the copy
// bandwidth instead of the 0.9 and more of this layout).
template <typename TY, bool SIGNED, bool UNIFORM>
__global__ void __launch_bounds__(kThreads) DequantizeKernel(const uint8_t* __restrict__ q, TY* __restrict__ y, long long n,
                                                             SliceArgs a) {
  constexpr int PER = kPerRound<TY>;
  const long long base = (long long)blockIdx.x * (kThreads * PER * kRounds) + threadIdx.x * PER;
  Words<PER> w[kRounds];
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const long long i = base + (long long)r * (kThreads * PER);
    if (i + PER <= n) w[r].Load(q + i);
  }
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const long long i = base + (long long)r * (kThreads * PER);
    if (i + PER <= n) {
      float v[PER], s, zp;
      if (UNIFORM) {
        // One scale for the thread's bytes.  byte -> float without a conversion or an integer add: a byte permute drops
        // the byte into the low byte of the bit pattern of 2^23 (signed bytes are offset by 128 first, b ^ 0x80 = b + 128),
        // which IS the float 2^23 + b; one exact subtraction takes 2^23 (+ 128) off again.  Then the same two roundings as
        // everywhere: minus zero point, times scale (a zero point of 0 subtracts exactly, so both cases share the code).
        SliceConsts(a, i, &s, &zp);
        const float off = SIGNED ? 8388736.f : 8388608.f;  // 2^23 + 128 | 2^23
#pragma unroll
        for (int j = 0; j < PER / 4; ++j) {
          const uint32_t word = SIGNED ? (w[r].w[j] ^ 0x80808080u) : w[r].w[j];
          v[4 * j + 0] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650));
          v[4 * j + 1] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7651));
          v[4 * j + 2] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7652));
          v[4 * j + 3] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7653));
        }
#pragma unroll
        for (int b = 0; b < PER; ++b) v[b] = __fmul_rn(__fsub_rn(__fsub_rn(v[b], off), zp), s);
      } else {
#pragma unroll
        for (int b = 0; b < PER; ++b) {
          const uint32_t byte = (w[r].w[b / 4] >> (8 * (b % 4))) & 0xff;
          SliceConsts(a, i + b, &s, &zp);
          v[b] = __fmul_rn(__fsub_rn(SmallIntToFloat(SIGNED ? int(int8_t(byte)) : int(byte)), zp), s);
        }
      }
      StoreRound<TY>(y + i, v);
    } else {
      for (long long e = i; e < n; ++e) {
        float s, zp;
        SliceConsts(a, e, &s, &zp);
        const float f = SmallIntToFloat(SIGNED ? int(int8_t(q[e])) : int(q[e]));
        y[e] = FromFloat<TY>(__fmul_rn(__fsub_rn(f, zp), s));
      }
    }
  }
}

template <typename TY, bool SIGNED>
__global__ void __launch_bounds__(kThreads) DequantizeScalarKernel(const uint8_t* __restrict__ q, TY* __restrict__ y,
                                                                   long long n, SliceArgs a) {
  long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
  const long long stride = (long long)gridDim.x * kThreads;
  for (; i < n; i += stride) {
    float s, zp;
    SliceConsts(a, i, &s, &zp);
    const float f = SIGNED ? float(int(int8_t(q[i]))) : float(q[i]);
    y[i] = FromFloat<TY>(__fmul_rn(__fsub_rn(f, zp), s));
  }
}

inline bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int GridFor(long long n_groups) { return int((n_groups + kThreads - 1) / kThreads); }

template <typename TX, bool SIGNED, int KIND>
int LaunchQuantize(const void* x, void* q, long long n, const SliceArgs& a, cudaStream_t st) {
  const TX* xp = static_cast<const TX*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
  if (!Aligned16(x) || !Aligned16(q)) {
    const int blocks = int(std::min<long long>((n + kThreads - 1) / kThreads, (long long)SmCount() * 16));
    QuantizeScalarKernel<TX, SIGNED, KIND><<<blocks, kThreads, 0, st>>>(xp, qp, n, a);
    return CheckLaunch("QuantizeScalarKernel");
  }
  const long long groups = (n + kVec * kGroups<TX> - 1) / (kVec * kGroups<TX>);  // one thread each
  const bool uniform = a.nslice <= 1 || (a.inner % kVec) == 0;
  if (uniform)
    QuantizeKernel<TX, SIGNED, KIND, true><<<GridFor(groups), kThreads, 0, st>>>(xp, qp, n, a);
  else
    QuantizeKernel<TX, SIGNED, KIND, false><<<GridFor(groups), kThreads, 0, st>>>(xp, qp, n, a);
  return CheckLaunch("QuantizeKernel");
}

template <typename TX, bool SIGNED>
int DispatchQuantKind(int kind, const void* x, void* q, long long n, const SliceArgs& a, cudaStream_t st) {
  switch (kind) {
    case ITEXB_QUANT_SCALED: return LaunchQuantize<TX, SIGNED, ITEXB_QUANT_SCALED>(x, q, n, a, st);
    case ITEXB_QUANT_MIN_FIRST_LEGACY: return LaunchQuantize<TX, SIGNED, ITEXB_QUANT_MIN_FIRST_LEGACY>(x, q, n, a, st);
    case ITEXB_QUANT_MIN_FIRST_CLASSIC: return LaunchQuantize<TX, SIGNED, ITEXB_QUANT_MIN_FIRST_CLASSIC>(x, q, n, a, st);
    default: return SetError(ITEXB_INVALID_ARGUMENT, "quantize: unknown kind %d", kind);
  }
}

template <typename TY, bool SIGNED>
int LaunchDequantize(const void* q, void* y, long long n, const SliceArgs& a, cudaStream_t st) {
  const uint8_t* qp = static_cast<const uint8_t*>(q);
  TY* yp = static_cast<TY*>(y);
  if (!Aligned16(q) || !Aligned16(y)) {
    const int blocks = int(std::min<long long>((n + kThreads - 1) / kThreads, (long long)SmCount() * 16));
    DequantizeScalarKernel<TY, SIGNED><<<blocks, kThreads, 0, st>>>(qp, yp, n, a);
    return CheckLaunch("DequantizeScalarKernel");
  }
  constexpr long long kPerBlock = (long long)kThreads * kPerRound<TY> * kRounds;
  const int grid = int((n + kPerBlock - 1) / kPerBlock);
  const bool uniform = a.nslice <= 1 || (a.inner % kPerRound<TY>) == 0;  // a thread's elements of a round share a slice
  if (uniform)
    DequantizeKernel<TY, SIGNED, true><<<grid, kThreads, 0, st>>>(qp, yp, n, a);
  else
    DequantizeKernel<TY, SIGNED, false><<<grid, kThreads, 0, st>>>(qp, yp, n, a);
  return CheckLaunch("DequantizeKernel");
}

int CheckSliceArgs(const char* who, int64_t n, int64_t inner, int64_t nslice, const float* scale) {
  ITEXB_REQUIRE(n >= 0, ITEXB_INVALID_ARGUMENT, "%s: negative element count", who);
  ITEXB_REQUIRE(nslice >= 1 && inner >= 1, ITEXB_INVALID_ARGUMENT, "%s: inner and nslice must be >= 1", who);
  ITEXB_REQUIRE(nslice == 1 || scale != nullptr, ITEXB_INVALID_ARGUMENT,
                "%s: a device scale vector is required when nslice > 1", who);
  return ITEXB_OK;
}

// ---- float atomics on ordered bit patterns -----------------------------------------
__device__ __forceinline__ void AtomicMaxFloat(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void AtomicMinFloat(float* addr, float v) {
  if (v >= 0.f) atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__device__ __forceinline__ float WarpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float WarpMin(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__global__ void MinMaxInitKernel(float* mm) {
  mm[0] = __int_as_float(0x7f800000);
  mm[1] = __int_as_float(0xff800000);
}

template <typename TX>
__global__ void __launch_bounds__(kThreads) MinMaxKernel(const TX* __restrict__ x, long long n, float* __restrict__ mm,
                                                         bool vec) {
  float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);
  const long long stride = (long long)gridDim.x * kThreads;
  if (vec) {
    const long long groups = n / kVec;
    for (long long g = (long long)blockIdx.x * kThreads + threadIdx.x; g < groups; g += stride) {
      float v[kVec];
      Load16<TX>(x + g * kVec, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) { lo = fminf(lo, v[j]); hi = fmaxf(hi, v[j]); }
    }
    for (long long i = groups * kVec + (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
      const float f = ToFloat<TX>(x[i]);
      lo = fminf(lo, f); hi = fmaxf(hi, f);
    }
  } else {
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
      const float f = ToFloat<TX>(x[i]);
      lo = fminf(lo, f); hi = fmaxf(hi, f);
    }
  }
  __shared__ float s_lo[kThreads / 32], s_hi[kThreads / 32];
  lo = WarpMin(lo); hi = WarpMax(hi);
  if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    lo = threadIdx.x < kThreads / 32 ? s_lo[threadIdx.x] : __int_as_float(0x7f800000);
    hi = threadIdx.x < kThreads / 32 ? s_hi[threadIdx.x] : __int_as_float(0xff800000);
    lo = WarpMin(lo); hi = WarpMax(hi);
    if (threadIdx.x == 0) { AtomicMinFloat(mm, lo); AtomicMaxFloat(mm + 1, hi); }
  }
}

// Host math of QuantizeV2 SCALED restated on the device for a device-resident range:
// AdjustInputMinMaxRange then GetScaleAndZeropointAndAlignMinMax (quantize branch).
__device__ __forceinline__ void DynamicScale(const float* mm, float emr, bool is_signed, float* scale, float* omin,
                                             float* omax) {
  const float min_in = mm[0], max_in = mm[1];
  const float adj_min = fminf(0.f, min_in);
  const float eps = __fmul_rn(fmaxf(1.f, fmaxf(fabsf(min_in), fabsf(max_in))), emr);
  const float adj_max = fmaxf(0.f, fmaxf(max_in, __fadd_rn(adj_min, eps)));
  const float abs_range = fmaxf(fabsf(adj_min), fabsf(adj_max));
  *scale = __fdiv_rn(is_signed ? 127.f : 255.f, abs_range);
  *omin = is_signed ? -abs_range : 0.f;
  *omax = abs_range;
}

template <typename TX, bool SIGNED>
__global__ void __launch_bounds__(kThreads) QuantizeDynamicKernel(const TX* __restrict__ x, uint8_t* __restrict__ q,
                                                                  long long n, const float* __restrict__ mm, float emr,
                                                                  float* __restrict__ out3, const float* __restrict__ weight_range,
                                                                  int n_scales, float* __restrict__ scales) {
  float s, omin, omax;
  DynamicScale(mm, emr, SIGNED, &s, &omin, &omax);
  if (blockIdx.x == 0 && threadIdx.x == 0 && out3 != nullptr) { out3[0] = s; out3[1] = omin; out3[2] = omax; }
  if (blockIdx.x == 0 && scales != nullptr) {
    // the consuming matmul's per-channel output scales (same formula as MatMulScalesDynamicKernel)
    const float range_input = fmaxf(fabsf(omin), fabsf(omax));
    const float denom = __fmul_rn(SIGNED ? 127.f : 255.f, 127.f);
    for (int j = threadIdx.x; j < n_scales; j += kThreads) scales[j] = __fdiv_rn(__fmul_rn(range_input, weight_range[j]), denom);
  }
  const long long i0 = ((long long)blockIdx.x * kThreads + threadIdx.x) * kVec;
  if (i0 >= n) return;
  if (i0 + kVec <= n) {
    float v[kVec];
    int r[kVec];
    Load16<TX>(x + i0, v);
#pragma unroll
    for (int j = 0; j < kVec; ++j) r[j] = SatRne8<SIGNED>(__fmul_rn(v[j], s));
    StoreBytes16(q + i0, r);
  } else {
    for (long long i = i0; i < n; ++i) q[i] = uint8_t(SatRne8<SIGNED>(__fmul_rn(ToFloat<TX>(x[i]), s)));
  }
}

// scales[j] = (range_input * range_weight[j]) / (max_int8_input * 127): the per-channel output scale of the
// fused matmul ops with the activation range read on the device (range3 = what QuantizeDynamicKernel wrote).
__global__ void MatMulScalesDynamicKernel(const float* __restrict__ range3, const float* __restrict__ weight_range, int n,
                                          float max_int8_input, float* __restrict__ scales) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const float range_input = fmaxf(fabsf(range3[1]), fabsf(range3[2]));
  scales[j] = __fdiv_rn(__fmul_rn(range_input, weight_range[j]), __fmul_rn(max_int8_input, 127.f));
}

// ---- FP8 ----------------------------------------------------------------------------
template <bool E4M3> __device__ __forceinline__ uint8_t FloatToFp8Sat(float f) { return FloatToFp8Bits(f, E4M3); }
template <bool E4M3> __device__ __forceinline__ float Fp8ToFloat(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, E4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// y = fp8(float(x) * scale[0]); amax[0] = max(amax[0], max|x|)
// GELU of the FP8 path, the formula of itex/core/kernels/gpu/fp8/fp8_gelu_gpu.h:29-34.
__device__ __forceinline__ float Fp8PathGelu(float v) {
  return __fmul_rn(v, __fadd_rn(0.5f, __fmul_rn(0.5f, tanhf(__fmul_rn(v, __fadd_rn(0.79788456f, __fmul_rn(__fmul_rn(0.03567741f, v), v)))))));
}

// GELU = false: y = fp8(x * scale); GELU = true: y = fp8(gelu(x) * scale).  amax is raised to max|x| resp. max|gelu(x)|.
template <typename TX, bool E4M3, bool GELU = false>
__global__ void __launch_bounds__(kThreads) Fp8QuantizeKernel(const TX* __restrict__ x, uint8_t* __restrict__ y, long long n,
                                                              const float* __restrict__ scale, float* __restrict__ amax,
                                                              bool vec) {
  const float s = __ldg(scale);
  float m = 0.f;
  const long long stride = (long long)gridDim.x * kThreads;
  if (vec) {
    constexpr int G = 1;  // (two groups per thread for 16-bit inputs, as in QuantizeKernel, measured 1-3 % slower here)
    const long long groups = n / (kVec * G);
    for (long long g = (long long)blockIdx.x * kThreads + threadIdx.x; g < groups; g += stride) {
      float v[G][kVec];
#pragma unroll
      for (int h = 0; h < G; ++h) Load16<TX>(x + (g * G + h) * kVec, v[h]);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        int r[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float f = GELU ? Fp8PathGelu(v[h][j]) : v[h][j];
          m = fmaxf(m, fabsf(f));
          r[j] = FloatToFp8Sat<E4M3>(__fmul_rn(f, s));
        }
        StoreBytes16(y + (g * G + h) * kVec, r);
      }
    }
    for (long long i = groups * (kVec * G) + (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
      const float f = GELU ? Fp8PathGelu(ToFloat<TX>(x[i])) : ToFloat<TX>(x[i]);
      m = fmaxf(m, fabsf(f));
      y[i] = FloatToFp8Sat<E4M3>(__fmul_rn(f, s));
    }
  } else {
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
      const float f = GELU ? Fp8PathGelu(ToFloat<TX>(x[i])) : ToFloat<TX>(x[i]);
      m = fmaxf(m, fabsf(f));
      y[i] = FloatToFp8Sat<E4M3>(__fmul_rn(f, s));
    }
  }
  if (amax == nullptr) return;
  __shared__ float s_m[kThreads / 32];
  m = WarpMax(m);
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < kThreads / 32 ? s_m[threadIdx.x] : 0.f;
    m = WarpMax(m);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));  // m >= 0
  }
}

// y = T(float(x) * scale_inv[0]).  The layout of DequantizeKernel: 16-byte stores, whole sectors per warp instruction.
// Two FP8 bytes convert to a pair of halves in one instruction (exact: every FP8 value is a half), then to fp32.
template <typename TY, bool E4M3>
__global__ void __launch_bounds__(kThreads) Fp8DequantizeKernel(const uint8_t* __restrict__ x, TY* __restrict__ y, long long n,
                                                                const float* __restrict__ scale_inv) {
  constexpr int PER = kPerRound<TY>;
  const float s = __ldg(scale_inv);
  const long long base = (long long)blockIdx.x * (kThreads * PER * kRounds) + threadIdx.x * PER;
  Words<PER> w[kRounds];
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const long long i = base + (long long)r * (kThreads * PER);
    if (i + PER <= n) w[r].Load(x + i);
  }
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const long long i = base + (long long)r * (kThreads * PER);
    if (i + PER <= n) {
      float v[PER];
#pragma unroll
      for (int j = 0; j < PER / 2; ++j) {
        const uint32_t pair = (w[r].w[j / 2] >> (16 * (j % 2))) & 0xffffu;
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)pair, E4M3 ? __NV_E4M3 : __NV_E5M2);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
        v[2 * j] = __fmul_rn(f.x, s);
        v[2 * j + 1] = __fmul_rn(f.y, s);
      }
      StoreRound<TY>(y + i, v);
    } else {
      for (long long e = i; e < n; ++e) y[e] = FromFloat<TY>(__fmul_rn(Fp8ToFloat<E4M3>(x[e]), s));
    }
  }
}

template <typename TY, bool E4M3>
__global__ void __launch_bounds__(kThreads) Fp8DequantizeScalarKernel(const uint8_t* __restrict__ x, TY* __restrict__ y, long long n,
                                                                      const float* __restrict__ scale_inv) {
  const float s = __ldg(scale_inv);
  const long long stride = (long long)gridDim.x * kThreads;
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
    y[i] = FromFloat<TY>(__fmul_rn(Fp8ToFloat<E4M3>(x[i]), s));
}

// One thread per meta slot.  floor(log2(.)) is taken on the fp32-rounded logarithm like
// the TensorFlow expression it restates; 2^|exp| is exact for integer exponents.
__global__ void Fp8AmaxScaleUpdateKernel(float* __restrict__ hist, float* __restrict__ scale, float* __restrict__ scale_inv,
                                         int hlen, int n, float fp8_max, float margin, int algo) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float amax = hist[j];
  if (algo == 0)
    for (int r = 1; r < hlen; ++r) amax = fmaxf(amax, hist[(long long)r * n + j]);
  const float old = scale[j];
  const float ratio = __fdiv_rn(fp8_max, amax);
  const float lg = float(log2(double(ratio)));
  const float e = __fsub_rn(floorf(lg), margin);
  float sf = rintf(exp2f(fabsf(e)));
  sf = (amax > 0.f) ? sf : old;
  sf = (isfinite(amax)) ? sf : old;
  sf = (e < 0.f) ? __fdiv_rn(1.f, sf) : sf;
  // roll(-1, axis 0): row r takes row r+1, last row takes row 0; then row 0 is zeroed.
  const float first = hist[j];
  for (int r = 0; r + 1 < hlen; ++r) hist[(long long)r * n + j] = hist[(long long)(r + 1) * n + j];
  hist[(long long)(hlen - 1) * n + j] = first;
  hist[j] = 0.f;
  scale[j] = sf;
  scale_inv[j] = __fdiv_rn(1.f, sf);
}

// ---- one-time packers ---------------------------------------------------------------
// [batch][k,n] -> [batch][n,k_pad] through a 64x64 shared tile (+4 bytes of row padding against bank conflicts).
// vec_load / vec_store: 4 bytes per thread along n (source) and along k (destination) when pitch and base allow.
__global__ void __launch_bounds__(256) PackWeightsKnKernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                           long long k, long long n, long long k_pad, long long src_stride,
                                                           long long dst_stride, bool vec_load, bool vec_store) {
  __shared__ __align__(16) uint8_t tile[64][68];
  src += (long long)blockIdx.z * src_stride;
  dst += (long long)blockIdx.z * dst_stride;
  const long long k0 = (long long)blockIdx.y * 64, n0 = (long long)blockIdx.x * 64;
  if (vec_load) {
    for (int t = threadIdx.x; t < 64 * 16; t += 256) {
      const int r = t >> 4, c = (t & 15) * 4;  // r: k, c: n
      const long long kk = k0 + r, nn = n0 + c;
      uint32_t v = 0;
      if (kk < k && nn < n) v = __ldg(reinterpret_cast<const uint32_t*>(src + kk * n + nn));  // n % 4 == 0: nn + 3 < n
      *reinterpret_cast<uint32_t*>(&tile[r][c]) = v;
    }
  } else {
    for (int t = threadIdx.x; t < 64 * 64; t += 256) {
      const int r = t >> 6, c = t & 63;  // r: k, c: n (coalesced along n)
      const long long kk = k0 + r, nn = n0 + c;
      tile[r][c] = (kk < k && nn < n) ? src[kk * n + nn] : uint8_t(0);
    }
  }
  __syncthreads();
  if (vec_store) {
    for (int t = threadIdx.x; t < 64 * 16; t += 256) {
      const int r = t >> 4, c = (t & 15) * 4;  // r: n, c: k
      const long long nn = n0 + r, kk = k0 + c;
      if (nn < n && kk < k_pad) {  // k_pad % 4 == 0: kk + 3 < k_pad
        const uint32_t v = uint32_t(tile[c][r]) | (uint32_t(tile[c + 1][r]) << 8) | (uint32_t(tile[c + 2][r]) << 16) |
                           (uint32_t(tile[c + 3][r]) << 24);
        *reinterpret_cast<uint32_t*>(dst + nn * k_pad + kk) = v;
      }
    }
  } else {
    for (int t = threadIdx.x; t < 64 * 64; t += 256) {
      const int r = t >> 6, c = t & 63;  // r: n, c: k (coalesced along k)
      const long long nn = n0 + r, kk = k0 + c;
      if (nn < n && kk < k_pad) dst[nn * k_pad + kk] = tile[c][r];
    }
  }
}

// out[i] = in[broadcast index of i]: `rank` output dims (outermost first) with the input's element strides,
// 0 where the input has extent 1.  One element per thread; T is the 2- or 4-byte storage type.
struct BroadcastShape {
  int rank;
  long long dims[ITEXB_MAX_DIMS];
  long long strides[ITEXB_MAX_DIMS];
};
template <typename T>
__global__ void BroadcastKernel(const T* __restrict__ in, T* __restrict__ out, long long total, BroadcastShape s) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, src = 0;
#pragma unroll
    for (int d = ITEXB_MAX_DIMS - 1; d >= 0; --d) {
      if (d < s.rank) {
        const long long q = rem / s.dims[d];
        src += (rem - q * s.dims[d]) * s.strides[d];
        rem = q;
      }
    }
    out[i] = __ldg(in + src);
  }
}

__global__ void ColsumS8Kernel(const int8_t* __restrict__ b, int32_t* __restrict__ colsum, long long k, long long n) {
  const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  int s = 0;
  for (long long i = 0; i < k; ++i) s += int(b[i * n + j]);
  colsum[j] = s;
}

// HWIO [kh,kw,c,co] -> [co][k_pad]: k = (tap * c_pad + channel), zero padded per tap (c_pad > c) and
// at the row end (k_pad = kh*kw*c_pad rounded up to 16).
__global__ void PackFilterKernel(const uint8_t* __restrict__ f, uint8_t* __restrict__ dst, int taps, int c, int co, int c_pad,
                                 int k_pad) {
  const long long total = (long long)co * k_pad;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int kk = int(i % k_pad);
    const int o = int(i / k_pad);
    const int t = kk / c_pad, ci = kk - t * c_pad;
    dst[i] = (t < taps && ci < c) ? f[((long long)t * c + ci) * co + o] : uint8_t(0);
  }
}

}  // namespace

int LaunchBroadcast(const void* in, const int64_t* in_dims, int in_rank, void* out, const int64_t* out_dims, int out_rank,
                    int elem_bytes, cudaStream_t stream) {
  ITEXB_REQUIRE(in != nullptr && out != nullptr && in_rank <= out_rank && out_rank <= ITEXB_MAX_DIMS && (elem_bytes == 2 || elem_bytes == 4),
                ITEXB_INVALID_ARGUMENT, "broadcast: bad arguments");
  BroadcastShape s{};
  s.rank = out_rank;
  long long total = 1, stride = 1;
  for (int d = out_rank - 1; d >= 0; --d) {
    const int id = d - (out_rank - in_rank);
    const long long extent = id >= 0 ? in_dims[id] : 1;
    ITEXB_REQUIRE(extent == out_dims[d] || extent == 1, ITEXB_INVALID_ARGUMENT, "broadcast: extent %lld does not broadcast to %lld",
                  extent, (long long)out_dims[d]);
    s.dims[d] = out_dims[d];
    s.strides[d] = extent == 1 ? 0 : stride;
    stride *= extent;
    total *= out_dims[d];
  }
  if (total == 0) return ITEXB_OK;
  const int blocks = int(std::max<long long>(1, std::min<long long>((total + 255) / 256, (long long)SmCount() * 16)));
  if (elem_bytes == 4) BroadcastKernel<uint32_t><<<blocks, 256, 0, stream>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), total, s);
  else BroadcastKernel<uint16_t><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), total, s);
  return CheckLaunch("BroadcastKernel");
}

}  // namespace itexb

using namespace itexb;

extern "C" {

int itexb_quantize(const void* x, int x_dtype, void* q, int q_dtype, int64_t n, int64_t inner, int64_t nslice, int kind,
                   const float* scale, const float* shift, float scale_host, float shift_host, itexb_stream_t stream) {
  ITEXB_RETURN_IF_ERROR(CheckSliceArgs("quantize", n, inner, nslice, scale));
  ITEXB_REQUIRE(IsInt8(q_dtype), ITEXB_INVALID_ARGUMENT, "quantize: output type %s is not qint8/quint8", DtypeName(q_dtype));
  if (n == 0) return ITEXB_OK;
  ITEXB_REQUIRE(x != nullptr && q != nullptr, ITEXB_INVALID_ARGUMENT, "quantize: NULL tensor");
  SliceArgs a{scale, shift, scale_host, shift_host, (long long)inner, (long long)nslice};
  cudaStream_t st = AsCuda(stream);
  const bool sg = IsSigned8(q_dtype);
  switch (x_dtype) {
    case ITEXB_DT_FLOAT:
      return sg ? DispatchQuantKind<float, true>(kind, x, q, n, a, st) : DispatchQuantKind<float, false>(kind, x, q, n, a, st);
    case ITEXB_DT_BFLOAT16:
      return sg ? DispatchQuantKind<__nv_bfloat16, true>(kind, x, q, n, a, st)
                : DispatchQuantKind<__nv_bfloat16, false>(kind, x, q, n, a, st);
    case ITEXB_DT_HALF:
      return sg ? DispatchQuantKind<__half, true>(kind, x, q, n, a, st) : DispatchQuantKind<__half, false>(kind, x, q, n, a, st);
    default:
      return SetError(ITEXB_INVALID_ARGUMENT, "quantize: input type %s is not float/bfloat16/half", DtypeName(x_dtype));
  }
}

int itexb_dequantize(const void* q, int q_dtype, void* y, int y_dtype, int64_t n, int64_t inner, int64_t nslice,
                     const float* scale, const float* zp, float scale_host, float zp_host, itexb_stream_t stream) {
  ITEXB_RETURN_IF_ERROR(CheckSliceArgs("dequantize", n, inner, nslice, scale));
  ITEXB_REQUIRE(IsInt8(q_dtype), ITEXB_INVALID_ARGUMENT, "dequantize: input type %s is not qint8/quint8", DtypeName(q_dtype));
  if (n == 0) return ITEXB_OK;
  ITEXB_REQUIRE(q != nullptr && y != nullptr, ITEXB_INVALID_ARGUMENT, "dequantize: NULL tensor");
  SliceArgs a{scale, zp, scale_host, zp_host, (long long)inner, (long long)nslice};
  cudaStream_t st = AsCuda(stream);
  const bool sg = IsSigned8(q_dtype);
  switch (y_dtype) {
    case ITEXB_DT_FLOAT:
      return sg ? LaunchDequantize<float, true>(q, y, n, a, st) : LaunchDequantize<float, false>(q, y, n, a, st);
    case ITEXB_DT_BFLOAT16:
      return sg ? LaunchDequantize<__nv_bfloat16, true>(q, y, n, a, st) : LaunchDequantize<__nv_bfloat16, false>(q, y, n, a, st);
    case ITEXB_DT_HALF:
      return sg ? LaunchDequantize<__half, true>(q, y, n, a, st) : LaunchDequantize<__half, false>(q, y, n, a, st);
    default:
      return SetError(ITEXB_INVALID_ARGUMENT, "dequantize: output type %s is not float/bfloat16/half", DtypeName(y_dtype));
  }
}

int itexb_minmax_init(float* minmax, itexb_stream_t stream) {
  ITEXB_REQUIRE(minmax != nullptr, ITEXB_INVALID_ARGUMENT, "minmax_init: NULL pointer");
  MinMaxInitKernel<<<1, 1, 0, AsCuda(stream)>>>(minmax);
  return CheckLaunch("MinMaxInitKernel");
}

int itexb_minmax(const void* x, int x_dtype, int64_t n, float* minmax, itexb_stream_t stream) {
  ITEXB_REQUIRE(minmax != nullptr && n >= 0, ITEXB_INVALID_ARGUMENT, "minmax: bad arguments");
  if (n == 0) return ITEXB_OK;
  const bool vec = Aligned16(x);
  const long long work = vec ? (n + kVec - 1) / kVec : n;
  const int blocks = int(std::max<long long>(1, std::min<long long>((work + kThreads - 1) / kThreads, (long long)SmCount() * 8)));
  cudaStream_t st = AsCuda(stream);
  if (x_dtype == ITEXB_DT_FLOAT)
    MinMaxKernel<float><<<blocks, kThreads, 0, st>>>(static_cast<const float*>(x), n, minmax, vec);
  else if (x_dtype == ITEXB_DT_BFLOAT16)
    MinMaxKernel<__nv_bfloat16><<<blocks, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, minmax, vec);
  else
    return SetError(ITEXB_INVALID_ARGUMENT, "minmax: input type %s is not float/bfloat16", DtypeName(x_dtype));
  return CheckLaunch("MinMaxKernel");
}

int itexb_quantize_dynamic(const void* x, int x_dtype, void* q, int q_dtype, int64_t n, const float* minmax,
                           float ensure_minimum_range, float* out3, itexb_stream_t stream) {
  return itexb_quantize_dynamic_scales(x, x_dtype, q, q_dtype, n, minmax, ensure_minimum_range, out3, nullptr, 0, nullptr, stream);
}

int itexb_quantize_dynamic_scales(const void* x, int x_dtype, void* q, int q_dtype, int64_t n, const float* minmax,
                                  float ensure_minimum_range, float* out3, const float* weight_range, int32_t n_scales,
                                  float* scales, itexb_stream_t stream) {
  ITEXB_REQUIRE(scales == nullptr || (weight_range != nullptr && n_scales > 0), ITEXB_INVALID_ARGUMENT,
                "quantize_dynamic_scales: scales needs weight_range and a positive count");
  ITEXB_REQUIRE(IsInt8(q_dtype), ITEXB_INVALID_ARGUMENT, "quantize_dynamic: output type %s is not qint8/quint8",
                DtypeName(q_dtype));
  ITEXB_REQUIRE(minmax != nullptr && n >= 0, ITEXB_INVALID_ARGUMENT, "quantize_dynamic: bad arguments");
  ITEXB_REQUIRE(Aligned16(x) && Aligned16(q), ITEXB_INVALID_ARGUMENT, "quantize_dynamic: tensors must be 16-byte aligned");
  if (n == 0) return ITEXB_OK;
  const int grid = GridFor((n + kVec - 1) / kVec);
  cudaStream_t st = AsCuda(stream);
  const bool sg = IsSigned8(q_dtype);
  uint8_t* qp = static_cast<uint8_t*>(q);
  if (x_dtype == ITEXB_DT_FLOAT) {
    auto xp = static_cast<const float*>(x);
    if (sg) QuantizeDynamicKernel<float, true><<<grid, kThreads, 0, st>>>(xp, qp, n, minmax, ensure_minimum_range, out3, weight_range, n_scales, scales);
    else QuantizeDynamicKernel<float, false><<<grid, kThreads, 0, st>>>(xp, qp, n, minmax, ensure_minimum_range, out3, weight_range, n_scales, scales);
  } else if (x_dtype == ITEXB_DT_BFLOAT16) {
    auto xp = static_cast<const __nv_bfloat16*>(x);
    if (sg) QuantizeDynamicKernel<__nv_bfloat16, true><<<grid, kThreads, 0, st>>>(xp, qp, n, minmax, ensure_minimum_range, out3, weight_range, n_scales, scales);
    else QuantizeDynamicKernel<__nv_bfloat16, false><<<grid, kThreads, 0, st>>>(xp, qp, n, minmax, ensure_minimum_range, out3, weight_range, n_scales, scales);
  } else {
    return SetError(ITEXB_INVALID_ARGUMENT, "quantize_dynamic: input type %s is not float/bfloat16", DtypeName(x_dtype));
  }
  return CheckLaunch("QuantizeDynamicKernel");
}

int itexb_matmul_scales_dynamic(const float* range3, const float* weight_range, int32_t n, int a_dtype, float* scales,
                                itexb_stream_t stream) {
  ITEXB_REQUIRE(range3 != nullptr && weight_range != nullptr && scales != nullptr && n > 0, ITEXB_INVALID_ARGUMENT,
                "matmul_scales_dynamic: bad arguments");
  ITEXB_REQUIRE(IsInt8(a_dtype), ITEXB_INVALID_ARGUMENT, "matmul_scales_dynamic: activation type %s is not 8-bit", DtypeName(a_dtype));
  MatMulScalesDynamicKernel<<<(n + 127) / 128, 128, 0, AsCuda(stream)>>>(range3, weight_range, n, IsSigned8(a_dtype) ? 127.f : 255.f, scales);
  return CheckLaunch("MatMulScalesDynamicKernel");
}

int itexb_pack_weights_kn_batched(const void* b_kn, void* b_nk, int64_t k, int64_t n, int64_t k_pad, int64_t batch,
                                  int64_t src_stride, int64_t dst_stride, itexb_stream_t stream) {
  ITEXB_REQUIRE(b_kn != nullptr && b_nk != nullptr && k > 0 && n > 0 && k_pad >= k && batch > 0 && batch <= 65535 && src_stride >= 0 &&
                    dst_stride >= 0,
                ITEXB_INVALID_ARGUMENT, "pack_weights_kn: bad arguments");
  const bool vec_load = n % 4 == 0 && src_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(b_kn) & 3) == 0;
  const bool vec_store = k_pad % 4 == 0 && dst_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(b_nk) & 3) == 0;
  dim3 grid((unsigned)((n + 63) / 64), (unsigned)((k_pad + 63) / 64), (unsigned)batch);
  PackWeightsKnKernel<<<grid, 256, 0, AsCuda(stream)>>>(static_cast<const uint8_t*>(b_kn), static_cast<uint8_t*>(b_nk), k, n, k_pad,
                                                        src_stride, dst_stride, vec_load, vec_store);
  return CheckLaunch("PackWeightsKnKernel");
}

int itexb_pack_weights_kn(const void* b_kn, void* b_nk, int64_t k, int64_t n, int64_t k_pad, itexb_stream_t stream) {
  return itexb_pack_weights_kn_batched(b_kn, b_nk, k, n, k_pad, 1, 0, 0, stream);
}

int itexb_colsum_s8(const int8_t* b_kn, int32_t* colsum, int64_t k, int64_t n, itexb_stream_t stream) {
  ITEXB_REQUIRE(b_kn != nullptr && colsum != nullptr && k > 0 && n > 0, ITEXB_INVALID_ARGUMENT, "colsum_s8: bad arguments");
  ColsumS8Kernel<<<(unsigned)((n + 127) / 128), 128, 0, AsCuda(stream)>>>(b_kn, colsum, k, n);
  return CheckLaunch("ColsumS8Kernel");
}

int itexb_pack_filter_hwio(const void* f_hwio, void* f_packed, int32_t kh, int32_t kw, int32_t c, int32_t co, int32_t c_pad,
                           itexb_stream_t stream) {
  ITEXB_REQUIRE(f_hwio != nullptr && f_packed != nullptr && kh > 0 && kw > 0 && c > 0 && co > 0 && c_pad >= c,
                ITEXB_INVALID_ARGUMENT, "pack_filter_hwio: bad arguments");
  const int k_pad = (kh * kw * c_pad + 15) / 16 * 16;
  const long long total = (long long)co * k_pad;
  const int blocks = int(std::min<long long>((total + 255) / 256, (long long)SmCount() * 8));
  PackFilterKernel<<<blocks, 256, 0, AsCuda(stream)>>>(static_cast<const uint8_t*>(f_hwio), static_cast<uint8_t*>(f_packed),
                                                      kh * kw, c, co, c_pad, k_pad);
  return CheckLaunch("PackFilterKernel");
}

int itexb_fp8_quantize(const void* x, int x_dtype, void* y, int fp8_dtype, int64_t n, const float* scale, float* amax,
                       itexb_stream_t stream) {
  ITEXB_REQUIRE(IsFp8(fp8_dtype), ITEXB_INVALID_ARGUMENT, "fp8_quantize: fp8_dtype must be E4M3 or E5M2");
  ITEXB_REQUIRE(scale != nullptr && n >= 0, ITEXB_INVALID_ARGUMENT, "fp8_quantize: bad arguments");
  if (n == 0) return ITEXB_OK;
  const bool vec = Aligned16(x) && Aligned16(y);
  const long long work = vec ? (n + kVec - 1) / kVec : n;
  const int blocks = int(std::max<long long>(1, std::min<long long>((work + kThreads - 1) / kThreads, (long long)SmCount() * 16)));
  cudaStream_t st = AsCuda(stream);
  uint8_t* yp = static_cast<uint8_t*>(y);
  const bool e4 = fp8_dtype == ITEXB_DT_FP8_E4M3;
#define ITEXB_FP8Q(TX)                                                                                         \
  do {                                                                                                         \
    if (e4) Fp8QuantizeKernel<TX, true><<<blocks, kThreads, 0, st>>>(static_cast<const TX*>(x), yp, n, scale, amax, vec); \
    else Fp8QuantizeKernel<TX, false><<<blocks, kThreads, 0, st>>>(static_cast<const TX*>(x), yp, n, scale, amax, vec);   \
  } while (0)
  if (x_dtype == ITEXB_DT_FLOAT) ITEXB_FP8Q(float);
  else if (x_dtype == ITEXB_DT_BFLOAT16) ITEXB_FP8Q(__nv_bfloat16);
  else if (x_dtype == ITEXB_DT_HALF) ITEXB_FP8Q(__half);
  else return SetError(ITEXB_INVALID_ARGUMENT, "fp8_quantize: input type %s is not float/bfloat16/half", DtypeName(x_dtype));
#undef ITEXB_FP8Q
  return CheckLaunch("Fp8QuantizeKernel");
}

int itexb_fp8_gelu(const void* x, int x_dtype, void* y, int fp8_dtype, int64_t n, const float* scale, float* amax,
                   itexb_stream_t stream) {
  ITEXB_REQUIRE(IsFp8(fp8_dtype), ITEXB_INVALID_ARGUMENT, "fp8_gelu: fp8_dtype must be E4M3 or E5M2");
  ITEXB_REQUIRE(scale != nullptr && n >= 0, ITEXB_INVALID_ARGUMENT, "fp8_gelu: bad arguments");
  if (n == 0) return ITEXB_OK;
  const bool vec = Aligned16(x) && Aligned16(y);
  const long long work = vec ? (n + kVec - 1) / kVec : n;
  const int blocks = int(std::max<long long>(1, std::min<long long>((work + kThreads - 1) / kThreads, (long long)SmCount() * 16)));
  cudaStream_t st = AsCuda(stream);
  uint8_t* yp = static_cast<uint8_t*>(y);
  const bool e4 = fp8_dtype == ITEXB_DT_FP8_E4M3;
#define ITEXB_FP8G(TX)                                                                                                  \
  do {                                                                                                                  \
    if (e4) Fp8QuantizeKernel<TX, true, true><<<blocks, kThreads, 0, st>>>(static_cast<const TX*>(x), yp, n, scale, amax, vec); \
    else Fp8QuantizeKernel<TX, false, true><<<blocks, kThreads, 0, st>>>(static_cast<const TX*>(x), yp, n, scale, amax, vec);   \
  } while (0)
  if (x_dtype == ITEXB_DT_FLOAT) ITEXB_FP8G(float);
  else if (x_dtype == ITEXB_DT_BFLOAT16) ITEXB_FP8G(__nv_bfloat16);
  else if (x_dtype == ITEXB_DT_HALF) ITEXB_FP8G(__half);
  else return SetError(ITEXB_INVALID_ARGUMENT, "fp8_gelu: input type %s is not float/bfloat16/half", DtypeName(x_dtype));
#undef ITEXB_FP8G
  return CheckLaunch("Fp8GeluKernel");
}

int itexb_fp8_dequantize(const void* x, int fp8_dtype, void* y, int y_dtype, int64_t n, const float* scale_inv,
                         itexb_stream_t stream) {
  ITEXB_REQUIRE(IsFp8(fp8_dtype), ITEXB_INVALID_ARGUMENT, "fp8_dequantize: fp8_dtype must be E4M3 or E5M2");
  ITEXB_REQUIRE(scale_inv != nullptr && n >= 0, ITEXB_INVALID_ARGUMENT, "fp8_dequantize: bad arguments");
  if (n == 0) return ITEXB_OK;
  const bool vec = Aligned16(x) && Aligned16(y);
  cudaStream_t st = AsCuda(stream);
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  const bool e4 = fp8_dtype == ITEXB_DT_FP8_E4M3;
#define ITEXB_FP8D(TY)                                                                                                   \
  do {                                                                                                                   \
    if (vec) {                                                                                                           \
      constexpr long long kPerBlock = (long long)kThreads * kPerRound<TY> * kRounds;                                     \
      const int grid = int((n + kPerBlock - 1) / kPerBlock);                                                             \
      if (e4) Fp8DequantizeKernel<TY, true><<<grid, kThreads, 0, st>>>(xp, static_cast<TY*>(y), n, scale_inv);           \
      else Fp8DequantizeKernel<TY, false><<<grid, kThreads, 0, st>>>(xp, static_cast<TY*>(y), n, scale_inv);             \
    } else {                                                                                                             \
      const int blocks = int(std::min<long long>((n + kThreads - 1) / kThreads, (long long)SmCount() * 16));             \
      if (e4) Fp8DequantizeScalarKernel<TY, true><<<blocks, kThreads, 0, st>>>(xp, static_cast<TY*>(y), n, scale_inv);   \
      else Fp8DequantizeScalarKernel<TY, false><<<blocks, kThreads, 0, st>>>(xp, static_cast<TY*>(y), n, scale_inv);     \
    }                                                                                                                    \
  } while (0)
  if (y_dtype == ITEXB_DT_FLOAT) ITEXB_FP8D(float);
  else if (y_dtype == ITEXB_DT_BFLOAT16) ITEXB_FP8D(__nv_bfloat16);
  else if (y_dtype == ITEXB_DT_HALF) ITEXB_FP8D(__half);
  else return SetError(ITEXB_INVALID_ARGUMENT, "fp8_dequantize: output type %s is not float/bfloat16/half", DtypeName(y_dtype));
#undef ITEXB_FP8D
  return CheckLaunch("Fp8DequantizeKernel");
}

int itexb_fp8_amax_and_scale_update(float* amax_history, float* scale, float* scale_inv, int32_t history_len, int32_t n,
                                    float fp8_max, float margin, int32_t algo, itexb_stream_t stream) {
  ITEXB_REQUIRE(amax_history && scale && scale_inv && history_len >= 1 && n >= 1, ITEXB_INVALID_ARGUMENT,
                "fp8_amax_and_scale_update: bad arguments");
  ITEXB_REQUIRE(algo == 0 || algo == 1, ITEXB_INVALID_ARGUMENT,
                "We only support the fp8 recipe with 'max' or 'most_recent' amax_compute_algo");
  Fp8AmaxScaleUpdateKernel<<<(n + 63) / 64, 64, 0, AsCuda(stream)>>>(amax_history, scale, scale_inv, history_len, n, fp8_max,
                                                                    margin, algo);
  return CheckLaunch("Fp8AmaxScaleUpdateKernel");
}

}  // extern "C"
