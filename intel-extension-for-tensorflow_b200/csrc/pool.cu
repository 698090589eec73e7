// NHWC 8-bit max / average pooling for sm_100a (HBM-bound: one read of the input window
// per output, 16 channels per thread as 16-byte vectors when the channel count allows).
#include <algorithm>

#include "common.h"

namespace itexb {
namespace {

// 16-bit lane arithmetic on packed pairs (one instruction each on this architecture).
__device__ __forceinline__ uint32_t Max16x2(uint32_t a, uint32_t b, bool is_signed) {
  uint32_t r;
  if (is_signed) asm("max.s16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// prmt in its default mode: a selector nibble with bit 3 set replicates the selected byte's sign bit.
__device__ __forceinline__ uint32_t Prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t Add16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.s16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// 16 channels of one tap folded into eight accumulator words of two 16-bit lanes: byte permutes widen the bytes
// (zero- or sign-extending), packed 16-bit max / add combines them.
template <bool SIGNED, bool AVG>
__device__ __forceinline__ void FoldTap(uint32_t (&acc)[8], const uint4& v) {
  constexpr uint32_t kSel01 = SIGNED ? 0x9180u : 0x4140u, kSel23 = SIGNED ? 0xB3A2u : 0x4342u;  // bytes 0,1 | 2,3 -> 16-bit lanes
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t lo = Prmt(w[q], 0u, kSel01), hi = Prmt(w[q], 0u, kSel23);
    acc[2 * q] = AVG ? Add16x2(acc[2 * q], lo) : Max16x2(acc[2 * q], lo, SIGNED);
    acc[2 * q + 1] = AVG ? Add16x2(acc[2 * q + 1], hi) : Max16x2(acc[2 * q + 1], hi, SIGNED);
  }
}
// The accumulator's 16 lanes -> 16 output bytes (average: divide by the number of taps inside the image, clamp,
// round half to even).
template <bool SIGNED, bool AVG>
__device__ __forceinline__ uint4 FinishPool(const uint32_t (&acc)[8], int count) {
  uint32_t o[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t word = 0;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const uint32_t lane16 = (acc[2 * q + (h >> 1)] >> (16 * (h & 1))) & 0xffffu;
      int r = SIGNED ? int(int16_t(lane16)) : int(lane16);
      if (AVG) {
        float f = __fdiv_rn(float(r), float(max(count, 1)));
        f = fminf(fmaxf(f, SIGNED ? -128.f : 0.f), SIGNED ? 127.f : 255.f);
        r = __float2int_rn(f);
      }
      word |= uint32_t(r & 0xff) << (8 * h);
    }
    o[q] = word;
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}
template <bool SIGNED, bool AVG> __device__ __forceinline__ uint32_t PoolIdentityLanes() { return AVG ? 0u : (SIGNED ? 0xff80ff80u : 0u); }
template <bool SIGNED, bool AVG> __device__ __forceinline__ uint32_t PoolIdentityBytes() { return AVG ? 0u : (SIGNED ? 0x80808080u : 0u); }

// Windows of at most 3 x 3 (the max pooling after a ResNet stem): one thread per output pixel and 16 channels,
// all nine taps requested before the first is used (one load in flight per thread made the kernel a chain of
// kh*kw memory latencies: 3x3/2 max pooling of [32,112,112,64] took 32 us for 32 MB).
template <bool SIGNED, bool AVG>
__global__ void __launch_bounds__(256) PoolSmallKernel(itexb_pool_params_t p) {
  const int cv = p.c >> 4;
  const long long total = (long long)p.n * p.oh * p.ow * cv;
  const uint32_t idb = PoolIdentityBytes<SIGNED, AVG>();
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int cc = int(i % cv);
    const long long pix = i / cv;
    const int ox = int(pix % p.ow);
    const int oy = int((pix / p.ow) % p.oh);
    const int b = int(pix / ((long long)p.ow * p.oh));
    const int ix0 = ox * p.stride_w - p.pad_left, iy0 = oy * p.stride_h - p.pad_top;
    const uint8_t* base = static_cast<const uint8_t*>(p.x) + (long long)b * p.h * p.w * p.c + cc * 16;
    uint4 v[9];
    int count = 0;
#pragma unroll
    for (int ky = 0; ky < 3; ++ky)
#pragma unroll
      for (int kx = 0; kx < 3; ++kx) {
        const int iy = iy0 + ky, ix = ix0 + kx;
        const bool in = ky < p.kh && kx < p.kw && iy >= 0 && iy < p.h && ix >= 0 && ix < p.w;
        count += in ? 1 : 0;
        v[ky * 3 + kx] = in ? __ldg(reinterpret_cast<const uint4*>(base + ((long long)iy * p.w + ix) * p.c)) : make_uint4(idb, idb, idb, idb);
      }
    uint32_t acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = PoolIdentityLanes<SIGNED, AVG>();
#pragma unroll
    for (int t = 0; t < 9; ++t) FoldTap<SIGNED, AVG>(acc, v[t]);
    *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + pix * p.c + cc * 16) = FinishPool<SIGNED, AVG>(acc, count);
  }
}

// Larger windows (the 7 x 7 global average pooling): a block of 8 warps works on 32 consecutive units (output
// pixel x 16 channels); warp r takes the window rows r, r+8, ... of all 32 (coalesced: the 32 lanes read 512
// consecutive bytes of a pixel, or neighbouring pixels), eight taps of a row in flight at a time, and the eight
// partial results meet in shared memory.  Window sums fit 16 bits for up to 257 taps of unsigned input (257 * 255 = 65535)
// and 256 taps of signed input (256 * -128 = -32768): the host checks.
template <bool SIGNED, bool AVG>
__global__ void __launch_bounds__(256) PoolRowsKernel(itexb_pool_params_t p) {
  __shared__ uint32_t red[8][32][9];
  const int cv = p.c >> 4;
  const long long total = (long long)p.n * p.oh * p.ow * cv;
  const int r = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t idb = PoolIdentityBytes<SIGNED, AVG>();
  for (long long i0 = (long long)blockIdx.x * 32; i0 < total; i0 += (long long)gridDim.x * 32) {
    const long long i = i0 + lane;
    const bool live = i < total;
    const int cc = int((live ? i : 0) % cv);
    const long long pix = (live ? i : 0) / cv;
    const int ox = int(pix % p.ow);
    const int oy = int((pix / p.ow) % p.oh);
    const int b = int(pix / ((long long)p.ow * p.oh));
    const int ix0 = ox * p.stride_w - p.pad_left;
    uint32_t acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = PoolIdentityLanes<SIGNED, AVG>();
    int count = 0;
    for (int ky = r; ky < p.kh; ky += 8) {
      const int iy = oy * p.stride_h + ky - p.pad_top;
      if (!live || iy < 0 || iy >= p.h) continue;
      const uint8_t* row = static_cast<const uint8_t*>(p.x) + (((long long)b * p.h + iy) * p.w) * p.c + cc * 16;
      for (int kx0 = 0; kx0 < p.kw; kx0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int ix = ix0 + kx0 + t;
          const bool in = kx0 + t < p.kw && ix >= 0 && ix < p.w;
          count += in ? 1 : 0;
          v[t] = in ? __ldg(reinterpret_cast<const uint4*>(row + (long long)ix * p.c)) : make_uint4(idb, idb, idb, idb);
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) FoldTap<SIGNED, AVG>(acc, v[t]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[r][lane][j] = acc[j];
    red[r][lane][8] = uint32_t(count);
    __syncthreads();
    if (r == 0 && live) {
#pragma unroll 1
      for (int rr = 1; rr < 8; ++rr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = AVG ? Add16x2(acc[j], red[rr][lane][j]) : Max16x2(acc[j], red[rr][lane][j], SIGNED);
        count += int(red[rr][lane][8]);
      }
      *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + pix * p.c + cc * 16) = FinishPool<SIGNED, AVG>(acc, count);
    }
    __syncthreads();
  }
}

template <bool SIGNED, bool AVG>
__global__ void __launch_bounds__(256) PoolScalarKernel(itexb_pool_params_t p) {
  const long long total = (long long)p.n * p.oh * p.ow * p.c;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int ch = int(i % p.c);
    const long long pix = i / p.c;
    const int ox = int(pix % p.ow);
    const int oy = int((pix / p.ow) % p.oh);
    const int b = int(pix / ((long long)p.ow * p.oh));
    int acc = AVG ? 0 : (SIGNED ? -128 : 0), count = 0;
    for (int ky = 0; ky < p.kh; ++ky) {
      const int iy = oy * p.stride_h + ky - p.pad_top;
      if (iy < 0 || iy >= p.h) continue;
      for (int kx = 0; kx < p.kw; ++kx) {
        const int ix = ox * p.stride_w + kx - p.pad_left;
        if (ix < 0 || ix >= p.w) continue;
        ++count;
        const uint8_t byte = static_cast<const uint8_t*>(p.x)[(((long long)b * p.h + iy) * p.w + ix) * p.c + ch];
        const int e = SIGNED ? int(int8_t(byte)) : int(byte);
        acc = AVG ? acc + e : max(acc, e);
      }
    }
    if (AVG) {
      float f = __fdiv_rn(float(acc), float(max(count, 1)));
      f = fminf(fmaxf(f, SIGNED ? -128.f : 0.f), SIGNED ? 127.f : 255.f);
      acc = __float2int_rn(f);
    }
    static_cast<uint8_t*>(p.out)[i] = uint8_t(acc & 0xff);
  }
}

}  // namespace
}  // namespace itexb

using namespace itexb;

extern "C" int itexb_pool2d(const itexb_pool_params_t* p, itexb_stream_t stream) {
  ITEXB_REQUIRE(p != nullptr, ITEXB_INVALID_ARGUMENT, "pool2d: params is NULL");
  ITEXB_REQUIRE(p->n >= 0 && p->h > 0 && p->w > 0 && p->c > 0 && p->kh > 0 && p->kw > 0 && p->stride_h > 0 && p->stride_w > 0 &&
                    p->oh > 0 && p->ow > 0,
                ITEXB_INVALID_ARGUMENT, "pool2d: bad dimensions");
  ITEXB_REQUIRE(IsInt8(p->dtype), ITEXB_INVALID_ARGUMENT, "pool2d: type %s is not qint8/quint8", DtypeName(p->dtype));
  if (p->n == 0) return ITEXB_OK;
  ITEXB_REQUIRE(p->x != nullptr && p->out != nullptr, ITEXB_INVALID_ARGUMENT, "pool2d: NULL tensor");
  const bool vec = p->c % 16 == 0 && ((reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->out)) & 15) == 0 &&
                   (long long)p->kh * p->kw <= (IsSigned8(p->dtype) ? 256 : 257);  // 16-bit window sums: 257 * 255, 256 * -128
  const long long work = (long long)p->n * p->oh * p->ow * (vec ? p->c / 16 : p->c);
  const bool small = p->kh <= 3 && p->kw <= 3;
  const long long want_blocks = (vec && !small) ? (work + 31) / 32 : (work + 255) / 256;
  const int blocks = int(std::max<long long>(1, std::min<long long>(want_blocks, (long long)SmCount() * 32)));
  cudaStream_t st = AsCuda(stream);
  const bool sg = IsSigned8(p->dtype);
#define ITEXB_POOL(K)                                                     \
  do {                                                                    \
    if (sg && p->is_avg) K<true, true><<<blocks, 256, 0, st>>>(*p);       \
    else if (sg) K<true, false><<<blocks, 256, 0, st>>>(*p);              \
    else if (p->is_avg) K<false, true><<<blocks, 256, 0, st>>>(*p);       \
    else K<false, false><<<blocks, 256, 0, st>>>(*p);                     \
  } while (0)
  if (vec && small) ITEXB_POOL(PoolSmallKernel);
  else if (vec) ITEXB_POOL(PoolRowsKernel);
  else ITEXB_POOL(PoolScalarKernel);
#undef ITEXB_POOL
  return CheckLaunch("PoolKernel");
}
