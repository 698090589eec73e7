// NHWC 8-bit max / average pooling for sm_100a (HBM-bound: one read of the input window
// per output, 16 channels per thread as one 16-byte vector when the channel count allows).
#include <algorithm>

#include "common.h"

namespace itexb {
namespace {

template <bool SIGNED, bool AVG>
__global__ void __launch_bounds__(256) PoolVecKernel(itexb_pool_params_t p) {
  const int cv = p.c >> 4;
  const long long total = (long long)p.n * p.oh * p.ow * cv;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int cc = int(i % cv);
    const long long pix = i / cv;
    const int ox = int(pix % p.ow);
    const int oy = int((pix / p.ow) % p.oh);
    const int b = int(pix / ((long long)p.ow * p.oh));
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = AVG ? 0 : (SIGNED ? -128 : 0);
    int count = 0;
    for (int ky = 0; ky < p.kh; ++ky) {
      const int iy = oy * p.stride_h + ky - p.pad_top;
      if (iy < 0 || iy >= p.h) continue;
      for (int kx = 0; kx < p.kw; ++kx) {
        const int ix = ox * p.stride_w + kx - p.pad_left;
        if (ix < 0 || ix >= p.w) continue;
        ++count;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x) +
                                                             (((long long)b * p.h + iy) * p.w + ix) * p.c + cc * 16));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t byte = (w[j >> 2] >> (8 * (j & 3))) & 0xff;
          const int e = SIGNED ? int(int8_t(byte)) : int(byte);
          acc[j] = AVG ? acc[j] + e : max(acc[j], e);
        }
      }
    }
    uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int r = acc[j];
      if (AVG) {
        float f = __fdiv_rn(float(acc[j]), float(max(count, 1)));
        f = fminf(fmaxf(f, SIGNED ? -128.f : 0.f), SIGNED ? 127.f : 255.f);
        r = __float2int_rn(f);
      }
      o[j >> 2] |= uint32_t(r & 0xff) << (8 * (j & 3));
    }
    *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + pix * p.c + cc * 16) = make_uint4(o[0], o[1], o[2], o[3]);
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
  const bool vec = p->c % 16 == 0 && ((reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->out)) & 15) == 0;
  const long long work = (long long)p->n * p->oh * p->ow * (vec ? p->c / 16 : p->c);
  const int blocks = int(std::max<long long>(1, std::min<long long>((work + 255) / 256, (long long)SmCount() * 32)));
  cudaStream_t st = AsCuda(stream);
  const bool sg = IsSigned8(p->dtype);
#define ITEXB_POOL(K)                                                     \
  do {                                                                    \
    if (sg && p->is_avg) K<true, true><<<blocks, 256, 0, st>>>(*p);       \
    else if (sg) K<true, false><<<blocks, 256, 0, st>>>(*p);              \
    else if (p->is_avg) K<false, true><<<blocks, 256, 0, st>>>(*p);       \
    else K<false, false><<<blocks, 256, 0, st>>>(*p);                     \
  } while (0)
  if (vec) ITEXB_POOL(PoolVecKernel);
  else ITEXB_POOL(PoolScalarKernel);
#undef ITEXB_POOL
  return CheckLaunch("PoolKernel");
}
