// NHWC x HWIO int8 convolution for sm_100a, lowered onto the tcgen05 GEMM kernel.
//
// Four lowerings share the MMA main loop and the fused epilogue; itexb_conv2d picks one from the geometry
// and the channel pitch of the packed filter:
//   * pointwise (1x1, stride 1, no padding, channels a multiple of 16): the input IS the
//     [n*h*w, c] A operand; nothing is staged.
//   * TMA im2col (channels a multiple of 16, filter taps packed at a pitch of c rounded up to 128): the
//     producer thread issues one 4-D im2col tensor load per k-block - 128 output pixels x 128 channels of one
//     filter tap - from a tensor map whose pixel bounding box and traversal strides describe the convolution;
//     padding, rows past the end and channels past c read as zeros.  No scratch, no gather instructions.
//   * cp.async gather (channels a multiple of 16, densely packed filter): four extra warps of the GEMM
//     kernel copy the A tile of each k-block from the NHWC input in 16-byte pieces (zero fill for padding)
//     into the swizzled shared-memory layout.  No scratch either.
//   * other channel counts (e.g. an RGB stem): a gather kernel writes the [n*oh*ow, round_up(kh*kw*c, 16)]
//     patch matrix (zero fill for padding) into caller-provided scratch, then the GEMM runs on it.  Scratch
//     traffic is kh*kw times the input; the caller sizes it with itexb_conv2d_workspace_bytes().
#include <algorithm>
#include <mutex>

#include "common.h"
#include "gemm_sm100.h"

namespace itexb {
namespace {

struct GatherArgs {
  const uint8_t* x;
  uint8_t* ws;
  int n, h, w, c, kh, kw, oh, ow, c_pad;
  int stride_h, stride_w, dil_h, dil_w, pad_top, pad_left;
  long long m;       // n*oh*ow
  int chunks;        // 16-byte chunks per patch row = kh*kw*c_pad/16
};

// One thread per 16-byte chunk of the patch matrix (c % 16 == 0 and c_pad == c).
__global__ void __launch_bounds__(256) GatherPatchesVecKernel(GatherArgs a) {
  const long long total = a.m * a.chunks;
  const int cpt = a.c_pad >> 4;  // chunks per tap
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long pix = i / a.chunks;
    const int ch = int(i - pix * a.chunks);
    const int tap = ch / cpt, cc = ch - tap * cpt;
    const int ky = tap / a.kw, kx = tap - ky * a.kw;
    const int ox = int(pix % a.ow);
    const int oy = int((pix / a.ow) % a.oh);
    const int b = int(pix / ((long long)a.ow * a.oh));
    const int iy = oy * a.stride_h + ky * a.dil_h - a.pad_top;
    const int ix = ox * a.stride_w + kx * a.dil_w - a.pad_left;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (iy >= 0 && iy < a.h && ix >= 0 && ix < a.w)
      v = __ldg(reinterpret_cast<const uint4*>(a.x + (((long long)b * a.h + iy) * a.w + ix) * a.c + cc * 16));
    reinterpret_cast<uint4*>(a.ws)[i] = v;
  }
}

// Any channel count (e.g. 3 for an RGB stem) with the dense layout c_pad == c: one thread per
// (pixel, filter row).  With dilation 1 the kw*c bytes of one filter row are contiguous in the NHWC
// input, so the thread copies one run (clipped at the left/right border, zeros elsewhere); the last
// filter row's thread also zeroes the row tail up to the 16-byte multiple.
__global__ void __launch_bounds__(256) GatherPatchesRowKernel(GatherArgs a) {
  const long long kp = (long long)a.chunks * 16;
  const int run = a.kw * a.c;
  const long long total = a.m * a.kh;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long pix = i / a.kh;
    const int ky = int(i - pix * a.kh);
    const int ox = int(pix % a.ow);
    const int oy = int((pix / a.ow) % a.oh);
    const int b = int(pix / ((long long)a.ow * a.oh));
    const int iy = oy * a.stride_h + ky * a.dil_h - a.pad_top;
    uint8_t* dst = a.ws + pix * kp + (long long)ky * run;
    const bool row_in = iy >= 0 && iy < a.h;
    const uint8_t* src_row = a.x + ((long long)b * a.h + (row_in ? iy : 0)) * a.w * a.c;
    for (int kx = 0; kx < a.kw; ++kx) {
      const int ix = ox * a.stride_w + kx * a.dil_w - a.pad_left;
      const bool in = row_in && ix >= 0 && ix < a.w;
      for (int ci = 0; ci < a.c; ++ci) dst[kx * a.c + ci] = in ? __ldg(src_row + (long long)ix * a.c + ci) : uint8_t(0);
    }
    if (ky == a.kh - 1)
      for (long long t = (long long)a.kh * run; t < kp; ++t) a.ws[pix * kp + t] = 0;
  }
}

// Few-channel stem convolutions (e.g. 7x7x3, stride 2): the filter shape is a template parameter.
// A block builds TP consecutive output pixels of one output row in three phases:
//   1. the KH input rows the pixels touch go to shared memory as aligned 32-bit words (a few edge
//      words byte by byte, zero outside the image);
//   2. each thread pulls the KH runs of KW*C bytes of its pixel into registers - aligned word reads
//      plus one byte permute per word for the run's phase inside its first word - and composes the
//      patch row from them: every word of the row takes its bytes from at most three of those
//      registers at compile-time positions, i.e. one or two byte permutes;
//   3. the TP patch rows are written with consecutive threads on consecutive 16-byte units.
// `pitch` is the distance of patch rows in the workspace: a multiple of 128 bytes, because TMA reads
// 128-byte boxes whose rows straddle two cache lines at half the rate (measured on the GEMM that
// consumes this matrix: 148 us at a pitch of 160 bytes, 83 us at 256).  Dilation 1.
template <int KH, int KW, int C, int TP>
__global__ void __launch_bounds__(TP) GatherPatchesStemKernel(GatherArgs a, int pitch) {
  constexpr int kRun = KW * C;                            // bytes of one filter row
  constexpr int kBytes = KH * kRun;                       // bytes of one patch
  constexpr int kRowBytes = (kBytes + 15) / 16 * 16;      // patch row as written (zero padded)
  constexpr int kDW = (kRun + 3) / 4;                     // registers holding one run
  constexpr int kLW = (kRun + 3 + 3) / 4;                 // words read to cover a run at any phase
  extern __shared__ __align__(16) uint8_t s_mem[];
  const int tiles_x = (a.ow + TP - 1) / TP;
  const int tile = blockIdx.x % tiles_x;
  const int oy = (blockIdx.x / tiles_x) % a.oh;
  const int b = blockIdx.x / (tiles_x * a.oh);
  const int ox0 = tile * TP;
  const int span = (TP - 1) * a.stride_w + KW;            // input columns the tile touches
  const int row_words = (span * C + 3) / 4 + 1;           // words per staged input row (any phase)
  const int start = (ox0 * a.stride_w - a.pad_left) * C;  // byte offset of the window in an image row, may be negative
  const int phase = ((start % 4) + 4) % 4;
  const int start_al = start - phase;                     // word-aligned (the image rows are: w*C % 4 == 0, checked by the host)
  const int image_row_bytes = a.w * C;
  uint32_t* s_in = reinterpret_cast<uint32_t*>(s_mem);    // [KH][row_words]
  // All of a thread's words are requested before the first is stored: with one load in flight per thread the
  // block's lifetime was a chain of 2*KH memory latencies (the kernel ran at a third of the DRAM rate).
  constexpr int kPerRow = 2;  // words per thread and input row; the host checks row_words <= kPerRow * TP
  uint32_t v[KH * kPerRow];
#pragma unroll
  for (int ky = 0; ky < KH; ++ky) {
    const int iy = oy * a.stride_h + ky - a.pad_top;
    const bool row_in = iy >= 0 && iy < a.h;
    const uint8_t* g_row = a.x + ((long long)b * a.h + (row_in ? iy : 0)) * image_row_bytes;
#pragma unroll
    for (int p = 0; p < kPerRow; ++p) {
      const int wi = threadIdx.x + p * TP;
      const int gb = start_al + 4 * wi;
      uint32_t word = 0;
      if (row_in && wi < row_words) {
        if (gb >= 0 && gb + 4 <= image_row_bytes) {
          word = __ldg(reinterpret_cast<const uint32_t*>(g_row + gb));
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t)
            if (gb + t >= 0 && gb + t < image_row_bytes) word |= uint32_t(__ldg(g_row + gb + t)) << (8 * t);
        }
      }
      v[ky * kPerRow + p] = word;
    }
  }
#pragma unroll
  for (int ky = 0; ky < KH; ++ky)
#pragma unroll
    for (int p = 0; p < kPerRow; ++p)
      if (threadIdx.x + p * TP < row_words) s_in[ky * row_words + threadIdx.x + p * TP] = v[ky * kPerRow + p];
  __syncthreads();
  // phase 2: runs into registers
  const int o = phase + threadIdx.x * a.stride_w * C;     // byte offset of this pixel's runs in a staged row
  const int w0 = o >> 2;
  const uint32_t sel = 0x3210u + 0x1111u * uint32_t(o & 3);
  uint32_t d[KH * kDW];
#pragma unroll
  for (int r = 0; r < KH; ++r) {
    uint32_t wv[kLW + 1];
#pragma unroll
    for (int i = 0; i < kLW; ++i) wv[i] = s_in[r * row_words + w0 + i];
    wv[kLW] = 0;
#pragma unroll
    for (int i = 0; i < kDW; ++i) d[r * kDW + i] = __byte_perm(wv[i], wv[i + 1], sel);
  }
  // compose the patch row; byte k of it is byte (k % kRun) & 3 of register (k / kRun) * kDW + ((k % kRun) >> 2)
  uint4* s_out = reinterpret_cast<uint4*>(s_mem + ((KH * row_words * 4 + 15) / 16) * 16);
  uint4* dst = s_out + threadIdx.x * (kRowBytes / 16);
#pragma unroll
  for (int u = 0; u < kRowBytes / 16; ++u) {
    uint32_t w[4];
#pragma unroll
    for (int qq = 0; qq < 4; ++qq) {
      const int k0 = (u * 4 + qq) * 4;                    // compile-time after unrolling, like everything derived from it
      uint32_t word = 0;
      if (k0 < kBytes) {
        const int r0 = (k0 / kRun) * kDW + ((k0 % kRun) >> 2);
        int r1 = -1, r2 = -1;
#pragma unroll
        for (int t = 1; t < 4; ++t) {
          const int k = k0 + t;
          if (k < kBytes) {
            const int rg = (k / kRun) * kDW + ((k % kRun) >> 2);
            if (rg != r0) {
              if (r1 < 0) r1 = rg;
              else if (rg != r1 && r2 < 0) r2 = rg;
            }
          }
        }
        uint32_t sel1 = 0, sel2 = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int k = k0 + t;
          uint32_t n1 = 0, n2 = uint32_t(t);
          if (k < kBytes) {
            const int rg = (k / kRun) * kDW + ((k % kRun) >> 2);
            const uint32_t sb = uint32_t((k % kRun) & 3);
            if (rg == r0) n1 = sb;
            else if (rg == r1) n1 = 4u + sb;
            else n2 = 4u + sb;
          }
          sel1 |= n1 << (4 * t);
          sel2 |= n2 << (4 * t);
        }
        word = __byte_perm(d[r0], d[r1 < 0 ? r0 : r1], sel1);
        if (r2 >= 0) word = __byte_perm(word, d[r2], sel2);
        if (k0 + 4 > kBytes) word &= (1u << (8 * (kBytes - k0))) - 1u;  // zero padding after the last patch byte
      }
      w[qq] = word;
    }
    dst[u] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __syncthreads();
  const int pixels = min(TP, a.ow - ox0);
  uint8_t* out = a.ws + (((long long)b * a.oh + oy) * a.ow + ox0) * pitch;
  constexpr int kUnits = kRowBytes / 16;
  for (int i = threadIdx.x; i < pixels * kUnits; i += TP) {
    const int pix = i / kUnits, u = i - pix * kUnits;
    *reinterpret_cast<uint4*>(out + (long long)pix * pitch + 16 * u) = s_out[i];
  }
}

bool IsPointwise(const itexb_conv_params_t& p) {
  return p.kh == 1 && p.kw == 1 && p.stride_h == 1 && p.stride_w == 1 && p.pad_top == 0 && p.pad_left == 0 &&
         p.oh == p.h && p.ow == p.w && p.c % 16 == 0 && p.c_pad == p.c;
}

// Geometry the TMA im2col path can express: 16-byte channel runs, traversal strides up to 8, box
// corners and tap offsets within the signed 8-bit fields of the tensor map and the instruction.
bool Im2colGeometryOk(const itexb_conv_params_t& p) {
  if (IsPointwise(p) || p.c % 16 != 0 || p.stride_h > 8 || p.stride_w > 8) return false;
  const int up_w = (p.ow - 1) * p.stride_w - p.pad_left - p.w + 1, up_h = (p.oh - 1) * p.stride_h - p.pad_top - p.h + 1;
  const auto in8 = [](int v) { return v >= -128 && v <= 127; };
  return in8(-p.pad_left) && in8(-p.pad_top) && in8(up_w) && in8(up_h) && (p.kw - 1) * p.dil_w <= 127 && (p.kh - 1) * p.dil_h <= 127 &&
         p.w + up_w + p.pad_left > 0 && p.h + up_h + p.pad_top > 0 && (long long)p.h * p.w * p.c < (1ll << 40);
}

// Channels per tap the packed filter should have: c rounded up to the 128 bytes of a k-block when
// the TMA im2col path will run (each k-block is then one tap), c otherwise.
// The k-blocks of the im2col path are one tap wide: 128 bytes (128-byte swizzle), or for filters of at most
// 64 channels 64 or 32 bytes with the swizzle of that width, so that a 64-channel 3x3 layer neither fills shared
// memory with nor multiplies 64 zero channels per tap.
int Im2colCPad(int c) { return c <= 32 ? 32 : (c <= 64 ? 64 : (c + 127) / 128 * 128); }
int FilterCPad(const itexb_conv_params_t& p) { return Im2colGeometryOk(p) ? Im2colCPad(p.c) : p.c; }

bool IsIm2col(const itexb_conv_params_t& p) { return Im2colGeometryOk(p) && p.c_pad == Im2colCPad(p.c); }

int Validate(const itexb_conv_params_t& p) {
  ITEXB_REQUIRE(p.n >= 0 && p.h > 0 && p.w > 0 && p.c > 0 && p.kh > 0 && p.kw > 0 && p.co > 0, ITEXB_INVALID_ARGUMENT,
                "conv2d: bad tensor dimensions");
  ITEXB_REQUIRE(p.stride_h > 0 && p.stride_w > 0 && p.dil_h > 0 && p.dil_w > 0, ITEXB_INVALID_ARGUMENT,
                "conv2d: strides and dilations must be positive");
  ITEXB_REQUIRE(p.oh > 0 && p.ow > 0, ITEXB_INVALID_ARGUMENT, "conv2d: empty output");
  ITEXB_REQUIRE(p.c_pad == p.c || (p.c_pad == Im2colCPad(p.c) && Im2colGeometryOk(p)), ITEXB_INVALID_ARGUMENT,
                "conv2d: c_pad must be what itexb_conv2d_filter_c_pad returns (%d or c=%d), got %d", FilterCPad(p), p.c, p.c_pad);
  ITEXB_REQUIRE(IsInt8(p.x_dtype), ITEXB_INVALID_ARGUMENT, "conv2d: input type %s is not qint8/quint8", DtypeName(p.x_dtype));
  return ValidateEpilogue("conv2d", p.ep, p.out_dtype, false, p.co);
}

}  // namespace
}  // namespace itexb

using namespace itexb;

// Channel counts that are a multiple of 16 are gathered inside the GEMM kernel (16-byte runs);
// nothing is staged in global memory for them.  That kernel keeps 32-bit byte offsets into the
// input and 15-bit tap masks per axis, hence the size limits.
static bool IsImplicit(const itexb_conv_params_t& p) {
  return p.c % 16 == 0 && p.c_pad == p.c && p.kh <= 15 && p.kw <= 15 &&
         (long long)p.n * p.h * p.w * p.c < (1ll << 31);
}

extern "C" int32_t itexb_conv2d_filter_c_pad(const itexb_conv_params_t* p) { return p == nullptr ? 0 : FilterCPad(*p); }

// The 7x7x3 stem has its own patch builder (GatherPatchesStemKernel).
static bool IsStem(const itexb_conv_params_t& p) {
  return p.kh == 7 && p.kw == 7 && p.c == 3 && p.c_pad == 3 && p.dil_h == 1 && p.dil_w == 1 && p.stride_w <= 2 && (p.w * p.c) % 4 == 0;
}
// Distance of patch rows in the workspace: the row length (a multiple of 16 bytes), or for the stem the next
// multiple of 128, which TMA reads at twice the rate (the padding is never written or read).
static size_t PatchPitch(const itexb_conv_params_t& p) {
  const size_t kp = (size_t(p.kh) * p.kw * p.c_pad + 15) / 16 * 16;
  return IsStem(p) ? (kp + 127) / 128 * 128 : kp;
}

extern "C" size_t itexb_conv2d_workspace_bytes(const itexb_conv_params_t* p) {
  if (p == nullptr || IsPointwise(*p) || IsIm2col(*p) || IsImplicit(*p)) return 0;
  return size_t(p->n) * p->oh * p->ow * PatchPitch(*p);
}

extern "C" int itexb_conv2d(const itexb_conv_params_t* p, itexb_stream_t stream) {
  ITEXB_REQUIRE(p != nullptr, ITEXB_INVALID_ARGUMENT, "conv2d: params is NULL");
  ITEXB_RETURN_IF_ERROR(Validate(*p));
  if (p->n == 0) return ITEXB_OK;
  ITEXB_REQUIRE(p->x && p->filter_packed && p->out, ITEXB_INVALID_ARGUMENT, "conv2d: NULL tensor");
  cudaStream_t st = AsCuda(stream);
  const long long m = (long long)p->n * p->oh * p->ow;
  ITEXB_REQUIRE(m < (1ll << 31), ITEXB_INVALID_ARGUMENT, "conv2d: more than 2^31 output pixels");
  const int kp = (p->kh * p->kw * p->c_pad + 15) / 16 * 16;  // patch-matrix row length / packed-filter row pitch
  long long lda = kp;                                        // patch-matrix row pitch
  const void* a_ptr = p->x;
  const bool im2col = IsIm2col(*p);
  const bool implicit = !im2col && !IsPointwise(*p) && IsImplicit(*p);
  if (implicit || im2col) {
    ITEXB_REQUIRE((reinterpret_cast<uintptr_t>(p->x) & 15) == 0, ITEXB_INVALID_ARGUMENT, "conv2d: input must be 16-byte aligned");
  } else if (!IsPointwise(*p)) {
    ITEXB_REQUIRE(p->workspace != nullptr, ITEXB_INVALID_ARGUMENT, "conv2d: workspace of %zu bytes is required",
                  itexb_conv2d_workspace_bytes(p));
    ITEXB_REQUIRE((reinterpret_cast<uintptr_t>(p->workspace) & 15) == 0, ITEXB_INVALID_ARGUMENT,
                  "conv2d: workspace must be 16-byte aligned");
    GatherArgs a{};
    a.x = static_cast<const uint8_t*>(p->x);
    a.ws = static_cast<uint8_t*>(p->workspace);
    a.n = p->n; a.h = p->h; a.w = p->w; a.c = p->c; a.kh = p->kh; a.kw = p->kw; a.oh = p->oh; a.ow = p->ow; a.c_pad = p->c_pad;
    a.stride_h = p->stride_h; a.stride_w = p->stride_w; a.dil_h = p->dil_h; a.dil_w = p->dil_w;
    a.pad_top = p->pad_top; a.pad_left = p->pad_left;
    a.m = m;
    a.chunks = kp / 16;
    const bool vec = p->c % 16 == 0 && p->c_pad == p->c && (reinterpret_cast<uintptr_t>(p->x) & 15) == 0;
    const long long work = vec ? m * a.chunks : m * (long long)p->kh;
    const int blocks = int(std::max<long long>(1, std::min<long long>((work + 255) / 256, (long long)SmCount() * 32)));
    if (vec) {
      GatherPatchesVecKernel<<<blocks, 256, 0, st>>>(a);
    } else if (IsStem(*p)) {
      ITEXB_REQUIRE((reinterpret_cast<uintptr_t>(p->x) & 3) == 0, ITEXB_INVALID_ARGUMENT, "conv2d: input must be 4-byte aligned");
      constexpr int kTP = 64;
      const int tiles_x = (p->ow + kTP - 1) / kTP;
      const int row_words = (((kTP - 1) * p->stride_w + 7) * 3 + 3) / 4 + 1;  // <= 2 * kTP for stride_w <= 2
      const size_t smem = (size_t(7) * row_words * 4 + 15) / 16 * 16 + size_t(kTP) * 160;  // input window + staged patch rows
      lda = (long long)PatchPitch(*p);
      GatherPatchesStemKernel<7, 7, 3, kTP><<<unsigned(p->n) * p->oh * tiles_x, kTP, smem, st>>>(a, int(lda));
    } else {
      GatherPatchesRowKernel<<<blocks, 256, 0, st>>>(a);
    }
    ITEXB_RETURN_IF_ERROR(CheckLaunch("GatherPatchesKernel"));
    a_ptr = p->workspace;
  } else {
    ITEXB_REQUIRE((reinterpret_cast<uintptr_t>(p->x) & 15) == 0, ITEXB_INVALID_ARGUMENT, "conv2d: input must be 16-byte aligned");
  }
  ITEXB_REQUIRE((reinterpret_cast<uintptr_t>(p->filter_packed) & 15) == 0, ITEXB_INVALID_ARGUMENT,
                "conv2d: packed filter must be 16-byte aligned");
  CUtensorMap ta, tb;
  const int bn = PickBN(p->co);
  ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tb, p->filter_packed, p->co, kp, kp, bn, 1, 0, (im2col && p->c_pad < 128) ? p->c_pad : 128));
  if (implicit) ta = tb;  // unused: the kernel gathers A itself
  else if (im2col) ITEXB_RETURN_IF_ERROR(EncodeIm2colMap(&ta, *p));
  // A patch matrix with padded rows is described to TMA as lda bytes wide: boxes that lie partly outside the
  // tensor are read at half the rate (measured 155 us against 83 us on the stem), and what the padding holds
  // does not matter - the filter's rows end at kp, so TMA zero-fills the filter bytes it is multiplied with.
  else ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&ta, a_ptr, m, lda, lda, 128));
  TailMaps tail;
  tail.box = (implicit || im2col) ? 0 : TailBox(kp);
  if (tail.box != 0) {
    ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tail.a, a_ptr, m, kp, lda, 128, 1, 0, tail.box));
    ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tail.b, p->filter_packed, p->co, kp, kp, bn, 1, 0, tail.box));
  }
  GemmArgs g{};
  if (implicit || im2col) {
    g.conv_mode = im2col ? kConvIm2col : kConvGather; g.conv_cpad = p->c_pad; g.conv_kh = p->kh; g.conv_c = p->c; g.conv_h = p->h; g.conv_w = p->w; g.kw = p->kw; g.oh = p->oh; g.ow = p->ow;
    g.stride_h = p->stride_h; g.stride_w = p->stride_w; g.dil_h = p->dil_h; g.dil_w = p->dil_w;
    g.pad_top = p->pad_top; g.pad_left = p->pad_left;
    g.conv_x = p->x;
  }
  g.m = int(m); g.n = p->co; g.k = kp;
  g.out_dtype = p->out_dtype;
  g.out = p->out; g.ldo = p->co;
  g.ep = p->ep;
  if (g.ep.summand != nullptr && g.ep.ld_summand == 0) g.ep.ld_summand = p->co;
  g.status_word = p->status_word;
  g.idesc = MakeInstrDesc(p->x_dtype, ITEXB_DT_QINT8, bn);
  return LaunchGemm(ta, tb, g, bn, false, st, tail.box != 0 ? &tail : nullptr);
}

// ---------------------------------------------------------------------------------------
// Convolution for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the moment they need a convolution:
// a plugin running inside another framework's memory arena (every byte on the device is
// already owned by that framework's allocator and a second allocator would fragment or
// exhaust it), code running between the begin and end of a stream capture (allocation is
// illegal there), or a latency-critical serving loop that has to be allocation-free by
// policy.  For them the patch matrix of the general lowering lives in a fixed array inside
// the library's own device image instead of in caller-provided scratch.
//
// The array costs ITEXB_STATIC_SCRATCH_BYTES on every GPU that loads the library, for the
// life of the process, so it is kept modest; convolutions that need more are refused with
// a clear status and must use itexb_conv2d with caller scratch.
//
// In host code `g_conv_scratch` is only a stand-in symbol, not a device address: handing it
// to a kernel would fault (or, where the GPU can reach host memory, silently use the wrong
// memory).  The real address is asked from the runtime once per device, with that device
// current, by cudaGetSymbolAddress.
// ---------------------------------------------------------------------------------------
namespace itexb {
namespace {

static __device__ __align__(256) unsigned char g_conv_scratch[ITEXB_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up on first use).
int StaticScratchAddress(void** ptr) {
  int dev = 0;
  ITEXB_CUDA(cudaGetDevice(&dev));
  ITEXB_REQUIRE(dev >= 0 && dev < kMaxDevices, ITEXB_INVALID_ARGUMENT, "conv2d_static_scratch: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    ITEXB_CUDA(cudaGetSymbolAddress(&p, g_conv_scratch));
    ITEXB_REQUIRE(p != nullptr, ITEXB_INTERNAL, "conv2d_static_scratch: cudaGetSymbolAddress returned a null address");
    g_scratch_ptr[dev] = p;
  }
  *ptr = g_scratch_ptr[dev];
  return ITEXB_OK;
}

}  // namespace
}  // namespace itexb

extern "C" int itexb_conv2d_static_scratch(const itexb_conv_params_t* p, itexb_stream_t stream) {
  ITEXB_REQUIRE(p != nullptr, ITEXB_INVALID_ARGUMENT, "conv2d_static_scratch: params is NULL");
  ITEXB_RETURN_IF_ERROR(Validate(*p));  // bad dimensions are an argument error, not a scratch-size one
  // The array's address is looked up on the current device, so the stream has to belong to it: a stream of another GPU
  // would run the kernels there with this GPU's address.
  int cur = 0, sdev = 0;
  ITEXB_CUDA(cudaGetDevice(&cur));
  if (stream != nullptr) {
    ITEXB_CUDA(cudaStreamGetDevice(AsCuda(stream), &sdev));
    ITEXB_REQUIRE(sdev == cur, ITEXB_INVALID_ARGUMENT,
                  "conv2d_static_scratch: the stream belongs to device %d but device %d is current; make the stream's device current", sdev, cur);
  }
  const size_t need = itexb_conv2d_workspace_bytes(p);
  ITEXB_REQUIRE(need <= size_t(ITEXB_STATIC_SCRATCH_BYTES), ITEXB_RESOURCE_EXHAUSTED,
                "conv2d_static_scratch: this convolution needs %zu bytes of scratch, the built-in array holds %zu; "
                "use itexb_conv2d with caller-provided scratch",
                need, size_t(ITEXB_STATIC_SCRATCH_BYTES));
  itexb_conv_params_t q = *p;
  q.workspace = nullptr;
  if (need > 0) ITEXB_RETURN_IF_ERROR(StaticScratchAddress(&q.workspace));
  // The gather kernel writes every byte of the region it uses (zeros where the window hangs
  // over the border), so nothing left by an earlier call can leak into this one.
  return itexb_conv2d(&q, stream);
}
