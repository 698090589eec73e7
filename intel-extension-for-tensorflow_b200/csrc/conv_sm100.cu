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

// Few-channel stem convolutions (e.g. 7x7x3, stride 2): the filter shape is a template parameter,
// so every byte position of the 16-byte-aligned patch row is a compile-time offset into a
// shared-memory copy of the input window.  A block builds TP consecutive output pixels of one
// output row: it loads the KH input rows they touch once (coalesced), then each thread assembles
// its patch row in registers and writes it as 16-byte vectors.  Dilation 1.
template <int KH, int KW, int C, int TP>
__global__ void __launch_bounds__(TP) GatherPatchesStemKernel(GatherArgs a) {
  constexpr int kRun = KW * C;                         // bytes of one filter row
  constexpr int kRowPitch = (KH * kRun + 15) / 16 * 16;  // patch-matrix pitch
  extern __shared__ __align__(16) uint8_t s_in[];      // [KH][span * C], then the staged patch rows
  const int tiles_x = (a.ow + TP - 1) / TP;
  const int tile = blockIdx.x % tiles_x;
  const int oy = (blockIdx.x / tiles_x) % a.oh;
  const int b = blockIdx.x / (tiles_x * a.oh);
  const int ox0 = tile * TP;
  const int span = (TP - 1) * a.stride_w + KW;         // input columns the tile touches
  const int ix0 = ox0 * a.stride_w - a.pad_left;
  const int row_bytes = span * C;
  for (int i = threadIdx.x; i < KH * row_bytes; i += TP) {
    const int ky = i / row_bytes, r = i - ky * row_bytes;
    const int ix = ix0 + r / C, ci = r % C;
    const int iy = oy * a.stride_h + ky - a.pad_top;
    uint8_t v = 0;
    if (iy >= 0 && iy < a.h && ix >= 0 && ix < a.w) v = __ldg(a.x + (((long long)b * a.h + iy) * a.w + ix) * C + ci);
    s_in[i] = v;
  }
  __syncthreads();
  // Each thread assembles the patch row of one pixel into the shared staging tile; the block then
  // writes the tile - TP consecutive patch rows are one contiguous run of the patch matrix - with
  // consecutive threads on consecutive 16-byte units, so that every store instruction fills whole
  // sectors (a thread storing its own row would write 16 bytes every kRowPitch bytes).
  uint4* s_out = reinterpret_cast<uint4*>(s_in + ((KH * row_bytes + 15) / 16) * 16);
  const uint8_t* base = s_in + threadIdx.x * a.stride_w * C;
  uint4* dst = s_out + threadIdx.x * (kRowPitch / 16);
#pragma unroll
  for (int u = 0; u < kRowPitch / 16; ++u) {
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t word = 0;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        constexpr int dummy = 0;
        const int k = u * 16 + q * 4 + t;               // compile-time after unrolling
        if (k < KH * kRun) word |= uint32_t(base[(k / kRun) * row_bytes + (k % kRun)]) << (8 * t);
        (void)dummy;
      }
      w[q] = word;
    }
    dst[u] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __syncthreads();
  const int pixels = min(TP, a.ow - ox0);
  uint4* out = reinterpret_cast<uint4*>(a.ws + (((long long)b * a.oh + oy) * a.ow + ox0) * kRowPitch);
  for (int i = threadIdx.x; i < pixels * (kRowPitch / 16); i += TP) out[i] = s_out[i];
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
int FilterCPad(const itexb_conv_params_t& p) { return Im2colGeometryOk(p) ? (p.c + 127) / 128 * 128 : p.c; }

bool IsIm2col(const itexb_conv_params_t& p) { return Im2colGeometryOk(p) && p.c_pad == (p.c + 127) / 128 * 128; }

int Validate(const itexb_conv_params_t& p) {
  ITEXB_REQUIRE(p.n >= 0 && p.h > 0 && p.w > 0 && p.c > 0 && p.kh > 0 && p.kw > 0 && p.co > 0, ITEXB_INVALID_ARGUMENT,
                "conv2d: bad tensor dimensions");
  ITEXB_REQUIRE(p.stride_h > 0 && p.stride_w > 0 && p.dil_h > 0 && p.dil_w > 0, ITEXB_INVALID_ARGUMENT,
                "conv2d: strides and dilations must be positive");
  ITEXB_REQUIRE(p.oh > 0 && p.ow > 0, ITEXB_INVALID_ARGUMENT, "conv2d: empty output");
  ITEXB_REQUIRE(p.c_pad == p.c || (p.c_pad == (p.c + 127) / 128 * 128 && Im2colGeometryOk(p)), ITEXB_INVALID_ARGUMENT,
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

extern "C" size_t itexb_conv2d_workspace_bytes(const itexb_conv_params_t* p) {
  if (p == nullptr || IsPointwise(*p) || IsIm2col(*p) || IsImplicit(*p)) return 0;
  return size_t(p->n) * p->oh * p->ow * ((size_t(p->kh) * p->kw * p->c_pad + 15) / 16 * 16);
}

extern "C" int itexb_conv2d(const itexb_conv_params_t* p, itexb_stream_t stream) {
  ITEXB_REQUIRE(p != nullptr, ITEXB_INVALID_ARGUMENT, "conv2d: params is NULL");
  ITEXB_RETURN_IF_ERROR(Validate(*p));
  if (p->n == 0) return ITEXB_OK;
  ITEXB_REQUIRE(p->x && p->filter_packed && p->out, ITEXB_INVALID_ARGUMENT, "conv2d: NULL tensor");
  cudaStream_t st = AsCuda(stream);
  const long long m = (long long)p->n * p->oh * p->ow;
  ITEXB_REQUIRE(m < (1ll << 31), ITEXB_INVALID_ARGUMENT, "conv2d: more than 2^31 output pixels");
  const int kp = (p->kh * p->kw * p->c_pad + 15) / 16 * 16;  // patch-matrix / packed-filter row pitch
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
    } else if (p->kh == 7 && p->kw == 7 && p->c == 3 && p->dil_h == 1 && p->dil_w == 1 && p->stride_w <= 4) {
      constexpr int kTP = 64;
      const int tiles_x = (p->ow + kTP - 1) / kTP;
      const size_t smem = (size_t(7) * ((kTP - 1) * p->stride_w + 7) * 3 + 15) / 16 * 16 + size_t(kTP) * 160;  // input window + staged patch rows
      GatherPatchesStemKernel<7, 7, 3, kTP><<<unsigned(p->n) * p->oh * tiles_x, kTP, smem, st>>>(a);
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
  ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tb, p->filter_packed, p->co, kp, kp, bn));
  if (implicit) ta = tb;  // unused: the kernel gathers A itself
  else if (im2col) ITEXB_RETURN_IF_ERROR(EncodeIm2colMap(&ta, *p));
  else ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&ta, a_ptr, m, kp, kp, 128));
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
  return LaunchGemm(ta, tb, g, bn, false, st);
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
