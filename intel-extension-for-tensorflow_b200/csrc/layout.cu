// Transposition of quantized tensors for sm_100a: the data movement between the quantized matmuls of a
// transformer graph ([B,S,H,D] <-> [B,H,S,D], K^T).  HBM-bound byte work: every path reads and writes whole
// 16-byte (or at least 4-byte) units per lane.
#include <algorithm>

#include "common.h"

namespace itexb {
namespace {

constexpr int kMaxRank = ITEXB_TRANSPOSE_MAX_RANK;

struct Shape {
  int rank;
  long long out_dims[kMaxRank];    // extents of the output, outermost first
  long long in_stride[kMaxRank];   // input stride (in units) of each output dimension
};

// The innermost dimension keeps its place: the tensor is a permutation of rows of 16-byte units.  IDX = unsigned when
// the unit count fits 32 bits (the divisions of the index walk are then a fraction of the 64-bit ones' cost).
template <typename IDX>
__global__ void __launch_bounds__(256) PermuteRowsKernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long total, Shape s) {
  const IDX stride = IDX(gridDim.x) * blockDim.x;
  for (IDX i = IDX(blockIdx.x) * blockDim.x + threadIdx.x; i < IDX(total); i += stride) {
    IDX rest = i, src = 0;
#pragma unroll 1
    for (int d = s.rank - 1; d >= 0; --d) {
      const IDX ext = IDX(s.out_dims[d]);
      const IDX q = rest / ext;
      src += (rest - q * ext) * IDX(s.in_stride[d]);
      rest = q;
    }
    __stcs(y + i, __ldcs(x + src));
  }
}

// Rows of `width` 16-byte units copied from a dense source into a destination with a longer row pitch, starting at unit
// `col0` of every destination row: one input of a concatenation along an inner axis.
__global__ void __launch_bounds__(256) CopyRowsKernel(const uint4* __restrict__ x, uint4* __restrict__ y, unsigned total, unsigned width,
                                                      unsigned dpitch, unsigned col0) {
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const unsigned r = i / width;
    __stcs(y + (size_t)r * dpitch + col0 + (i - r * width), __ldcs(x + i));
  }
}

// Batched transposition of the two innermost dimensions of a byte tensor, [batch, rows, cols] -> [batch, cols, rows],
// in 64 x 64 tiles.  A thread loads a 4 x 4 block of bytes as four words (a half-warp reads 64 contiguous bytes of a
// row), transposes it in registers with byte permutes, and leaves the four words of the transposed block in shared
// memory; after the barrier every thread assembles 16 contiguous bytes of one output row, so four lanes write a
// whole 64-byte run.  Edge tiles and unaligned rows go byte by byte.
__global__ void __launch_bounds__(256) TransposeBytes2dKernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, long long rows,
                                                              long long cols, Shape outer) {
  __shared__ uint32_t tile[64 * 16];  // [output row within the tile][word], words XOR-swizzled by (row >> 2)
  // blockIdx.z walks the outer (batch) dimensions of the OUTPUT; their input offset comes from the strides
  long long rest = blockIdx.z, boff = 0;
#pragma unroll 1
  for (int d = outer.rank - 1; d >= 0; --d) {
    const long long q = rest / outer.out_dims[d];
    boff += (rest - q * outer.out_dims[d]) * outer.in_stride[d];
    rest = q;
  }
  const uint8_t* xb = x + boff;
  uint8_t* yb = y + (long long)blockIdx.z * rows * cols;
  const long long r0 = (long long)blockIdx.y * 64, c0 = (long long)blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // the thread's 4 x 4 block: rows 4ty.., columns 4tx..
  const bool full = r0 + 64 <= rows && c0 + 64 <= cols && (cols & 3) == 0 && (rows & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(xb) & 3) == 0 && (reinterpret_cast<uintptr_t>(yb) & 15) == 0;
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long r = r0 + 4 * ty + j, c = c0 + 4 * tx;
    if (full) {
      w[j] = *reinterpret_cast<const uint32_t*>(xb + r * cols + c);
    } else {
      w[j] = 0u;
      for (int b = 0; b < 4; ++b)
        if (r < rows && c + b < cols) w[j] |= uint32_t(xb[r * cols + c + b]) << (8 * b);
    }
  }
  // 4 x 4 byte transposition: t[k] holds byte k of w[0..3]
  const uint32_t a0 = __byte_perm(w[0], w[1], 0x5140), a1 = __byte_perm(w[0], w[1], 0x7362);  // (w0.b0 w1.b0 w0.b1 w1.b1), (.. b2 .. b3)
  const uint32_t b0 = __byte_perm(w[2], w[3], 0x5140), b1 = __byte_perm(w[2], w[3], 0x7362);
  const uint32_t t[4] = {__byte_perm(a0, b0, 0x5410), __byte_perm(a0, b0, 0x7632), __byte_perm(a1, b1, 0x5410), __byte_perm(a1, b1, 0x7632)};
#pragma unroll
  for (int k = 0; k < 4; ++k) tile[(4 * tx + k) * 16 + (ty ^ tx)] = t[k];  // output row 4tx + k, bytes 4ty .. 4ty+3
  __syncthreads();
  const int orow = threadIdx.x >> 2, q = threadIdx.x & 3;  // 16 bytes: output row orow, input rows 16q .. 16q+15
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = tile[orow * 16 + ((4 * q + i) ^ (orow >> 2))];
  const long long c = c0 + orow, r = r0 + 16 * q;
  if (full) {
    __stcs(reinterpret_cast<uint4*>(yb + c * rows + r), make_uint4(o[0], o[1], o[2], o[3]));
  } else if (c < cols) {
    for (int b = 0; b < 16; ++b)
      if (r + b < rows) yb[c * rows + r + b] = uint8_t(o[b >> 2] >> (8 * (b & 3)));
  }
}

// Anything else: one element of `esz` bytes per thread, writes coalesced.
__global__ void __launch_bounds__(256) PermuteElementsKernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, long long total, int esz,
                                                             Shape s) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long rest = i, src = 0;
#pragma unroll 1
    for (int d = s.rank - 1; d >= 0; --d) {
      const long long q = rest / s.out_dims[d];
      src += (rest - q * s.out_dims[d]) * s.in_stride[d];
      rest = q;
    }
    for (int b = 0; b < esz; ++b) y[i * esz + b] = x[src * esz + b];
  }
}

}  // namespace
}  // namespace itexb

using namespace itexb;

extern "C" int itexb_transpose(const itexb_transpose_params_t* p, itexb_stream_t stream) {
  ITEXB_REQUIRE(p != nullptr, ITEXB_INVALID_ARGUMENT, "transpose: params is NULL");
  ITEXB_REQUIRE(p->rank >= 0 && p->rank <= kMaxRank, ITEXB_INVALID_ARGUMENT, "transpose: rank must be 0..%d, got %d", kMaxRank, p->rank);
  ITEXB_REQUIRE(p->elem_size == 1 || p->elem_size == 2 || p->elem_size == 4, ITEXB_INVALID_ARGUMENT, "transpose: elem_size must be 1, 2 or 4");
  long long total = 1;
  bool seen[kMaxRank] = {};
  for (int d = 0; d < p->rank; ++d) {
    ITEXB_REQUIRE(p->dims[d] >= 0, ITEXB_INVALID_ARGUMENT, "transpose: negative dimension");
    ITEXB_REQUIRE(p->perm[d] >= 0 && p->perm[d] < p->rank && !seen[p->perm[d]], ITEXB_INVALID_ARGUMENT,
                  "transpose: perm is not a permutation of 0..%d", p->rank - 1);
    seen[p->perm[d]] = true;
    total *= p->dims[d];
  }
  if (total == 0) return ITEXB_OK;
  ITEXB_REQUIRE(p->x != nullptr && p->y != nullptr, ITEXB_INVALID_ARGUMENT, "transpose: NULL tensor");
  cudaStream_t st = AsCuda(stream);
  // input strides in elements, then the output's view: extent and input stride per output dimension, with extent-1
  // dimensions dropped and output dimensions that are also adjacent in the input merged
  long long in_stride[kMaxRank];
  {
    long long sdim = 1;
    for (int d = p->rank - 1; d >= 0; --d) { in_stride[d] = sdim; sdim *= p->dims[d]; }
  }
  long long od[kMaxRank], os[kMaxRank];
  int r = 0;
  for (int d = 0; d < p->rank; ++d) {
    const long long ext = p->dims[p->perm[d]], str = in_stride[p->perm[d]];
    if (ext == 1) continue;
    if (r > 0 && os[r - 1] == ext * str) { od[r - 1] *= ext; os[r - 1] = str; }  // previous dimension steps over exactly this one
    else { od[r] = ext; os[r] = str; ++r; }
  }
  if (r == 0 || (r == 1 && os[0] == 1)) {  // the permutation moves nothing
    ITEXB_CUDA(cudaMemcpyAsync(p->y, p->x, size_t(total) * p->elem_size, cudaMemcpyDeviceToDevice, st));
    return ITEXB_OK;
  }
  const int esz = p->elem_size;
  const auto grid_for = [](long long n) { return int(std::max<long long>(1, std::min<long long>((n + 255) / 256, (long long)SmCount() * 16))); };
  // (1) the innermost dimension stays innermost and is a whole number of 16-byte units
  if (os[r - 1] == 1 && (od[r - 1] * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(p->x) & 15) == 0 && (reinterpret_cast<uintptr_t>(p->y) & 15) == 0) {
    bool ok = true;
    Shape s{};
    s.rank = r;
    const long long unit = 16 / esz;  // elements per 16-byte unit
    for (int d = 0; d < r; ++d) {
      s.out_dims[d] = d == r - 1 ? od[d] / unit : od[d];
      if (d < r - 1 && os[d] % unit != 0) ok = false;
      s.in_stride[d] = d == r - 1 ? 1 : os[d] / unit;
    }
    if (ok) {
      const long long units = total / unit;
      if (units < (1ll << 31))
        PermuteRowsKernel<unsigned><<<grid_for(units), 256, 0, st>>>(static_cast<const uint4*>(p->x), static_cast<uint4*>(p->y), units, s);
      else
        PermuteRowsKernel<long long><<<grid_for(units), 256, 0, st>>>(static_cast<const uint4*>(p->x), static_cast<uint4*>(p->y), units, s);
      return CheckLaunch("PermuteRowsKernel");
    }
  }
  // (2) bytes, the two innermost output dimensions are the two innermost input dimensions swapped
  if (esz == 1 && r >= 2 && os[r - 2] == 1 && os[r - 1] == od[r - 2]) {
    const long long rows = od[r - 1], cols = od[r - 2];  // of the INPUT's inner matrix [rows, cols]
    long long batches = 1;
    Shape outer{};
    outer.rank = r - 2;
    for (int d = 0; d < r - 2; ++d) { outer.out_dims[d] = od[d]; outer.in_stride[d] = os[d]; batches *= od[d]; }
    if (batches <= 65535 && (rows + 63) / 64 <= 65535) {
      dim3 grid(unsigned((cols + 63) / 64), unsigned((rows + 63) / 64), unsigned(batches));
      TransposeBytes2dKernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(p->x), static_cast<uint8_t*>(p->y), rows, cols, outer);
      return CheckLaunch("TransposeBytes2dKernel");
    }
  }
  // (3) anything else
  Shape s{};
  s.rank = r;
  for (int d = 0; d < r; ++d) { s.out_dims[d] = od[d]; s.in_stride[d] = os[d]; }
  PermuteElementsKernel<<<grid_for(total), 256, 0, st>>>(static_cast<const uint8_t*>(p->x), static_cast<uint8_t*>(p->y), total, esz, s);
  return CheckLaunch("PermuteElementsKernel");
}

// One input of a concatenation: `outer` rows of `width` bytes into rows of `dpitch` bytes at byte offset `col`.
extern "C" int itexb_copy_rows(const void* src, void* dst, int64_t outer, int64_t width, int64_t dpitch, int64_t col, itexb_stream_t stream) {
  ITEXB_REQUIRE(outer >= 0 && width >= 0 && dpitch >= width && col >= 0 && col + width <= dpitch, ITEXB_INVALID_ARGUMENT, "copy_rows: bad geometry");
  if (outer == 0 || width == 0) return ITEXB_OK;
  ITEXB_REQUIRE(src != nullptr && dst != nullptr, ITEXB_INVALID_ARGUMENT, "copy_rows: NULL pointer");
  cudaStream_t st = AsCuda(stream);
  const long long units = outer * (width / 16);
  if (((width | dpitch | col) & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0 && units < (1ll << 31) &&
      outer * (dpitch / 16) < (1ll << 40)) {
    const int grid = int(std::max<long long>(1, std::min<long long>((units + 255) / 256, (long long)SmCount() * 16)));
    CopyRowsKernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), unsigned(units), unsigned(width / 16),
                                         unsigned(dpitch / 16), unsigned(col / 16));
    return CheckLaunch("CopyRowsKernel");
  }
  ITEXB_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(dst) + col, size_t(dpitch), src, size_t(width), size_t(width), size_t(outer),
                               cudaMemcpyDeviceToDevice, st));
  return ITEXB_OK;
}
