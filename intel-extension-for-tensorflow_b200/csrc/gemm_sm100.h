// Internal interface of the tcgen05 GEMM / implicit-GEMM convolution kernels.
#ifndef ITEXB_CSRC_GEMM_SM100_H_
#define ITEXB_CSRC_GEMM_SM100_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include "itexb200.h"

namespace itexb {

// Kernel argument block (by value in parameter space).
// Division by a divisor fixed per launch: see MakeFastDiv.
struct FastDiv { unsigned mul, shift; };
FastDiv MakeFastDiv(unsigned d);

struct GemmArgs {
  int m, n, k;          // k in bytes = elements (8-bit operands)
  int out_dtype;
  void* out;
  long long ldo;        // elements
  itexb_epilogue_t ep;
  int* status_word;     // set non-zero when a bounded wait expired
  long long wait_limit; // cycles a wait on one pipeline stage may take before the kernel gives up (set by LaunchGemm)
  long long wait_limit_acc;  // the same for the waits that sit behind the MMA issuer - the epilogue's on a whole accumulator,
                             // the producers' on a stage's release: twice as long, so that the role that is actually
                             // starved reports first (set by LaunchGemm)
  int debug_skip_kb;    // test hook: the producer leaves out this k-block of each CTA's first tile (-1: none; set by LaunchGemm)
  unsigned idesc;       // tcgen05 instruction descriptor
  int vec_store;        // output rows are 16-byte aligned (set by LaunchGemm)
  int tma_store;        // epilogue writes through shared memory + TMA stores (set by LaunchGemm)
  int out_esz;          // bytes per output element (set by LaunchGemm)
  int out_kind;         // epilogue instantiation (set by LaunchGemm)
  int ep_mode;          // epilogue loop specialisation (set by LaunchGemm)
  int preset;           // accumulators start from the bit pattern of 1.5 * 2^23 instead of zero (set by LaunchGemm)
  int tail_box;         // 0, or the width (64 | 32 bytes) of a narrower last k-block (set by LaunchGemm)
  int group_m;          // tile rows per rasterisation group (set by LaunchGemm)
  FastDiv div_per_batch, div_per_group, div_group_m;  // dividers of the tile walk (set by LaunchGemm)
  int num_peers;        // fused all-gather: every output block is also stored to the same offset of peer_out[0 .. num_peers)
  void* peer_out[ITEXB_MAX_PEERS];
  int batch;            // independent GEMMs in this launch (third coordinate of the tensor maps); 0 is read as 1
  long long batch_rows_out;  // rows of `out` (and of the summand) from one batch to the next
  unsigned long long neg_zero2;  // two fp32 -0 (set by LaunchGemm): a run-time value the assembler cannot fold
  // Implicit-GEMM convolution (conv_mode != kConvNone): row m of A is output pixel m of the NHWC tensor
  // conv_x; column k = tap * conv_cpad + channel, tap = ky * kw + kx.  kConvGather: conv_cpad == conv_c and
  // four extra warps gather the A tile with cp.async.  kConvIm2col: conv_cpad is conv_c rounded up to 128
  // and the A tile of a k-block (one tap, 128 channels) is one TMA im2col load through the map `ta`.
  int conv_mode, conv_cpad;
  int conv_c, conv_h, conv_w, conv_kh, kw, oh, ow;
  int stride_h, stride_w, dil_h, dil_w, pad_top, pad_left;
  const void* conv_x;
};

enum : int { kConvNone = 0, kConvGather = 1, kConvIm2col = 2 };

// 4-D im2col tensor map over an NHWC 8-bit tensor: box = 128 channels x 128 pixels, 128-byte swizzle,
// zero fill outside; the pixel bounding box and traversal strides describe the convolution.
int EncodeIm2colMap(CUtensorMap* map, const itexb_conv_params_t& p);
// 3-D tiled tensor map over a (batched) K-major 8-bit operand: dims {k, rows, batch}, row pitch `ld` bytes, batch pitch
// batch_stride bytes, box {128 bytes, box_rows, 1}, 128-byte
// swizzle, zero fill outside.
// box_k: bytes of K per box - 128 (128-byte swizzle), or 64 / 32 with the swizzle of that width for a narrow last k-block.
int EncodeOperandMap(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows, int64_t batch = 1,
                     int64_t batch_stride = 0, int box_k = 128);
// A last k-block of at most 64 bytes (k % 128 in 16..64) is loaded through its own pair of maps with 64- or 32-byte
// boxes: TMA reads boxes that lie partly outside the tensor at a fraction of its normal rate, and the narrow tile
// is half or a quarter of the shared-memory fill and MMA work.  TailBox returns 64, 32, or 0 when K has no such tail.
struct TailMaps { CUtensorMap a, b; int box; };
int TailBox(int64_t k);
unsigned MakeInstrDesc(int a_dtype, int b_dtype, int bn, int rows = 128);
int PickBN(int n);
// cg = 2: a pair of CTAs per 256 x bn tile; `tb` (and the tail's) then has boxes of bn / 2 rows and g.idesc 256 rows.
int LaunchGemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, int bn, bool f8, cudaStream_t st, const TailMaps* tail = nullptr,
               int cg = 1);
int ValidateEpilogue(const char* who, const itexb_epilogue_t& ep, int out_dtype, bool f8, int n);

}  // namespace itexb

#endif  // ITEXB_CSRC_GEMM_SM100_H_
