// int8 / FP8 GEMM for sm_100a: out[m][n] = epilogue(sum_k a[m][k] * b[n][k]).
//
// One persistent CTA per SM (640 threads; 768 in the cp.async convolution variant), warp-specialised:
//   warp 0      TMA producer   cp.async.bulk.tensor -> smem ring of 128 x 128-byte A tiles and BN x 128-byte
//                              B tiles (128-byte swizzle).  A is a tiled load of a matrix or, for
//                              convolutions, a 4-D im2col load of the NHWC input (one filter tap x 128
//                              channels per k-block).  A last k-block of at most 64 bytes, and every
//                              k-block of a convolution whose taps have at most 64 channels, is 64 or 32
//                              bytes wide with the swizzle of that width
//   warp 1      MMA issuer     tcgen05.mma.cta_group::1.kind::i8 | kind::f8f6f4, 128 x BN x 32 per
//                              instruction, operands read from smem through UMMA descriptors,
//                              accumulators (s32 | f32) in tensor memory
//   warp 2      TMEM allocator (2 accumulator stages of BN columns, so the epilogue of tile i
//                              overlaps the main loop of tile i+1)
//   warps 4-19  epilogue       four warps per TMEM lane quarter (= four per scheduler); each takes every
//                              fourth column block: tcgen05.ld (32 lanes x 16 columns) -> scale / bias
//                              (staged in smem per tile column) / sum / ReLU / activation -> conversion ->
//                              swizzled staging tile in smem -> one TMA store per block (direct stores
//                              when rows are unaligned).  The loop is compiled in three forms (plain,
//                              8-bit summand, general) and chosen per launch
//   warps 20-23 (convolutions with densely packed filters only) gather the A tile with cp.async
// Pipelines are mbarrier based: full[s]/empty[s] between producer and MMA issuer
// (tcgen05.commit releases a stage), tmem_full[a]/tmem_empty[a] between MMA issuer and
// epilogue.  Every wait is bounded: on expiry the kernel raises a status word, all roles
// leave their loops, TMEM is released and the kernel returns.
//
// Epilogue arithmetic: int->float uses the exact 1.5*2^23 adder trick (the conversion instructions
// run on the multi-function unit, the slowest pipe of this part and the first measured bottleneck),
// with the real conversion kept for accumulators beyond 2^22 (in the plain loop the accumulators start
// from that bit pattern, so the tensor core does the add); float->8-bit is one conversion to s32 per
// element and a saturating pack per pair.  Multiply and add stay separate roundings (bit-exactness with
// oneDNN).  The kernel is launched with programmatic stream serialization: everything before
// griddepcontrol.wait may overlap the previous kernel of the stream.
//
// No cluster launch and no multicast loads are used, so the same code runs unchanged in
// single- and multi-GPU jobs.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <string>

#include "common.h"
#include "fp8_cast.h"
#include "gemm_sm100.h"

namespace itexb {
namespace {

constexpr int kBM = 128;          // rows of a per tile = TMEM lanes
constexpr int kBK = 128;          // bytes of K per pipeline stage (one 128-byte swizzle row)
constexpr int kUmmaK = 32;        // bytes of K per tcgen05.mma
constexpr int kEpilogueWarps = 16;     // four per TMEM lane quarter = four per scheduler: their instruction streams hide each other's latencies
constexpr int kFirstGatherWarp = 4 + kEpilogueWarps;
constexpr int kThreads = 32 * kFirstGatherWarp;          // 4 control warps + the epilogue warps
constexpr int kThreadsConv = kThreads + 128;            // ... + 4 warps that gather the convolution's A operand (one thread per tile row)
constexpr int kGatherThreads = 128;
constexpr int kStagingPerWarp = 2048;  // bytes of output staging each epilogue warp owns
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr long long kWaitLimitCycles = 4000000000ll;  // ~2 s at 2 GHz; the default of GemmArgs::wait_limit

enum : int { kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3, kErrSmemAlign = 4 };

// CG = 2: a pair of CTAs (a cluster of two) works on one 256 x BN tile.  Each CTA holds 128 rows of A, HALF of the B
// tile and the accumulators of its own 128 rows; the tensor cores of the pair read both halves of B, so a CTA fetches a
// third less per k-block and the ring is deeper.
template <int BN, int CG = 1> struct Cfg {
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = (BN / CG) * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;   // 4 (BN=256), 6 (128; 256 as a pair), 8 (64)
  // Accumulators in tensor memory: 2 stages of SUP sub-tiles of BN columns (a power of two >= 32, at most the 512 there are).
  template <int SUP> static constexpr int kTmemCols = 2 * BN * SUP < 32 ? 32 : 2 * BN * SUP;
  static constexpr int kSumBars = kEpilogueWarps * 4;          // one per epilogue warp and staging buffer (summand loads)
  static constexpr int kAccBars = 2 * 4;                       // accumulator full / empty barriers: 2 stages x up to 4 sub-tiles
  static constexpr int kBarrierBytes = (2 * kStages + 2 * kAccBars + 2 + kSumBars) * 8 + 16;
  static constexpr int kParamBytes = 2 * BN * 4;               // the tile's per-column scales and biases
  static constexpr int kStagingBytes = kEpilogueWarps * kStagingPerWarp;
  // No slack for aligning the base: dynamic shared memory is declared 1024-byte aligned and the kernel checks it.
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kParamBytes + kBarrierBytes;
  static_assert(kSmemBytes <= 232448, "over the 227 KB a block may have");
};

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarArriveExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the wait expired or another role already gave up;
// in the first case it also publishes `code` to the status word.
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word, int code,
                                         const long long& limit) {
  if (MbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (MbarTryWait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {  // read from the kernel's parameter space only here, every 256 polls
        *abort_flag = 1;
        if (status_word != nullptr) atomicCAS(status_word, 0, code);
        return false;
      }
    }
  }
}

// ---- CTA pairs (CG = 2) ----
__device__ __forceinline__ uint32_t ClusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t MapToCta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrival on a barrier of either CTA of the pair.  What it publishes are tensor-memory reads, ordered by the
// tcgen05 fence before it, so the default semantics do (a cluster-scope release here was measured to cost the
// epilogue warps about a microsecond per tile).
__device__ __forceinline__ void MbarArriveCluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void ClusterSync() {
  __syncwarp();  // the aligned forms want the whole warp at the same instruction
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int N> __device__ __forceinline__ void CpAsyncWaitGroup() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void TmaLoad3d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// The same into this CTA's shared memory, but the bytes are counted on a barrier that may live in the pair's other CTA
// (`bar` is a shared::cluster address).
__device__ __forceinline__ void TmaLoad3dPair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// One k-block of a convolution's A operand: 128 channels from c0 of the pixels that start at
// base position (w, h, n) and follow the map's traversal strides, displaced by the filter tap's
// offset (off_w, off_h); positions outside the image read zeros.
__device__ __forceinline__ void TmaLoadIm2col(uint32_t dst, const void* tmap, uint32_t bar, int c0, int w, int h, int n, int off_w, int off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(w), "r"(h), "r"(n), "h"(uint16_t(off_w)), "h"(uint16_t(off_h))
      : "memory");
}

// CG = 2: one warp of EACH CTA of the pair issues these, with the same slot offset and column count.
template <int CG> __device__ __forceinline__ void TmemAlloc(uint32_t slot_smem, uint32_t cols) {
  if (CG == 2) asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
  else asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
template <int CG> __device__ __forceinline__ void TmemRelinquish() {
  if (CG == 2) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int CG> __device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t cols) {
  if (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Pair MMAs: one arrival on the barrier at shared::cluster address `bar` (either CTA's) once every MMA issued so far
// has completed in both CTAs.
__device__ __forceinline__ void TcCommitPair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <bool F8, int CG = 1>
__device__ __forceinline__ void UmmaSS(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (CG == 2) {
    // 256 x BN x 32 across the pair: rows 0-127 from this CTA's A tile into its tensor memory, rows 128-255 from the
    // other CTA's into that one's; B's rows 0 .. BN/2-1 from this CTA's shared memory, the rest from the other's.
    if (F8) {
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
          "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
          : "memory");
    } else {
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
          "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
          : "memory");
    }
    return;
  }
  if (F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  }
}

// K-major operand tile whose rows are 128 bytes, stored with the 128-byte swizzle TMA
// writes: 8-row groups are 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t UmmaDescSw128(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}
// The same for a tile whose rows are 64 or 32 bytes (64- / 32-byte swizzle): 8-row groups are 8 * row_bytes
// apart and the layout field says which swizzle the rows were written with (4: 64 bytes, 6: 32 bytes).
__device__ __forceinline__ uint64_t UmmaDescNarrow(uint32_t smem_addr, int row_bytes) {
  return uint64_t((smem_addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t((8 * row_bytes) >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(row_bytes == 64 ? 4 : 6) << 61);
}


// Tile rasterisation: the tile grid is walked in super-groups of group_m tile rows, column by column inside a
// group, so that the 148 tiles in flight share operand panels in L2.
// A batched launch lays the batches' tile grids one after the other.
// Every role walks the tile list once per tile, the sixteen epilogue warps included, and a 64-column tile is
// only one slice of work per warp: the four divisions here were a third of a narrow tile's instructions, so
// the three whose divisor is fixed for the launch use a multiplier prepared on the host (the fourth only
// differs in the last, shorter group).
__device__ __forceinline__ int DivBy(int x, const FastDiv& d) {  // x >= 0
  return d.mul == 0u ? x : int(__umulhi(uint32_t(x), d.mul) >> d.shift);
}
__device__ __forceinline__ void TileCoords(int t, const GemmArgs& g, int tiles_m, int tiles_n, int* tm, int* tn, int* batch) {
  const int per_batch = tiles_m * tiles_n;
  const int b = DivBy(t, g.div_per_batch);
  t -= b * per_batch;
  *batch = b;
  const int per_group = g.group_m * tiles_n;
  const int grp = DivBy(t, g.div_per_group);
  const int first_m = grp * g.group_m;
  const int r = t - grp * per_group;
  if (first_m + g.group_m <= tiles_m) {
    const int c = DivBy(r, g.div_group_m);
    *tn = c;
    *tm = first_m + (r - c * g.group_m);
  } else {
    const int rows = tiles_m - first_m;
    *tn = r / rows;
    *tm = first_m + r % rows;
  }
}

// ---------------------------------------------------------------------------------------
// Epilogue.  The unit of work is a slice: 32 rows (one per lane) x 16 columns.  The slice
// code is one short loop body that every slice of every tile re-executes, so it stays in the
// instruction cache (a fully unrolled 32-column body executed once per block was measured to
// be fetch-bound: ~3000 cycles per block for a few hundred instructions).  The output type
// is a template parameter, chosen once per launch; everything else is a uniform run-time flag.
// ---------------------------------------------------------------------------------------
constexpr float kMagic = 12582912.f;        // 1.5 * 2^23
constexpr int kMagicBits = 0x4B400000;

// int -> float is done on the fp32 adder with the 1.5*2^23 trick (exact for |a| <= 2^22), because the
// conversion instructions run on the multi-function unit, the slowest pipe of this part (measured
// 71 % busy, everything else idle, when every conversion went through it).
//
// float -> 8-bit: round-to-nearest-even conversion to s32 (out-of-range values clamp, NaN gives 0) and the saturating pack of
// four s32 into four 8-bit lanes: one conversion-unit instruction per element plus two packs per four,
// against two conversion-unit instructions per element for a direct float -> 8-bit conversion.
__device__ __forceinline__ int RneS32(float f) {
  int r;
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(r) : "f"(f));
  return r;
}
template <bool SIGNED> __device__ __forceinline__ uint32_t PackSat8(int e0, int e1, int e2, int e3) {
  uint32_t hi, r;
  if (SIGNED) {
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(e3), "r"(e2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(e1), "r"(e0), "r"(hi));
  } else {
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(e3), "r"(e2), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(e1), "r"(e0), "r"(hi));
  }
  return r;
}
// Low bytes of a, b, c, d -> one word (byte-permute unit: 3 instructions per 4 outputs).
__device__ __forceinline__ uint32_t PackLowBytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Packed fp32 pairs: one instruction rounds both lanes exactly like the scalar operation.
__device__ __forceinline__ uint64_t Pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void Unpack2(uint64_t p, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p)); }
__device__ __forceinline__ uint64_t Fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t Add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ bool DtypeIs8(int dt) {
  return dt == ITEXB_DT_QUINT8 || dt == ITEXB_DT_UINT8 || dt == ITEXB_DT_QINT8 || dt == ITEXB_DT_INT8;
}

__device__ __forceinline__ float LoadSummand(const void* p, int dt, long long idx) {
  switch (dt) {
    case ITEXB_DT_QUINT8: case ITEXB_DT_UINT8: return float(static_cast<const uint8_t*>(p)[idx]);
    case ITEXB_DT_QINT8: case ITEXB_DT_INT8: return float(int(static_cast<const int8_t*>(p)[idx]));
    case ITEXB_DT_BFLOAT16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    case ITEXB_DT_HALF: return __half2float(static_cast<const __half*>(p)[idx]);
    default: return static_cast<const float*>(p)[idx];
  }
}

// Columns of one epilogue block (the unit one warp converts, stages and stores with one TMA store).  The four warps
// that share a row quarter are spread over the sup sub-tiles of an accumulator stage, 4 / sup warps per sub-tile, and
// every one of them must find a block there.  Tiles of 128 or more columns: 16 columns of a 4-byte output, 32 of a
// narrower one.  64-column tiles: the tile's columns divided among its 4 / sup warps, at most 64 bytes per row - a
// single sub-tile per stage leaves each warp a 16-column block (stores of 16-byte row fragments, which is what
// stacking four sub-tiles per stage avoids: then one warp owns whole 64-column rows of one sub-tile).  The 8-bit
// summand loop wants two staging buffers per warp (the summand of the next block lands while this one is
// converted), which caps its rows at 32 bytes.
__host__ __device__ constexpr int OutBlockCols(int bn, int esz, int sup, bool sum8) {
  // 64-byte rows where that leaves every epilogue warp of a row quarter a block (8-bit outputs: 256-column tiles only;
  // 401408 x 256 x 64 -> u8 47.3 -> 45.3 us, 128-column tiles 14.5 -> 16.6 with two of four warps idle); the 8-bit
  // summand loop keeps 32-byte rows for its two buffers
  if (bn != 64) return esz == 4 ? 16 : ((esz == 1 && bn == 256 && !sum8) ? 64 : 32);
  int cols = bn / (4 / sup);                       // 16, 32 or 64
  const int max_cols = (sum8 ? 32 : 64) / esz;     // row bytes the staging buffers allow
  return cols < max_cols ? cols : (max_cols < 16 ? 16 : max_cols);
}
// Epilogue loop specialisations (template parameter, chosen per launch by LaunchGemm).
enum : int { kEpGeneral = 0, kEpPlain = 1, kEpSum8 = 2, kEpGelu = 3 };
// Output kinds (template parameter of the epilogue).
enum : int { kOutRaw = 0, kOutF32, kOutBF16, kOutF16, kOutS32, kOutU8, kOutS8, kOutFP8 };
template <int OK> struct OutBytes { static constexpr int v = (OK == kOutRaw || OK == kOutF32 || OK == kOutS32) ? 4 : ((OK == kOutBF16 || OK == kOutF16) ? 2 : 1); };

// 16 consecutive outputs of one row -> packed words (16, 8 or 4 of them).
template <int OK>
__device__ __forceinline__ void Convert16(const float (&v)[16], uint32_t (&w)[16], bool e4m3, float out_scale) {
  if (OK == kOutF32) {
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = __float_as_uint(v[j]);
  } else if (OK == kOutBF16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else if (OK == kOutF16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else if (OK == kOutS32) {
    // oneDNN converts the fp32 tail to s32 with saturation and RNE (rare output type: conversion unit).
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float f = v[j];
      w[j] = uint32_t(f >= 2147483648.f ? 2147483647 : (f <= -2147483648.f ? (-2147483647 - 1) : __float2int_rn(f)));
    }
  } else if (OK == kOutU8 || OK == kOutS8) {
    // One saturating conversion instruction per element.  Sending half of them through the main pipes instead
    // (clamp, clamp, magic add) to relieve the conversion unit was measured slower: issue slots, not that unit, limit.
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = PackSat8<OK == kOutS8>(RneS32(v[4 * j]), RneS32(v[4 * j + 1]), RneS32(v[4 * j + 2]), RneS32(v[4 * j + 3]));
  } else if (OK == kOutFP8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t q[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) q[t] = (uint32_t)FloatToFp8Bits(__fmul_rn(v[4 * j + t], out_scale), e4m3);
      w[j] = PackLowBytes(q[0], q[1], q[2], q[3]);
    }
  }
}

// 16 per-column parameters from the tile's staged copy in shared memory (all lanes read the same
// address: broadcast, no bank conflict).
__device__ __forceinline__ void LoadStaged16(const float* __restrict__ p, float (&out)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = reinterpret_cast<const float4*>(p)[i];
    out[4 * i] = t.x; out[4 * i + 1] = t.y; out[4 * i + 2] = t.z; out[4 * i + 3] = t.w;
  }
}

__device__ __forceinline__ void TmemLd16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Waits for this thread's outstanding tcgen05.ld.  The registers are listed as in/out
// operands so that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void TmemLdWait16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// Writes `value` to 16 consecutive TMEM columns of this warp's 32 lanes, and the wait for such stores.
__device__ __forceinline__ void TmemSt16Same(uint32_t taddr, uint32_t value) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
      "r"(value)
      : "memory");
}
__device__ __forceinline__ void TmemStWait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void TmaStore3d(const void* tmap, uint32_t src_smem, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap), "r"(src_smem), "r"(c0),
               "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void TmaStore2d(const void* tmap, uint32_t src_smem, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src_smem), "r"(c0),
               "r"(c1)
               : "memory");
}
__device__ __forceinline__ void TmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Blocks until at most `pending` of this thread's store groups are still reading shared memory.
__device__ __forceinline__ void TmaStoreWaitRead(int pending) {
  if (pending >= 3) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
  else if (pending == 2) asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
  else if (pending == 1) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
  else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void TmaStoreWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Element-wise post-op on 16 values, out of line so that the slice loop every launch executes stays
// short.  The switch is on a launch-uniform value and sits outside the unrolled loops, so a launch
// executes one short straight-line case.  The transcendental cases use the hardware exponential and reciprocal: a few ulp,
// inside the 1e-5 the parity tests allow.
#define ITEXB_ACT_CASE(KIND, EXPR)                                     \
  case KIND:                                                           \
    _Pragma("unroll") for (int j = 0; j < 16; ++j) {                   \
      const float x = v[j];                                            \
      v[j] = __fmul_rn((EXPR), post_scale);                            \
    }                                                                  \
    break;
__device__ __forceinline__ float GeluTanh(float x) {
  // 0.5 x (1 + tanh(u)) = x / (1 + exp(-2u)), u = sqrt(2/pi) (x + 0.044715 x^3)
  const float u = __fmul_rn(__fmul_rn(0.7978845608028654f, x), __fmaf_rn(0.044715f, __fmul_rn(x, x), 1.f));
  return __fdividef(x, __fadd_rn(1.f, __expf(__fmul_rn(-2.f, u))));
}
struct Float16 { float v[16]; };
__device__ __noinline__ Float16 ApplyActivation16(Float16 in, int kind, float alpha, float beta, float post_scale) {
  float (&v)[16] = in.v;
  switch (kind) {
    ITEXB_ACT_CASE(ITEXB_ACT_RELU, x > 0.f ? x : __fmul_rn(x, alpha))
    ITEXB_ACT_CASE(ITEXB_ACT_CLIP, fminf(fmaxf(x, alpha), beta))
    ITEXB_ACT_CASE(ITEXB_ACT_GELU_ERF, __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.f, erff(__fmul_rn(x, 0.70710678118654752f)))))
    ITEXB_ACT_CASE(ITEXB_ACT_GELU_TANH, GeluTanh(x))
    ITEXB_ACT_CASE(ITEXB_ACT_SIGMOID, __fdividef(1.f, __fadd_rn(1.f, __expf(-x))))
    ITEXB_ACT_CASE(ITEXB_ACT_TANH, tanhf(x))
    ITEXB_ACT_CASE(ITEXB_ACT_ELU, x > 0.f ? x : __fmul_rn(alpha, expm1f(x)))
    ITEXB_ACT_CASE(ITEXB_ACT_SWISH, __fdividef(x, __fadd_rn(1.f, __expf(__fmul_rn(-alpha, x)))))
    ITEXB_ACT_CASE(ITEXB_ACT_LINEAR, __fadd_rn(__fmul_rn(alpha, x), beta))
    default: break;
  }
  return in;
}
#undef ITEXB_ACT_CASE

// Fused all-gather.  The epilogue warps only store the tile locally (TMA stores, as in every launch).  Two warps that
// are otherwise idle copy each finished tile from the local output - still in L2 - to the same place of every
// peer's buffer: one 16-byte load per lane and row, then one 16-byte store per lane and peer, so that every store
// instruction of the warp writes 512 contiguous bytes of one row (NVLink wants long runs: the same bytes pushed as
// 64-byte row fragments straight from the epilogue's staging tiles, by per-lane stores or by TMA stores through peer
// tensor maps, moved at ~300 GB/s and held the epilogue up for as long).  The epilogue warps count a tile in
// `stored` once their stores of it have completed; the copying warps wait for 16 counts per tile.
__device__ __forceinline__ uint32_t LdAcquireShared(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(SmemAddr(p)) : "memory");
  return v;
}
__device__ __forceinline__ void RedReleaseShared(uint32_t* p, uint32_t v) {
  asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(SmemAddr(p)), "r"(v) : "memory");
}

// What an epilogue warp needs to know; filled once per launch.
struct EpilogueCtx {
  const float* scale;   // per-column scale vector or nullptr
  const float* bias;    // per-column bias vector or nullptr
  float scalar_scale;   // used when scale == nullptr (1 when there is no scale at all)
  bool acc_small;       // |accumulator| <= 2^22 follows from k alone
  bool relu;            // apply max(f, 0) (skipped when an unsigned clamp does it anyway)
  bool sum_bytes_vec;   // summand is 1-byte with 16-byte aligned rows: one 16-byte load per slice
  bool e4m3;            // FP8 output format
  float out_scale;      // FP8 output scale
  float post_scale;     // multiplier after the activation
  uint8_t* stage;       // this warp's staging memory
  uint32_t sum_flip;    // 8-bit summand: XOR mask (0x80 per byte when signed), the float bit pattern the bytes are
  uint32_t sum_base_bits;  //   dropped into, and the packed constant that takes the pattern's value off again
  uint64_t sum_off2;
};

// The persistent loop of one epilogue warp.  Warp (q, sub) owns TMEM lanes 32q..32q+31 (the
// quarter its warp id may read) and the column blocks sub, sub+4, ... of every tile.  A block
// is 16 columns of a 4-byte output or 32 columns of a narrower one; it is produced as 16-column
// slices into a swizzled staging tile (32 rows of 64 or 32 bytes) that one TMA store then
// writes; edges are clipped by the tensor map.  Without TMA-legal output rows the slices go
// straight to global memory.
template <int BN, bool F8, int OK, int MODE, int SUP, int CG>
__device__ __forceinline__ void EpilogueLoop(const GemmArgs& g, const CUtensorMap* tma_out, const CUtensorMap* tma_sum, uint32_t* stored,
                                             uint8_t* s_stage,
                                             float* s_par, uint64_t* tmem_full_bar, uint64_t* tmem_empty_bar, uint64_t* par_bar,
                                             uint64_t* sum_bar, volatile int* abort_flag, uint32_t tmem_base, int warp, int lane, int tiles_m,
                                             int tiles_n, int num_tiles) {
  constexpr int esz = OutBytes<OK>::v;
  constexpr int units = esz;                          // 16-byte units per 16-column slice
  constexpr int bcols = OutBlockCols(BN, esz, SUP, MODE == kEpSum8);  // columns per block
  constexpr int slices = bcols / 16;
  constexpr int row_bytes = bcols * esz;              // 64, 64, 32 (BN = 64: 64, 32, 16)
  constexpr int row_units = row_bytes / 16;
  constexpr int buf_bytes = 32 * row_bytes;
  constexpr int nbuf = kStagingPerWarp / buf_bytes;   // staging buffers per warp: 1 (64-byte rows), 2 or 4
  const int q = warp & 3;
  const int sub = (warp - 4) >> 2;
  constexpr int W = 4 / SUP;            // warps of a row quarter that share one sub-tile
  const int j = sub / W;                // this warp's sub-tile within every accumulator stage
  const int c_first = sub % W;          // ... and its first block there; it takes every W-th
  const int tiles_m_real = (g.m + kBM - 1) / kBM;  // tiles_m counts super rows of SUP * CG tile rows each
  // CTA pairs: the pair's unit is two consecutive tile rows, this CTA's is number `rank` of them; the accumulator-empty
  // barriers the MMA issuer waits on are those of the pair's first CTA.
  const int rank = CG == 2 ? int(ClusterCtaRank()) : 0;
  const int tfirst = int(blockIdx.x) / CG, tstep = int(gridDim.x) / CG;
  auto release_acc = [&](int a) {  // one arrival on accumulator stage a's empty barrier (the first CTA's, in a pair)
    if (CG == 2) MbarArriveCluster(MapToCta(SmemAddr(&tmem_empty_bar[a]), 0));
    else MbarArrive(SmemAddr(&tmem_empty_bar[a]));
  };
  constexpr bool PLAIN = MODE == kEpPlain || MODE == kEpGelu, SUM8 = MODE == kEpSum8;  // kEpGelu: the plain loop + tanh-GELU
  const bool tma_store = MODE != kEpGeneral || g.tma_store;
  EpilogueCtx e;
  const bool has_alpha = g.ep.alpha_a != nullptr && g.ep.alpha_b != nullptr;
  e.scalar_scale = 1.f;
  e.scale = nullptr;
  if (has_alpha) e.scalar_scale = __fmul_rn(__ldg(g.ep.alpha_a), __ldg(g.ep.alpha_b));
  else if (g.ep.scale_count == 1) e.scalar_scale = __ldg(g.ep.scale);
  else if (g.ep.scale_count > 1) e.scale = g.ep.scale;
  e.bias = g.ep.bias;
  e.acc_small = !F8 && (long long)g.k * 255 * 128 < (1ll << 22);
  e.relu = g.ep.relu && !(g.ep.mid_dtype == 0 && OK == kOutU8);  // max(f, 0) is implied by the clamp to [0, 255]
  e.sum_bytes_vec = g.ep.summand != nullptr && DtypeIs8(g.ep.summand_dtype) && g.ep.ld_summand % 16 == 0 &&
                    (reinterpret_cast<uintptr_t>(g.ep.summand) & 15) == 0;
  e.e4m3 = g.out_dtype == ITEXB_DT_FP8_E4M3;
  e.out_scale = g.ep.out_scale != nullptr ? __ldg(g.ep.out_scale) : 1.f;
  e.post_scale = g.ep.post_scale == 0.f ? 1.f : g.ep.post_scale;
  e.stage = s_stage + (warp - 4) * kStagingPerWarp;
  const bool sum_signed = g.ep.summand_dtype == ITEXB_DT_QINT8 || g.ep.summand_dtype == ITEXB_DT_INT8;
  e.sum_flip = sum_signed ? 0x80808080u : 0u;
  e.sum_base_bits = sum_signed ? uint32_t(kMagicBits) : 0x4B000000u;  // 1.5 * 2^23 | 2^23
  {
    const float off = sum_signed ? -(kMagic + 128.f) : -8388608.f;
    e.sum_off2 = Pack2(off, off);
  }
  const int swz = (lane / (8 / row_units)) % row_units;  // this lane's XOR term of the staging swizzle
  int acc = 0;
  uint32_t acc_phase = 0, seq = 0;
  float thread_amax = 0.f;
  // Per-column scale and bias of the current tile column live in shared memory (s_par[0..BN) scales,
  // s_par[BN..2BN) biases): fetched from global memory once per change of tile column by the 512
  // epilogue threads together, instead of once per slice by every warp (that global-load latency,
  // ~480 cycles per slice, was the largest single item of the epilogue).  par_bar[0] counts the warps
  // that have written their part, par_bar[1] the warps that are done reading the old contents.
  const bool staged = OK != kOutRaw;
  const int et = threadIdx.x - 4 * 32;      // 0..511 among the epilogue threads
  int last_tn = -1;
  uint32_t reloads = 0;

  // Preset accumulators (int8 kinds with a converting epilogue): both TMEM stages start out holding the bit
  // pattern of 1.5 * 2^23 in every column instead of zero and the MMA always accumulates, so what the epilogue
  // reads is already the float 1.5 * 2^23 + acc of the adder trick - the integer add per element is done by the
  // tensor core.  Each warp re-arms the columns it has read with one TMEM store per slice; the first arming
  // happens here and is published through the accumulator-empty barriers the MMA warp waits on.
  constexpr bool preset = !F8 && OK != kOutRaw && MODE != kEpGeneral;  // == g.preset, known at compile time here
  if (preset) {
    // each warp arms what it will read and re-arm later: its blocks of its sub-tile, in both stages
#pragma unroll 1
    for (int a = 0; a < 2; ++a)
#pragma unroll 1
      for (int c = c_first * bcols; c < BN; c += bcols * W)
#pragma unroll 1
        for (int sl = 0; sl < slices; ++sl)
          TmemSt16Same(tmem_base + uint32_t((a * SUP + j) * BN + c + 16 * sl) + (uint32_t(q * 32) << 16), uint32_t(kMagicBits));
    TmemStWait();
    TcFenceBefore();
    __syncwarp();
    if (lane == 0) {
      release_acc(j);
      release_acc(SUP + j);
    }
  }

  // Sum8: the summand block of an output block is brought by TMA into the very staging buffer the block's output
  // will be written to (same rows, same swizzle), one block ahead, so each lane finds its 16 summand bytes where
  // it is about to store its 16 output bytes: no per-lane global loads (they touched 32 half-used sectors per
  // instruction) and no latency on the slice's path.  sum_bar[buffer] completes when the block has landed.
  uint64_t* my_sum_bar = sum_bar + (warp - 4) * 4;
  bool give_up = false;
  bool sum_pref = false;  // the load for block number `seq` (the next one this warp processes) is already on its way
  auto issue_sum = [&](int col0, int brow0, int bbt, uint32_t s) {
    const uint32_t b = s & uint32_t(nbuf - 1);
    const uint32_t bar = SmemAddr(&my_sum_bar[b]);
    MbarArriveExpectTx(bar, uint32_t(buf_bytes));
    TmaLoad3d(SmemAddr(e.stage + b * buf_bytes), tma_sum, bar, col0 * esz, brow0, bbt);
  };

  for (int t = tfirst; t < num_tiles; t += tstep) {
    int tm, tn, bt;
    TileCoords(t, g, tiles_m, tiles_n, &tm, &tn, &bt);
    if (g.num_peers > 0 && t != tfirst && lane == 0) {
      // fused all-gather: this warp's stores of the previous tile have completed -> one count for the copying warp.
      // Done here, where the warp would otherwise only wait for the next accumulator.
      TmaStoreWaitAll();
      RedReleaseShared(stored, 1u);
    }
    if (staged && tn != last_tn) {
      bool pok = true;
      if (reloads > 0) pok = MbarWait(SmemAddr(&par_bar[1]), (reloads - 1) & 1, abort_flag, g.status_word, kErrEpilogue, g.wait_limit);
      if (!__all_sync(0xffffffffu, pok)) break;
      if (et < 2 * BN) {
        const int j = et < BN ? et : et - BN;
        const int col = tn * BN + j;
        float v;
        if (et < BN) v = (e.scale != nullptr && col < g.n) ? __ldg(e.scale + col) : e.scalar_scale;
        else v = (e.bias != nullptr && col < g.n) ? __ldg(e.bias + col) : 0.f;
        s_par[et] = v;
      }
      __syncwarp();
      if (lane == 0) MbarArrive(SmemAddr(&par_bar[0]));
      pok = MbarWait(SmemAddr(&par_bar[0]), reloads & 1, abort_flag, g.status_word, kErrEpilogue, g.wait_limit);
      if (!__all_sync(0xffffffffu, pok)) break;
      ++reloads;
      last_tn = tn;
    }
    const int nblocks = min(BN / bcols, (g.n - tn * BN + bcols - 1) / bcols);  // blocks holding real columns
    const bool ok = MbarWait(SmemAddr(&tmem_full_bar[acc * SUP + j]), acc_phase, abort_flag, g.status_word, kErrEpilogue, g.wait_limit_acc);
    if (!__all_sync(0xffffffffu, ok)) break;  // warp-uniform: a lane gave up or saw another role give up
    TcFenceAfter();
    // One accumulator stage holds SUP tiles of consecutive tile rows (sub-tile j in columns j*BN ...); each warp works
    // on one of them.  For 64-column tiles that gives a warp whole rows of its sub-tile (one TMA store of full rows per
    // warp and stage) where a single tile per stage left it a 16-column fragment.
    do {
    const int tmr = (tm * SUP + j) * CG + rank;
    if (tmr >= tiles_m_real) break;  // the MMA issuer left these columns untouched (still armed); the hand-over takes place all the same
    const int row0 = tmr * kBM + q * 32;  // first row of this warp's 32-row block
    const bool row_ok = row0 + lane < g.m;
    const long long row = (long long)bt * g.batch_rows_out + row0 + lane;  // row of `out` / the summand across batches
    const uint32_t taddr = tmem_base + uint32_t((acc * SUP + j) * BN) + (uint32_t(q * 32) << 16);
    if (row0 >= g.m) {
      // No row of this warp is stored, but the MMA still accumulated onto its lanes: re-arm them too.
      if (preset) {
#pragma unroll 1
        for (int c = c_first * bcols; c < BN; c += bcols * W)
#pragma unroll 1
          for (int sl = 0; sl < slices; ++sl) TmemSt16Same(taddr + uint32_t(c + 16 * sl), uint32_t(kMagicBits));
      }
    } else {
#pragma unroll 1
      for (int c = c_first; c < nblocks; c += W) {
        const int col0 = tn * BN + c * bcols;
        uint8_t* buf = e.stage + (seq & uint32_t(nbuf - 1)) * buf_bytes;
        bool sum_pref_next = false;
        if constexpr (SUM8) {
          if (!sum_pref) {  // first block of the launch, or the block before could not look ahead
            if (lane == 0) {
              TmaStoreWaitRead(nbuf - 1);  // the store that last used this buffer has read it
              issue_sum(col0, row0, bt, seq);
            }
          }
          const bool sok = MbarWait(SmemAddr(&my_sum_bar[seq & uint32_t(nbuf - 1)]), (seq / uint32_t(nbuf)) & 1u, abort_flag,
                                    g.status_word, kErrEpilogue, g.wait_limit);
          if (!__all_sync(0xffffffffu, sok)) { give_up = true; break; }
        }
#pragma unroll 1
        for (int sl = 0; sl < slices; ++sl) {
          const int col = col0 + 16 * sl;
          if (col >= g.n) break;
          if constexpr (SUM8) if (sl == slices - 1) {
            // look one block ahead: the next block of this sub-tile, or this warp's first block in the next stage it
            // works on.  A guess of "none" is always safe (the block then fetches its own summand); a
            // block is only ever announced when it is exactly the one this warp processes next.
            int ncol0 = -1, nrow0 = 0, nbt = 0;
            if (c + W < nblocks) {
              ncol0 = col0 + bcols * W; nrow0 = row0; nbt = bt;
            } else if (t + tstep < num_tiles) {
              int ntm, ntn;
              TileCoords(t + tstep, g, tiles_m, tiles_n, &ntm, &ntn, &nbt);
              nrow0 = ((ntm * SUP + j) * CG + rank) * kBM + q * 32;  // < m implies that the tile row exists
              if (nrow0 < g.m && ntn * BN + c_first * bcols < g.n) ncol0 = ntn * BN + c_first * bcols;
            }
            if (ncol0 >= 0) {
              if (lane == 0) {
                TmaStoreWaitRead(nbuf - 2);  // the next buffer's last store (nbuf - 1 blocks ago) has read it
                issue_sum(ncol0, nrow0, nbt, seq + 1);
              }
              sum_pref_next = true;
            }
          }
          uint32_t r[16];
          TmemLd16(taddr + uint32_t(c * bcols + 16 * sl), r);
          uint32_t w[16];
          if (OK == kOutRaw) {
            TmemLdWait16(r);
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = r[j];
          } else {
            // general loop: the 16 summand bytes of this slice are requested first, their latency is the longest
            const bool sum_vec = MODE == kEpGeneral && e.sum_bytes_vec && row_ok && col + 16 <= g.n;
            uint4 s4 = make_uint4(0u, 0u, 0u, 0u);
            if (SUM8) {
              s4 = *reinterpret_cast<const uint4*>(buf + lane * row_bytes + ((uint32_t(sl * units) ^ uint32_t(swz)) << 4));
            } else if (sum_vec) {
              s4 = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(g.ep.summand) + (row * g.ep.ld_summand + col)));
            }
            float sc[16], bi[16];
            LoadStaged16(s_par + (c * bcols + 16 * sl), sc);  // in flight together with the TMEM load
            LoadStaged16(s_par + BN + (c * bcols + 16 * sl), bi);
            TmemLdWait16(r);
            if (preset) TmemSt16Same(taddr + uint32_t(c * bcols + 16 * sl), uint32_t(kMagicBits));  // re-arm what was just read
            float v[16];
            bool shifted = false;  // v still carries the +1.5*2^23 of the adder trick
            if (F8) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            } else {
              // int32 -> fp32: exact adder trick when every accumulator is within +-2^22 (always
              // true when k is small enough, otherwise checked), the conversion instruction otherwise
              bool big = false;
              if (!e.acc_small) {
                // largest and smallest of the 16 accumulators, three operands per instruction
                int mx = __vimax3_s32(int(r[0]), int(r[1]), int(r[2])), mn = __vimin3_s32(int(r[0]), int(r[1]), int(r[2]));
#pragma unroll
                for (int j = 3; j < 15; j += 2) {
                  mx = __vimax3_s32(mx, int(r[j]), int(r[j + 1]));
                  mn = __vimin3_s32(mn, int(r[j]), int(r[j + 1]));
                }
                mx = max(mx, int(r[15]));
                mn = min(mn, int(r[15]));
                const int base = preset ? kMagicBits : 0;  // preset accumulators carry the pattern already
                big = mx >= base + (1 << 22) || mn < base - (1 << 22);
              }
              if (!big) {
                shifted = true;
                if (preset) {
#pragma unroll
                  for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                } else {
#pragma unroll
                  for (int j = 0; j < 16; ++j) v[j] = __int_as_float(int(r[j]) + kMagicBits);
                }
              } else {
                // volatile keeps the slow conversions inside this branch (a preset accumulator that wrapped
                // around wraps back in the subtraction)
                const uint32_t base = preset ? uint32_t(kMagicBits) : 0u;
#pragma unroll
                for (int j = 0; j < 16; ++j) asm volatile("cvt.rn.f32.s32 %0, %1;" : "=f"(v[j]) : "r"(r[j] - base));
              }
            }
            // separate multiply and add: the order and rounding of oneDNN's scale-then-bias tail.
            // A missing scale multiplies by 1 and a missing bias adds 0, both exact.
            // Two columns per instruction for the un-shift and the multiply (packed fp32).
            const uint64_t unshift = shifted ? Pack2(-kMagic, -kMagic) : Pack2(-0.f, -0.f);  // x + (-0) == x for every x
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint64_t p = Pack2(v[2 * j], v[2 * j + 1]);
              if (!F8) p = Add2(p, unshift);
              // A packed multiply feeding a packed add is contracted into a packed fused multiply-add by the
              // assembler even with .rn on both (measured: 25 % of results differ in the last bit), which would
              // break bit-exactness; so is a fused multiply-add whose addend is a literal -0.  The product is
              // therefore formed by a fused multiply-add with a -0 the assembler cannot see (a kernel argument):
              // it rounds x*s exactly like the multiply and keeps the sign of a zero product, and a fused
              // multiply-add feeding an add cannot be contracted further.
              p = Fma2(p, Pack2(sc[2 * j], sc[2 * j + 1]), g.neg_zero2);
              p = Add2(p, Pack2(bi[2 * j], bi[2 * j + 1]));
              Unpack2(p, v[2 * j], v[2 * j + 1]);
            }
            if (SUM8 || (!PLAIN && g.ep.summand != nullptr && row_ok)) {
              const long long sb = row * g.ep.ld_summand + col;
              if (SUM8 || sum_vec) {  // SUM8: rows past m carry zero bytes and are never stored
                // 16 summand bytes -> fp32 without conversion instructions: the byte permute drops each byte into
                // the low byte of the bit pattern of a power of two P >= 2^23, i.e. builds the float P + byte, and
                // one exact add takes P off again (unsigned bytes: P = 2^23; signed bytes are offset by 128 first,
                // b ^ 0x80 = b + 128, on 1.5 * 2^23, and the add takes 1.5 * 2^23 + 128 off).  Then ONE fused
                // multiply-add  v = summand * sum_scale + v : the sum post-op of oneDNN's kernels is a fused
                // multiply-add (a single rounding), which shows on rounding ties - a handful of elements in ten
                // million - and is what the oracle and the real-oneDNN fixture pin.  Two columns per instruction.
                const uint32_t sw[4] = {s4.x ^ e.sum_flip, s4.y ^ e.sum_flip, s4.z ^ e.sum_flip, s4.w ^ e.sum_flip};
                const uint64_t ss2 = Pack2(g.ep.sum_scale, g.ep.sum_scale);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const uint32_t word = sw[j >> 1];
                  const float f0 = __uint_as_float(__byte_perm(word, e.sum_base_bits, (j & 1) ? 0x7652 : 0x7650));
                  const float f1 = __uint_as_float(__byte_perm(word, e.sum_base_bits, (j & 1) ? 0x7653 : 0x7651));
                  uint64_t t = Add2(Pack2(f0, f1), e.sum_off2);
                  t = Fma2(t, ss2, Pack2(v[2 * j], v[2 * j + 1]));
                  Unpack2(t, v[2 * j], v[2 * j + 1]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (!SUM8 && col + j < g.n) v[j] = __fmaf_rn(g.ep.sum_scale, LoadSummand(g.ep.summand, g.ep.summand_dtype, sb + j), v[j]);
              }
            }
            if (e.relu) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = fmaxf(v[j], 0.f);
            }
            if constexpr (MODE == kEpGelu) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(GeluTanh(v[j]), e.post_scale);
            }
            if (MODE == kEpGeneral && g.ep.activation != ITEXB_ACT_NONE) {
              Float16 t;
#pragma unroll
              for (int j = 0; j < 16; ++j) t.v[j] = v[j];
              t = ApplyActivation16(t, g.ep.activation, g.ep.act_alpha, g.ep.act_beta, e.post_scale);
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = t.v[j];
            }
            if (MODE == kEpGeneral && g.ep.mid_dtype == ITEXB_DT_BFLOAT16) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
            } else if (MODE == kEpGeneral && g.ep.mid_dtype == ITEXB_DT_HALF) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __half2float(__float2half_rn(v[j]));
            }
            if (OK == kOutFP8 && row_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (col + j < g.n) thread_amax = fmaxf(thread_amax, fabsf(v[j]));
            }
            Convert16<OK>(v, w, e.e4m3, e.out_scale);
          }
          if (tma_store) {
            if (sl == 0) {
              // the store that last used this staging buffer must have finished reading it
              if (lane == 0) TmaStoreWaitRead(nbuf - 1);
              __syncwarp();
            }
            // 16-byte unit j of staging row r lives at unit j ^ ((r / (8/row_units)) % row_units): the
            // layout a TMA store with a 64/32-byte swizzle reads
            uint8_t* srow = buf + lane * row_bytes;
#pragma unroll
            for (int u = 0; u < units; ++u)
              *reinterpret_cast<uint4*>(srow + (((sl * units + u) ^ swz) << 4)) = make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
          } else if (row_ok) {
            uint8_t* o = static_cast<uint8_t*>(g.out) + (row * g.ldo + col) * esz;
            if (g.vec_store && col + 16 <= g.n) {
#pragma unroll
              for (int u = 0; u < units; ++u) reinterpret_cast<uint4*>(o)[u] = make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (col + j < g.n) {
                  if (esz == 4) reinterpret_cast<uint32_t*>(o)[j] = w[j];
                  else if (esz == 2) reinterpret_cast<uint16_t*>(o)[j] = uint16_t(w[j >> 1] >> (16 * (j & 1)));
                  else o[j] = uint8_t(w[j >> 2] >> (8 * (j & 3)));
                }
              }
            }
          }
        }
        if (tma_store) {
          FenceProxyAsyncShared();
          __syncwarp();
          if (lane == 0) {
            TmaStore3d(tma_out, SmemAddr(buf), col0 * esz, row0, bt);  // rows >= m and columns >= n are clipped
            TmaStoreCommit();
          }
          ++seq;
          sum_pref = sum_pref_next;
        }
      }
      if (give_up) break;
    }
    } while (false);  // this warp's sub-tile
    if (give_up) break;
    if (preset) TmemStWait();  // the re-armed columns are in place before the MMA warp may accumulate onto them
    TcFenceBefore();
    __syncwarp();
    if (lane == 0) {
      // one arrival per warp: all its lanes have read their rows
      release_acc(acc * SUP + j);
      if (staged && tiles_n > 1 && t + tstep < num_tiles) {  // one tile column: the parameters never change
        int ntm, ntn, nbt;
        TileCoords(t + tstep, g, tiles_m, tiles_n, &ntm, &ntn, &nbt);
        if (ntn != tn) MbarArrive(SmemAddr(&par_bar[1]));  // this warp is done with the staged parameters
      }
    }
    acc ^= 1;
    if (acc == 0) acc_phase ^= 1;
  }
  if (tma_store && lane == 0) TmaStoreWaitAll();  // staging memory stays valid until the last store has read it
  if (g.num_peers > 0 && lane == 0 && !give_up && tfirst < num_tiles) RedReleaseShared(stored, 1u);  // the last tile
  if (OK == kOutFP8 && g.ep.amax != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) thread_amax = fmaxf(thread_amax, __shfl_xor_sync(0xffffffffu, thread_amax, o));
    if (lane == 0 && thread_amax > 0.f) atomicMax(reinterpret_cast<int*>(g.ep.amax), __float_as_int(thread_amax));
  }
}

// ---------------------------------------------------------------------------------------
// The kernel.  CONV selects how the producer addresses the A operand: a plain [m,k]
// matrix (2-D map) or NHWC pixels gathered per filter tap (see conv section below).
// ---------------------------------------------------------------------------------------
template <int BN, bool F8, int CONV, int SUP, int CG>
__global__ void __launch_bounds__(CONV == kConvGather ? kThreadsConv : kThreads, 1)
GemmKernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
           const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_a_tail,
           const __grid_constant__ CUtensorMap tma_b_tail, const __grid_constant__ CUtensorMap tma_sum, const __grid_constant__ GemmArgs g) {
  using C = Cfg<BN, CG>;
  static_assert(CG == 1 || (CG == 2 && CONV == kConvNone && SUP == 1), "CTA pairs serve plain GEMMs, one tile per accumulator stage");
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((SmemAddr(smem) & 1023u) != 0) {
    // the swizzled operand tiles need a 1024-byte aligned base; refuse rather than compute garbage
    // (the offset is the same in every CTA of the grid, so a pair leaves together)
    if (threadIdx.x == 0 && g.status_word != nullptr) atomicCAS(g.status_word, 0, kErrSmemAlign);
    return;
  }
  uint8_t* s_stage = smem + C::kStages * C::kStageBytes;  // the epilogue warps' staging tiles, 1024-aligned
  float* s_par = reinterpret_cast<float*>(s_stage + C::kStagingBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_par) + C::kParamBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tmem_full_bar = bars + 2 * C::kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + C::kAccBars;   // [stage * SUP + sub-tile], like tmem_full_bar
  uint64_t* par_bar = tmem_empty_bar + C::kAccBars;
  uint64_t* sum_bar = par_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sum_bar + C::kSumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* stored = tmem_slot + 2;  // fused all-gather: epilogue warps that have completed their stores, summed over tiles

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  static_assert(SUP == 1 || SUP == 2 || SUP == 4, "sub-tiles per accumulator stage");
  static_assert(2 * BN * SUP <= 512, "tensor memory has 512 columns");
  static_assert(CONV != kConvGather || SUP == 1, "the cp.async gather variant walks single tiles");
  const int tiles_m_real = (g.m + kBM - 1) / kBM;
  const int tiles_m = (tiles_m_real + SUP * CG - 1) / (SUP * CG);  // super rows: the unit of the tile walk is SUP (CG) consecutive tile rows
  const int rank = CG == 2 ? int(ClusterCtaRank()) : 0;  // this CTA's place in its pair
  const int tfirst = int(blockIdx.x) / CG, tstep = int(gridDim.x) / CG;
  const int tiles_n = (g.n + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * g.batch;
  // bytes of K per k-block: 128, or in the im2col path 64 / 32 when a filter tap has that many (padded) channels
  const int kb_bytes = (CONV == kConvIm2col && g.conv_cpad < kBK) ? g.conv_cpad : kBK;
  const int num_kb = (g.k + kb_bytes - 1) / kb_bytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      MbarInit(SmemAddr(&full_bar[s]), CONV == kConvGather ? 1 + kGatherThreads : 1);  // B's TMA arrival (+ one per gather thread)
      MbarInit(SmemAddr(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2 * SUP; ++a) {
      // every sub-tile of an accumulator stage is handed over by itself: to the kEpilogueWarps / SUP warps that work on
      // it, and back (a pair's issuer waits for both CTAs' epilogue warps)
      MbarInit(SmemAddr(&tmem_full_bar[a]), 1);
      MbarInit(SmemAddr(&tmem_empty_bar[a]), (kEpilogueWarps / SUP) * CG);
    }
    for (int a = 0; a < 2; ++a) MbarInit(SmemAddr(&par_bar[a]), kEpilogueWarps);
    for (int i = 0; i < C::kSumBars; ++i) MbarInit(SmemAddr(&sum_bar[i]), 1);
    *abort_flag = 0;
    *stored = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    TmemAlloc<CG>(SmemAddr(tmem_slot), C::template kTmemCols<SUP>);
    TmemRelinquish<CG>();
  }
  TcFenceBefore();
  __syncthreads();
  if (CG == 2) ClusterSync();  // the other CTA's barriers are initialised before anything signals them
  TcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: the set-up above (barriers, TMEM allocation) may run while the previous kernel of
  // the stream is still finishing; nothing below touches global memory before that kernel's writes are visible.
  // The kernel after this one may start its own set-up as soon as an SM is free of this grid.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = tfirst; t < num_tiles && ok; t += tstep) {
      int tms, tn, bt;
      TileCoords(t, g, tiles_m, tiles_n, &tms, &tn, &bt);
      for (int j = 0; j < SUP && ok; ++j) {
      const int tm = (tms * SUP + j) * CG + rank;
      if (CG == 1 && tm >= tiles_m_real) break;  // (a pair always loads: rows past the end read as zeros)
      int w0 = 0, h0 = 0, n0 = 0, c0 = 0, kx = 0, ky = 0;  // im2col: base position of the tile's first pixel, position in K
      if (CONV == kConvIm2col) {
        const int pix = tm * kBM;
        const int rest = pix / g.ow;
        w0 = (pix - rest * g.ow) * g.stride_w - g.pad_left;
        n0 = rest / g.oh;
        h0 = (rest - n0 * g.oh) * g.stride_h - g.pad_top;
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = MbarWait(SmemAddr(&empty_bar[stage]), phase ^ 1, abort_flag, g.status_word, kErrProducer, g.wait_limit_acc);
        if (!ok) break;
        if (CG == 1 && kb == g.debug_skip_kb && t == int(blockIdx.x) && j == 0) {
          // Test hook: this k-block never arrives (neither its expect_tx nor its copies are issued), so the MMA issuer's
          // wait on it runs out and the kernel has to take its give-up path with nothing of this stage in flight.
          if (CONV == kConvIm2col) {
            c0 += kb_bytes;
            if (c0 >= g.conv_cpad) { c0 = 0; if (++kx == g.kw) { kx = 0; ++ky; } }
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
          continue;
        }
        uint8_t* sa = smem + stage * C::kStageBytes;
        if (CG == 2) {
          // Both CTAs' copies are counted on the first CTA's barrier, which its producer arms for the bytes of both.
          const uint32_t fb = MapToCta(SmemAddr(&full_bar[stage]), 0);
          const bool tail = g.tail_box != 0 && kb == num_kb - 1;
          if (rank == 0) MbarArriveExpectTx(SmemAddr(&full_bar[stage]), tail ? uint32_t(2 * (kBM + BN / 2) * g.tail_box) : uint32_t(2 * C::kStageBytes));
          TmaLoad3dPair(SmemAddr(sa), tail ? &tma_a_tail : &tma_a, fb, kb * kBK, tm * kBM, bt);
          TmaLoad3dPair(SmemAddr(sa + C::kABytes), tail ? &tma_b_tail : &tma_b, fb, kb * kBK, tn * BN + rank * (BN / 2), bt);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
          continue;
        }
        const uint32_t fb = SmemAddr(&full_bar[stage]);
        if (CONV == kConvGather) {
          MbarArriveExpectTx(fb, C::kBBytes);  // the A tile is gathered by the last four warps
        } else if (CONV == kConvIm2col) {
          MbarArriveExpectTx(fb, uint32_t((kBM + BN) * kb_bytes));
          TmaLoadIm2col(SmemAddr(sa), &tma_a, fb, c0, w0, h0, n0, kx * g.dil_w, ky * g.dil_h);
          c0 += kb_bytes;
          if (c0 >= g.conv_cpad) { c0 = 0; if (++kx == g.kw) { kx = 0; ++ky; } }
          TmaLoad3d(SmemAddr(sa + C::kABytes), &tma_b, fb, kb * kb_bytes, tn * BN, bt);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
          continue;
        } else if (g.tail_box != 0 && kb == num_kb - 1) {
          // the last k-block is 64 or 32 bytes wide: narrower boxes (nothing outside the tensor is touched) into
          // tiles with the matching narrower swizzle
          MbarArriveExpectTx(fb, uint32_t((kBM + BN) * g.tail_box));
          TmaLoad3d(SmemAddr(sa), &tma_a_tail, fb, kb * kBK, tm * kBM, bt);
          TmaLoad3d(SmemAddr(sa + C::kABytes), &tma_b_tail, fb, kb * kBK, tn * BN, bt);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
          continue;
        } else {
          MbarArriveExpectTx(fb, C::kStageBytes);
          TmaLoad3d(SmemAddr(sa), &tma_a, fb, kb * kBK, tm * kBM, bt);
        }
        TmaLoad3d(SmemAddr(sa + C::kABytes), &tma_b, fb, kb * kBK, tn * BN, bt);
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
      }  // sub-tiles
    }
    if (CG == 2 && ok) {
      // The issuer's releases of the last stages arrive from the other CTA: this CTA's shared memory has to outlive them.
      for (int i = 0; i < C::kStages && ok; ++i) {
        ok = MbarWait(SmemAddr(&empty_bar[stage]), phase ^ 1, abort_flag, g.status_word, kErrProducer, g.wait_limit_acc);
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok) {
      // Copies already issued land within microseconds; give them a bounded ~200 us
      // before the CTA tears its shared memory down.
      const long long t0 = clock64();
      while (clock64() - t0 < 400000) {}
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = tfirst; t < num_tiles && ok; t += tstep) {
      int tms = 0;
      if (SUP > 1) {
        int tn_unused, bt_unused;
        TileCoords(t, g, tiles_m, tiles_n, &tms, &tn_unused, &bt_unused);
      }
      for (int j = 0; j < SUP && ok; ++j) {
      // Without preset the first use of each accumulator finds its barrier "already released" (parity trick);
      // with preset it waits for the epilogue warps' arming of it, one phase earlier throughout.
      ok = MbarWait(SmemAddr(&tmem_empty_bar[acc * SUP + j]), g.preset ? acc_phase : acc_phase ^ 1, abort_flag, g.status_word, kErrMma, g.wait_limit);
      if (!ok) break;
      TcFenceAfter();
      const uint32_t d_tmem = tmem_base + uint32_t((acc * SUP + j) * BN);
      // a sub-tile past the last tile row gets no MMAs, but its hand-over still takes place: the barriers stay in step
      const int num_kb_j = (SUP > 1 && tms * SUP + j >= tiles_m_real) ? 0 : num_kb;
      for (int kb = 0; kb < num_kb_j; ++kb) {
        ok = MbarWait(SmemAddr(&full_bar[stage]), phase, abort_flag, g.status_word, kErrMma, g.wait_limit);
        if (!ok) break;
        TcFenceAfter();
        uint8_t* sa = smem + stage * C::kStageBytes;
        const int narrow = (CONV == kConvIm2col && kb_bytes < kBK) ? kb_bytes
                           : ((CONV == kConvNone && g.tail_box != 0 && kb == num_kb - 1) ? g.tail_box : 0);
        if (narrow != 0) {
          const uint64_t a_desc = UmmaDescNarrow(SmemAddr(sa), narrow);
          const uint64_t b_desc = UmmaDescNarrow(SmemAddr(sa + C::kABytes), narrow);
          for (int k = 0; k < narrow / kUmmaK; ++k)
            UmmaSS<F8, CG>(d_tmem, a_desc + uint64_t(k * (kUmmaK >> 4)), b_desc + uint64_t(k * (kUmmaK >> 4)), g.idesc,
                       ((kb | k) != 0 || g.preset) ? 1u : 0u);
        } else {
          const uint64_t a_desc = UmmaDescSw128(SmemAddr(sa));
          const uint64_t b_desc = UmmaDescSw128(SmemAddr(sa + C::kABytes));
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            UmmaSS<F8, CG>(d_tmem, a_desc + uint64_t(k * (kUmmaK >> 4)), b_desc + uint64_t(k * (kUmmaK >> 4)), g.idesc,
                       ((kb | k) != 0 || g.preset) ? 1u : 0u);
        }
        // stage reusable once these MMAs have read it (in both CTAs of a pair)
        if (CG == 2) {
          TcCommitPair(SmemAddr(&empty_bar[stage]));
          TcCommitPair(MapToCta(SmemAddr(&empty_bar[stage]), 1));
        } else {
          TcCommit(SmemAddr(&empty_bar[stage]));
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      // this sub-tile's accumulator is complete
      if (CG == 2) {
        TcCommitPair(SmemAddr(&tmem_full_bar[acc * SUP + j]));
        TcCommitPair(MapToCta(SmemAddr(&tmem_full_bar[acc * SUP + j]), 1));
      } else {
        TcCommit(SmemAddr(&tmem_full_bar[acc * SUP + j]));
      }
      }  // sub-tiles
      if (!ok) break;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if ((warp == 2 || warp == 3) && CONV == kConvNone && g.num_peers > 0) {
    // ---------------- fused all-gather: copy finished tiles to the peers ----------------
    // Two warps, half of a tile's rows each; twelve 16-byte loads per lane in flight (12 rows of 512 bytes per round
    // when the tile is full): what bounds a copying warp is the latency of its loads, not the stores that follow them.
    const int esz = g.out_esz;
    const long long pitch = g.ldo * esz;
    uint8_t* const local = static_cast<uint8_t*>(g.out);
    const int half = warp - 2;
    uint32_t want = 0;
    bool ok = true;
    for (int t = tfirst; t < num_tiles && ok; t += tstep) {
      int tms, tn, bt;
      TileCoords(t, g, tiles_m, tiles_n, &tms, &tn, &bt);
      want += uint32_t(kEpilogueWarps);
      if (LdAcquireShared(stored) < want) {
        const long long t0 = clock64();
        for (uint32_t it = 1; LdAcquireShared(stored) < want; ++it) {
          if ((it & 63u) == 0) {
            if (*abort_flag) { ok = false; break; }
            if (clock64() - t0 > g.wait_limit_acc) {
              *abort_flag = 1;
              if (g.status_word != nullptr) atomicCAS(g.status_word, 0, kErrEpilogue);
              ok = false;
              break;
            }
          }
          __nanosleep(100);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      for (int j = 0; j < SUP * CG; ++j) {
        if (CG == 2 && j != rank) continue;   // a pair's CTAs copy their own tile rows
        const int row0 = (tms * SUP * CG + j) * kBM + half * (kBM / 2);
        if (row0 >= g.m) break;
        const int rows = min(kBM / 2, g.m - row0);
        const int cpr = (min(BN, g.n - tn * BN) * esz) >> 4;           // 16-byte chunks per row of this tile (n * esz % 16 == 0)
        const long long base = ((long long)bt * g.batch_rows_out + row0) * pitch + (long long)tn * BN * esz;
        const int chunks = rows * cpr;
        if (cpr == 32) {
          // full tile rows (512 bytes): twelve rows per round, one row per instruction
          const uint8_t* src = local + base + lane * 16;
          for (int r0 = 0; r0 < rows; r0 += 12) {
            uint4 v[12];
#pragma unroll
            for (int u = 0; u < 12; ++u)
              if (r0 + u < rows) v[u] = __ldcg(reinterpret_cast<const uint4*>(src + (long long)(r0 + u) * pitch));
#pragma unroll 1
            for (int p = 0; p < g.num_peers; ++p) {
              uint8_t* const dst = static_cast<uint8_t*>(g.peer_out[p]) + base + lane * 16;
#pragma unroll
              for (int u = 0; u < 12; ++u)
                if (r0 + u < rows) *reinterpret_cast<uint4*>(dst + (long long)(r0 + u) * pitch) = v[u];
            }
          }
          continue;
        }
        for (int c0 = 0; c0 < chunks; c0 += 128) {
          uint4 v[4];
          long long off[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * 32 + lane;
            const int r = c / cpr;
            off[u] = base + r * pitch + (long long)(c - r * cpr) * 16;
            if (c < chunks) v[u] = __ldcg(reinterpret_cast<const uint4*>(local + off[u]));
          }
#pragma unroll 1
          for (int p = 0; p < g.num_peers; ++p) {
            uint8_t* const dst = static_cast<uint8_t*>(g.peer_out[p]);
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (c0 + u * 32 + lane < chunks) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
          }
        }
      }
    }
  } else if (CONV == kConvGather && warp >= kFirstGatherWarp) {
    // ---------------- implicit-GEMM A producer (convolution) ----------------
    // Every k-block these 128 threads copy the 128 x 128-byte A tile straight from the NHWC input
    // into the positions the 128-byte swizzle gives them (what a TMA load would have written),
    // 16 bytes per cp.async, zero-filled for padding, rows past the end and the K tail.  Thread g
    // owns 16-byte column g%8 of rows g/8, g/8+16, ..., so a warp reads four whole 128-byte runs
    // and the position in K (filter tap and channel) is the same for all eight of its copies.
    // Per tile each thread keeps, for its eight rows, the byte offset of the receptive field's
    // corner and a bit mask of the taps that fall inside the image (bits 0-14: kx, 16-30: ky).
    // Completion is tracked per thread: once the group issued kStages-2 stages ago has landed, a
    // proxy fence makes it visible to the tensor core and the thread arrives on that stage's barrier.
    const int gi = threadIdx.x - kFirstGatherWarp * 32;
    const int j = gi & 7, rbase = gi >> 3;
    const uint32_t dst_off = uint32_t(rbase) * 128u + (uint32_t(j ^ (rbase & 7)) << 4);
    const uint8_t* __restrict__ x = static_cast<const uint8_t*>(g.conv_x);
    constexpr int kLag = C::kStages - 2;  // groups a thread keeps in flight before it signals the oldest stage
    int stage = 0, sig_stage = 0;
    uint32_t phase = 0;
    long long issued = 0, signaled = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn, bt_unused;
      TileCoords(t, g, tiles_m, tiles_n, &tm, &tn, &bt_unused);
      uint32_t msk[8], off[8];
      {
        int pix = tm * kBM + rbase;  // m < 2^31 is checked by the host
        int ox = pix % g.ow;
        const int rest = pix / g.ow;
        int oy = rest % g.oh;
        int b = rest / g.oh;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int iy0 = oy * g.stride_h - g.pad_top, ix0 = ox * g.stride_w - g.pad_left;
          uint32_t ym = 0, xm = 0;
          for (int ky = 0; ky < g.conv_kh; ++ky) ym |= uint32_t(uint32_t(iy0 + ky * g.dil_h) < uint32_t(g.conv_h)) << ky;
          for (int kx = 0; kx < g.kw; ++kx) xm |= uint32_t(uint32_t(ix0 + kx * g.dil_w) < uint32_t(g.conv_w)) << kx;
          msk[i] = pix < g.m ? (ym << 16) | xm : 0u;
          // modulo 2^32; exact once a valid tap's offset is added (the host bounds the input size)
          off[i] = uint32_t((b * g.conv_h + iy0) * g.conv_w + ix0) * uint32_t(g.conv_c);
          pix += 16;
          ox += 16;
          while (ox >= g.ow) { ox -= g.ow; if (++oy == g.oh) { oy = 0; ++b; } }
        }
      }
      // Position in K of this thread's column: channel ci inside tap (ky, kx); 128 bytes further per k-block.
      int ci = j * 16, kx = 0, ky = 0;
      while (ci >= g.conv_c) { ci -= g.conv_c; if (++kx == g.kw) { kx = 0; ++ky; } }
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = MbarWait(SmemAddr(&empty_bar[stage]), phase ^ 1, abort_flag, g.status_word, kErrProducer, g.wait_limit_acc);
        if (!ok) break;
        const uint32_t dst = SmemAddr(smem + stage * C::kStageBytes) + dst_off;
        const uint32_t tap_off = uint32_t((ky * g.dil_h * g.conv_w + kx * g.dil_w) * g.conv_c + ci);
        const uint32_t shx = ky < g.conv_kh ? uint32_t(kx) : 31u, shy = ky < g.conv_kh ? uint32_t(16 + ky) : 31u;  // bit 31 is never set
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool in = ((msk[i] >> shx) & (msk[i] >> shy) & 1u) != 0;
          const uint8_t* src = x + (in ? uint32_t(off[i] + tap_off) : 0u);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + uint32_t(i) * 2048u), "l"(src), "r"(in ? 16u : 0u)
                       : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        ++issued;
        if (issued - signaled > kLag) {
          CpAsyncWaitGroup<kLag>();
          FenceProxyAsyncShared();
          MbarArrive(SmemAddr(&full_bar[sig_stage]));
          ++signaled;
          if (++sig_stage == C::kStages) sig_stage = 0;
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        ci += kBK;
        while (ci >= g.conv_c) { ci -= g.conv_c; if (++kx == g.kw) { kx = 0; ++ky; } }
      }
    }
    CpAsyncWaitGroup<0>();
    FenceProxyAsyncShared();
    while (signaled < issued) {
      MbarArrive(SmemAddr(&full_bar[sig_stage]));
      ++signaled;
      if (++sig_stage == C::kStages) sig_stage = 0;
    }
  } else if (warp >= 4 && warp < kFirstGatherWarp) {
    // ---------------- epilogue ----------------
#define ITEXB_EP_ARGS g, &tma_out, &tma_sum, stored, s_stage, s_par, tmem_full_bar, tmem_empty_bar, par_bar, sum_bar, abort_flag, tmem_base, warp, lane, tiles_m, tiles_n, num_tiles
    switch (g.out_kind) {
      case kOutRaw: EpilogueLoop<BN, F8, kOutRaw, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS); break;
      case kOutF32:
        if (g.ep_mode == kEpPlain) EpilogueLoop<BN, F8, kOutF32, kEpPlain, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpGelu) EpilogueLoop<BN, F8, kOutF32, kEpGelu, SUP, CG>(ITEXB_EP_ARGS);
        else EpilogueLoop<BN, F8, kOutF32, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS);
        break;
      case kOutBF16:
        if (g.ep_mode == kEpPlain) EpilogueLoop<BN, F8, kOutBF16, kEpPlain, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpGelu) EpilogueLoop<BN, F8, kOutBF16, kEpGelu, SUP, CG>(ITEXB_EP_ARGS);
        else EpilogueLoop<BN, F8, kOutBF16, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS);
        break;
      case kOutF16:
        if (g.ep_mode == kEpPlain) EpilogueLoop<BN, F8, kOutF16, kEpPlain, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpGelu) EpilogueLoop<BN, F8, kOutF16, kEpGelu, SUP, CG>(ITEXB_EP_ARGS);
        else EpilogueLoop<BN, F8, kOutF16, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS);
        break;
      case kOutS32:
        if (g.ep_mode == kEpPlain) EpilogueLoop<BN, F8, kOutS32, kEpPlain, SUP, CG>(ITEXB_EP_ARGS);
        else EpilogueLoop<BN, F8, kOutS32, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS);
        break;
      case kOutU8:
        if (g.ep_mode == kEpPlain) EpilogueLoop<BN, F8, kOutU8, kEpPlain, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpSum8) EpilogueLoop<BN, F8, kOutU8, kEpSum8, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpGelu) EpilogueLoop<BN, F8, kOutU8, kEpGelu, SUP, CG>(ITEXB_EP_ARGS);
        else EpilogueLoop<BN, F8, kOutU8, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS);
        break;
      case kOutS8:
        if (g.ep_mode == kEpPlain) EpilogueLoop<BN, F8, kOutS8, kEpPlain, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpSum8) EpilogueLoop<BN, F8, kOutS8, kEpSum8, SUP, CG>(ITEXB_EP_ARGS);
        else if (g.ep_mode == kEpGelu) EpilogueLoop<BN, F8, kOutS8, kEpGelu, SUP, CG>(ITEXB_EP_ARGS);
        else EpilogueLoop<BN, F8, kOutS8, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS);
        break;
      default: EpilogueLoop<BN, F8, kOutFP8, kEpGeneral, SUP, CG>(ITEXB_EP_ARGS); break;
    }
  }

  TcFenceBefore();
  __syncthreads();
  // A pair leaves together: neither CTA's shared memory or tensor memory goes away while the other may still signal
  // a barrier in it or have MMAs in flight on it.
  if (CG == 2) ClusterSync();
  if (warp == 2) {
    TcFenceAfter();
    TmemDealloc<CG>(tmem_base, C::template kTmemCols<SUP>);
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn GetEncodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

template <int BN, bool F8, int CONV, int SUP, int CG = 1>
int Launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tat, const CUtensorMap& tbt,
           const CUtensorMap& ts, const GemmArgs& g, cudaStream_t st) {
  using C = Cfg<BN, CG>;
  const unsigned threads = CONV == kConvGather ? kThreadsConv : kThreads;
  // The opt-in shared-memory size is a per-device function attribute; set it when the device changes.
  static thread_local int last_dev = -1;
  static thread_local int max_pairs = 0;  // CG = 2: pairs of CTAs the device runs at once
  int dev = 0;
  ITEXB_CUDA(cudaGetDevice(&dev));
  if (dev != last_dev) {
    ITEXB_CUDA(cudaFuncSetAttribute(GemmKernel<BN, F8, CONV, SUP, CG>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    if (CG == 2) {
      cudaLaunchConfig_t q{};
      q.gridDim = dim3(unsigned(SmCount() & ~1));
      q.blockDim = dim3(threads);
      q.dynamicSmemBytes = C::kSmemBytes;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int n = 0;
      ITEXB_CUDA(cudaOccupancyMaxActiveClusters(&n, GemmKernel<BN, F8, CONV, SUP, CG>, &q));
      ITEXB_REQUIRE(n >= 1, ITEXB_FAILED_PRECONDITION, "GemmKernel: the device cannot co-schedule a pair of CTAs");
      max_pairs = n;
    }
    last_dev = dev;
  }
  const int tiles = (((g.m + kBM - 1) / kBM + SUP * CG - 1) / (SUP * CG)) * ((g.n + BN - 1) / BN) * g.batch;
  const int grid = CG == 2 ? 2 * std::max(1, std::min(tiles, max_pairs)) : std::max(1, std::min(tiles, SmCount()));
  // Launched with programmatic stream serialization (ITEXB_PDL=0 turns it off): back-to-back GEMM launches of a
  // layer graph overlap one kernel's set-up with the tail of the one before.
  static const bool pdl = [] {
    const char* e = std::getenv("ITEXB_PDL");
    return e == nullptr || e[0] != '0';
  }();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (CG == 2) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  ITEXB_CUDA(cudaLaunchKernelEx(&cfg, GemmKernel<BN, F8, CONV, SUP, CG>, ta, tb, to, tat, tbt, ts, g));
  return CheckLaunch("GemmKernel");
}

}  // namespace

int TailBox(int64_t k) {
  const int t = int(k % kBK);
  return (t == 0 || t > 64) ? 0 : (t <= 32 ? 32 : 64);
}

int EncodeOperandMap(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows, int64_t batch,
                     int64_t batch_stride, int box_k) {
  EncodeTiledFn enc = GetEncodeTiled();
  ITEXB_REQUIRE(enc != nullptr, ITEXB_FAILED_PRECONDITION, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  if (batch <= 1) { batch = 1; batch_stride = rows * ld; }
  const cuuint64_t dims[3] = {cuuint64_t(k), cuuint64_t(rows), cuuint64_t(batch)};
  const cuuint64_t strides[2] = {cuuint64_t(ld), cuuint64_t(batch_stride)};
  const cuuint32_t box[3] = {cuuint32_t(box_k), cuuint32_t(box_rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = box_k == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (box_k == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ITEXB_REQUIRE(r == CUDA_SUCCESS, ITEXB_INTERNAL, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld k=%lld ld=%lld)",
                int(r), (long long)rows, (long long)k, (long long)ld);
  return ITEXB_OK;
}

using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*,
                                    const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int EncodeIm2colMap(CUtensorMap* map, const itexb_conv_params_t& p) {
  static EncodeIm2colFn enc = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &f, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      enc = reinterpret_cast<EncodeIm2colFn>(f);
    else
      (void)cudaGetLastError();
  });
  ITEXB_REQUIRE(enc != nullptr, ITEXB_FAILED_PRECONDITION, "cuTensorMapEncodeIm2col is not available from the CUDA driver");
  const cuuint64_t dims[4] = {cuuint64_t(p.c), cuuint64_t(p.w), cuuint64_t(p.h), cuuint64_t(p.n)};
  const cuuint64_t strides[3] = {cuuint64_t(p.c), cuuint64_t(p.w) * p.c, cuuint64_t(p.h) * p.w * p.c};
  // The base position of output pixel (oy, ox) is (oy*stride - pad_top, ox*stride - pad_left); the box
  // corners bound it to the oh x ow positions of one image so that a run of pixels wraps like the output.
  const int lower[2] = {-p.pad_left, -p.pad_top};
  const int upper[2] = {(p.ow - 1) * p.stride_w - p.pad_left - p.w + 1, (p.oh - 1) * p.stride_h - p.pad_top - p.h + 1};
  const cuuint32_t estr[4] = {1, cuuint32_t(p.stride_w), cuuint32_t(p.stride_h), 1};
  const int box_c = p.c_pad < kBK ? p.c_pad : kBK;  // 128 channels per box, or a whole (padded) tap of 64 / 32
  const CUtensorMapSwizzle sw = box_c == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (box_c == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(p.x), dims, strides, lower, upper, cuuint32_t(box_c),
                   cuuint32_t(kBM), estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ITEXB_REQUIRE(r == CUDA_SUCCESS, ITEXB_INTERNAL,
                "cuTensorMapEncodeIm2col failed with CUresult %d (n=%d h=%d w=%d c=%d corners [%d,%d] [%d,%d] strides %d,%d)", int(r), p.n,
                p.h, p.w, p.c, lower[0], lower[1], upper[0], upper[1], p.stride_w, p.stride_h);
  return ITEXB_OK;
}

// Tensor map for the epilogue's TMA stores: the output as a byte matrix {n*esz, m} with
// row pitch ldo*esz, box = one warp block of 32 rows x 16 (4-byte) or 32 (narrower) elements,
// swizzle matching the staging tile's row width (64 or 32 bytes).
static int EncodeOutputMap(CUtensorMap* map, void* base, int64_t m, int64_t n, int64_t ldo, int esz, int bn, int sup, bool sum8, int64_t batch,
                           int64_t batch_rows) {
  EncodeTiledFn enc = GetEncodeTiled();
  ITEXB_REQUIRE(enc != nullptr, ITEXB_FAILED_PRECONDITION, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  const cuuint64_t dims[3] = {cuuint64_t(n) * esz, cuuint64_t(m), cuuint64_t(batch)};
  const cuuint64_t strides[2] = {cuuint64_t(ldo) * esz, cuuint64_t(batch_rows) * ldo * esz};
  const int row_bytes = OutBlockCols(bn, esz, sup, sum8) * esz;  // staging rows of 64, 32 or 16 bytes, swizzled over their own width
  const cuuint32_t box[3] = {cuuint32_t(row_bytes), 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ITEXB_REQUIRE(r == CUDA_SUCCESS, ITEXB_INTERNAL, "cuTensorMapEncodeTiled (output) failed with CUresult %d", int(r));
  return ITEXB_OK;
}

uint32_t MakeInstrDesc(int a_dtype, int b_dtype, int bn, int rows) {
  const bool f8 = IsFp8(a_dtype);
  uint32_t a_fmt, b_fmt, c_fmt;
  if (f8) {
    a_fmt = a_dtype == ITEXB_DT_FP8_E4M3 ? 0u : 1u;
    b_fmt = b_dtype == ITEXB_DT_FP8_E4M3 ? 0u : 1u;
    c_fmt = 1u;  // f32 accumulate
  } else {
    a_fmt = IsSigned8(a_dtype) ? 1u : 0u;
    b_fmt = IsSigned8(b_dtype) ? 1u : 0u;
    c_fmt = 2u;  // s32 accumulate
  }
  // [4,6) D format, [7,10) A format, [10,13) B format, bits 15/16 = 0: both operands K-major,
  // [17,23) N>>3, [24,29) M>>4 (128 rows, or 256 across a pair of CTAs).
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(rows >> 4) << 24);
}

// floor(x / d) for 0 <= x < 2^31 as umulhi(x, mul) >> shift, with mul = ceil(2^(32 + shift) / d) and
// shift = ceil(log2 d) - 1 (d >= 2; mul == 0 marks d == 1).  The rounding error of mul adds less than
// x / 2^(32 + shift) * d < 1/d to the quotient's fraction, so the floor is exact.
FastDiv MakeFastDiv(uint32_t d) {
  FastDiv f{0u, 0u};
  if (d <= 1u) return f;
  uint32_t lg = 0;
  while ((1ull << lg) < d) ++lg;
  f.shift = lg - 1;
  f.mul = uint32_t(((1ull << (31 + lg)) + d - 1) / d);
  return f;
}

int PickBN(int n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

// Sub-tiles per accumulator stage (1, 2 or 4; 2 * bn * sup <= 512 columns of tensor memory).  Narrow tiles carry little
// epilogue work per barrier round trip, so several consecutive tile rows share one; what that costs is coarser work
// units, so the largest factor is taken that keeps the last wave of the persistent grid reasonably full.
// ITEXB_GEMM_SUP forces a value (for measurements).
static int PickSup(int bn, bool single_only, int tiles_m, int tiles_n, int batch) {
  const int max_sup = single_only ? 1 : (bn == 64 ? 4 : (bn == 128 ? 2 : 1));
  static const int forced = [] {
    const char* e = std::getenv("ITEXB_GEMM_SUP");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (forced == 1 || forced == 2 || forced == 4) return std::min(forced, max_sup);
  const long long sms = SmCount();
  const long long tiles = (long long)tiles_m * tiles_n * batch;
  int best = 1;
  double best_eff = 0.0;
  for (int sup = max_sup; sup >= 1; sup /= 2) {
    const long long units = (long long)((tiles_m + sup - 1) / sup) * tiles_n * batch;
    if (sup > 1 && units < sms) continue;  // not enough units to occupy every SM
    const long long waves = (units + sms - 1) / sms;
    const double eff = double(tiles) / double(waves * sms * sup);
    if (eff >= 0.85) return sup;
    if (eff > best_eff) { best_eff = eff; best = sup; }
  }
  return best;
}

// Test hooks (itexb_debug_set): process-wide, read at every launch.
static std::atomic<long long> g_wait_limit_cycles{0};  // 0: the default
static std::atomic<int> g_debug_skip_kb{-1};
long long GemmWaitLimitCycles() {
  const long long limit = g_wait_limit_cycles.load(std::memory_order_relaxed);
  return limit > 0 ? limit : kWaitLimitCycles;
}

// A pair of CTAs per 256 x 256 tile (each loads half of B) for plain GEMMs that have enough such tiles and write 4-byte
// outputs.  Measured on B200, pair against single: 8192^3 -> f32 0.350-0.358 ms against 0.373-0.395 (1.03 of the
// library's kernel instead of 0.96-0.98); 12288 x 4096 x 1024 -> f32 59.8 us against 64.0, raw accumulators 57.1
// against 65.7; but -> u8 53.1 against 49.7 and -> bf16 54.7 against 51.6 (the same 6-7 % at 12288 x 1024 x 4096 and
// 12288 x 3072 x 1024): the pair's issuer waits for the slower of two epilogues, which only the launches whose
// epilogue is bound by its stores win back through the third less operand traffic.
// ITEXB_GEMM_CTA_PAIR=0 (or itexb_debug_set("gemm_cta_pair", 0)) turns it off, 1 takes it wherever the kernel allows
// (tests and measurements), -1 is this rule.
static std::atomic<int> g_cta_pair{-2};  // -2: not set through itexb_debug_set, the environment decides
int PickCtaGroup(int m, int n, int batch, int bn, bool gather, int out_esz) {
  static const int from_env = [] {
    const char* e = std::getenv("ITEXB_GEMM_CTA_PAIR");
    return e != nullptr ? std::atoi(e) : -1;
  }();
  const int set = g_cta_pair.load(std::memory_order_relaxed);
  const int forced = set != -2 ? set : from_env;
  if (forced == 0 || bn != 256 || gather) return 1;
  if (g_debug_skip_kb.load(std::memory_order_relaxed) >= 0) return 1;  // the test hook lives in the single-CTA producer
  const int tiles_m_real = (m + kBM - 1) / kBM;
  if (tiles_m_real % 2 != 0) return 1;  // every pair gets two real tile rows
  if (forced == 1) return 2;
  if (out_esz != 4) return 1;
  const long long pairs = (long long)(tiles_m_real / 2) * ((n + bn - 1) / bn) * std::max(batch, 1);
  return pairs >= 2ll * (SmCount() / 2) ? 2 : 1;
}

int LaunchGemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, int bn, bool f8, cudaStream_t st, const TailMaps* tail, int cg) {
  const CUtensorMap& tat = tail != nullptr ? tail->a : ta;  // placeholders when there is no narrow last k-block
  const CUtensorMap& tbt = tail != nullptr ? tail->b : tb;
  g.tail_box = (tail != nullptr && g.conv_mode == kConvNone) ? tail->box : 0;
  // Output addressing: TMA stores from a staged tile when the rows are 16-byte aligned,
  // otherwise per-thread stores straight from registers.
  g.out_esz = g.ep.raw_acc ? 4 : DtypeSize(g.out_dtype);
  if (g.ep.raw_acc) g.out_kind = kOutRaw;
  else switch (g.out_dtype) {
    case ITEXB_DT_FLOAT: g.out_kind = kOutF32; break;
    case ITEXB_DT_BFLOAT16: g.out_kind = kOutBF16; break;
    case ITEXB_DT_HALF: g.out_kind = kOutF16; break;
    case ITEXB_DT_QINT32: case ITEXB_DT_INT32: g.out_kind = kOutS32; break;
    case ITEXB_DT_QUINT8: case ITEXB_DT_UINT8: g.out_kind = kOutU8; break;
    case ITEXB_DT_QINT8: case ITEXB_DT_INT8: g.out_kind = kOutS8; break;
    default: g.out_kind = kOutFP8; break;
  }
  // m-tiles per rasterisation group, measured: wide tile grids want tall groups (8192^3: 32 beats 16 by 2 %, 8 loses 3 %),
  // narrow ones short groups (n = 4096: 8 beats 16 by 1-2 %)
  const int tiles_n = (g.n + bn - 1) / bn;
  const int tiles_m_real = (g.m + kBM - 1) / kBM;
  if (g.batch <= 1) { g.batch = 1; g.batch_rows_out = g.m; }
  // Measured (B200, u8 output): stacking sub-tiles pays where a tile is all epilogue - one or two k-blocks: 401408 x 64
  // with K = 64 26.8 -> 20.6 us, the 7x7x3 stem's GEMM (K = 160) 120.6 -> 99.8 us - and costs a few per cent where the
  // main loop matters (K = 256: 27.2 -> 28.9 us; 3x3 convolutions of 64 channels, K = 576: 72.7 -> 76.4 us), because the
  // MMA issuer then waits for a whole stage of sub-tiles to be drained.
  const int sup = cg == 2 ? 1 : PickSup(bn, f8 || g.conv_mode == kConvGather || g.k > 192, tiles_m_real, tiles_n, g.batch);
  const int tiles_m = (tiles_m_real + sup * cg - 1) / (sup * cg);  // the tile walk's rows are super rows of `sup` (`cg`) tile rows
  g.group_m = tiles_n >= 32 ? 32 : (tiles_n <= 16 ? 8 : 16);
  if (cg == 2) g.group_m = tiles_n >= 32 ? 16 : 8;  // rows of pairs (8192^3: 16 -> 0.350 ms, 8 -> 0.356, 32 -> 0.415, 4 -> 0.377)
  {
    static const int forced_group = [] {  // ITEXB_GEMM_GROUP_M: measurements
      const char* e = std::getenv("ITEXB_GEMM_GROUP_M");
      return e != nullptr ? std::atoi(e) : 0;
    }();
    if (forced_group > 0) g.group_m = forced_group;
  }
  g.div_per_batch = MakeFastDiv(uint32_t(tiles_m) * uint32_t(tiles_n));
  g.div_per_group = MakeFastDiv(uint32_t(g.group_m) * uint32_t(tiles_n));
  g.div_group_m = MakeFastDiv(uint32_t(g.group_m));
  g.neg_zero2 = 0x8000000080000000ull;
  const long long limit = g_wait_limit_cycles.load(std::memory_order_relaxed);
  g.wait_limit = limit > 0 ? limit : kWaitLimitCycles;
  g.wait_limit_acc = 2 * g.wait_limit;
  g.debug_skip_kb = g_debug_skip_kb.load(std::memory_order_relaxed);
  g.vec_store = ((reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && (g.ldo * g.out_esz) % 16 == 0) ? 1 : 0;
  g.tma_store = g.vec_store;
  // The common epilogues run loops compiled without the rest (the loop is bound by instruction fetch: the same
  // arithmetic is 15-20 % faster without the untaken branches around it).  Plain: scale, bias, ReLU, conversion,
  // TMA stores.  Sum8: the same plus an 8-bit summand read 16 bytes at a time into an 8-bit output (the
  // residual additions of a quantized ResNet).
  g.ep_mode = kEpGeneral;
  if (g.tma_store && g.ep.activation == ITEXB_ACT_NONE && g.ep.mid_dtype == 0 && !g.ep.raw_acc) {
    const int sd = g.ep.summand_dtype;
    const bool sum8 = sd == ITEXB_DT_QUINT8 || sd == ITEXB_DT_UINT8 || sd == ITEXB_DT_QINT8 || sd == ITEXB_DT_INT8;
    if (g.ep.summand == nullptr) g.ep_mode = kEpPlain;
    else if ((g.out_kind == kOutU8 || g.out_kind == kOutS8) && sum8 && g.n % 16 == 0 && g.ep.ld_summand % 16 == 0 &&
             (reinterpret_cast<uintptr_t>(g.ep.summand) & 15) == 0)
      g.ep_mode = kEpSum8;
  }
  // tanh-GELU after scale and bias, nothing else (the FFN-up layer of a transformer): the plain loop with the activation
  // inlined instead of the general loop's out-of-line activation call (12288 x 4096 x 1024 -> bf16: see the kernel table)
  if (g.tma_store && g.ep.activation == ITEXB_ACT_GELU_TANH && g.ep.mid_dtype == 0 && !g.ep.raw_acc && g.ep.summand == nullptr && !g.ep.relu &&
      (g.out_kind == kOutF32 || g.out_kind == kOutBF16 || g.out_kind == kOutF16 || g.out_kind == kOutU8 || g.out_kind == kOutS8))
    g.ep_mode = kEpGelu;
  g.preset = (!f8 && g.ep_mode != kEpGeneral) ? 1 : 0;
  CUtensorMap to;
  CUtensorMap tsum;  // Sum8: the summand seen through the output's geometry (same boxes, same swizzle)
  if (g.ep_mode == kEpSum8)
    ITEXB_RETURN_IF_ERROR(EncodeOutputMap(&tsum, const_cast<void*>(g.ep.summand), g.m, g.n, g.ep.ld_summand, 1, bn, sup, true, g.batch, g.batch_rows_out));
  else tsum = ta;  // unused by the kernel
  if (g.tma_store)
    ITEXB_RETURN_IF_ERROR(EncodeOutputMap(&to, g.out, g.m, g.n, g.ldo, g.out_esz, bn, sup, g.ep_mode == kEpSum8, g.batch, g.batch_rows_out));
  else to = ta;  // unused by the kernel
  if (g.num_peers > 0)
    ITEXB_REQUIRE(g.tma_store, ITEXB_INVALID_ARGUMENT, "gemm: the fused all-gather needs 16-byte aligned output rows");
  if (g.conv_mode == kConvGather) {
    if (bn == 256) return Launch<256, false, kConvGather, 1>(ta, tb, to, tat, tbt, tsum, g, st);
    if (bn == 128) return Launch<128, false, kConvGather, 1>(ta, tb, to, tat, tbt, tsum, g, st);
    return Launch<64, false, kConvGather, 1>(ta, tb, to, tat, tbt, tsum, g, st);
  }
  if (cg == 2) {
    ITEXB_REQUIRE(bn == 256 && g.conv_mode == kConvNone && tiles_m_real % 2 == 0 && g.num_peers == 0, ITEXB_INTERNAL,
                  "LaunchGemm: a CTA pair was asked for a launch it does not serve");
    if (f8) return Launch<256, true, kConvNone, 1, 2>(ta, tb, to, tat, tbt, tsum, g, st);
    return Launch<256, false, kConvNone, 1, 2>(ta, tb, to, tat, tbt, tsum, g, st);
  }
  if (f8) {
    if (bn == 256) return Launch<256, true, kConvNone, 1>(ta, tb, to, tat, tbt, tsum, g, st);
    if (bn == 128) return Launch<128, true, kConvNone, 1>(ta, tb, to, tat, tbt, tsum, g, st);
    return Launch<64, true, kConvNone, 1>(ta, tb, to, tat, tbt, tsum, g, st);
  }
  const bool im2col = g.conv_mode == kConvIm2col;
#define ITEXB_LAUNCH(BN_, SUP_)                                                                     \
  return im2col ? Launch<BN_, false, kConvIm2col, SUP_>(ta, tb, to, tat, tbt, tsum, g, st)          \
                : Launch<BN_, false, kConvNone, SUP_>(ta, tb, to, tat, tbt, tsum, g, st)
  if (bn == 256) { ITEXB_LAUNCH(256, 1); }
  if (bn == 128) {
    if (sup == 2) { ITEXB_LAUNCH(128, 2); }
    ITEXB_LAUNCH(128, 1);
  }
  if (sup == 4) { ITEXB_LAUNCH(64, 4); }
  if (sup == 2) { ITEXB_LAUNCH(64, 2); }
  ITEXB_LAUNCH(64, 1);
#undef ITEXB_LAUNCH
}

int ValidateEpilogue(const char* who, const itexb_epilogue_t& ep, int out_dtype, bool f8, int n) {
  ITEXB_REQUIRE(ep.scale_count == 0 || ep.scale_count == 1 || ep.scale_count == n, ITEXB_INVALID_ARGUMENT,
                "%s: scale_count must be 0, 1 or n (%d), got %d", who, n, ep.scale_count);
  ITEXB_REQUIRE(ep.scale_count == 0 || ep.scale != nullptr, ITEXB_INVALID_ARGUMENT, "%s: scale is NULL", who);
  ITEXB_REQUIRE((ep.alpha_a == nullptr) == (ep.alpha_b == nullptr), ITEXB_INVALID_ARGUMENT,
                "%s: alpha_a and alpha_b must be given together", who);
  switch (out_dtype) {
    case ITEXB_DT_FLOAT: case ITEXB_DT_BFLOAT16: case ITEXB_DT_HALF: break;
    case ITEXB_DT_QINT32: case ITEXB_DT_INT32: case ITEXB_DT_QUINT8: case ITEXB_DT_UINT8: case ITEXB_DT_QINT8: case ITEXB_DT_INT8:
      ITEXB_REQUIRE(!f8, ITEXB_INVALID_ARGUMENT, "%s: integer outputs need int8 operands", who);
      break;
    case ITEXB_DT_FP8_E4M3: case ITEXB_DT_FP8_E5M2:
      ITEXB_REQUIRE(ep.out_scale != nullptr, ITEXB_INVALID_ARGUMENT, "%s: FP8 output needs out_scale", who);
      break;
    default: return SetError(ITEXB_INVALID_ARGUMENT, "%s: unsupported output type %s", who, DtypeName(out_dtype));
  }
  if (ep.raw_acc)
    ITEXB_REQUIRE(!f8 && (out_dtype == ITEXB_DT_QINT32 || out_dtype == ITEXB_DT_INT32), ITEXB_INVALID_ARGUMENT,
                  "%s: raw_acc needs int8 operands and a qint32 output", who);
  if (ep.summand != nullptr) {
    const int sd = ep.summand_dtype;
    ITEXB_REQUIRE(IsInt8(sd) || sd == ITEXB_DT_FLOAT || sd == ITEXB_DT_BFLOAT16 || sd == ITEXB_DT_HALF, ITEXB_INVALID_ARGUMENT,
                  "%s: unsupported summand type %s", who, DtypeName(sd));
  }
  return ITEXB_OK;
}

}  // namespace itexb

using namespace itexb;

extern "C" int itexb_debug_set(const char* key, int64_t value) {
  ITEXB_REQUIRE(key != nullptr, ITEXB_INVALID_ARGUMENT, "debug_set: key is NULL");
  const std::string k(key);
  if (k == "gemm_wait_limit_cycles") {
    ITEXB_REQUIRE(value >= 0, ITEXB_INVALID_ARGUMENT, "debug_set: gemm_wait_limit_cycles must be >= 0 (0 restores the default)");
    g_wait_limit_cycles.store(value, std::memory_order_relaxed);
  } else if (k == "gemm_cta_pair") {
    ITEXB_REQUIRE(value >= -1 && value <= 1, ITEXB_INVALID_ARGUMENT, "debug_set: gemm_cta_pair must be -1 (automatic), 0 (never) or 1 (wherever possible)");
    g_cta_pair.store(int(value), std::memory_order_relaxed);
  } else if (k == "gemm_skip_kblock") {
    ITEXB_REQUIRE(value >= -1 && value < (1ll << 30), ITEXB_INVALID_ARGUMENT, "debug_set: gemm_skip_kblock must be -1 (off) or a k-block index");
    g_debug_skip_kb.store(int(value), std::memory_order_relaxed);
  } else {
    return SetError(ITEXB_NOT_FOUND, "debug_set: unknown key '%s'", key);
  }
  return ITEXB_OK;
}

extern "C" int itexb_gemm(const itexb_gemm_params_t* p, itexb_stream_t stream) {
  ITEXB_REQUIRE(p != nullptr, ITEXB_INVALID_ARGUMENT, "gemm: params is NULL");
  ITEXB_REQUIRE(p->m >= 0 && p->n >= 0 && p->k >= 0, ITEXB_INVALID_ARGUMENT, "gemm: negative dimension");
  const bool f8 = IsFp8(p->a_dtype);
  if (f8)
    ITEXB_REQUIRE(IsFp8(p->b_dtype), ITEXB_INVALID_ARGUMENT, "gemm: FP8 a needs FP8 b, got %s", DtypeName(p->b_dtype));
  else
    ITEXB_REQUIRE(IsInt8(p->a_dtype) && IsInt8(p->b_dtype), ITEXB_INVALID_ARGUMENT, "gemm: operands must be 8-bit (%s x %s)",
                  DtypeName(p->a_dtype), DtypeName(p->b_dtype));
  ITEXB_RETURN_IF_ERROR(ValidateEpilogue("gemm", p->ep, p->out_dtype, f8, p->n));
  if (p->m == 0 || p->n == 0) return ITEXB_OK;
  ITEXB_REQUIRE(p->k > 0, ITEXB_INVALID_ARGUMENT, "gemm: k must be positive");
  ITEXB_REQUIRE(p->a && p->b && p->out, ITEXB_INVALID_ARGUMENT, "gemm: NULL operand");
  ITEXB_REQUIRE(p->lda >= p->k && p->ldb >= p->k && p->ldo >= p->n, ITEXB_INVALID_ARGUMENT, "gemm: leading dimension too small");
  ITEXB_REQUIRE(p->lda % 16 == 0 && p->ldb % 16 == 0 && (reinterpret_cast<uintptr_t>(p->a) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(p->b) & 15) == 0,
                ITEXB_INVALID_ARGUMENT, "gemm: a and b must be 16-byte aligned with lda/ldb multiples of 16 (TMA rule)");
  const int64_t batch = p->batch > 1 ? p->batch : 1;
  if (batch > 1) {
    ITEXB_REQUIRE(p->stride_a % 16 == 0 && p->stride_b % 16 == 0 && p->stride_a > 0 && p->stride_b > 0, ITEXB_INVALID_ARGUMENT,
                  "gemm: batch strides of a and b must be positive multiples of 16 bytes");
    ITEXB_REQUIRE(p->stride_out >= int64_t(p->m) * p->ldo && p->stride_out % p->ldo == 0, ITEXB_INVALID_ARGUMENT,
                  "gemm: stride_out must be a multiple of ldo and at least m*ldo");
    ITEXB_REQUIRE(batch * ((p->m + kBM - 1) / kBM) * ((p->n + 63) / 64) < (1ll << 31), ITEXB_INVALID_ARGUMENT, "gemm: too many tiles");
  }
  CUtensorMap ta, tb;
  int bn = PickBN(p->n);
  {
    static const int forced_bn = [] {  // ITEXB_GEMM_BN: measurements
      const char* e = std::getenv("ITEXB_GEMM_BN");
      return e != nullptr ? std::atoi(e) : 0;
    }();
    if ((forced_bn == 64 || forced_bn == 128 || forced_bn == 256) && forced_bn < bn) bn = forced_bn;
  }
  const int cg = PickCtaGroup(p->m, p->n, int(batch), bn, p->num_peers > 0, p->ep.raw_acc ? 4 : DtypeSize(p->out_dtype));  // 2: each CTA of a pair loads half of a B tile
  // A launch whose 256-column tiles would leave more than half of the SMs without one takes 128-column tiles: twice the
  // CTAs, the same time per wave (4096 x 512 x 14336 FP8: 41.2 against 43.3 us), and in a fused all-gather twice as
  // many SMs copying.
  if (cg == 1 && bn == 256 && 2ll * ((p->m + kBM - 1) / kBM) * ((p->n + 255) / 256) * batch <= SmCount()) bn = 128;
  ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&ta, p->a, p->m, p->k, p->lda, kBM, batch, p->stride_a));
  ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tb, p->b, p->n, p->k, p->ldb, bn / cg, batch, p->stride_b));
  TailMaps tail;
  tail.box = TailBox(p->k);
  if (tail.box != 0) {
    ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tail.a, p->a, p->m, p->k, p->lda, kBM, batch, p->stride_a, tail.box));
    ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tail.b, p->b, p->n, p->k, p->ldb, bn / cg, batch, p->stride_b, tail.box));
  }
  GemmArgs g{};
  g.batch = int(batch);
  g.batch_rows_out = batch > 1 ? p->stride_out / p->ldo : p->m;
  g.m = p->m; g.n = p->n; g.k = p->k;
  g.out_dtype = p->out_dtype;
  g.out = p->out; g.ldo = p->ldo;
  g.ep = p->ep;
  g.status_word = p->status_word;
  g.idesc = MakeInstrDesc(p->a_dtype, p->b_dtype, bn, kBM * cg);
  if (p->num_peers > 0) {
    ITEXB_REQUIRE(p->num_peers <= ITEXB_MAX_PEERS && p->peer_out != nullptr, ITEXB_INVALID_ARGUMENT, "gemm: num_peers must be at most %d with peer_out given",
                  ITEXB_MAX_PEERS);
    const int esz = p->ep.raw_acc ? 4 : DtypeSize(p->out_dtype);
    ITEXB_REQUIRE(batch == 1 && (int64_t(p->n) * esz) % 16 == 0 && (p->ldo * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(p->out) & 15) == 0,
                  ITEXB_INVALID_ARGUMENT, "gemm: the fused all-gather needs a single GEMM whose output rows are 16-byte aligned multiples of 16 bytes");
    g.num_peers = p->num_peers;
    for (int i = 0; i < p->num_peers; ++i) {
      ITEXB_REQUIRE(p->peer_out[i] != nullptr && (reinterpret_cast<uintptr_t>(p->peer_out[i]) & 15) == 0, ITEXB_INVALID_ARGUMENT,
                    "gemm: peer_out[%d] must be a 16-byte aligned device pointer", i);
      g.peer_out[i] = p->peer_out[i];
    }
  }
  return LaunchGemm(ta, tb, g, bn, f8, AsCuda(stream), tail.box != 0 ? &tail : nullptr, cg);
}
