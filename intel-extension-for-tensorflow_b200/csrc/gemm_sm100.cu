// int8 / FP8 GEMM for sm_100a: out[m][n] = epilogue(sum_k a[m][k] * b[n][k]).
//
// One persistent CTA per SM, warp-specialised:
//   warp 0   TMA producer   cp.async.bulk.tensor (2-D tiled, 128-byte swizzle) -> smem ring
//   warp 1   MMA issuer     tcgen05.mma.cta_group::1.kind::i8 | kind::f8f6f4, 128 x BN x 32 per
//                           instruction, operands read from smem through UMMA descriptors,
//                           accumulators (s32 | f32) in tensor memory
//   warp 2   TMEM allocator (2 accumulator stages of BN columns, so the epilogue of tile i
//                           overlaps the main loop of tile i+1)
//   warps 4-7 epilogue      tcgen05.ld 32 lanes x 32 columns per warp, scale/bias/sum/ReLU,
//                           conversion, 16-byte stores
// Pipelines are mbarrier based: full[s]/empty[s] between producer and MMA issuer
// (tcgen05.commit releases a stage), tmem_full[a]/tmem_empty[a] between MMA issuer and
// epilogue.  Every wait is bounded: on expiry the kernel raises a status word, all roles
// leave their loops, TMEM is released and the kernel returns.
//
// No cluster launch and no multicast loads are used, so the same code runs unchanged in
// single- and multi-GPU jobs.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>

#include "common.h"
#include "gemm_sm100.h"

namespace itexb {
namespace {

constexpr int kBM = 128;          // rows of a per tile = TMEM lanes
constexpr int kBK = 128;          // bytes of K per pipeline stage (one 128-byte swizzle row)
constexpr int kUmmaK = 32;        // bytes of K per tcgen05.mma
constexpr int kThreads = 256;
constexpr int kEpilogueThreads = 128;
constexpr int kGroupM = 16;       // tile rasterisation: m-tiles per L2 super-group
constexpr long long kWaitLimitCycles = 4000000000ll;  // ~2 s at 2 GHz

enum : int { kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3 };

template <int BN> struct Cfg {
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;   // 4 (BN=256), 6 (128), 8 (64)
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // power of two >= 32
  static constexpr int kParamBytes = 2 * 2 * BN * 4;           // scale + bias, per accumulator stage
  static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kParamBytes + kBarrierBytes;
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
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word, int code) {
  if (MbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (MbarTryWait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        if (status_word != nullptr) atomicCAS(status_word, 0, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void TmaLoad2d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void TmemAlloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <bool F8>
__device__ __forceinline__ void UmmaSS(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
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

// 32 lanes x 32 consecutive 32-bit columns: register j of lane l = D[lane_base + l][col + j].
__device__ __forceinline__ void TmemLd32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void TmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile whose rows are 128 bytes, stored with the 128-byte swizzle TMA
// writes: 8-row groups are 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t UmmaDescSw128(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}

__device__ __forceinline__ void EpilogueBarrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// Epilogue math and stores
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ int SatRneInt(float f, float lo, float hi) {
  f = f < lo ? lo : (f > hi ? hi : f);
  return __float2int_rn(f);
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

__device__ __forceinline__ uint32_t Pack4(int a, int b, int c, int d) {
  return uint32_t(a & 0xff) | (uint32_t(b & 0xff) << 8) | (uint32_t(c & 0xff) << 16) | (uint32_t(d & 0xff) << 24);
}

// Converts and stores 32 consecutive outputs of one row.  `ncols` (<= 32) columns are in
// range; `vec` says the row segment is 16-byte aligned and complete.
__device__ __forceinline__ void StoreRow32(const GemmArgs& g, const float (&v)[32], long long row, int col0, int ncols,
                                           bool vec, float* thread_amax, float out_scale) {
  const long long base = row * g.ldo + col0;
  switch (g.out_dtype) {
    case ITEXB_DT_FLOAT: {
      float* o = static_cast<float*>(g.out) + base;
      if (vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(o)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      } else {
        for (int j = 0; j < ncols; ++j) o[j] = v[j];
      }
      break;
    }
    case ITEXB_DT_BFLOAT16: {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(g.out) + base;
      if (vec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t*>(&h);
          }
          reinterpret_cast<uint4*>(o)[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        for (int j = 0; j < ncols; ++j) o[j] = __float2bfloat16_rn(v[j]);
      }
      break;
    }
    case ITEXB_DT_HALF: {
      __half* o = static_cast<__half*>(g.out) + base;
      if (vec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __half2 h = __floats2half2_rn(v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
            w[t] = *reinterpret_cast<uint32_t*>(&h);
          }
          reinterpret_cast<uint4*>(o)[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        for (int j = 0; j < ncols; ++j) o[j] = __float2half_rn(v[j]);
      }
      break;
    }
    case ITEXB_DT_QINT32: case ITEXB_DT_INT32: {
      // oneDNN converts the fp32 tail to s32 with saturation and RNE.
      int* o = static_cast<int*>(g.out) + base;
      int q[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float f = v[j];
        q[j] = f >= 2147483648.f ? 2147483647 : (f <= -2147483648.f ? (-2147483647 - 1) : __float2int_rn(f));
      }
      if (vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) reinterpret_cast<int4*>(o)[j] = make_int4(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
      } else {
        for (int j = 0; j < ncols; ++j) o[j] = q[j];
      }
      break;
    }
    case ITEXB_DT_QUINT8: case ITEXB_DT_UINT8: case ITEXB_DT_QINT8: case ITEXB_DT_INT8: {
      const bool sg = (g.out_dtype == ITEXB_DT_QINT8 || g.out_dtype == ITEXB_DT_INT8);
      const float lo = sg ? -128.f : 0.f, hi = sg ? 127.f : 255.f;
      uint8_t* o = static_cast<uint8_t*>(g.out) + base;
      int q[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) q[j] = SatRneInt(v[j], lo, hi);
      if (vec) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
          reinterpret_cast<uint4*>(o)[j] =
              make_uint4(Pack4(q[16 * j], q[16 * j + 1], q[16 * j + 2], q[16 * j + 3]),
                         Pack4(q[16 * j + 4], q[16 * j + 5], q[16 * j + 6], q[16 * j + 7]),
                         Pack4(q[16 * j + 8], q[16 * j + 9], q[16 * j + 10], q[16 * j + 11]),
                         Pack4(q[16 * j + 12], q[16 * j + 13], q[16 * j + 14], q[16 * j + 15]));
      } else {
        for (int j = 0; j < ncols; ++j) o[j] = uint8_t(q[j]);
      }
      break;
    }
    case ITEXB_DT_FP8_E4M3: case ITEXB_DT_FP8_E5M2: {
      const __nv_fp8_interpretation_t kind = g.out_dtype == ITEXB_DT_FP8_E4M3 ? __NV_E4M3 : __NV_E5M2;
      uint8_t* o = static_cast<uint8_t*>(g.out) + base;
      int q[32];
      float m = *thread_amax;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols) m = fmaxf(m, fabsf(v[j]));
        q[j] = (int)__nv_cvt_float_to_fp8(__fmul_rn(v[j], out_scale), __NV_SATFINITE, kind);
      }
      *thread_amax = m;
      if (vec) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
          reinterpret_cast<uint4*>(o)[j] =
              make_uint4(Pack4(q[16 * j], q[16 * j + 1], q[16 * j + 2], q[16 * j + 3]),
                         Pack4(q[16 * j + 4], q[16 * j + 5], q[16 * j + 6], q[16 * j + 7]),
                         Pack4(q[16 * j + 8], q[16 * j + 9], q[16 * j + 10], q[16 * j + 11]),
                         Pack4(q[16 * j + 12], q[16 * j + 13], q[16 * j + 14], q[16 * j + 15]));
      } else {
        for (int j = 0; j < ncols; ++j) o[j] = uint8_t(q[j]);
      }
      break;
    }
    default: break;
  }
}

__device__ __forceinline__ void TileCoords(int t, int tiles_m, int tiles_n, int* tm, int* tn) {
  const int per_group = kGroupM * tiles_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int rows = min(kGroupM, tiles_m - first_m);
  const int r = t - g * per_group;
  *tm = first_m + r % rows;
  *tn = r / rows;
}

// ---------------------------------------------------------------------------------------
// The kernel.  CONV selects how the producer addresses the A operand: a plain [m,k]
// matrix (2-D map) or NHWC pixels gathered per filter tap (see conv section below).
// ---------------------------------------------------------------------------------------
template <int BN, bool F8>
__global__ void __launch_bounds__(kThreads, 1)
GemmKernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmArgs g) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_scale = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);  // [2][BN]
  float* s_bias = s_scale + 2 * BN;                                              // [2][BN]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + 2 * BN);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tmem_full_bar = bars + 2 * C::kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* ep_decision = abort_flag + 1;  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (g.m + kBM - 1) / kBM;
  const int tiles_n = (g.n + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (g.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      MbarInit(SmemAddr(&full_bar[s]), 1);
      MbarInit(SmemAddr(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      MbarInit(SmemAddr(&tmem_full_bar[a]), 1);
      MbarInit(SmemAddr(&tmem_empty_bar[a]), kEpilogueThreads);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    TmemAlloc(SmemAddr(tmem_slot), C::kTmemCols);
    TmemRelinquish();
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      TileCoords(t, tiles_m, tiles_n, &tm, &tn);
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = MbarWait(SmemAddr(&empty_bar[stage]), phase ^ 1, abort_flag, g.status_word, kErrProducer);
        if (!ok) break;
        const uint32_t fb = SmemAddr(&full_bar[stage]);
        uint8_t* sa = smem + stage * C::kStageBytes;
        MbarArriveExpectTx(fb, C::kStageBytes);
        TmaLoad2d(SmemAddr(sa), &tma_a, fb, kb * kBK, tm * kBM);
        TmaLoad2d(SmemAddr(sa + C::kABytes), &tma_b, fb, kb * kBK, tn * BN);
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok) {
      // Copies already issued land within microseconds; give them a bounded ~200 us
      // before the CTA tears its shared memory down.
      const long long t0 = clock64();
      while (clock64() - t0 < 400000) {}
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      ok = MbarWait(SmemAddr(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, g.status_word, kErrMma);
      if (!ok) break;
      TcFenceAfter();
      const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = MbarWait(SmemAddr(&full_bar[stage]), phase, abort_flag, g.status_word, kErrMma);
        if (!ok) break;
        TcFenceAfter();
        uint8_t* sa = smem + stage * C::kStageBytes;
        const uint64_t a_desc = UmmaDescSw128(SmemAddr(sa));
        const uint64_t b_desc = UmmaDescSw128(SmemAddr(sa + C::kABytes));
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k)
          UmmaSS<F8>(d_tmem, a_desc + uint64_t(k * (kUmmaK >> 4)), b_desc + uint64_t(k * (kUmmaK >> 4)), g.idesc,
                     (kb | k) != 0 ? 1u : 0u);
        TcCommit(SmemAddr(&empty_bar[stage]));  // stage reusable once these MMAs have read it
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      TcCommit(SmemAddr(&tmem_full_bar[acc]));  // accumulator complete
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (warp >= 4) {
    // ---------------- epilogue ----------------
    const int et = threadIdx.x - 4 * 32;  // 0..127
    const int q = warp & 3;               // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    float thread_amax = 0.f;
    float alpha = 1.f;
    const bool has_alpha = g.ep.alpha_a != nullptr && g.ep.alpha_b != nullptr;
    if (has_alpha) alpha = __fmul_rn(__ldg(g.ep.alpha_a), __ldg(g.ep.alpha_b));
    const bool has_scale = has_alpha || g.ep.scale_count > 0;
    const float out_scale = g.ep.out_scale != nullptr ? __ldg(g.ep.out_scale) : 1.f;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int tm, tn;
      TileCoords(t, tiles_m, tiles_n, &tm, &tn);
      float* sc = s_scale + acc * BN;
      float* bi = s_bias + acc * BN;
      for (int i = et; i < BN; i += kEpilogueThreads) {
        const int n = tn * BN + i;
        float s = 1.f, b = 0.f;
        if (n < g.n) {
          if (has_alpha) s = alpha;
          else if (g.ep.scale_count > 1) s = __ldg(g.ep.scale + n);
          else if (g.ep.scale_count == 1) s = __ldg(g.ep.scale);
          if (g.ep.bias != nullptr) b = __ldg(g.ep.bias + n);
        }
        sc[i] = s;
        bi[i] = b;
      }
      MbarWait(SmemAddr(&tmem_full_bar[acc]), acc_phase, abort_flag, g.status_word, kErrEpilogue);
      // One thread samples the abort flag so that all 128 take the same branch.
      if (et == 0) ep_decision[acc] = *abort_flag;
      EpilogueBarrier();  // scale/bias and the decision are visible
      if (ep_decision[acc]) break;
      TcFenceAfter();
      const long long row = (long long)tm * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + uint32_t(acc * BN) + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        TmemLd32(taddr + uint32_t(c * 32), r);
        TmemLdWait();
        const int col0 = tn * BN + c * 32;
        const int ncols = min(32, g.n - col0);
        if (row < g.m && ncols > 0) {
          const bool vec = g.vec_store && ncols == 32;
          if (g.ep.raw_acc) {
            int* o = static_cast<int*>(g.out) + row * g.ldo + col0;
            if (vec) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                reinterpret_cast<int4*>(o)[j] = make_int4(int(r[4 * j]), int(r[4 * j + 1]), int(r[4 * j + 2]), int(r[4 * j + 3]));
            } else {
              for (int j = 0; j < ncols; ++j) o[j] = int(r[j]);
            }
          } else {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float f = F8 ? __uint_as_float(r[j]) : float(int(r[j]));
              if (has_scale) f = __fmul_rn(f, sc[c * 32 + j]);
              if (g.ep.bias != nullptr) f = __fadd_rn(f, bi[c * 32 + j]);
              v[j] = f;
            }
            if (g.ep.summand != nullptr) {
              const long long sb = row * g.ep.ld_summand + col0;
              for (int j = 0; j < ncols; ++j)
                v[j] = __fadd_rn(v[j], __fmul_rn(g.ep.sum_scale, LoadSummand(g.ep.summand, g.ep.summand_dtype, sb + j)));
            }
            if (g.ep.relu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
            }
            if (g.ep.mid_dtype == ITEXB_DT_BFLOAT16) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
            } else if (g.ep.mid_dtype == ITEXB_DT_HALF) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __half2float(__float2half_rn(v[j]));
            }
            StoreRow32(g, v, row, col0, ncols, vec, &thread_amax, out_scale);
          }
        }
      }
      TcFenceBefore();
      MbarArrive(SmemAddr(&tmem_empty_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (g.ep.amax != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) thread_amax = fmaxf(thread_amax, __shfl_xor_sync(0xffffffffu, thread_amax, o));
      if (lane == 0 && thread_amax > 0.f) atomicMax(reinterpret_cast<int*>(g.ep.amax), __float_as_int(thread_amax));
    }
  }

  TcFenceBefore();
  __syncthreads();
  if (warp == 2) {
    TcFenceAfter();
    TmemDealloc(tmem_base, C::kTmemCols);
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

template <int BN, bool F8>
int Launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, cudaStream_t st) {
  using C = Cfg<BN>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(GemmKernel<BN, F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  });
  // The attribute is per device; set it again when the current device changed (cheap).
  static thread_local int last_dev = -1;
  int dev = 0;
  ITEXB_CUDA(cudaGetDevice(&dev));
  if (dev != last_dev) {
    ITEXB_CUDA(cudaFuncSetAttribute(GemmKernel<BN, F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    last_dev = dev;
  }
  ITEXB_CUDA(attr_err);
  const int tiles = ((g.m + kBM - 1) / kBM) * ((g.n + BN - 1) / BN);
  const int grid = std::max(1, std::min(tiles, SmCount()));
  GemmKernel<BN, F8><<<grid, kThreads, C::kSmemBytes, st>>>(ta, tb, g);
  return CheckLaunch("GemmKernel");
}

}  // namespace

int EncodeOperandMap(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  EncodeTiledFn enc = GetEncodeTiled();
  ITEXB_REQUIRE(enc != nullptr, ITEXB_FAILED_PRECONDITION, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld)};
  const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ITEXB_REQUIRE(r == CUDA_SUCCESS, ITEXB_INTERNAL, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld k=%lld ld=%lld)",
                int(r), (long long)rows, (long long)k, (long long)ld);
  return ITEXB_OK;
}

uint32_t MakeInstrDesc(int a_dtype, int b_dtype, int bn) {
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
  // [17,23) N>>3, [24,29) M>>4.
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
}

int PickBN(int n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

int LaunchGemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, int bn, bool f8, cudaStream_t st) {
  if (f8) {
    if (bn == 256) return Launch<256, true>(ta, tb, g, st);
    if (bn == 128) return Launch<128, true>(ta, tb, g, st);
    return Launch<64, true>(ta, tb, g, st);
  }
  if (bn == 256) return Launch<256, false>(ta, tb, g, st);
  if (bn == 128) return Launch<128, false>(ta, tb, g, st);
  return Launch<64, false>(ta, tb, g, st);
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
  CUtensorMap ta, tb;
  const int bn = PickBN(p->n);
  ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&ta, p->a, p->m, p->k, p->lda, kBM));
  ITEXB_RETURN_IF_ERROR(EncodeOperandMap(&tb, p->b, p->n, p->k, p->ldb, bn));
  GemmArgs g{};
  g.m = p->m; g.n = p->n; g.k = p->k;
  g.out_dtype = p->out_dtype;
  g.out = p->out; g.ldo = p->ldo;
  g.ep = p->ep;
  g.status_word = p->status_word;
  g.idesc = MakeInstrDesc(p->a_dtype, p->b_dtype, bn);
  const int osz = (p->ep.raw_acc ? 4 : DtypeSize(p->out_dtype));
  g.vec_store = ((reinterpret_cast<uintptr_t>(p->out) & 15) == 0 && (p->ldo * osz) % 16 == 0) ? 1 : 0;
  return LaunchGemm(ta, tb, g, bn, f8, AsCuda(stream));
}
