// Shared internals of libitexb200: status plumbing, dtype helpers, launch accounting.
#ifndef ITEXB_CSRC_COMMON_H_
#define ITEXB_CSRC_COMMON_H_

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "itexb200.h"

namespace itexb {

// Records `msg` as the calling thread's last error and returns `code`.
int SetError(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
const char* LastError();

extern std::atomic<uint64_t> g_launch_count;
inline void CountLaunch(uint64_t n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }

inline int CudaStatus(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return ITEXB_OK;
  return SetError(e == cudaErrorMemoryAllocation ? ITEXB_RESOURCE_EXHAUSTED : ITEXB_INTERNAL, "%s: %s (%s)", what,
                  cudaGetErrorString(e), cudaGetErrorName(e));
}

#define ITEXB_CUDA(expr)                                        \
  do {                                                          \
    int _st = ::itexb::CudaStatus((expr), #expr);               \
    if (_st != ITEXB_OK) return _st;                            \
  } while (0)

#define ITEXB_RETURN_IF_ERROR(expr) \
  do {                              \
    int _st = (expr);               \
    if (_st != ITEXB_OK) return _st;\
  } while (0)

#define ITEXB_REQUIRE(cond, code, ...)                          \
  do {                                                          \
    if (!(cond)) return ::itexb::SetError((code), __VA_ARGS__); \
  } while (0)

// Checks the launch that was just issued (configuration errors surface here).
inline int CheckLaunch(const char* kernel) {
  CountLaunch();
  return CudaStatus(cudaGetLastError(), kernel);
}

inline int DtypeSize(int dt) {
  switch (dt) {
    case ITEXB_DT_FLOAT: case ITEXB_DT_INT32: case ITEXB_DT_QINT32: return 4;
    case ITEXB_DT_INT64: return 8;
    case ITEXB_DT_BFLOAT16: case ITEXB_DT_HALF: return 2;
    case ITEXB_DT_UINT8: case ITEXB_DT_INT8: case ITEXB_DT_QINT8: case ITEXB_DT_QUINT8:
    case ITEXB_DT_FP8_E4M3: case ITEXB_DT_FP8_E5M2: return 1;
    default: return 0;
  }
}

inline const char* DtypeName(int dt) {
  switch (dt) {
    case ITEXB_DT_FLOAT: return "float";
    case ITEXB_DT_INT32: return "int32";
    case ITEXB_DT_INT64: return "int64";
    case ITEXB_DT_UINT8: return "uint8";
    case ITEXB_DT_INT8: return "int8";
    case ITEXB_DT_QINT8: return "qint8";
    case ITEXB_DT_QUINT8: return "quint8";
    case ITEXB_DT_QINT32: return "qint32";
    case ITEXB_DT_BFLOAT16: return "bfloat16";
    case ITEXB_DT_HALF: return "half";
    case ITEXB_DT_FP8_E4M3: return "fp8_e4m3";
    case ITEXB_DT_FP8_E5M2: return "fp8_e5m2";
    default: return "invalid";
  }
}

inline bool IsSigned8(int dt) { return dt == ITEXB_DT_QINT8 || dt == ITEXB_DT_INT8; }
inline bool IsUnsigned8(int dt) { return dt == ITEXB_DT_QUINT8 || dt == ITEXB_DT_UINT8; }
inline bool IsInt8(int dt) { return IsSigned8(dt) || IsUnsigned8(dt); }
inline bool IsFp8(int dt) { return dt == ITEXB_DT_FP8_E4M3 || dt == ITEXB_DT_FP8_E5M2; }

inline cudaStream_t AsCuda(itexb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// While any stream of the process is being captured into a CUDA graph in the default ("global") capture mode, calls
// that are not stream operations - event queries, host or device allocations - are refused and invalidate the capture.
// Bookkeeping calls that only concern work outside the capture (has an earlier upload landed? may a freed block be
// reused?) are made with this guard, which switches the calling thread to the relaxed mode for its lifetime.
struct RelaxedCaptureMode {
  cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
  RelaxedCaptureMode() { if (cudaThreadExchangeStreamCaptureMode(&mode) != cudaSuccess) (void)cudaGetLastError(); }
  ~RelaxedCaptureMode() { if (cudaThreadExchangeStreamCaptureMode(&mode) != cudaSuccess) (void)cudaGetLastError(); }
  RelaxedCaptureMode(const RelaxedCaptureMode&) = delete;
  RelaxedCaptureMode& operator=(const RelaxedCaptureMode&) = delete;
};
inline bool IsCapturing(cudaStream_t stream) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) (void)cudaGetLastError();
  return cap != cudaStreamCaptureStatusNone;
}

// Number of SMs of the current device (cached per device ordinal).
int SmCount();

}  // namespace itexb

#endif  // ITEXB_CSRC_COMMON_H_
