// Device runtime of libitexb200: streams, events, copies and a caching device
// allocator.  Plays the role of the StreamExecutor callback table the reference
// fills in itex/core/devices/gpu/gpu_device_plugin.cc:26-376 and of its BFC
// allocator (itex/core/devices/bfc_allocator.cc:76-140), rewritten over the CUDA
// runtime.  One allocator per device ordinal; freed blocks are kept in
// size-class bins and reused (no driver call on the steady-state path).
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace itexb {

std::atomic<uint64_t> g_launch_count{0};

static thread_local std::string t_last_error;

int SetError(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_last_error = buf;
  return code;
}
const char* LastError() { return t_last_error.c_str(); }

int SmCount() {
  static std::mutex mu;
  static std::unordered_map<int, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  std::lock_guard<std::mutex> l(mu);
  auto it = cache.find(dev);
  if (it != cache.end()) return it->second;
  int n = 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 148;
  cache[dev] = n;
  return n;
}

namespace {

// Rounds a request to its size class: 512 B steps up to 1 MiB, then 2 MiB steps.
size_t SizeClass(size_t bytes) {
  if (bytes == 0) bytes = 1;
  if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);
  const size_t g = size_t(2) << 20;
  return (bytes + g - 1) / g * g;
}

class CachingAllocator {
 public:
  explicit CachingAllocator(int ordinal) : ordinal_(ordinal) {
    const char* lim = std::getenv("ITEXB_LIMIT_MEMORY_MB");
    if (lim != nullptr && *lim) stats_.bytes_limit = int64_t(std::atoll(lim)) << 20;
  }

  int Allocate(size_t bytes, void** ptr) {
    const size_t cls = SizeClass(bytes);
    std::lock_guard<std::mutex> l(mu_);
    SweepPendingLocked();
    auto it = free_.find(cls);
    void* p = nullptr;
    if (it != free_.end() && !it->second.empty()) {
      p = it->second.back();
      it->second.pop_back();
    } else {
      if (stats_.bytes_limit > 0 && stats_.bytes_reserved + int64_t(cls) > stats_.bytes_limit) {
        TrimLocked();
        if (stats_.bytes_reserved + int64_t(cls) > stats_.bytes_limit)
          return SetError(ITEXB_RESOURCE_EXHAUSTED,
                          "device %d: allocating %zu bytes exceeds the %lld-byte limit (ITEXB_LIMIT_MEMORY_MB)",
                          ordinal_, bytes, (long long)stats_.bytes_limit);
      }
      int prev = 0;
      ITEXB_CUDA(cudaGetDevice(&prev));
      if (prev != ordinal_) ITEXB_CUDA(cudaSetDevice(ordinal_));
      cudaError_t e = cudaMalloc(&p, cls);
      if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        TrimLocked();
        e = cudaMalloc(&p, cls);
      }
      if (prev != ordinal_) (void)cudaSetDevice(prev);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return SetError(ITEXB_RESOURCE_EXHAUSTED, "device %d: cudaMalloc(%zu) failed: %s", ordinal_, cls,
                        cudaGetErrorString(e));
      }
      stats_.bytes_reserved += int64_t(cls);
    }
    live_[p] = cls;
    stats_.num_allocs++;
    stats_.bytes_in_use += int64_t(cls);
    if (stats_.bytes_in_use > stats_.peak_bytes_in_use) stats_.peak_bytes_in_use = stats_.bytes_in_use;
    if (int64_t(cls) > stats_.largest_alloc_size) stats_.largest_alloc_size = int64_t(cls);
    *ptr = p;
    return ITEXB_OK;
  }

  int Deallocate(void* p) {
    if (p == nullptr) return ITEXB_OK;
    std::lock_guard<std::mutex> l(mu_);
    auto it = live_.find(p);
    if (it == live_.end()) return SetError(ITEXB_INVALID_ARGUMENT, "deallocate: %p was not allocated by device %d", p, ordinal_);
    free_[it->second].push_back(p);
    stats_.bytes_in_use -= int64_t(it->second);
    live_.erase(it);
    return ITEXB_OK;
  }

  // The block returns to the free lists only after the work queued on `stream` up to now has finished: an event is
  // recorded and Allocate looks at it before handing the block out again.  On a capturing stream no event can be
  // queried later, so the block waits for the next Trim (which synchronizes the device first).
  int DeallocateAfter(void* p, cudaStream_t stream) {
    if (p == nullptr) return ITEXB_OK;
    std::lock_guard<std::mutex> l(mu_);
    auto it = live_.find(p);
    if (it == live_.end()) return SetError(ITEXB_INVALID_ARGUMENT, "deallocate: %p was not allocated by device %d", p, ordinal_);
    Pending pd{p, it->second, nullptr};
    if (!IsCapturing(stream)) {
      int prev = 0;
      const bool switched = cudaGetDevice(&prev) == cudaSuccess && prev != ordinal_ && cudaSetDevice(ordinal_) == cudaSuccess;
      if (cudaEventCreateWithFlags(&pd.ev, cudaEventDisableTiming) != cudaSuccess || cudaEventRecord(pd.ev, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        if (pd.ev != nullptr) (void)cudaEventDestroy(pd.ev);
        pd.ev = nullptr;
      }
      if (switched) (void)cudaSetDevice(prev);
    }
    pending_.push_back(pd);
    stats_.bytes_in_use -= int64_t(it->second);
    live_.erase(it);
    return ITEXB_OK;
  }

  int Trim() {
    std::lock_guard<std::mutex> l(mu_);
    TrimLocked();
    return ITEXB_OK;
  }

  itexb_allocator_stats_t Stats() {
    std::lock_guard<std::mutex> l(mu_);
    return stats_;
  }

 private:
  struct Pending {
    void* ptr;
    size_t cls;
    cudaEvent_t ev;  // nullptr: no event could be recorded; released by Trim only
  };

  // Moves the blocks whose event has completed to the free lists.
  void SweepPendingLocked() {
    if (pending_.empty()) return;
    RelaxedCaptureMode relaxed;  // the events belong to work outside any capture
    size_t keep = 0;
    for (size_t i = 0; i < pending_.size(); ++i) {
      Pending& pd = pending_[i];
      bool done = false;
      if (pd.ev != nullptr) {
        const cudaError_t e = cudaEventQuery(pd.ev);
        if (e == cudaSuccess) done = true;
        else if (e != cudaErrorNotReady) (void)cudaGetLastError();
      }
      if (done) {
        (void)cudaEventDestroy(pd.ev);
        free_[pd.cls].push_back(pd.ptr);
      } else {
        pending_[keep++] = pd;
      }
    }
    pending_.resize(keep);
  }

  void TrimLocked() {
    if (!pending_.empty()) {
      int prev = 0;
      const bool switched = cudaGetDevice(&prev) == cudaSuccess && prev != ordinal_ && cudaSetDevice(ordinal_) == cudaSuccess;
      if (cudaDeviceSynchronize() == cudaSuccess) {
        for (Pending& pd : pending_) {
          if (pd.ev != nullptr) (void)cudaEventDestroy(pd.ev);
          free_[pd.cls].push_back(pd.ptr);
        }
        pending_.clear();
      } else {
        (void)cudaGetLastError();
      }
      if (switched) (void)cudaSetDevice(prev);
    }
    for (auto& kv : free_) {
      for (void* p : kv.second) {
        if (cudaFree(p) == cudaSuccess) stats_.bytes_reserved -= int64_t(kv.first);
      }
      kv.second.clear();
    }
  }

  int ordinal_;
  std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_;
  std::unordered_map<void*, size_t> live_;
  std::vector<Pending> pending_;
  itexb_allocator_stats_t stats_{};
};

CachingAllocator* AllocatorFor(int ordinal) {
  static std::mutex mu;
  static std::map<int, CachingAllocator*> table;
  std::lock_guard<std::mutex> l(mu);
  auto it = table.find(ordinal);
  if (it != table.end()) return it->second;
  auto* a = new CachingAllocator(ordinal);  // lives until process exit, like the device itself
  table[ordinal] = a;
  return a;
}

struct HostCallback {
  void (*fn)(void*);
  void* arg;
};
void CUDART_CB RunHostCallback(void* p) {
  auto* cb = static_cast<HostCallback*>(p);
  cb->fn(cb->arg);
  delete cb;
}

}  // namespace
}  // namespace itexb

using namespace itexb;

extern "C" {

const char* itexb_last_error(void) { return LastError(); }
const char* itexb_version(void) { return "itexb200 0.1 (sm_100a)"; }
uint64_t itexb_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int itexb_rt_device_count(int* count) {
  ITEXB_REQUIRE(count != nullptr, ITEXB_INVALID_ARGUMENT, "device_count: count is NULL");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    *count = 0;
    return SetError(ITEXB_FAILED_PRECONDITION, "no usable CUDA device: %s", cudaGetErrorString(e));
  }
  return ITEXB_OK;
}
int itexb_rt_set_device(int ordinal) { ITEXB_CUDA(cudaSetDevice(ordinal)); return ITEXB_OK; }
int itexb_rt_device_memory_usage(int ordinal, int64_t* free_bytes, int64_t* total_bytes) {
  int prev = 0;
  ITEXB_CUDA(cudaGetDevice(&prev));
  ITEXB_CUDA(cudaSetDevice(ordinal));
  size_t f = 0, t = 0;
  cudaError_t e = cudaMemGetInfo(&f, &t);
  (void)cudaSetDevice(prev);
  ITEXB_CUDA(e);
  if (free_bytes) *free_bytes = int64_t(f);
  if (total_bytes) *total_bytes = int64_t(t);
  return ITEXB_OK;
}
int itexb_rt_allocate(int ordinal, size_t bytes, void** ptr) {
  ITEXB_REQUIRE(ptr != nullptr, ITEXB_INVALID_ARGUMENT, "allocate: ptr is NULL");
  return AllocatorFor(ordinal)->Allocate(bytes, ptr);
}
int itexb_rt_deallocate(int ordinal, void* ptr) { return AllocatorFor(ordinal)->Deallocate(ptr); }
int itexb_rt_deallocate_after(int ordinal, void* ptr, itexb_stream_t stream) {
  return AllocatorFor(ordinal)->DeallocateAfter(ptr, AsCuda(stream));
}
int itexb_rt_host_allocate(size_t bytes, void** ptr) {
  ITEXB_REQUIRE(ptr != nullptr, ITEXB_INVALID_ARGUMENT, "host_allocate: ptr is NULL");
  ITEXB_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocDefault));
  return ITEXB_OK;
}
int itexb_rt_host_deallocate(void* ptr) {
  if (ptr) ITEXB_CUDA(cudaFreeHost(ptr));
  return ITEXB_OK;
}
int itexb_rt_allocator_stats(int ordinal, itexb_allocator_stats_t* stats) {
  ITEXB_REQUIRE(stats != nullptr, ITEXB_INVALID_ARGUMENT, "allocator_stats: stats is NULL");
  *stats = AllocatorFor(ordinal)->Stats();
  return ITEXB_OK;
}
int itexb_rt_trim(int ordinal) { return AllocatorFor(ordinal)->Trim(); }

int itexb_rt_create_stream(int ordinal, itexb_stream_t* stream) {
  ITEXB_REQUIRE(stream != nullptr, ITEXB_INVALID_ARGUMENT, "create_stream: stream is NULL");
  int prev = 0;
  ITEXB_CUDA(cudaGetDevice(&prev));
  ITEXB_CUDA(cudaSetDevice(ordinal));
  cudaStream_t s = nullptr;
  cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  (void)cudaSetDevice(prev);
  ITEXB_CUDA(e);
  *stream = s;
  return ITEXB_OK;
}
int itexb_rt_destroy_stream(itexb_stream_t stream) {
  if (stream) ITEXB_CUDA(cudaStreamDestroy(AsCuda(stream)));
  return ITEXB_OK;
}
int itexb_rt_stream_dependency(itexb_stream_t dependent, itexb_stream_t other) {
  cudaEvent_t ev = nullptr;
  ITEXB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ev, AsCuda(other));
  if (e == cudaSuccess) e = cudaStreamWaitEvent(AsCuda(dependent), ev, 0);
  (void)cudaEventDestroy(ev);
  ITEXB_CUDA(e);
  return ITEXB_OK;
}
int itexb_rt_stream_device(itexb_stream_t stream, int* ordinal) {
  ITEXB_REQUIRE(ordinal != nullptr, ITEXB_INVALID_ARGUMENT, "stream_device: ordinal is NULL");
  if (stream == nullptr) {
    ITEXB_CUDA(cudaGetDevice(ordinal));
  } else {
    ITEXB_CUDA(cudaStreamGetDevice(AsCuda(stream), ordinal));
  }
  return ITEXB_OK;
}
int itexb_rt_stream_status(itexb_stream_t stream) {
  cudaError_t e = cudaStreamQuery(AsCuda(stream));
  if (e == cudaSuccess || e == cudaErrorNotReady) return ITEXB_OK;
  return CudaStatus(e, "stream_status");
}
int itexb_rt_create_event(itexb_event_t* event) {
  ITEXB_REQUIRE(event != nullptr, ITEXB_INVALID_ARGUMENT, "create_event: event is NULL");
  cudaEvent_t ev = nullptr;
  ITEXB_CUDA(cudaEventCreate(&ev));
  *event = ev;
  return ITEXB_OK;
}
int itexb_rt_destroy_event(itexb_event_t event) {
  if (event) ITEXB_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return ITEXB_OK;
}
int itexb_rt_record_event(itexb_stream_t stream, itexb_event_t event) {
  ITEXB_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), AsCuda(stream)));
  return ITEXB_OK;
}
int itexb_rt_wait_for_event(itexb_stream_t stream, itexb_event_t event) {
  ITEXB_CUDA(cudaStreamWaitEvent(AsCuda(stream), static_cast<cudaEvent_t>(event), 0));
  return ITEXB_OK;
}
int itexb_rt_event_status(itexb_event_t event, int* complete) {
  ITEXB_REQUIRE(complete != nullptr, ITEXB_INVALID_ARGUMENT, "event_status: complete is NULL");
  cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
  if (e == cudaSuccess) { *complete = 1; return ITEXB_OK; }
  if (e == cudaErrorNotReady) { *complete = 0; return ITEXB_OK; }
  return CudaStatus(e, "event_status");
}
int itexb_rt_event_elapsed_ms(itexb_event_t start, itexb_event_t stop, float* ms) {
  ITEXB_REQUIRE(ms != nullptr, ITEXB_INVALID_ARGUMENT, "event_elapsed_ms: ms is NULL");
  ITEXB_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return ITEXB_OK;
}
int itexb_rt_memcpy_h2d(void* d, const void* s, size_t n, itexb_stream_t st) {
  ITEXB_CUDA(cudaMemcpyAsync(d, s, n, cudaMemcpyHostToDevice, AsCuda(st)));
  return ITEXB_OK;
}
int itexb_rt_memcpy_d2h(void* d, const void* s, size_t n, itexb_stream_t st) {
  ITEXB_CUDA(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToHost, AsCuda(st)));
  return ITEXB_OK;
}
int itexb_rt_memcpy_d2d(void* d, const void* s, size_t n, itexb_stream_t st) {
  ITEXB_CUDA(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, AsCuda(st)));
  return ITEXB_OK;
}
int itexb_rt_sync_memcpy_h2d(void* d, const void* s, size_t n) {
  ITEXB_CUDA(cudaMemcpy(d, s, n, cudaMemcpyHostToDevice));
  return ITEXB_OK;
}
int itexb_rt_sync_memcpy_d2h(void* d, const void* s, size_t n) {
  ITEXB_CUDA(cudaMemcpy(d, s, n, cudaMemcpyDeviceToHost));
  return ITEXB_OK;
}
int itexb_rt_sync_memcpy_d2d(void* d, const void* s, size_t n) {
  ITEXB_CUDA(cudaMemcpy(d, s, n, cudaMemcpyDeviceToDevice));
  return ITEXB_OK;
}
int itexb_rt_mem_zero(void* dev, size_t bytes, itexb_stream_t st) {
  ITEXB_CUDA(cudaMemsetAsync(dev, 0, bytes, AsCuda(st)));
  return ITEXB_OK;
}
int itexb_rt_memset(void* dev, uint8_t value, size_t bytes, itexb_stream_t st) {
  ITEXB_CUDA(cudaMemsetAsync(dev, value, bytes, AsCuda(st)));
  return ITEXB_OK;
}

}  // extern "C"

namespace itexb {
__global__ void Memset32Kernel(uint32_t* p, uint32_t v, size_t n) {
  size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) p[i] = v;
}
}  // namespace itexb

extern "C" {

int itexb_rt_memset32(void* dev, uint32_t pattern, size_t bytes, itexb_stream_t st) {
  ITEXB_REQUIRE(bytes % 4 == 0 && (reinterpret_cast<uintptr_t>(dev) & 3) == 0, ITEXB_INVALID_ARGUMENT,
                "memset32: pointer and size must be multiples of 4");
  const size_t n = bytes / 4;
  if (n == 0) return ITEXB_OK;
  const int threads = 256;
  const int blocks = int(std::min<size_t>((n + threads - 1) / threads, size_t(SmCount()) * 8));
  Memset32Kernel<<<blocks, threads, 0, AsCuda(st)>>>(static_cast<uint32_t*>(dev), pattern, n);
  return CheckLaunch("Memset32Kernel");
}
int itexb_rt_block_host_until_done(itexb_stream_t st) {
  ITEXB_CUDA(cudaStreamSynchronize(AsCuda(st)));
  return ITEXB_OK;
}
int itexb_rt_block_host_for_event(itexb_event_t ev) {
  ITEXB_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(ev)));
  return ITEXB_OK;
}
int itexb_rt_synchronize_all_activity(int ordinal) {
  int prev = 0;
  ITEXB_CUDA(cudaGetDevice(&prev));
  ITEXB_CUDA(cudaSetDevice(ordinal));
  cudaError_t e = cudaDeviceSynchronize();
  (void)cudaSetDevice(prev);
  ITEXB_CUDA(e);
  return ITEXB_OK;
}
int itexb_rt_host_callback(itexb_stream_t st, void (*fn)(void*), void* arg) {
  ITEXB_REQUIRE(fn != nullptr, ITEXB_INVALID_ARGUMENT, "host_callback: fn is NULL");
  auto* cb = new HostCallback{fn, arg};
  cudaError_t e = cudaLaunchHostFunc(AsCuda(st), RunHostCallback, cb);
  if (e != cudaSuccess) delete cb;
  ITEXB_CUDA(e);
  return ITEXB_OK;
}

int itexb_rt_ipc_export(void* dev_ptr, unsigned char handle[ITEXB_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == ITEXB_IPC_HANDLE_BYTES, "handle size");
  ITEXB_REQUIRE(dev_ptr != nullptr && handle != nullptr, ITEXB_INVALID_ARGUMENT, "ipc_export: NULL argument");
  cudaIpcMemHandle_t h;
  ITEXB_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
  std::memcpy(handle, &h, sizeof(h));
  return ITEXB_OK;
}
int itexb_rt_ipc_open(const unsigned char handle[ITEXB_IPC_HANDLE_BYTES], void** dev_ptr) {
  ITEXB_REQUIRE(dev_ptr != nullptr && handle != nullptr, ITEXB_INVALID_ARGUMENT, "ipc_open: NULL argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  ITEXB_CUDA(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return ITEXB_OK;
}
int itexb_rt_ipc_close(void* dev_ptr) {
  if (dev_ptr != nullptr) ITEXB_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  return ITEXB_OK;
}

}  // extern "C"

namespace itexb {
namespace {

struct FlagPtrs { int* p[ITEXB_MAX_PEERS + 1]; };

// Everything queued before this kernel on its stream has completed; the fence makes those writes (to local and peer
// memory) visible system-wide before the flags are.
__global__ void PeerSignalKernel(FlagPtrs f, int n, int value, const int* value_ptr) {
  if (value_ptr != nullptr) value += *value_ptr;
  __threadfence_system();
  const int i = threadIdx.x;
  if (i < n) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f.p[i]), "r"(value) : "memory");
  }
}

// One lane per flag; every wait is bounded.
__global__ void PeerWaitKernel(const int* flags, int n, int value, const int* value_ptr, int* status_word, long long limit) {
  if (value_ptr != nullptr) value += *value_ptr;
  const int i = threadIdx.x;
  bool ok = true;
  if (i < n) {
    const long long t0 = clock64();
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
      if (v >= value) break;
      if (clock64() - t0 > limit) { ok = false; break; }
      __nanosleep(200);
    }
  }
  if (!ok && status_word != nullptr) atomicCAS(status_word, 0, 5);
  __threadfence_system();
}

}  // namespace
long long GemmWaitLimitCycles();
}  // namespace itexb

__global__ void PeerAdvanceKernel(int* counter) { *counter += 1; }

extern "C" int itexb_peer_advance(int32_t* counter, itexb_stream_t stream) {
  ITEXB_REQUIRE(counter != nullptr, ITEXB_INVALID_ARGUMENT, "peer_advance: counter is NULL");
  PeerAdvanceKernel<<<1, 1, 0, AsCuda(stream)>>>(counter);
  return CheckLaunch("PeerAdvanceKernel");
}

extern "C" int itexb_peer_signal(int32_t* const* flag_ptrs, int32_t n, int32_t value, const int32_t* value_ptr, itexb_stream_t stream) {
  ITEXB_REQUIRE(flag_ptrs != nullptr && n >= 0 && n <= ITEXB_MAX_PEERS + 1, ITEXB_INVALID_ARGUMENT, "peer_signal: bad arguments");
  if (n == 0) return ITEXB_OK;
  FlagPtrs f{};
  for (int i = 0; i < n; ++i) {
    ITEXB_REQUIRE(flag_ptrs[i] != nullptr, ITEXB_INVALID_ARGUMENT, "peer_signal: flag pointer %d is NULL", i);
    f.p[i] = flag_ptrs[i];
  }
  PeerSignalKernel<<<1, 32, 0, AsCuda(stream)>>>(f, n, value, value_ptr);
  return CheckLaunch("PeerSignalKernel");
}

extern "C" int itexb_peer_wait(const int32_t* local_flags, int32_t n, int32_t value, const int32_t* value_ptr, int32_t* status_word,
                               itexb_stream_t stream) {
  ITEXB_REQUIRE(local_flags != nullptr && n >= 0 && n <= 32, ITEXB_INVALID_ARGUMENT, "peer_wait: bad arguments");
  if (n == 0) return ITEXB_OK;
  PeerWaitKernel<<<1, 32, 0, AsCuda(stream)>>>(local_flags, n, value, value_ptr, status_word, itexb::GemmWaitLimitCycles() / 2);
  return CheckLaunch("PeerWaitKernel");
}

