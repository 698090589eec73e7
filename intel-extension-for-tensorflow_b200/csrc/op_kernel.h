// Kernel SDK of the op layer: attribute access, the OpKernel base class, registration and
// the small device-side caches the quantized ops keep per instance.  The counterpart of
// the reference's OpKernel / OpKernelConstruction / OpKernelContext facade
// (itex/core/utils/op_kernel.h) reduced to what the hot-path ops use, and free of
// TensorFlow types so that it can be driven by a TF shim or by a test harness alike.
#ifndef ITEXB_CSRC_OP_KERNEL_H_
#define ITEXB_CSRC_OP_KERNEL_H_

#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "common.h"

namespace itexb {

// Read-only view of the attrs a node was created with.
class AttrMap {
 public:
  AttrMap(const itexb_attr_t* attrs, int n) : attrs_(attrs), n_(n) {}
  bool Has(const char* name) const { return Find(name) != nullptr; }
  int GetString(const char* name, std::string* v) const;
  int GetInt(const char* name, int64_t* v) const;
  int GetFloat(const char* name, float* v) const;
  int GetBool(const char* name, bool* v) const;
  int GetType(const char* name, int* v) const;
  int GetIntList(const char* name, std::vector<int64_t>* v) const;
  int GetStringList(const char* name, std::vector<std::string>* v) const;

 private:
  const itexb_attr_t* Find(const char* name) const;
  int Missing(const char* name, const char* want) const;
  const itexb_attr_t* attrs_;
  int n_;
};

struct OpSignature {
  int num_inputs;
  int num_outputs;
  uint32_t host_input_mask;
  uint32_t host_output_mask;
};

class OpKernel {
 public:
  virtual ~OpKernel() = default;
  // Validates attrs; a non-OK status makes itexb_op_create fail (the reference fails
  // construction through OP_REQUIRES on the OpKernelConstruction).
  virtual int Init(const AttrMap& attrs) = 0;
  virtual int Compute(itexb_op_context_t* ctx) = 0;
  const std::string& name() const { return name_; }
  void set_name(const std::string& n) { name_ = n; }
  std::mutex& mu() { return mu_; }

  // ---- device status word ------------------------------------------------------------
  // Every wait inside the GEMM / convolution kernels is bounded; a wait that runs out makes the kernel abandon its
  // tiles and write a role code (1 producer, 2 MMA issuer, 3 epilogue, 4 misaligned shared memory) into a status word.
  // Each op instance owns one such word in device memory and hands it to every launch it makes.  The op layer copies it
  // to pinned host memory behind the launch (asynchronously, with an event) and looks at the copy at the instance's next
  // Compute, after the stream synchronization of ITEXB_SYNC_EXEC / ITEXB_VERBOSE, in itexb_op_check and in
  // itexb_op_delete: a non-zero word becomes ITEXB_ABORTED with the role in the message (the reference turns a failed
  // primitive into errors::Aborted the same way, itex/core/kernels/common/quantize_op.h:409-416).
  // Returns the word for this call's launches (allocated and zeroed on first use), or nullptr if that failed.
  int* StatusWord(int ordinal, cudaStream_t stream);
  // Enqueues the read-back of the word behind what Compute launched (no-op when no launch took the word, or while the
  // stream is being captured into a graph: the word is sticky, a later call reads it).
  void QueueStatusReadback(cudaStream_t stream);
  // Looks at the last read-back: wait = false returns OK while the copy has not landed yet.
  int PollStatus(bool wait);
  void ReleaseStatus();

 private:
  std::string name_;
  std::mutex mu_;  // one Compute at a time per instance
  int* status_dev_ = nullptr;
  int* status_host_ = nullptr;      // pinned
  cudaEvent_t status_ev_ = nullptr;
  cudaStream_t status_stream_ = nullptr;
  int status_ordinal_ = 0;
  bool status_taken_ = false;       // a launch of the current Compute took the word
  bool status_pending_ = false;     // a read-back is in flight or unread
};

using OpFactory = std::function<OpKernel*()>;
void RegisterOp(const char* name, const OpSignature& sig, OpFactory factory);
struct OpRegistrar {
  OpRegistrar(const char* name, const OpSignature& sig, OpFactory f) { RegisterOp(name, sig, std::move(f)); }
};

// ---- context helpers ----------------------------------------------------------------
inline int64_t NumElements(const itexb_tensor_t& t) {
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) n *= t.dims[i];
  return n;
}
int RequireInputs(const itexb_op_context_t* ctx, int n, const char* op);
// Input `i` as host floats (HostMemory argument); fails when the tensor is not on the host.
int HostFloats(const itexb_op_context_t* ctx, int i, const char* op, const char* arg, const float** data, int64_t* count);
// Input `i` as host integers (an int32 or int64 HostMemory argument: shape, perm, axis).
int HostInts(const itexb_op_context_t* ctx, int i, const char* op, const char* arg, std::vector<int64_t>* v);
int RequireDevice(const itexb_op_context_t* ctx, int i, const char* op, const char* arg);
int AllocateOutput(itexb_op_context_t* ctx, int index, int dtype, const int64_t* dims, int rank, bool on_host, itexb_tensor_t* out);
int AllocateTemp(itexb_op_context_t* ctx, size_t bytes, bool on_host, void** ptr);

// Device copy of a small host fp32 vector, re-uploaded (asynchronously, from pinned
// staging, on the op's stream) only when the host values change.  Same job as the
// reference's HostDataCache (itex/core/kernels/common/host_data_cache.h:36-97) without
// its blocking memcpy().wait(): a ring of staging slots guarded by events lets the host
// run ahead of the device.
class DeviceVectorCache {
 public:
  DeviceVectorCache() = default;
  ~DeviceVectorCache();
  DeviceVectorCache(const DeviceVectorCache&) = delete;
  DeviceVectorCache& operator=(const DeviceVectorCache&) = delete;
  // One instance serves one device; calls may come from several streams: a hit from a stream other than the one
  // that carried the upload first waits (on the device) for that upload's event.
  int Get(int ordinal, cudaStream_t stream, const float* host, size_t n, const float** dev);

 private:
  static constexpr int kSlots = 4;
  struct Slot {
    float* pinned = nullptr;
    float* dev = nullptr;
    size_t cap = 0;
    cudaEvent_t ev = nullptr;
    cudaStream_t stream = nullptr;   // the stream that carried the last upload into this slot
    bool used = false;
    bool landed = false;             // the upload's event has been seen complete
  };
  Slot slots_[kSlots];
  int cur_ = -1;
  int ordinal_ = 0;
  std::vector<float> last_;
};

// A persistent device buffer owned by a kernel instance (weights packed once, scaled bias).
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  ~DeviceBuffer() { Release(); }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  // `stream`: the stream the buffer's users run on.  A buffer that has to grow (or move to another device) is returned
  // to the allocator stream-ordered, so kernels already queued on that stream keep reading valid memory.
  int Ensure(int ordinal, size_t bytes, cudaStream_t stream);
  void Release();
  void* data() const { return ptr_; }
  size_t size() const { return bytes_; }

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
  int ordinal_ = 0;
  cudaStream_t stream_ = nullptr;
};

// ---- device-side bias preparation (bias_prep.cu) --------------------------------------
enum BiasPrepMode : int {
  kBiasCopy = 0,           // out = float(bias)
  kBiasMul = 1,            // out = float(bias) * f[j]
  kBiasMinFirstFloat = 2,  // out = bias + (float(colsum)*qmin / f[j])
  kBiasMinFirstInt8 = 3,   // out = bias*f[j]*g[j] + (float(colsum)*qmin*g[j])
  kBiasMinFirstS32 = 4     // out = bias*f[j] + (float(colsum)*qmin)
};
// f and g are device vectors of f_count / g_count (1 or n) entries.
int LaunchBiasPrep(int mode, const void* bias, int bias_dtype, const int32_t* colsum, const float* f, int f_count, const float* g,
                   int g_count, float qmin, float* out, int n, cudaStream_t stream);

// out = in broadcast to out_dims (numpy rules, trailing dims aligned); 2- or 4-byte elements (pointwise.cu).
int LaunchBroadcast(const void* in, const int64_t* in_dims, int in_rank, void* out, const int64_t* out_dims, int out_rank,
                    int elem_bytes, cudaStream_t stream);

}  // namespace itexb

#define ITEXB_REGISTER_OP(op_name, cls, nin, nout, hin, hout) \
  static ::itexb::OpRegistrar ITEXB_CONCAT(reg_, __COUNTER__)(op_name, ::itexb::OpSignature{nin, nout, hin, hout}, [] { return static_cast<::itexb::OpKernel*>(new cls); })
#define ITEXB_CONCAT_(a, b) a##b
#define ITEXB_CONCAT(a, b) ITEXB_CONCAT_(a, b)

#endif  // ITEXB_CSRC_OP_KERNEL_H_
