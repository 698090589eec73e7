// Op registry, attribute access, per-instance caches and the C-ABI of the op layer
// (itexb_op_* and itexb_simple_context_* of include/itexb200.h).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

#include "op_kernel.h"

namespace itexb {

// One NVTX range per op call, named after the op type: what a timeline tool shows in place of the reference's
// AnnotatedTraceMe around Compute (itex/core/utils/op_kernel.h:970-972).  NVTX 3 is header-only and does nothing
// unless a tool has injected itself into the process.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

// ---- AttrMap --------------------------------------------------------------------------
const itexb_attr_t* AttrMap::Find(const char* name) const {
  for (int i = 0; i < n_; ++i)
    if (attrs_[i].name != nullptr && std::strcmp(attrs_[i].name, name) == 0) return &attrs_[i];
  return nullptr;
}
int AttrMap::Missing(const char* name, const char* want) const {
  return SetError(ITEXB_INVALID_ARGUMENT, "attr '%s' of type %s is missing or has another type", name, want);
}
int AttrMap::GetString(const char* name, std::string* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_STRING || a->s == nullptr) return Missing(name, "string");
  *v = a->s;
  return ITEXB_OK;
}
int AttrMap::GetInt(const char* name, int64_t* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_INT) return Missing(name, "int");
  *v = a->i;
  return ITEXB_OK;
}
int AttrMap::GetFloat(const char* name, float* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_FLOAT) return Missing(name, "float");
  *v = a->f;
  return ITEXB_OK;
}
int AttrMap::GetBool(const char* name, bool* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_BOOL) return Missing(name, "bool");
  *v = a->i != 0;
  return ITEXB_OK;
}
int AttrMap::GetType(const char* name, int* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_TYPE) return Missing(name, "type");
  *v = int(a->i);
  return ITEXB_OK;
}
int AttrMap::GetIntList(const char* name, std::vector<int64_t>* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_INT_LIST) return Missing(name, "list(int)");
  v->assign(a->list_i, a->list_i + a->list_len);
  return ITEXB_OK;
}
int AttrMap::GetStringList(const char* name, std::vector<std::string>* v) const {
  const itexb_attr_t* a = Find(name);
  if (a == nullptr || a->type != ITEXB_ATTR_STRING_LIST) return Missing(name, "list(string)");
  v->clear();
  for (int i = 0; i < a->list_len; ++i) v->emplace_back(a->list_s[i]);
  return ITEXB_OK;
}

// ---- registry -------------------------------------------------------------------------
namespace {
struct Entry {
  OpSignature sig;
  OpFactory factory;
};
std::map<std::string, Entry>& Registry() {
  static std::map<std::string, Entry>* r = new std::map<std::string, Entry>();
  return *r;
}
}  // namespace

void RegisterOp(const char* name, const OpSignature& sig, OpFactory factory) { Registry()[name] = Entry{sig, std::move(factory)}; }

// ---- context helpers ------------------------------------------------------------------
int RequireInputs(const itexb_op_context_t* ctx, int n, const char* op) {
  ITEXB_REQUIRE(ctx != nullptr && ctx->inputs != nullptr, ITEXB_INVALID_ARGUMENT, "%s: context has no inputs", op);
  ITEXB_REQUIRE(ctx->num_inputs == n, ITEXB_INVALID_ARGUMENT, "%s expects %d inputs, got %d", op, n, ctx->num_inputs);
  ITEXB_REQUIRE(ctx->allocate_output != nullptr, ITEXB_INVALID_ARGUMENT, "%s: context has no allocate_output", op);
  return ITEXB_OK;
}
int HostFloats(const itexb_op_context_t* ctx, int i, const char* op, const char* arg, const float** data, int64_t* count) {
  const itexb_tensor_t& t = ctx->inputs[i];
  ITEXB_REQUIRE(t.on_host, ITEXB_INVALID_ARGUMENT, "%s: input '%s' (#%d) is a HostMemory argument but was passed in device memory",
                op, arg, i);
  ITEXB_REQUIRE(t.dtype == ITEXB_DT_FLOAT, ITEXB_INVALID_ARGUMENT, "%s: input '%s' must be float, is %s", op, arg,
                DtypeName(t.dtype));
  *count = NumElements(t);
  ITEXB_REQUIRE(*count >= 1 && t.data != nullptr, ITEXB_INVALID_ARGUMENT, "%s: input '%s' is empty", op, arg);
  *data = static_cast<const float*>(t.data);
  return ITEXB_OK;
}
int HostInts(const itexb_op_context_t* ctx, int i, const char* op, const char* arg, std::vector<int64_t>* v) {
  const itexb_tensor_t& t = ctx->inputs[i];
  ITEXB_REQUIRE(t.on_host, ITEXB_INVALID_ARGUMENT, "%s: input '%s' (#%d) is a HostMemory argument but was passed in device memory",
                op, arg, i);
  ITEXB_REQUIRE(t.dtype == ITEXB_DT_INT32 || t.dtype == ITEXB_DT_INT64, ITEXB_INVALID_ARGUMENT, "%s: input '%s' must be int32 or int64, is %s",
                op, arg, DtypeName(t.dtype));
  const int64_t n = NumElements(t);
  ITEXB_REQUIRE(n == 0 || t.data != nullptr, ITEXB_INVALID_ARGUMENT, "%s: input '%s' has no data", op, arg);
  v->resize(size_t(n));
  for (int64_t j = 0; j < n; ++j)
    (*v)[size_t(j)] = t.dtype == ITEXB_DT_INT32 ? int64_t(static_cast<const int32_t*>(t.data)[j]) : static_cast<const int64_t*>(t.data)[j];
  return ITEXB_OK;
}
int RequireDevice(const itexb_op_context_t* ctx, int i, const char* op, const char* arg) {
  ITEXB_REQUIRE(!ctx->inputs[i].on_host, ITEXB_INVALID_ARGUMENT, "%s: input '%s' (#%d) must be in device memory", op, arg, i);
  return ITEXB_OK;
}
int AllocateOutput(itexb_op_context_t* ctx, int index, int dtype, const int64_t* dims, int rank, bool on_host,
                   itexb_tensor_t* out) {
  ITEXB_REQUIRE(rank <= ITEXB_MAX_DIMS, ITEXB_INVALID_ARGUMENT, "output rank %d exceeds %d", rank, ITEXB_MAX_DIMS);
  std::memset(out, 0, sizeof(*out));
  out->dtype = dtype;
  out->rank = rank;
  for (int i = 0; i < rank; ++i) out->dims[i] = dims[i];
  out->on_host = on_host ? 1 : 0;
  int st = ctx->allocate_output(ctx->user, index, out);
  if (st != ITEXB_OK) return st;
  ITEXB_REQUIRE(out->data != nullptr || NumElements(*out) == 0, ITEXB_RESOURCE_EXHAUSTED, "allocate_output(%d) returned no memory",
                index);
  return ITEXB_OK;
}
int AllocateTemp(itexb_op_context_t* ctx, size_t bytes, bool on_host, void** ptr) {
  ITEXB_REQUIRE(ctx->allocate_temp != nullptr, ITEXB_INVALID_ARGUMENT, "context has no allocate_temp");
  int st = ctx->allocate_temp(ctx->user, bytes, on_host ? 1 : 0, ptr);
  if (st != ITEXB_OK) return st;
  ITEXB_REQUIRE(*ptr != nullptr, ITEXB_RESOURCE_EXHAUSTED, "allocate_temp(%zu) returned no memory", bytes);
  return ITEXB_OK;
}

// ---- DeviceVectorCache ------------------------------------------------------------------
DeviceVectorCache::~DeviceVectorCache() {
  for (Slot& s : slots_) {
    if (s.ev) (void)cudaEventDestroy(s.ev);
    if (s.pinned) (void)cudaFreeHost(s.pinned);
    if (s.dev) (void)itexb_rt_deallocate(ordinal_, s.dev);
  }
}

int DeviceVectorCache::Get(int ordinal, cudaStream_t stream, const float* host, size_t n, const float** dev) {
  ITEXB_REQUIRE(n > 0, ITEXB_INVALID_ARGUMENT, "DeviceVectorCache: empty vector");
  if (cur_ >= 0 && ordinal != ordinal_) {
    // The instance moved to another device: nothing cached here is reachable from there.  The old device's slots are
    // returned once its queued work is done.
    for (Slot& s : slots_) {
      if (s.used) ITEXB_CUDA(cudaEventSynchronize(s.ev));
      if (s.dev) ITEXB_RETURN_IF_ERROR(itexb_rt_deallocate(ordinal_, s.dev));
      s.dev = nullptr;
      if (s.pinned) ITEXB_CUDA(cudaFreeHost(s.pinned));
      s.pinned = nullptr;
      s.cap = 0;
      s.used = false;
    }
    cur_ = -1;
    last_.clear();
  }
  if (cur_ >= 0 && last_.size() == n && std::memcmp(last_.data(), host, n * sizeof(float)) == 0) {
    Slot& hit = slots_[cur_];
    // Another stream than the one that carried the upload: order this stream behind the upload, unless it has landed
    // already.  A stream that is being captured into a graph may not wait on work outside the capture, so there the
    // host waits instead (once: afterwards the event reads as complete).
    if (hit.stream != stream && !hit.landed) {
      RelaxedCaptureMode relaxed;
      const cudaError_t q = cudaEventQuery(hit.ev);
      if (q == cudaErrorNotReady) {
        if (!IsCapturing(stream)) ITEXB_CUDA(cudaStreamWaitEvent(stream, hit.ev, 0));
        else ITEXB_CUDA(cudaEventSynchronize(hit.ev));
      } else {
        ITEXB_CUDA(q);
        hit.landed = true;
      }
    }
    *dev = hit.dev;
    return ITEXB_OK;
  }
  ordinal_ = ordinal;
  ITEXB_REQUIRE(!IsCapturing(stream), ITEXB_FAILED_PRECONDITION,
                "a scale or range vector changed while the stream is being captured into a CUDA graph: run the op once with these "
                "values before the capture (the upload's staging memory is reused later and cannot belong to a graph)");
  const int next = (cur_ + 1) % kSlots;
  Slot& s = slots_[next];
  if (s.used) ITEXB_CUDA(cudaEventSynchronize(s.ev));  // only if the host is 4 uploads ahead
  if (s.cap < n) {
    if (s.pinned) ITEXB_CUDA(cudaFreeHost(s.pinned));
    // kernels queued on the slot's stream four uploads ago may still read the old vector: stream-ordered free
    if (s.dev) ITEXB_RETURN_IF_ERROR(itexb_rt_deallocate_after(ordinal, s.dev, s.stream));
    s.pinned = nullptr;
    s.dev = nullptr;
    s.cap = 0;
    ITEXB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&s.pinned), n * sizeof(float), cudaHostAllocDefault));
    void* d = nullptr;
    ITEXB_RETURN_IF_ERROR(itexb_rt_allocate(ordinal, n * sizeof(float), &d));
    s.dev = static_cast<float*>(d);
    s.cap = n;
  }
  if (s.ev == nullptr) ITEXB_CUDA(cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming));
  std::memcpy(s.pinned, host, n * sizeof(float));
  ITEXB_CUDA(cudaMemcpyAsync(s.dev, s.pinned, n * sizeof(float), cudaMemcpyHostToDevice, stream));
  ITEXB_CUDA(cudaEventRecord(s.ev, stream));
  s.used = true;
  s.landed = false;
  s.stream = stream;
  cur_ = next;
  last_.assign(host, host + n);
  *dev = s.dev;
  return ITEXB_OK;
}

// ---- DeviceBuffer -----------------------------------------------------------------------
int DeviceBuffer::Ensure(int ordinal, size_t bytes, cudaStream_t stream) {
  if (ptr_ != nullptr && bytes_ >= bytes && ordinal_ == ordinal) {
    stream_ = stream;
    return ITEXB_OK;
  }
  Release();
  ITEXB_RETURN_IF_ERROR(itexb_rt_allocate(ordinal, bytes, &ptr_));
  bytes_ = bytes;
  ordinal_ = ordinal;
  stream_ = stream;
  return ITEXB_OK;
}
void DeviceBuffer::Release() {
  // Work queued on the users' stream may still read the buffer (a GEMM launched by the previous Compute).
  if (ptr_ != nullptr) (void)itexb_rt_deallocate_after(ordinal_, ptr_, stream_);
  ptr_ = nullptr;
  bytes_ = 0;
}

// ---- OpKernel: device status word -------------------------------------------------------
namespace {

// Pinned host words for the status read-backs come from one process-wide pool: a page of them is pinned at a time and
// never unpinned, so creating and deleting kernel instances pins and unpins nothing (unpinning synchronizes the device
// and is not allowed while any stream of the thread captures a graph).
class StatusSlots {
 public:
  int* Take() {
    std::lock_guard<std::mutex> l(mu_);
    if (free_.empty()) {
      RelaxedCaptureMode relaxed;
      int* page = nullptr;
      constexpr int kWords = 1024;
      if (cudaHostAlloc(reinterpret_cast<void**>(&page), kWords * sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
      }
      for (int i = kWords - 1; i >= 0; --i) free_.push_back(page + i);
    }
    int* w = free_.back();
    free_.pop_back();
    *w = 0;
    return w;
  }
  void Give(int* w) {
    if (w == nullptr) return;
    std::lock_guard<std::mutex> l(mu_);
    free_.push_back(w);
  }

 private:
  std::mutex mu_;
  std::vector<int*> free_;
};

StatusSlots& Slots() {
  static StatusSlots* s = new StatusSlots();  // outlives every kernel instance, static destruction order included
  return *s;
}

// A deleted instance whose last read-back had not landed yet: its words stay reserved until the event completes, and
// a give-up they report is written to stderr (nobody is left to return a status to).
struct Orphan {
  cudaEvent_t ev;
  int* host;
  int* dev;
  int ordinal;
  cudaStream_t stream;
  std::string name;
};
std::mutex g_orphan_mu;
std::vector<Orphan> g_orphans;

void SweepOrphans() {
  std::lock_guard<std::mutex> l(g_orphan_mu);
  if (g_orphans.empty()) return;
  RelaxedCaptureMode relaxed;
  size_t keep = 0;
  for (size_t i = 0; i < g_orphans.size(); ++i) {
    Orphan& o = g_orphans[i];
    const cudaError_t e = cudaEventQuery(o.ev);
    if (e == cudaErrorNotReady) {
      if (keep != i) g_orphans[keep] = std::move(o);
      ++keep;
      continue;
    }
    if (e != cudaSuccess) (void)cudaGetLastError();
    if (e == cudaSuccess && *o.host != 0)
      std::fprintf(stderr, "itexb: %s (deleted): a kernel gave up on a bounded wait (status %d) and left its output incomplete\n",
                   o.name.c_str(), *o.host);
    (void)cudaEventDestroy(o.ev);
    Slots().Give(o.host);
    (void)itexb_rt_deallocate_after(o.ordinal, o.dev, o.stream);
  }
  g_orphans.resize(keep);
}

}  // namespace

int* OpKernel::StatusWord(int ordinal, cudaStream_t stream) {
  if (status_dev_ != nullptr && status_ordinal_ != ordinal) ReleaseStatus();
  if (status_dev_ == nullptr) {
    // First use inside a graph capture: the zeroing below would become a graph node instead of running now.  This
    // call goes without a status word; the instance gets one at its first Compute outside a capture.
    if (IsCapturing(stream)) return nullptr;
    SweepOrphans();
    void* d = nullptr;
    if (itexb_rt_allocate(ordinal, sizeof(int), &d) != ITEXB_OK) return nullptr;
    status_host_ = Slots().Take();
    if (status_host_ == nullptr || cudaMemsetAsync(d, 0, sizeof(int), stream) != cudaSuccess ||
        cudaEventCreateWithFlags(&status_ev_, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      (void)itexb_rt_deallocate_after(ordinal, d, stream);
      Slots().Give(status_host_);
      status_host_ = nullptr;
      status_ev_ = nullptr;
      return nullptr;
    }
    status_dev_ = static_cast<int*>(d);
    status_ordinal_ = ordinal;
  }
  status_taken_ = true;
  status_stream_ = stream;
  return status_dev_;
}

void OpKernel::QueueStatusReadback(cudaStream_t stream) {
  if (!status_taken_ || status_dev_ == nullptr) return;
  status_taken_ = false;
  if (IsCapturing(stream)) return;
  if (cudaMemcpyAsync(status_host_, status_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream) == cudaSuccess &&
      cudaEventRecord(status_ev_, stream) == cudaSuccess)
    status_pending_ = true;
  else
    (void)cudaGetLastError();
}

int OpKernel::PollStatus(bool wait) {
  if (!status_pending_) return ITEXB_OK;
  RelaxedCaptureMode relaxed;  // the read-back was queued outside any capture
  if (wait) {
    ITEXB_CUDA(cudaEventSynchronize(status_ev_));
  } else {
    const cudaError_t e = cudaEventQuery(status_ev_);
    if (e == cudaErrorNotReady) return ITEXB_OK;
    ITEXB_CUDA(e);
  }
  status_pending_ = false;
  const int code = *status_host_;
  if (code == 0) return ITEXB_OK;
  *status_host_ = 0;
  (void)cudaMemsetAsync(status_dev_, 0, sizeof(int), status_stream_);  // later launches report again
  static const char* const kRoles[] = {"", "TMA producer", "MMA issuer", "epilogue", "shared-memory alignment check"};
  return SetError(ITEXB_ABORTED,
                  "%s: a kernel of an earlier Compute gave up on a bounded wait (status %d, %s) and left its output incomplete",
                  name_.c_str(), code, code >= 1 && code <= 4 ? kRoles[code] : "unknown role");
}

void OpKernel::ReleaseStatus() {
  if (status_dev_ != nullptr) {
    if (status_pending_) {
      // the read-back is still in flight: the words are handed over and released once its event has completed
      std::lock_guard<std::mutex> l(g_orphan_mu);
      g_orphans.push_back(Orphan{status_ev_, status_host_, status_dev_, status_ordinal_, status_stream_, name_});
    } else {
      RelaxedCaptureMode relaxed;
      if (status_ev_ != nullptr) (void)cudaEventDestroy(status_ev_);
      Slots().Give(status_host_);
      (void)itexb_rt_deallocate_after(status_ordinal_, status_dev_, status_stream_);
    }
  }
  status_ev_ = nullptr;
  status_host_ = nullptr;
  status_dev_ = nullptr;
  status_pending_ = status_taken_ = false;
}

}  // namespace itexb

using namespace itexb;

struct itexb_op {
  std::unique_ptr<OpKernel> kernel;
};

// The default context: outputs and temporaries from the runtime allocator.
struct itexb_simple_context {
  itexb_op_context_t ctx;
  int ordinal;
  std::vector<itexb_tensor_t> outputs;
  std::vector<std::pair<void*, bool>> owned;  // (pointer, on_host)
  std::vector<std::pair<void*, bool>> temps;
};

namespace {

int SimpleAlloc(itexb_simple_context* c, size_t bytes, bool on_host, void** ptr) {
  if (on_host) return itexb_rt_host_allocate(bytes, ptr);
  return itexb_rt_allocate(c->ordinal, bytes, ptr);
}
void SimpleFree(itexb_simple_context* c, void* p, bool on_host) {
  if (on_host) (void)itexb_rt_host_deallocate(p);
  else (void)itexb_rt_deallocate(c->ordinal, p);
}

int SimpleAllocateOutput(void* user, int index, itexb_tensor_t* out) {
  auto* c = static_cast<itexb_simple_context*>(user);
  ITEXB_REQUIRE(index >= 0 && index < 64, ITEXB_INVALID_ARGUMENT, "output index %d out of range", index);
  const size_t bytes = size_t(std::max<int64_t>(NumElements(*out), 0)) * DtypeSize(out->dtype);
  void* p = nullptr;
  ITEXB_RETURN_IF_ERROR(SimpleAlloc(c, std::max<size_t>(bytes, 1), out->on_host != 0, &p));
  out->data = p;
  c->owned.emplace_back(p, out->on_host != 0);
  if (int(c->outputs.size()) <= index) c->outputs.resize(index + 1, itexb_tensor_t{});
  c->outputs[index] = *out;
  return ITEXB_OK;
}

int SimpleAllocateTemp(void* user, size_t bytes, int on_host, void** ptr) {
  auto* c = static_cast<itexb_simple_context*>(user);
  ITEXB_RETURN_IF_ERROR(SimpleAlloc(c, std::max<size_t>(bytes, 1), on_host != 0, ptr));
  c->temps.emplace_back(*ptr, on_host != 0);
  return ITEXB_OK;
}

void ReleaseList(itexb_simple_context* c, std::vector<std::pair<void*, bool>>* l) {
  for (auto& p : *l) SimpleFree(c, p.first, p.second);
  l->clear();
}

}  // namespace

extern "C" {

const char* const* itexb_op_list(void) {
  static std::vector<const char*>* names = [] {
    auto* v = new std::vector<const char*>();
    for (auto& kv : Registry()) v->push_back(kv.first.c_str());
    v->push_back(nullptr);
    return v;
  }();
  return names->data();
}

int itexb_op_signature(const char* op_name, int* num_inputs, int* num_outputs, uint32_t* host_input_mask,
                       uint32_t* host_output_mask) {
  ITEXB_REQUIRE(op_name != nullptr, ITEXB_INVALID_ARGUMENT, "op_signature: op_name is NULL");
  auto it = Registry().find(op_name);
  ITEXB_REQUIRE(it != Registry().end(), ITEXB_NOT_FOUND, "Op type not registered '%s'", op_name);
  if (num_inputs) *num_inputs = it->second.sig.num_inputs;
  if (num_outputs) *num_outputs = it->second.sig.num_outputs;
  if (host_input_mask) *host_input_mask = it->second.sig.host_input_mask;
  if (host_output_mask) *host_output_mask = it->second.sig.host_output_mask;
  return ITEXB_OK;
}

int itexb_op_create(const char* op_name, const itexb_attr_t* attrs, int num_attrs, itexb_op_t** op) {
  ITEXB_REQUIRE(op_name != nullptr && op != nullptr, ITEXB_INVALID_ARGUMENT, "op_create: NULL argument");
  *op = nullptr;
  auto it = Registry().find(op_name);
  ITEXB_REQUIRE(it != Registry().end(), ITEXB_NOT_FOUND, "Op type not registered '%s'", op_name);
  std::unique_ptr<OpKernel> k(it->second.factory());
  k->set_name(op_name);
  AttrMap am(attrs, attrs == nullptr ? 0 : num_attrs);
  int st = k->Init(am);
  if (st != ITEXB_OK) return st;
  *op = new itexb_op{std::move(k)};
  return ITEXB_OK;
}

int itexb_op_compute(itexb_op_t* op, itexb_op_context_t* ctx) {
  ITEXB_REQUIRE(op != nullptr && ctx != nullptr, ITEXB_INVALID_ARGUMENT, "op_compute: NULL argument");
  std::lock_guard<std::mutex> lock(op->kernel->mu());
  // Without a usable device the op still runs its host-side checks (and then fails at
  // its first launch), so argument errors are reported the same way everywhere.
  int prev = ctx->device_ordinal;
  if (cudaGetDevice(&prev) != cudaSuccess) {
    (void)cudaGetLastError();
    prev = ctx->device_ordinal;
  }
  if (prev != ctx->device_ordinal) ITEXB_CUDA(cudaSetDevice(ctx->device_ordinal));
  // ITEXB_VERBOSE (the reference's ITEX_VERBOSE, itex/core/utils/op_kernel.h:880-906 and op_kernel.cc:972-980): run the op
  // to completion and print "type,name,nanoseconds" per call.  A node has no name at this boundary, so the second field is
  // the kernel instance's address.
  static const bool verbose = [] {
    const char* e = std::getenv("ITEXB_VERBOSE");
    return e != nullptr && std::atoll(e) != 0;
  }();
  const auto t0 = std::chrono::steady_clock::now();
  // A launch of an earlier Compute of this instance that gave up on a bounded wait is reported now (its read-back has
  // landed by the time the host gets here in all but back-to-back calls; otherwise the call after this one reports it).
  int st = op->kernel->PollStatus(false);
  if (st == ITEXB_OK) {
    NvtxRange range(op->kernel->name().c_str());
    st = op->kernel->Compute(ctx);
    op->kernel->QueueStatusReadback(AsCuda(ctx->stream));
  }
  if (st == ITEXB_OK && (verbose || std::getenv("ITEXB_SYNC_EXEC") != nullptr)) {
    st = CudaStatus(cudaStreamSynchronize(AsCuda(ctx->stream)), verbose ? "ITEXB_VERBOSE" : "ITEXB_SYNC_EXEC");
    if (st == ITEXB_OK) st = op->kernel->PollStatus(true);
  }
  if (verbose) {
    const long long ns = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
    std::fprintf(stderr, "%s,%p,%lld\n", op->kernel->name().c_str(), static_cast<void*>(op->kernel.get()), ns);
  }
  if (prev != ctx->device_ordinal) (void)cudaSetDevice(prev);
  return st;
}

int itexb_op_check(itexb_op_t* op, int wait) {
  ITEXB_REQUIRE(op != nullptr, ITEXB_INVALID_ARGUMENT, "op_check: op is NULL");
  std::lock_guard<std::mutex> lock(op->kernel->mu());
  return op->kernel->PollStatus(wait != 0);
}

void itexb_op_delete(itexb_op_t* op) {
  if (op == nullptr) return;
  // Last chance to learn that a launch of this instance gave up: there is no status to return, so it is written to
  // stderr (and left in itexb_last_error for the calling thread).  A read-back still in flight is not waited for: its
  // words go to the orphan list, which reports the same way once the event has completed.
  if (op->kernel->PollStatus(false) != ITEXB_OK) std::fprintf(stderr, "itexb_op_delete: %s\n", LastError());
  op->kernel->ReleaseStatus();
  delete op;
  SweepOrphans();
}

int itexb_simple_context_create(int device_ordinal, itexb_stream_t stream, itexb_simple_context_t** c) {
  ITEXB_REQUIRE(c != nullptr, ITEXB_INVALID_ARGUMENT, "simple_context_create: NULL argument");
  auto* s = new itexb_simple_context();
  s->ordinal = device_ordinal;
  std::memset(&s->ctx, 0, sizeof(s->ctx));
  s->ctx.user = s;
  s->ctx.device_ordinal = device_ordinal;
  s->ctx.stream = stream;
  s->ctx.allocate_output = SimpleAllocateOutput;
  s->ctx.allocate_temp = SimpleAllocateTemp;
  *c = s;
  return ITEXB_OK;
}

itexb_op_context_t* itexb_simple_context_begin(itexb_simple_context_t* c, const itexb_tensor_t* inputs, int num_inputs) {
  if (c == nullptr) return nullptr;
  c->ctx.inputs = inputs;
  c->ctx.num_inputs = num_inputs;
  c->outputs.clear();
  return &c->ctx;
}

int itexb_simple_context_num_outputs(itexb_simple_context_t* c) { return c == nullptr ? 0 : int(c->outputs.size()); }

const itexb_tensor_t* itexb_simple_context_output(itexb_simple_context_t* c, int index) {
  if (c == nullptr || index < 0 || index >= int(c->outputs.size())) return nullptr;
  return &c->outputs[index];
}

int itexb_simple_context_reset(itexb_simple_context_t* c) {
  ITEXB_REQUIRE(c != nullptr, ITEXB_INVALID_ARGUMENT, "simple_context_reset: NULL argument");
  // Temporaries and outputs may still be read by work queued on the stream.
  ITEXB_CUDA(cudaStreamSynchronize(AsCuda(c->ctx.stream)));
  ReleaseList(c, &c->temps);
  ReleaseList(c, &c->owned);
  c->outputs.clear();
  return ITEXB_OK;
}

void itexb_simple_context_destroy(itexb_simple_context_t* c) {
  if (c == nullptr) return;
  (void)cudaStreamSynchronize(AsCuda(c->ctx.stream));
  ReleaseList(c, &c->temps);
  ReleaseList(c, &c->owned);
  delete c;
}

}  // extern "C"
