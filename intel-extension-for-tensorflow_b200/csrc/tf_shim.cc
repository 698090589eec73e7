// TensorFlow PluggableDevice shim over the C-ABI of libitexb200: the two entry points TensorFlow's plugin loader needs
// from a shared object under site-packages/tensorflow-plugins/ to run this library's kernels -
//
//   SE_InitPlugin   the device: platform, stream executor and timer tables over itexb_rt_*
//                   (what itex/core/devices/gpu/gpu_device_plugin.cc:26-376 fills, listed at
//                   itex/core/wrapper/itex_gpu_wrapper.cc:190-228,269-299);
//   TF_InitKernel   op definitions (itexb_op_def; registration pattern itex/core/ops/nn_ops.cc:1070-1102) and kernels
//                   (TF_NewKernelBuilder + HostMemory, itex/core/utils/op_kernel.cc:887-918) for every name in
//                   itexb_op_list(), each kernel being create / compute / delete over itexb_op_create / _compute /
//                   _delete (callback signatures: itex/core/utils/op_kernel.h:710-714);
// (The third entry point a plugin may export, TF_InitGraph, is not in this file: its optimizer walks a serialized
// GraphDef, which needs the protobuf classes of the TensorFlow build; per node it only has to call itexb_rewrite_node.)
//
// This translation unit is compiled only where TensorFlow's C headers are on the include path (they are not part of
// this repository and this library never needs them); the build of libitexb200.so skips it otherwise.  It contains no
// arithmetic: every decision (attrs, shapes, HostMemory arguments, errors) is taken below the C-ABI, so that the same
// code path is exercised by the tests, which drive the C-ABI directly.
#if defined(__has_include)
#if __has_include("tensorflow/c/kernels.h") && __has_include("tensorflow/c/experimental/stream_executor/stream_executor.h")
#define ITEXB_HAVE_TENSORFLOW 1
#endif
#endif

#ifdef ITEXB_HAVE_TENSORFLOW

#include <array>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "itexb200.h"
#include "tensorflow/c/experimental/stream_executor/stream_executor.h"
#include "tensorflow/c/kernels.h"
#include "tensorflow/c/ops.h"
#include "tensorflow/c/tf_datatype.h"
#include "tensorflow/c/tf_status.h"
#include "tensorflow/c/tf_tensor.h"

// The plugin defines what SP_Stream / SP_Event / SP_Timer point to (gpu_device_plugin.h:23-26 in the reference).
struct SP_Stream_st {
  itexb_stream_t stream_handle;
};
struct SP_Event_st {
  itexb_event_t event_handle;
};
struct SP_Timer_st {
  itexb_event_t start, stop;
};

namespace {

constexpr char kDeviceType[] = "GPU";       // the device type graphs are placed on
constexpr char kPlatformName[] = "ITEXB200";

void SetStatus(TF_Status* status, int code) {
  // itexb_status_t uses TensorFlow's numbering of error codes
  if (status == nullptr) return;
  if (code == ITEXB_OK) TF_SetStatus(status, TF_OK, "");
  else TF_SetStatus(status, static_cast<TF_Code>(code), itexb_last_error());
}

// ------------------------------------------------------------------------------------------------------------------
// Device runtime: the SP_StreamExecutor callbacks, one line each over itexb_rt_*.
// ------------------------------------------------------------------------------------------------------------------
void DeviceCount(const SP_Platform*, int* count, TF_Status* status) { SetStatus(status, itexb_rt_device_count(count)); }

void CreateDevice(const SP_Platform*, SE_CreateDeviceParams* params, TF_Status* status) {
  params->device->struct_size = SP_DEVICE_STRUCT_SIZE;
  params->device->device_handle = nullptr;  // the ordinal says it all
  params->device->ordinal = params->ordinal;
  TF_SetStatus(status, TF_OK, "");
}
void DestroyDevice(const SP_Platform*, SP_Device* device) { device->ordinal = -1; }
void CreateDeviceFns(const SP_Platform*, SE_CreateDeviceFnsParams* params, TF_Status* status) {
  params->device_fns->struct_size = SP_DEVICE_FNS_STRUCT_SIZE;
  TF_SetStatus(status, TF_OK, "");
}
void DestroyDeviceFns(const SP_Platform*, SP_DeviceFns*) {}

void Allocate(const SP_Device* device, uint64_t size, int64_t /*memory_space*/, SP_DeviceMemoryBase* mem) {
  mem->struct_size = SP_DEVICE_MEMORY_BASE_STRUCT_SIZE;
  void* p = nullptr;
  if (itexb_rt_allocate(device->ordinal, size, &p) != ITEXB_OK) p = nullptr;  // TensorFlow reads a null opaque as out of memory
  mem->opaque = p;
  mem->size = size;
}
void Deallocate(const SP_Device* device, SP_DeviceMemoryBase* mem) {
  // TensorFlow frees a buffer only after the work that uses it has finished (it orders frees itself).
  (void)itexb_rt_deallocate(device->ordinal, mem->opaque);
  mem->opaque = nullptr;
  mem->size = 0;
}
void* HostMemoryAllocate(const SP_Device*, uint64_t size) {
  void* p = nullptr;
  return itexb_rt_host_allocate(size, &p) == ITEXB_OK ? p : nullptr;
}
void HostMemoryDeallocate(const SP_Device*, void* mem) { (void)itexb_rt_host_deallocate(mem); }

TF_Bool GetAllocatorStats(const SP_Device* device, SP_AllocatorStats* stats) {
  itexb_allocator_stats_t s;
  if (itexb_rt_allocator_stats(device->ordinal, &s) != ITEXB_OK) return false;
  stats->struct_size = SP_ALLOCATORSTATS_STRUCT_SIZE;
  stats->num_allocs = s.num_allocs;
  stats->bytes_in_use = s.bytes_in_use;
  stats->peak_bytes_in_use = s.peak_bytes_in_use;
  stats->largest_alloc_size = s.largest_alloc_size;
  stats->has_bytes_limit = s.bytes_limit > 0;
  stats->bytes_limit = s.bytes_limit;
  stats->bytes_reserved = s.bytes_reserved;
  stats->peak_bytes_reserved = s.bytes_reserved;
  stats->has_bytes_reservable_limit = false;
  stats->bytes_reservable_limit = 0;
  stats->largest_free_block_bytes = 0;
  return true;
}
TF_Bool DeviceMemoryUsage(const SP_Device* device, int64_t* free_bytes, int64_t* total_bytes) {
  return itexb_rt_device_memory_usage(device->ordinal, free_bytes, total_bytes) == ITEXB_OK;
}

void CreateStream(const SP_Device* device, SP_Stream* stream, TF_Status* status) {
  itexb_stream_t s = nullptr;
  const int st = itexb_rt_create_stream(device->ordinal, &s);
  if (st == ITEXB_OK) *stream = new SP_Stream_st{s};
  SetStatus(status, st);
}
void DestroyStream(const SP_Device*, SP_Stream stream) {
  if (stream == nullptr) return;
  (void)itexb_rt_destroy_stream(stream->stream_handle);
  delete stream;
}
void CreateStreamDependency(const SP_Device*, SP_Stream dependent, SP_Stream other, TF_Status* status) {
  SetStatus(status, itexb_rt_stream_dependency(dependent->stream_handle, other->stream_handle));
}
void GetStreamStatus(const SP_Device*, SP_Stream stream, TF_Status* status) { SetStatus(status, itexb_rt_stream_status(stream->stream_handle)); }

void CreateEvent(const SP_Device*, SP_Event* event, TF_Status* status) {
  itexb_event_t e = nullptr;
  const int st = itexb_rt_create_event(&e);
  if (st == ITEXB_OK) *event = new SP_Event_st{e};
  SetStatus(status, st);
}
void DestroyEvent(const SP_Device*, SP_Event event) {
  if (event == nullptr) return;
  (void)itexb_rt_destroy_event(event->event_handle);
  delete event;
}
SE_EventStatus GetEventStatus(const SP_Device*, SP_Event event) {
  int complete = 0;
  if (itexb_rt_event_status(event->event_handle, &complete) != ITEXB_OK) return SE_EVENT_ERROR;
  return complete ? SE_EVENT_COMPLETE : SE_EVENT_PENDING;
}
void RecordEvent(const SP_Device*, SP_Stream stream, SP_Event event, TF_Status* status) {
  SetStatus(status, itexb_rt_record_event(stream->stream_handle, event->event_handle));
}
void WaitForEvent(const SP_Device*, SP_Stream stream, SP_Event event, TF_Status* status) {
  SetStatus(status, itexb_rt_wait_for_event(stream->stream_handle, event->event_handle));
}

void CreateTimer(const SP_Device*, SP_Timer* timer, TF_Status* status) {
  itexb_event_t a = nullptr, b = nullptr;
  int st = itexb_rt_create_event(&a);
  if (st == ITEXB_OK) st = itexb_rt_create_event(&b);
  if (st == ITEXB_OK) *timer = new SP_Timer_st{a, b};
  SetStatus(status, st);
}
void DestroyTimer(const SP_Device*, SP_Timer timer) {
  if (timer == nullptr) return;
  (void)itexb_rt_destroy_event(timer->start);
  (void)itexb_rt_destroy_event(timer->stop);
  delete timer;
}
void StartTimer(const SP_Device*, SP_Stream stream, SP_Timer timer, TF_Status* status) {
  SetStatus(status, itexb_rt_record_event(stream->stream_handle, timer->start));
}
void StopTimer(const SP_Device*, SP_Stream stream, SP_Timer timer, TF_Status* status) {
  SetStatus(status, itexb_rt_record_event(stream->stream_handle, timer->stop));
}
uint64_t TimerNanoseconds(SP_Timer timer) {
  float ms = 0.f;
  if (itexb_rt_block_host_for_event(timer->stop) != ITEXB_OK || itexb_rt_event_elapsed_ms(timer->start, timer->stop, &ms) != ITEXB_OK) return 0;
  return static_cast<uint64_t>(static_cast<double>(ms) * 1e6);
}

void MemcpyDtoH(const SP_Device*, SP_Stream stream, void* host_dst, const SP_DeviceMemoryBase* device_src, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_memcpy_d2h(host_dst, device_src->opaque, size, stream->stream_handle));
}
void MemcpyHtoD(const SP_Device*, SP_Stream stream, SP_DeviceMemoryBase* device_dst, const void* host_src, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_memcpy_h2d(device_dst->opaque, host_src, size, stream->stream_handle));
}
void MemcpyDtoD(const SP_Device*, SP_Stream stream, SP_DeviceMemoryBase* device_dst, const SP_DeviceMemoryBase* device_src, uint64_t size,
                TF_Status* status) {
  SetStatus(status, itexb_rt_memcpy_d2d(device_dst->opaque, device_src->opaque, size, stream->stream_handle));
}
void SyncMemcpyDtoH(const SP_Device*, void* host_dst, const SP_DeviceMemoryBase* device_src, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_sync_memcpy_d2h(host_dst, device_src->opaque, size));
}
void SyncMemcpyHtoD(const SP_Device*, SP_DeviceMemoryBase* device_dst, const void* host_src, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_sync_memcpy_h2d(device_dst->opaque, host_src, size));
}
void SyncMemcpyDtoD(const SP_Device*, SP_DeviceMemoryBase* device_dst, const SP_DeviceMemoryBase* device_src, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_sync_memcpy_d2d(device_dst->opaque, device_src->opaque, size));
}
void BlockHostForEvent(const SP_Device*, SP_Event event, TF_Status* status) { SetStatus(status, itexb_rt_block_host_for_event(event->event_handle)); }
void BlockHostUntilDone(const SP_Device*, SP_Stream stream, TF_Status* status) {
  SetStatus(status, itexb_rt_block_host_until_done(stream->stream_handle));
}
void SynchronizeAllActivity(const SP_Device* device, TF_Status* status) { SetStatus(status, itexb_rt_synchronize_all_activity(device->ordinal)); }
void MemZero(const SP_Device*, SP_Stream stream, SP_DeviceMemoryBase* location, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_mem_zero(location->opaque, size, stream->stream_handle));
}
void Memset(const SP_Device*, SP_Stream stream, SP_DeviceMemoryBase* location, uint8_t pattern, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_memset(location->opaque, pattern, size, stream->stream_handle));
}
void Memset32(const SP_Device*, SP_Stream stream, SP_DeviceMemoryBase* location, uint32_t pattern, uint64_t size, TF_Status* status) {
  SetStatus(status, itexb_rt_memset32(location->opaque, pattern, size, stream->stream_handle));
}

struct HostCallbackArgs {
  SE_StatusCallbackFn fn;
  void* arg;
};
void RunHostCallback(void* p) {
  std::unique_ptr<HostCallbackArgs> a(static_cast<HostCallbackArgs*>(p));
  TF_Status* st = TF_NewStatus();
  a->fn(a->arg, st);
  TF_DeleteStatus(st);
}
TF_Bool HostCallback(const SP_Device*, SP_Stream stream, SE_StatusCallbackFn callback_fn, void* callback_arg) {
  auto* a = new HostCallbackArgs{callback_fn, callback_arg};
  if (itexb_rt_host_callback(stream->stream_handle, RunHostCallback, a) == ITEXB_OK) return true;
  delete a;
  return false;
}

void CreateStreamExecutor(const SP_Platform*, SE_CreateStreamExecutorParams* params, TF_Status* status) {
  SP_StreamExecutor* se = params->stream_executor;
  se->struct_size = SP_STREAMEXECUTOR_STRUCT_SIZE;
  se->allocate = Allocate;
  se->deallocate = Deallocate;
  se->host_memory_allocate = HostMemoryAllocate;
  se->host_memory_deallocate = HostMemoryDeallocate;
  se->get_allocator_stats = GetAllocatorStats;
  se->device_memory_usage = DeviceMemoryUsage;
  se->create_stream = CreateStream;
  se->destroy_stream = DestroyStream;
  se->create_stream_dependency = CreateStreamDependency;
  se->get_stream_status = GetStreamStatus;
  se->create_event = CreateEvent;
  se->destroy_event = DestroyEvent;
  se->get_event_status = GetEventStatus;
  se->record_event = RecordEvent;
  se->wait_for_event = WaitForEvent;
  se->create_timer = CreateTimer;
  se->destroy_timer = DestroyTimer;
  se->start_timer = StartTimer;
  se->stop_timer = StopTimer;
  se->memcpy_dtoh = MemcpyDtoH;
  se->memcpy_htod = MemcpyHtoD;
  se->memcpy_dtod = MemcpyDtoD;
  se->sync_memcpy_dtoh = SyncMemcpyDtoH;
  se->sync_memcpy_htod = SyncMemcpyHtoD;
  se->sync_memcpy_dtod = SyncMemcpyDtoD;
  se->block_host_until_done = BlockHostUntilDone;
  se->block_host_for_event = BlockHostForEvent;
  se->synchronize_all_activity = SynchronizeAllActivity;
  se->mem_zero = MemZero;
  se->memset = Memset;
  se->memset32 = Memset32;
  se->host_callback = HostCallback;
  TF_SetStatus(status, TF_OK, "");
}
void DestroyStreamExecutor(const SP_Platform*, SP_StreamExecutor*) {}
void CreateTimerFns(const SP_Platform*, SP_TimerFns* timer_fns, TF_Status* status) {
  timer_fns->nanoseconds = TimerNanoseconds;
  TF_SetStatus(status, TF_OK, "");
}
void DestroyTimerFns(const SP_Platform*, SP_TimerFns*) {}
void DestroyPlatform(SP_Platform*) {}
void DestroyPlatformFns(SP_PlatformFns*) {}

// ------------------------------------------------------------------------------------------------------------------
// Kernels: one itexb_op_t per node, created from the node's attrs.
// ------------------------------------------------------------------------------------------------------------------

// "name: type-spec [= default]" -> name and a coarse kind, enough to choose the TF_OpKernelConstruction_GetAttr* call.
struct AttrSpec {
  std::string name;
  int kind;  // itexb_attr_type_t, or -1 for kinds this path has no use for (list(type) of the list-typed inputs)
};

AttrSpec ParseAttrSpec(const char* spec) {
  AttrSpec a;
  const char* colon = std::strchr(spec, ':');
  a.name.assign(spec, colon != nullptr ? size_t(colon - spec) : std::strlen(spec));
  std::string type = colon != nullptr ? std::string(colon + 1) : std::string();
  const size_t eq = type.find('=');
  if (eq != std::string::npos) type.resize(eq);
  while (!type.empty() && type.front() == ' ') type.erase(type.begin());
  while (!type.empty() && type.back() == ' ') type.pop_back();
  if (type == "int") a.kind = ITEXB_ATTR_INT;
  else if (type == "float") a.kind = ITEXB_ATTR_FLOAT;
  else if (type == "bool") a.kind = ITEXB_ATTR_BOOL;
  else if (type == "string" || type.rfind("{'", 0) == 0 || type.rfind("{\"", 0) == 0) a.kind = ITEXB_ATTR_STRING;  // enumerated strings
  else if (type == "list(string)") a.kind = ITEXB_ATTR_STRING_LIST;
  else if (type.rfind("list(int)", 0) == 0) a.kind = ITEXB_ATTR_INT_LIST;
  else if (type.rfind("list(", 0) == 0) a.kind = -1;
  else a.kind = ITEXB_ATTR_TYPE;  // "type", "quantizedtype", "{float, bfloat16}" ...
  return a;
}

// The attrs of a node, read through the op's definition, in the form itexb_op_create takes.
struct AttrStore {
  std::vector<itexb_attr_t> attrs;
  std::vector<std::string> names, strings;
  std::vector<std::vector<int64_t>> int_lists;
  std::vector<std::vector<std::string>> string_lists;
  std::vector<std::vector<const char*>> string_list_ptrs;
};

bool ReadAttrs(TF_OpKernelConstruction* ctx, const itexb_op_def_t& def, AttrStore* out, TF_Status* status) {
  out->names.reserve(size_t(def.num_attrs));
  out->strings.reserve(size_t(def.num_attrs));
  out->int_lists.reserve(size_t(def.num_attrs));
  out->string_lists.reserve(size_t(def.num_attrs));
  out->string_list_ptrs.reserve(size_t(def.num_attrs));
  for (int i = 0; i < def.num_attrs; ++i) {
    const AttrSpec spec = ParseAttrSpec(def.attrs[i]);
    if (spec.kind < 0) continue;
    // a TensorFlow-defined op may declare fewer attrs than the twin definition lists
    if (!TF_OpKernelConstruction_HasAttr(ctx, spec.name.c_str(), status)) continue;
    out->names.push_back(spec.name);
    itexb_attr_t a;
    std::memset(&a, 0, sizeof(a));
    a.name = out->names.back().c_str();
    a.type = spec.kind;
    switch (spec.kind) {
      case ITEXB_ATTR_INT: {
        int64_t v = 0;
        TF_OpKernelConstruction_GetAttrInt64(ctx, a.name, &v, status);
        a.i = v;
        break;
      }
      case ITEXB_ATTR_FLOAT: TF_OpKernelConstruction_GetAttrFloat(ctx, a.name, &a.f, status); break;
      case ITEXB_ATTR_BOOL: {
        TF_Bool v = 0;
        TF_OpKernelConstruction_GetAttrBool(ctx, a.name, &v, status);
        a.i = v ? 1 : 0;
        break;
      }
      case ITEXB_ATTR_TYPE: {
        TF_DataType v = TF_FLOAT;
        TF_OpKernelConstruction_GetAttrType(ctx, a.name, &v, status);
        a.i = static_cast<int64_t>(v);  // itexb_dtype_t uses TensorFlow's DataType numbering
        break;
      }
      case ITEXB_ATTR_STRING: {
        int32_t list_size = 0, total_size = 0;
        TF_OpKernelConstruction_GetAttrSize(ctx, a.name, &list_size, &total_size, status);
        std::string s(size_t(total_size), '\0');
        if (total_size > 0) TF_OpKernelConstruction_GetAttrString(ctx, a.name, &s[0], size_t(total_size), status);
        out->strings.push_back(std::move(s));
        a.s = out->strings.back().c_str();
        break;
      }
      case ITEXB_ATTR_INT_LIST: {
        int32_t list_size = 0, total_size = 0;
        TF_OpKernelConstruction_GetAttrSize(ctx, a.name, &list_size, &total_size, status);
        out->int_lists.emplace_back(size_t(list_size));
        if (list_size > 0) TF_OpKernelConstruction_GetAttrInt64List(ctx, a.name, out->int_lists.back().data(), list_size, status);
        a.list_i = out->int_lists.back().data();
        a.list_len = list_size;
        break;
      }
      case ITEXB_ATTR_STRING_LIST: {
        int32_t list_size = 0, total_size = 0;
        TF_OpKernelConstruction_GetAttrSize(ctx, a.name, &list_size, &total_size, status);
        std::vector<char*> vals(size_t(list_size) + 1);
        std::vector<size_t> lens(size_t(list_size) + 1);
        std::vector<char> storage(size_t(total_size) + 1);
        if (list_size > 0)
          TF_OpKernelConstruction_GetAttrStringList(ctx, a.name, vals.data(), lens.data(), list_size, storage.data(), storage.size(), status);
        out->string_lists.emplace_back();
        for (int32_t j = 0; j < list_size; ++j) out->string_lists.back().emplace_back(vals[size_t(j)], lens[size_t(j)]);
        out->string_list_ptrs.emplace_back();
        for (const std::string& s : out->string_lists.back()) out->string_list_ptrs.back().push_back(s.c_str());
        a.list_s = out->string_list_ptrs.back().data();
        a.list_len = list_size;
        break;
      }
      default: break;
    }
    if (TF_GetCode(status) != TF_OK) return false;
    out->attrs.push_back(a);
  }
  return true;
}

struct ShimKernel {
  itexb_op_t* op = nullptr;
  std::string type;
};

// TensorFlow's create callback receives no op type, only the node.  Every registered op name therefore gets a create
// function of its own (slot I of a compile-time table), which knows its name from the table RegisterKernels filled - the
// job the reference's OpTypeFactory does with one create function per kernel class (op_kernel.cc:897).
constexpr int kMaxOps = 128;
const char* g_op_names[kMaxOps] = {};

void* CreateForType(TF_OpKernelConstruction* ctx, const char* type) {
  TF_Status* status = TF_NewStatus();
  std::unique_ptr<ShimKernel> k(new ShimKernel);
  k->type = type;
  itexb_op_def_t def;
  AttrStore store;
  int st = itexb_op_def(type, &def);
  if (st == ITEXB_OK && !ReadAttrs(ctx, def, &store, status)) {
    TF_OpKernelConstruction_Failure(ctx, status);
    TF_DeleteStatus(status);
    return nullptr;
  }
  if (st == ITEXB_OK) st = itexb_op_create(type, store.attrs.data(), int(store.attrs.size()), &k->op);
  if (st != ITEXB_OK) {  // construction errors (unsupported mode, type, fusion ...) surface like OP_REQUIRES in a constructor
    SetStatus(status, st);
    TF_OpKernelConstruction_Failure(ctx, status);
    TF_DeleteStatus(status);
    return nullptr;
  }
  TF_DeleteStatus(status);
  return k.release();
}

template <int I> void* KernelCreateSlot(TF_OpKernelConstruction* ctx) { return CreateForType(ctx, g_op_names[I]); }
using CreateFn = void* (*)(TF_OpKernelConstruction*);
template <int... I> constexpr std::array<CreateFn, sizeof...(I)> MakeCreateTable(std::integer_sequence<int, I...>) {
  return {{&KernelCreateSlot<I>...}};
}
constexpr std::array<CreateFn, kMaxOps> kCreateTable = MakeCreateTable(std::make_integer_sequence<int, kMaxOps>{});

// What one Compute needs to hand outputs and temporaries back to TensorFlow.
struct ComputeState {
  TF_OpKernelContext* ctx;
  TF_Status* status;
  std::vector<TF_Tensor*> owned;  // every handle obtained during this Compute; deleted at its end (the buffers live on in TF)
};

size_t ElementBytes(int dtype) {
  switch (dtype) {
    case ITEXB_DT_FLOAT: case ITEXB_DT_INT32: case ITEXB_DT_QINT32: return 4;
    case ITEXB_DT_BFLOAT16: case ITEXB_DT_HALF: return 2;
    case ITEXB_DT_INT64: return 8;
    default: return 1;
  }
}

int AllocateOutputCb(void* user, int index, itexb_tensor_t* out) {
  auto* cs = static_cast<ComputeState*>(user);
  int64_t n = 1;
  for (int i = 0; i < out->rank; ++i) n *= out->dims[i];
  // HostMemory outputs come back as host buffers because the kernel was registered with them as HostMemory
  TF_Tensor* t = TF_AllocateOutput(cs->ctx, index, static_cast<TF_DataType>(out->dtype), out->dims, out->rank, size_t(n) * ElementBytes(out->dtype),
                                   cs->status);
  if (TF_GetCode(cs->status) != TF_OK || t == nullptr) return ITEXB_RESOURCE_EXHAUSTED;
  cs->owned.push_back(t);
  out->data = TF_TensorData(t);
  return ITEXB_OK;
}

int AllocateTempCb(void* user, size_t bytes, int on_host, void** ptr) {
  auto* cs = static_cast<ComputeState*>(user);
  TF_AllocatorAttributes attrs;
  attrs.struct_size = TF_ALLOCATOR_ATTRIBUTES_STRUCT_SIZE;
  attrs.on_host = on_host ? 1 : 0;
  const int64_t dims[1] = {static_cast<int64_t>(bytes)};
  TF_Tensor* t = TF_AllocateTemp(cs->ctx, TF_UINT8, dims, 1, &attrs, cs->status);
  if (TF_GetCode(cs->status) != TF_OK || t == nullptr) return ITEXB_RESOURCE_EXHAUSTED;
  cs->owned.push_back(t);  // TensorFlow keeps a temporary alive until the stream has passed this op
  *ptr = TF_TensorData(t);
  return ITEXB_OK;
}

void KernelCompute(void* kernel, TF_OpKernelContext* ctx) {
  auto* k = static_cast<ShimKernel*>(kernel);
  TF_Status* status = TF_NewStatus();
  ComputeState cs{ctx, status, {}};
  int nin_decl = 0, nout_decl = 0;
  uint32_t host_in = 0, host_out = 0;
  (void)itexb_op_signature(k->type.c_str(), &nin_decl, &nout_decl, &host_in, &host_out);
  const int nin = TF_NumInputs(ctx);
  std::vector<itexb_tensor_t> inputs(size_t(nin > 0 ? nin : 1));
  bool ok = true;
  for (int i = 0; i < nin && ok; ++i) {
    TF_Tensor* t = nullptr;
    TF_GetInput(ctx, i, &t, status);
    if (TF_GetCode(status) != TF_OK || t == nullptr) { ok = false; break; }
    cs.owned.push_back(t);
    itexb_tensor_t& x = inputs[size_t(i)];
    std::memset(&x, 0, sizeof(x));
    x.dtype = static_cast<int32_t>(TF_TensorType(t));
    x.rank = TF_NumDims(t);
    if (x.rank > ITEXB_MAX_DIMS) {
      TF_SetStatus(status, TF_INVALID_ARGUMENT, "tensor rank exceeds ITEXB_MAX_DIMS");
      ok = false;
      break;
    }
    for (int d = 0; d < x.rank; ++d) x.dims[d] = TF_Dim(t, d);
    x.data = TF_TensorData(t);
    // Fixed-arity ops: the registered mask.  List-typed ops (mask 0, count -1): ranges are HostMemory lists, which
    // TensorFlow hands over as host tensors; the op checks per call that what it reads as a range is on the host, and
    // a float tensor of at most one element per output channel in one of the trailing positions is one.
    // QuantizedConcatV2 (values x N, axis, input_mins x N, input_maxes x N): everything after the N values.
    const bool concat = k->type.size() >= 17 && k->type.compare(k->type.size() - 17, 17, "QuantizedConcatV2") == 0;
    x.on_host = nin_decl >= 0 ? int((host_in >> i) & 1u)
                : concat      ? int(i >= (nin - 1) / 3)
                              : int(x.dtype == ITEXB_DT_FLOAT && i >= 2 && i >= nin - 6 && x.rank <= 1);
  }
  if (ok) {
    SP_Stream stream = TF_GetStream(ctx, status);
    itexb_op_context_t oc;
    std::memset(&oc, 0, sizeof(oc));
    oc.user = &cs;
    oc.num_inputs = nin;
    oc.inputs = inputs.data();
    oc.device_ordinal = 0;
    (void)itexb_rt_stream_device(stream->stream_handle, &oc.device_ordinal);
    oc.stream = stream->stream_handle;
    oc.allocate_output = AllocateOutputCb;
    oc.allocate_temp = AllocateTempCb;
    const int st = itexb_op_compute(k->op, &oc);
    if (st != ITEXB_OK && TF_GetCode(status) == TF_OK) SetStatus(status, st);
    ok = st == ITEXB_OK;
  }
  if (!ok) TF_OpKernelContext_Failure(ctx, status);  // never throws: the error travels in the context (op_kernel.cc:511-532)
  for (TF_Tensor* t : cs.owned) TF_DeleteTensor(t);
  TF_DeleteStatus(status);
}

void KernelDelete(void* kernel) {
  auto* k = static_cast<ShimKernel*>(kernel);
  if (k == nullptr) return;
  itexb_op_delete(k->op);
  delete k;
}

// "arg: T" -> "arg"
std::string ArgName(const char* spec) {
  const char* colon = std::strchr(spec, ':');
  return colon != nullptr ? std::string(spec, size_t(colon - spec)) : std::string(spec);
}

void RegisterOpDefinition(const itexb_op_def_t& def, TF_Status* status) {
  TF_OpDefinitionBuilder* b = TF_NewOpDefinitionBuilder(def.name);
  for (int i = 0; i < def.num_inputs; ++i) TF_OpDefinitionBuilderAddInput(b, def.inputs[i]);
  for (int i = 0; i < def.num_outputs; ++i) TF_OpDefinitionBuilderAddOutput(b, def.outputs[i]);
  for (int i = 0; i < def.num_attrs; ++i) TF_OpDefinitionBuilderAddAttr(b, def.attrs[i]);
  // shapes depend on run-time values (ranges, padding): unknown at graph construction, like the reference's unknown_shape_fn
  TF_OpDefinitionBuilderSetShapeInferenceFunction(b, [](TF_ShapeInferenceContext* c, TF_Status* s) { TF_ShapeInferenceContextSetUnknownShape(c, s); });
  TF_RegisterOpDefinition(b, status);
}

void RegisterKernel(int slot, const char* op_name, const itexb_op_def_t& def, TF_Status* status) {
  g_op_names[slot] = op_name;  // static storage of the library
  TF_KernelBuilder* b = TF_NewKernelBuilder(op_name, kDeviceType, kCreateTable[size_t(slot)], &KernelCompute, &KernelDelete);
  int nin = 0, nout = 0;
  uint32_t host_in = 0, host_out = 0;
  (void)itexb_op_signature(op_name, &nin, &nout, &host_in, &host_out);
  if (nin >= 0) {
    for (int i = 0; i < def.num_inputs && i < 32; ++i)
      if ((host_in >> i) & 1u) TF_KernelBuilder_HostMemory(b, ArgName(def.inputs[i]).c_str());
    for (int i = 0; i < def.num_outputs && i < 32; ++i)
      if ((host_out >> i) & 1u) TF_KernelBuilder_HostMemory(b, ArgName(def.outputs[i]).c_str());
  } else {
    // list-typed ops: the whole host_inputs / host_outputs lists (gpu/quantized_matmul.cc:137-182); QuantizedConcatV2:
    // axis, input_mins, input_maxes, output_min, output_max (common/quantized_concat_op.cc:251-268)
    const auto is_host = [](const std::string& a) {
      for (const char* prefix : {"host_", "min_", "max_", "input_min", "input_max", "output_min", "output_max"})
        if (a.rfind(prefix, 0) == 0) return true;
      return a == "axis";
    };
    for (int i = 0; i < def.num_inputs; ++i)
      if (is_host(ArgName(def.inputs[i]))) TF_KernelBuilder_HostMemory(b, ArgName(def.inputs[i]).c_str());
    for (int i = 0; i < def.num_outputs; ++i)
      if (is_host(ArgName(def.outputs[i]))) TF_KernelBuilder_HostMemory(b, ArgName(def.outputs[i]).c_str());
  }
  // No TypeConstraint: one kernel object serves every type combination the op layer implements and reports the others
  // at construction ("no kernel registered for T1=..."), which is where the reference's type matrix fails too.
  TF_RegisterKernelBuilder(op_name, b, status);
}

}  // namespace

extern "C" {

void SE_InitPlugin(SE_PlatformRegistrationParams* const params, TF_Status* const status) {
  params->platform->struct_size = SP_PLATFORM_STRUCT_SIZE;
  params->platform->name = kPlatformName;
  params->platform->type = kDeviceType;
  params->platform->supports_unified_memory = false;
  params->platform->use_bfc_allocator = false;  // allocations go through the plugin's own caching allocator
  params->platform_fns->get_device_count = DeviceCount;
  params->platform_fns->create_device = CreateDevice;
  params->platform_fns->destroy_device = DestroyDevice;
  params->platform_fns->create_device_fns = CreateDeviceFns;
  params->platform_fns->destroy_device_fns = DestroyDeviceFns;
  params->platform_fns->create_stream_executor = CreateStreamExecutor;
  params->platform_fns->destroy_stream_executor = DestroyStreamExecutor;
  params->platform_fns->create_timer_fns = CreateTimerFns;
  params->platform_fns->destroy_timer_fns = DestroyTimerFns;
  params->destroy_platform = DestroyPlatform;
  params->destroy_platform_fns = DestroyPlatformFns;
  TF_SetStatus(status, TF_OK, "");
}

void TF_InitKernel() {
  TF_Status* status = TF_NewStatus();
  int slot = 0;
  for (const char* const* name = itexb_op_list(); *name != nullptr && slot < kMaxOps; ++name) {
    itexb_op_def_t def;
    if (itexb_op_def(*name, &def) != ITEXB_OK) continue;
    if (def.defined_by_plugin) {
      RegisterOpDefinition(def, status);
      if (TF_GetCode(status) != TF_OK) continue;  // e.g. another plugin defined the op already: kernels of that name are theirs
    }
    RegisterKernel(slot++, *name, def, status);
  }
  TF_DeleteStatus(status);
}

}  // extern "C"

#endif  // ITEXB_HAVE_TENSORFLOW
