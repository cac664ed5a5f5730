// PJRT C API entry points of the B200 StableHLO executor (table layout: include/b2x_pjrt_c_api.h).
//
// What ryft-pjrt calls, and where: plugin loading crates/ryft-pjrt/src/plugins.rs:20-105; client creation
// clients.rs:671-825; buffers buffers.rs:2099-2150, 1237-1295; compile programs.rs:1245-1263; execute
// programs.rs:769-963; events events.rs:89-144.  All entry points are thread-safe.  There is no CPU execution path:
// when no CUDA device is usable, PJRT_Client_Create fails.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "nccl_dyn.h"
#include "objects.h"

using namespace b2x;

namespace b2x {

PJRT_Error* make_error(PJRT_Error_Code code, const std::string& msg) { return new PJRT_Error{code, msg}; }
PJRT_Error* cuda_error(cudaError_t e, const char* what) {
  PJRT_Error_Code code = (e == cudaErrorMemoryAllocation) ? PJRT_Error_Code_RESOURCE_EXHAUSTED : PJRT_Error_Code_INTERNAL;
  return make_error(code, std::string("CUDA error in ") + what + ": " + cudaGetErrorString(e));
}

PJRT_Buffer_Type to_pjrt_type(DType t) {
  switch (t) {
    case DType::PRED: return PJRT_Buffer_Type_PRED; case DType::S8: return PJRT_Buffer_Type_S8;
    case DType::S16: return PJRT_Buffer_Type_S16; case DType::S32: return PJRT_Buffer_Type_S32;
    case DType::S64: return PJRT_Buffer_Type_S64; case DType::U8: return PJRT_Buffer_Type_U8;
    case DType::U16: return PJRT_Buffer_Type_U16; case DType::U32: return PJRT_Buffer_Type_U32;
    case DType::U64: return PJRT_Buffer_Type_U64; case DType::F16: return PJRT_Buffer_Type_F16;
    case DType::BF16: return PJRT_Buffer_Type_BF16; case DType::F32: return PJRT_Buffer_Type_F32;
    case DType::F64: return PJRT_Buffer_Type_F64; default: return PJRT_Buffer_Type_INVALID;
  }
}
DType from_pjrt_type(PJRT_Buffer_Type t) {
  switch (t) {
    case PJRT_Buffer_Type_PRED: return DType::PRED; case PJRT_Buffer_Type_S8: return DType::S8;
    case PJRT_Buffer_Type_S16: return DType::S16; case PJRT_Buffer_Type_S32: return DType::S32;
    case PJRT_Buffer_Type_S64: return DType::S64; case PJRT_Buffer_Type_U8: return DType::U8;
    case PJRT_Buffer_Type_U16: return DType::U16; case PJRT_Buffer_Type_U32: return DType::U32;
    case PJRT_Buffer_Type_U64: return DType::U64; case PJRT_Buffer_Type_F16: return DType::F16;
    case PJRT_Buffer_Type_BF16: return DType::BF16; case PJRT_Buffer_Type_F32: return DType::F32;
    case PJRT_Buffer_Type_F64: return DType::F64; default: return DType::INVALID;
  }
}
}  // namespace b2x

// ---- events ---------------------------------------------------------------------------------------------------------

void PJRT_Event::set(PJRT_Error_Code c, const std::string& msg) {
  std::vector<std::pair<PJRT_Event_OnReadyCallback, void*>> cbs;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (ready) return;
    ready = true;
    code = c;
    message = msg;
    cbs.swap(callbacks);
  }
  cv.notify_all();
  for (auto& cb : cbs) cb.first(c == PJRT_Error_Code_OK ? nullptr : make_error(c, msg), cb.second);
}

static PJRT_Event* ready_event() {
  PJRT_Event* e = new PJRT_Event();
  e->ready = true;
  return e;
}

void PJRT_Client::post(Pending p) {
  if (p.event) p.event->ref();
  {
    std::lock_guard<std::mutex> lk(q_mu);
    queue.push_back(std::move(p));
  }
  q_cv.notify_one();
}

static void poller_main(PJRT_Client* c) {
  while (true) {
    PJRT_Client::Pending p;
    {
      std::unique_lock<std::mutex> lk(c->q_mu);
      c->q_cv.wait(lk, [&] { return c->stop || !c->queue.empty(); });
      if (c->queue.empty()) return;
      p = std::move(c->queue.front());
      c->queue.pop_front();
    }
    PJRT_Error_Code code = PJRT_Error_Code_OK;
    std::string msg;
    if (p.ev) {
      cudaSetDevice(p.ordinal);
      cudaError_t e = cudaEventSynchronize(p.ev);
      if (e != cudaSuccess) { code = PJRT_Error_Code_INTERNAL; msg = std::string("device work failed: ") + cudaGetErrorString(e); }
      cudaEventDestroy(p.ev);
    }
    if (p.finish) p.finish(&code, &msg);
    if (p.event) { p.event->set(code, msg); p.event->unref(); }
  }
}

PJRT_Client::~PJRT_Client() {
  {
    std::lock_guard<std::mutex> lk(q_mu);
    stop = true;
  }
  q_cv.notify_all();
  if (poller.joinable()) poller.join();
  nccl.reset();
  for (auto& d : device_storage) {
    if (!d->addressable) continue;
    cudaSetDevice(d->cuda_ordinal);
    cudaDeviceSynchronize();
    if (d->compute) cudaStreamDestroy(d->compute);
    if (d->h2d) cudaStreamDestroy(d->h2d);
    if (d->d2h) cudaStreamDestroy(d->d2h);
    if (d->comm) cudaStreamDestroy(d->comm);
    for (auto& r : d->recycled) { cudaEventDestroy(r.last_use); cudaFree(r.ptr); }
    d->recycled.clear();
    if (d->status_host) cudaFreeHost(d->status_host);
    for (void* p : d->staging_free) cudaFreeHost(p);
    d->staging_free.clear();
  }
}

PJRT_LoadedExecutable::~PJRT_LoadedExecutable() {
  for (size_t i = 0; i < per_device.size(); i++) {
    PerDevice& pd = per_device[i];
    cudaSetDevice(addressable[i]->cuda_ordinal);
    if (pd.arena || pd.consts) cudaStreamSynchronize(addressable[i]->compute);
    if (pd.arena) { cudaFree(pd.arena); addressable[i]->bytes_in_use -= (int64_t)pd.arena_bytes; }
    if (pd.consts) cudaFree(pd.consts);
    for (auto e : pd.coll_done) cudaEventDestroy(e);
    if (pd.fork) cudaEventDestroy(pd.fork);
    for (auto& exec : pd.timed) for (auto& ev : exec) { if (ev.first) cudaEventDestroy(ev.first); if (ev.second) cudaEventDestroy(ev.second); }
  }
}

// ---- helpers --------------------------------------------------------------------------------------------------------

#define B2X_CHECK_ARG(cond, msg) \
  do { if (!(cond)) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, msg); } while (0)

static void track_alloc(PJRT_Device* d, int64_t bytes) {
  int64_t now = d->bytes_in_use.fetch_add(bytes) + bytes;
  int64_t peak = d->peak_bytes.load();
  while (now > peak && !d->peak_bytes.compare_exchange_weak(peak, now)) {}
  d->num_allocs.fetch_add(1);
}

static PJRT_Error* alloc_buffer(PJRT_Device* dev, const TensorType& type, cudaStream_t stream, PJRT_Buffer** out) {
  PJRT_Buffer* b = new PJRT_Buffer();
  b->client = dev->client;
  b->device = dev;
  b->type = type;
  b->dims = type.dims;
  b->pjrt_type = to_pjrt_type(type.dtype);
  b->bytes = (size_t)type.byte_size();
  for (int i = type.rank() - 1; i >= 0; i--) b->minor_to_major.push_back(i);
  cudaError_t e = cudaSetDevice(dev->cuda_ordinal);
  if (e == cudaSuccess) e = cudaMallocAsync(&b->ptr, std::max<size_t>(b->bytes, 16), stream);
  if (e != cudaSuccess) { delete b; return cuda_error(e, "cudaMallocAsync (buffer)"); }
  track_alloc(dev, (int64_t)b->bytes);
  *out = b;
  return nullptr;
}

// Blocks until a late-defined buffer has had its last transfer enqueued (then `ready` covers it) or an error set.
static void await_definition(PJRT_Buffer* b) {
  std::shared_ptr<b2x_Definition> d = b->pending;
  if (!d) return;
  std::unique_lock<std::mutex> lk(d->mu);
  d->cv.wait(lk, [&] { return d->done; });
}

// A kernel whose bounded wait ran out leaves a non-zero code in the device's status word (mapped host memory).  The
// first completion on that device that finds it reports DEADLINE_EXCEEDED and clears the word, so that one expiry
// fails the work that observed it and not every execution and copy that follows.
static void report_expired_wait(PJRT_Device* dev, PJRT_Error_Code* code, std::string* msg) {
  if (!dev->status_host) return;
  const int32_t st = __atomic_exchange_n(&dev->status_host[0], 0, __ATOMIC_ACQ_REL);
  if (st == 0 || *code != PJRT_Error_Code_OK) return;
  *code = PJRT_Error_Code_DEADLINE_EXCEEDED;
  *msg = "a kernel gave up waiting on an internal barrier (status " + std::to_string(st) + ")";
}

static void release_buffer_memory(PJRT_Buffer* b) {
  if (!b->ptr) return;
  PJRT_Device* d = b->device;
  cudaSetDevice(d->cuda_ordinal);
  if (b->owns) {
    await_definition(b);
    // every use of the memory was enqueued on the compute stream, or on a transfer stream with a recorded event
    for (auto ev : b->pending_reads) { cudaStreamWaitEvent(d->compute, ev, 0); cudaEventDestroy(ev); }
    b->pending_reads.clear();
    if (b->ready) cudaStreamWaitEvent(d->compute, b->ready, 0);
    bool kept = false;
    if (b->from_host && b->bytes >= PJRT_Device::kMinRecycledBytes) {
      std::lock_guard<std::mutex> lk(d->recycle_mu);
      size_t held = 0;
      for (auto& r : d->recycled) held += r.bytes;
      if (d->recycled.size() < PJRT_Device::kMaxRecycled && held + b->bytes <= PJRT_Device::kMaxRecycledBytes) {
        cudaEvent_t ev = nullptr;
        if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess && cudaEventRecord(ev, d->compute) == cudaSuccess) {
          d->recycled.push_back({b->ptr, b->bytes, ev});
          kept = true;
        } else if (ev) {
          cudaEventDestroy(ev);
        }
      }
    }
    if (!kept) cudaFreeAsync(b->ptr, d->compute);
    d->bytes_in_use -= (int64_t)b->bytes;
  } else {
    for (auto ev : b->pending_reads) { cudaEventSynchronize(ev); cudaEventDestroy(ev); }
    b->pending_reads.clear();
    if (b->on_delete) { cudaStreamSynchronize(d->compute); b->on_delete(); }
  }
  b->ptr = nullptr;
}

// ---- error / plugin ---------------------------------------------------------------------------------------------------

static void Error_Destroy(PJRT_Error_Destroy_Args* a) { delete a->error; }
static void Error_Message(PJRT_Error_Message_Args* a) {
  a->message = a->error->message.data();
  a->message_size = a->error->message.size();
}
static PJRT_Error* Error_GetCode(PJRT_Error_GetCode_Args* a) { a->code = a->error->code; return nullptr; }
static PJRT_Error* Error_ForEachPayload(PJRT_Error_ForEachPayload_Args*) { return nullptr; }

static PJRT_Error* Plugin_Initialize(PJRT_Plugin_Initialize_Args*) { return nullptr; }
static PJRT_Error* Plugin_Attributes(PJRT_Plugin_Attributes_Args* a) {
  // Same attribute set as the reference's plugins report (crates/ryft-pjrt/src/lib.rs:575-577).
  static const int64_t cur[3] = {1, 16, 0}, min[3] = {0, 9, 0};
  static PJRT_NamedValue attrs[3];
  static std::once_flag once;
  std::call_once(once, [] {
    auto init = [](PJRT_NamedValue* v, const char* name) { memset(v, 0, sizeof(*v)); v->struct_size = sizeof(*v); v->name = name; v->name_size = strlen(name); };
    init(&attrs[0], "xla_version"); attrs[0].type = PJRT_NamedValue_kInt64; attrs[0].int64_value = 2; attrs[0].value_size = 1;
    init(&attrs[1], "stablehlo_current_version"); attrs[1].type = PJRT_NamedValue_kInt64List; attrs[1].int64_array_value = cur; attrs[1].value_size = 3;
    init(&attrs[2], "stablehlo_minimum_version"); attrs[2].type = PJRT_NamedValue_kInt64List; attrs[2].int64_array_value = min; attrs[2].value_size = 3;
  });
  a->attributes = attrs;
  a->num_attributes = 3;
  return nullptr;
}

// ---- events -----------------------------------------------------------------------------------------------------------

static PJRT_Error* Event_Create(PJRT_Event_Create_Args* a) { a->event = new PJRT_Event(); return nullptr; }
static PJRT_Error* Event_Set(PJRT_Event_Set_Args* a) {
  B2X_CHECK_ARG(a->event, "the event is null");
  {
    std::lock_guard<std::mutex> lk(a->event->mu);
    if (a->event->ready) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "the event has already been set");
  }
  a->event->set(a->error_code, a->error_message ? std::string(a->error_message, a->error_message_size) : std::string());
  return nullptr;
}
static PJRT_Error* Event_Destroy(PJRT_Event_Destroy_Args* a) { if (a->event) a->event->unref(); return nullptr; }
static PJRT_Error* Event_IsReady(PJRT_Event_IsReady_Args* a) {
  std::lock_guard<std::mutex> lk(a->event->mu);
  a->is_ready = a->event->ready;
  return nullptr;
}
static PJRT_Error* Event_Error(PJRT_Event_Error_Args* a) {
  std::lock_guard<std::mutex> lk(a->event->mu);
  if (!a->event->ready) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "the event is not ready yet");
  if (a->event->code == PJRT_Error_Code_OK) return nullptr;
  return make_error(a->event->code, a->event->message);
}
static PJRT_Error* Event_Await(PJRT_Event_Await_Args* a) {
  std::unique_lock<std::mutex> lk(a->event->mu);
  a->event->cv.wait(lk, [&] { return a->event->ready; });
  if (a->event->code == PJRT_Error_Code_OK) return nullptr;
  return make_error(a->event->code, a->event->message);
}
static PJRT_Error* Event_OnReady(PJRT_Event_OnReady_Args* a) {
  B2X_CHECK_ARG(a->callback, "the callback is null");
  PJRT_Error_Code code;
  std::string msg;
  {
    std::lock_guard<std::mutex> lk(a->event->mu);
    if (!a->event->ready) { a->event->callbacks.push_back({a->callback, a->user_arg}); return nullptr; }
    code = a->event->code;
    msg = a->event->message;
  }
  a->callback(code == PJRT_Error_Code_OK ? nullptr : make_error(code, msg), a->user_arg);
  return nullptr;
}

// ---- client -----------------------------------------------------------------------------------------------------------

static std::mutex g_client_mu;

static void fill_description(PJRT_Device* d, const cudaDeviceProp* prop, int cc_major, int cc_minor, int sms, size_t mem) {
  PJRT_DeviceDescription& dd = d->desc;
  dd.kind = prop ? prop->name : "NVIDIA GPU (remote)";
  dd.to_string = "CudaDevice(id=" + std::to_string(dd.id) + ")";
  dd.debug_string = "b200-stablehlo:" + dd.kind + ":id=" + std::to_string(dd.id) + ":process=" + std::to_string(dd.process_index);
  dd.attr_names = {"compute_capability", "core_count", "memory_bytes", "local_hardware_id"};
  dd.attr_strings = {std::to_string(cc_major) + "." + std::to_string(cc_minor)};
  dd.attributes.resize(4);
  for (auto& a : dd.attributes) { memset(&a, 0, sizeof(a)); a.struct_size = sizeof(a); }
  for (int i = 0; i < 4; i++) { dd.attributes[i].name = dd.attr_names[i].data(); dd.attributes[i].name_size = dd.attr_names[i].size(); }
  dd.attributes[0].type = PJRT_NamedValue_kString; dd.attributes[0].string_value = dd.attr_strings[0].data(); dd.attributes[0].value_size = dd.attr_strings[0].size();
  dd.attributes[1].type = PJRT_NamedValue_kInt64; dd.attributes[1].int64_value = sms; dd.attributes[1].value_size = 1;
  dd.attributes[2].type = PJRT_NamedValue_kInt64; dd.attributes[2].int64_value = (int64_t)mem; dd.attributes[2].value_size = 1;
  dd.attributes[3].type = PJRT_NamedValue_kInt64; dd.attributes[3].int64_value = dd.local_hardware_id; dd.attributes[3].value_size = 1;
}

static PJRT_Error* Client_Create(PJRT_Client_Create_Args* a) {
  std::lock_guard<std::mutex> lk(g_client_mu);
  int node_id = 0, num_nodes = 1;
  std::vector<int64_t> visible;
  bool have_visible = false;
  for (size_t i = 0; i < a->num_options; i++) {
    const PJRT_NamedValue& v = a->create_options[i];
    std::string name(v.name, v.name_size);
    if (name == "node_id" && v.type == PJRT_NamedValue_kInt64) node_id = (int)v.int64_value;
    else if (name == "num_nodes" && v.type == PJRT_NamedValue_kInt64) num_nodes = (int)v.int64_value;
    else if (name == "visible_devices" && v.type == PJRT_NamedValue_kInt64List) { visible.assign(v.int64_array_value, v.int64_array_value + v.value_size); have_visible = true; }
    // allocator, preallocate, memory_fraction, collective_memory_size, enable_mock_nccl, ... : accepted, not needed
  }
  if (const char* env = getenv("B2X_VISIBLE_DEVICES")) {
    visible.clear(); have_visible = true;
    std::stringstream ss(env); std::string tok;
    while (std::getline(ss, tok, ',')) if (!tok.empty()) visible.push_back(atoll(tok.c_str()));
  }
  int n_cuda = 0;
  cudaError_t e = cudaGetDeviceCount(&n_cuda);
  if (e != cudaSuccess || n_cuda == 0)
    return make_error(PJRT_Error_Code_FAILED_PRECONDITION,
                      std::string("no usable CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0") +
                          " (this plugin has no CPU execution path)");
  if (!have_visible) for (int i = 0; i < n_cuda; i++) visible.push_back(i);
  for (auto o : visible) B2X_CHECK_ARG(o >= 0 && o < n_cuda, "visible_devices names CUDA device " + std::to_string(o) + " but only " + std::to_string(n_cuda) + " exist");
  B2X_CHECK_ARG(!visible.empty(), "visible_devices is empty");
  B2X_CHECK_ARG(num_nodes >= 1 && node_id >= 0 && node_id < num_nodes, "node_id must be in [0, num_nodes)");

  std::unique_ptr<PJRT_Client> c(new PJRT_Client());
  c->process_index = node_id;
  c->num_processes = num_nodes;
  int rt = 0;
  cudaRuntimeGetVersion(&rt);
  c->platform_version = "cuda " + std::to_string(rt);
  c->kv_get = a->kv_get_callback; c->kv_get_arg = a->kv_get_user_arg;
  c->kv_put = a->kv_put_callback; c->kv_put_arg = a->kv_put_user_arg;
  const int local = (int)visible.size();
  // Global ids: process p owns [p * local, (p + 1) * local); every process must expose the same number of devices.
  for (int p = 0; p < num_nodes; p++) {
    for (int l = 0; l < local; l++) {
      std::unique_ptr<PJRT_Device> d(new PJRT_Device());
      d->client = c.get();
      d->desc.id = p * local + l;
      d->desc.process_index = p;
      d->addressable = (p == node_id);
      std::unique_ptr<PJRT_Memory> m(new PJRT_Memory());
      m->id = d->desc.id;
      m->device = d.get();
      m->devices = {d.get()};
      m->to_string = "DEVICE_" + std::to_string(m->id);
      m->debug_string = "device memory of device " + std::to_string(d->desc.id);
      d->memory = m.get();
      d->memories = {m.get()};
      if (d->addressable) {
        d->cuda_ordinal = (int)visible[l];
        d->desc.local_hardware_id = d->cuda_ordinal;
        B2X_CUDA(cudaSetDevice(d->cuda_ordinal));
        cudaDeviceProp prop;
        B2X_CUDA(cudaGetDeviceProperties(&prop, d->cuda_ordinal));
        if (prop.major != 10)
          return make_error(PJRT_Error_Code_FAILED_PRECONDITION, std::string("device ") + prop.name + " has compute capability " + std::to_string(prop.major) + "." +
                                std::to_string(prop.minor) + "; the kernels in this plugin are built for sm_100a only");
        B2X_CUDA(cudaStreamCreateWithFlags(&d->compute, cudaStreamNonBlocking));
        B2X_CUDA(cudaStreamCreateWithFlags(&d->h2d, cudaStreamNonBlocking));
        B2X_CUDA(cudaStreamCreateWithFlags(&d->d2h, cudaStreamNonBlocking));
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        B2X_CUDA(cudaStreamCreateWithPriority(&d->comm, cudaStreamNonBlocking, hi));
        B2X_CUDA(cudaHostAlloc((void**)&d->status_host, 64, cudaHostAllocMapped));
        memset(d->status_host, 0, 64);
        B2X_CUDA(cudaHostGetDevicePointer((void**)&d->status_dev, d->status_host, 0));
        cudaMemPool_t pool;
        B2X_CUDA(cudaDeviceGetDefaultMemPool(&pool, d->cuda_ordinal));
        uint64_t keep = UINT64_MAX;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        fill_description(d.get(), &prop, prop.major, prop.minor, prop.multiProcessorCount, prop.totalGlobalMem);
        c->addressable_devices.push_back(d.get());
        c->addressable_memories.push_back(m.get());
      } else {
        fill_description(d.get(), nullptr, 10, 0, 148, 0);
      }
      c->devices.push_back(d.get());
      c->device_storage.push_back(std::move(d));
      c->memory_storage.push_back(std::move(m));
    }
  }
  // peers of one process reach each other's memory directly (device-to-device copies, NCCL P2P)
  for (auto d : c->addressable_devices)
    for (auto o : c->addressable_devices) {
      if (d == o) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, d->cuda_ordinal, o->cuda_ordinal);
      if (can) { cudaSetDevice(d->cuda_ordinal); cudaError_t pe = cudaDeviceEnablePeerAccess(o->cuda_ordinal, 0); if (pe != cudaSuccess) cudaGetLastError(); }
    }
  c->nccl.reset(new NcclComms(c.get()));
  c->poller = std::thread(poller_main, c.get());
  a->client = c.release();
  return nullptr;
}

static PJRT_Error* Client_Destroy(PJRT_Client_Destroy_Args* a) {
  std::lock_guard<std::mutex> lk(g_client_mu);
  delete a->client;
  return nullptr;
}
static PJRT_Error* Client_PlatformName(PJRT_Client_PlatformName_Args* a) {
  a->platform_name = a->client->platform_name.data(); a->platform_name_size = a->client->platform_name.size(); return nullptr;
}
static PJRT_Error* Client_PlatformVersion(PJRT_Client_PlatformVersion_Args* a) {
  a->platform_version = a->client->platform_version.data(); a->platform_version_size = a->client->platform_version.size(); return nullptr;
}
static PJRT_Error* Client_ProcessIndex(PJRT_Client_ProcessIndex_Args* a) { a->process_index = a->client->process_index; return nullptr; }
static PJRT_Error* Client_Devices(PJRT_Client_Devices_Args* a) {
  a->devices = a->client->devices.data(); a->num_devices = a->client->devices.size(); return nullptr;
}
static PJRT_Error* Client_AddressableDevices(PJRT_Client_AddressableDevices_Args* a) {
  a->addressable_devices = a->client->addressable_devices.data(); a->num_addressable_devices = a->client->addressable_devices.size(); return nullptr;
}
static PJRT_Error* Client_LookupDevice(PJRT_Client_LookupDevice_Args* a) {
  for (auto d : a->client->devices) if (d->desc.id == a->id) { a->device = d; return nullptr; }
  return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "no device with id " + std::to_string(a->id));
}
static PJRT_Error* Client_LookupAddressableDevice(PJRT_Client_LookupAddressableDevice_Args* a) {
  for (auto d : a->client->addressable_devices) if (d->desc.local_hardware_id == a->local_hardware_id) { a->addressable_device = d; return nullptr; }
  return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "no addressable device with local hardware id " + std::to_string(a->local_hardware_id));
}
static PJRT_Error* Client_AddressableMemories(PJRT_Client_AddressableMemories_Args* a) {
  a->addressable_memories = a->client->addressable_memories.data(); a->num_addressable_memories = a->client->addressable_memories.size(); return nullptr;
}
static PJRT_Error* Client_DefaultDeviceAssignment(PJRT_Client_DefaultDeviceAssignment_Args* a) {
  const int n = a->num_replicas * a->num_partitions;
  B2X_CHECK_ARG(a->num_replicas >= 1 && a->num_partitions >= 1, "replica and partition counts must be positive");
  B2X_CHECK_ARG((size_t)n <= a->default_assignment_size, "the assignment buffer is too small");
  if (n > (int)a->client->devices.size())
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "a " + std::to_string(a->num_replicas) + "x" + std::to_string(a->num_partitions) +
                                                            " assignment needs " + std::to_string(n) + " devices but the client has " +
                                                            std::to_string(a->client->devices.size()));
  for (int i = 0; i < n; i++) a->default_assignment[i] = a->client->devices[i]->desc.id;
  return nullptr;
}
static PJRT_Error* Client_UpdateGlobalProcessInfo(PJRT_Client_UpdateGlobalProcessInfo_Args*) { return nullptr; }
static PJRT_Error* Client_DmaMap(PJRT_Client_DmaMap_Args* a) {
  cudaError_t e = cudaHostRegister(a->data, a->size, cudaHostRegisterDefault);
  if (e != cudaSuccess) { cudaGetLastError(); return cuda_error(e, "cudaHostRegister"); }
  return nullptr;
}
static PJRT_Error* Client_DmaUnmap(PJRT_Client_DmaUnmap_Args* a) {
  cudaError_t e = cudaHostUnregister(a->data);
  if (e != cudaSuccess) { cudaGetLastError(); return cuda_error(e, "cudaHostUnregister"); }
  return nullptr;
}

// ---- devices, memories --------------------------------------------------------------------------------------------------

static PJRT_Error* Device_GetDescription(PJRT_Device_GetDescription_Args* a) { a->device_description = &a->device->desc; return nullptr; }
static PJRT_Error* Device_IsAddressable(PJRT_Device_IsAddressable_Args* a) { a->is_addressable = a->device->addressable; return nullptr; }
static PJRT_Error* Device_LocalHardwareId(PJRT_Device_LocalHardwareId_Args* a) { a->local_hardware_id = a->device->desc.local_hardware_id; return nullptr; }
static PJRT_Error* Device_AddressableMemories(PJRT_Device_AddressableMemories_Args* a) {
  a->memories = a->device->memories.data(); a->num_memories = a->device->memories.size(); return nullptr;
}
static PJRT_Error* Device_DefaultMemory(PJRT_Device_DefaultMemory_Args* a) { a->memory = a->device->memory; return nullptr; }
static PJRT_Error* Device_MemoryStats(PJRT_Device_MemoryStats_Args* a) {
  PJRT_Device* d = a->device;
  if (!d->addressable) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "memory statistics are only available for addressable devices");
  size_t free_b = 0, total_b = 0;
  cudaSetDevice(d->cuda_ordinal);
  cudaMemGetInfo(&free_b, &total_b);
  a->bytes_in_use = d->bytes_in_use.load();
  a->peak_bytes_in_use = d->peak_bytes.load(); a->peak_bytes_in_use_is_set = true;
  a->num_allocs = d->num_allocs.load(); a->num_allocs_is_set = true;
  a->largest_alloc_size_is_set = false;
  a->bytes_limit = (int64_t)total_b; a->bytes_limit_is_set = true;
  a->bytes_reserved_is_set = false; a->peak_bytes_reserved_is_set = false; a->bytes_reservable_limit_is_set = false;
  a->largest_free_block_bytes = (int64_t)free_b; a->largest_free_block_bytes_is_set = true;
  a->pool_bytes_is_set = false; a->peak_pool_bytes_is_set = false;
  return nullptr;
}
static PJRT_Error* Device_GetAttributes(PJRT_Device_GetAttributes_Args* a) {
  a->attributes = a->device->desc.attributes.data(); a->num_attributes = a->device->desc.attributes.size();
  a->device_attributes = nullptr; a->attributes_deleter = nullptr;
  return nullptr;
}
// Marks a launch that has not started yet as failed (reference: crates/ryft-pjrt/src/devices.rs:257-303).
static PJRT_Error* Device_PoisonExecution(PJRT_Device_PoisonExecution_Args* a) {
  std::lock_guard<std::mutex> lk(a->device->poison_mu);
  a->device->poisoned[a->launch_id] = {a->error_code, a->error_message ? std::string(a->error_message, a->error_message_size) : std::string()};
  a->poisoned = true;
  return nullptr;
}
static PJRT_Error* DeviceDescription_Id(PJRT_DeviceDescription_Id_Args* a) { a->id = a->device_description->id; return nullptr; }
static PJRT_Error* DeviceDescription_ProcessIndex(PJRT_DeviceDescription_ProcessIndex_Args* a) { a->process_index = a->device_description->process_index; return nullptr; }
static PJRT_Error* DeviceDescription_Attributes(PJRT_DeviceDescription_Attributes_Args* a) {
  a->attributes = a->device_description->attributes.data(); a->num_attributes = a->device_description->attributes.size(); return nullptr;
}
static PJRT_Error* DeviceDescription_Kind(PJRT_DeviceDescription_Kind_Args* a) {
  a->device_kind = a->device_description->kind.data(); a->device_kind_size = a->device_description->kind.size(); return nullptr;
}
static PJRT_Error* DeviceDescription_DebugString(PJRT_DeviceDescription_DebugString_Args* a) {
  a->debug_string = a->device_description->debug_string.data(); a->debug_string_size = a->device_description->debug_string.size(); return nullptr;
}
static PJRT_Error* DeviceDescription_ToString(PJRT_DeviceDescription_ToString_Args* a) {
  a->to_string = a->device_description->to_string.data(); a->to_string_size = a->device_description->to_string.size(); return nullptr;
}
static PJRT_Error* Memory_Id(PJRT_Memory_Id_Args* a) { a->id = a->memory->id; return nullptr; }
// One memory kind, "device"; its id is a fixed non-zero number (FNV-1a of the kind name, 31 bits), as kind ids are
// compared for equality and tested for being non-zero by ryft (crates/ryft-pjrt/src/memories.rs:136-138, 354).
static constexpr int kDeviceMemoryKindId = 0x1b3c5a71;
static PJRT_Error* Memory_Kind_Id(PJRT_Memory_Kind_Id_Args* a) { a->kind_id = kDeviceMemoryKindId; return nullptr; }
static PJRT_Error* Memory_Kind(PJRT_Memory_Kind_Args* a) { a->kind = a->memory->kind.data(); a->kind_size = a->memory->kind.size(); return nullptr; }
static PJRT_Error* Memory_DebugString(PJRT_Memory_DebugString_Args* a) {
  a->debug_string = a->memory->debug_string.data(); a->debug_string_size = a->memory->debug_string.size(); return nullptr;
}
static PJRT_Error* Memory_ToString(PJRT_Memory_ToString_Args* a) { a->to_string = a->memory->to_string.data(); a->to_string_size = a->memory->to_string.size(); return nullptr; }
static PJRT_Error* Memory_AddressableByDevices(PJRT_Memory_AddressableByDevices_Args* a) {
  a->devices = a->memory->devices.data(); a->num_devices = a->memory->devices.size(); return nullptr;
}

// ---- buffers ----------------------------------------------------------------------------------------------------------

static PJRT_Error* resolve_device(PJRT_Client* c, PJRT_Device* device, PJRT_Memory* memory, PJRT_Device** out) {
  PJRT_Device* d = device ? device : (memory ? memory->device : nullptr);
  if (!d) d = c->addressable_devices.empty() ? nullptr : c->addressable_devices[0];
  if (!d || !d->addressable) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the target device is not addressable from this process");
  *out = d;
  return nullptr;
}

static PJRT_Error* Client_BufferFromHostBuffer(PJRT_Client_BufferFromHostBuffer_Args* a) {
  PJRT_Device* dev;
  B2X_RETURN_IF_ERROR(resolve_device(a->client, a->device, a->memory, &dev));
  DType dt = from_pjrt_type(a->type);
  if (dt == DType::INVALID) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "buffer element type " + std::to_string(a->type) + " is not supported");
  TensorType t;
  t.dtype = dt;
  t.dims.assign(a->dims, a->dims + a->num_dims);
  for (auto d : t.dims) B2X_CHECK_ARG(d >= 0, "negative dimension");
  const int es = dtype_size(dt);
  // dense major-to-minor unless strides say otherwise
  bool dense = true;
  if (a->byte_strides && a->num_byte_strides == a->num_dims) {
    int64_t acc = es;
    for (int i = (int)a->num_dims - 1; i >= 0; i--) { if (t.dims[i] != 1 && a->byte_strides[i] != acc) dense = false; acc *= t.dims[i]; }
  }
  PJRT_Buffer* b = nullptr;
  {
    // a block of this size that an earlier upload left behind and whose last use has finished
    const size_t want = (size_t)t.byte_size();
    void* reuse = nullptr;
    if (want >= PJRT_Device::kMinRecycledBytes) {
      std::lock_guard<std::mutex> lk(dev->recycle_mu);
      for (size_t i = 0; i < dev->recycled.size(); i++) {
        PJRT_Device::RecycledBlock& r = dev->recycled[i];
        if (r.bytes != want) continue;
        cudaSetDevice(dev->cuda_ordinal);
        if (cudaEventQuery(r.last_use) != cudaSuccess) { cudaGetLastError(); continue; }
        cudaEventDestroy(r.last_use);
        reuse = r.ptr;
        dev->recycled.erase(dev->recycled.begin() + (long)i);
        break;
      }
    }
    if (reuse) {
      b = new PJRT_Buffer();
      b->client = dev->client; b->device = dev; b->type = t; b->dims = t.dims; b->pjrt_type = to_pjrt_type(t.dtype);
      b->bytes = want;
      for (int i = t.rank() - 1; i >= 0; i--) b->minor_to_major.push_back(i);
      b->ptr = reuse;
      track_alloc(dev, (int64_t)b->bytes);
    } else {
      B2X_RETURN_IF_ERROR(alloc_buffer(dev, t, dev->h2d, &b));
    }
    b->from_host = true;
  }
  const void* src = a->data;
  std::vector<uint8_t> packed;
  if (!dense) {  // gather the strided host tensor into dense row-major order first
    packed.resize(b->bytes);
    std::vector<int64_t> idx(a->num_dims, 0);
    const int64_t n = t.num_elements();
    for (int64_t e = 0; e < n; e++) {
      int64_t off = 0;
      for (size_t d = 0; d < a->num_dims; d++) off += idx[d] * a->byte_strides[d];
      memcpy(packed.data() + e * es, (const char*)a->data + off, es);
      for (int d = (int)a->num_dims - 1; d >= 0; d--) { if (++idx[d] < t.dims[d]) break; idx[d] = 0; }
    }
    src = packed.data();
  }
  cudaError_t e = cudaSuccess;
  if (b->bytes) e = cudaMemcpyAsync(b->ptr, src, b->bytes, cudaMemcpyHostToDevice, dev->h2d);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b->ready, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventRecord(b->ready, dev->h2d);
  if (e != cudaSuccess) { release_buffer_memory(b); delete b; return cuda_error(e, "host to device copy"); }
  PJRT_Event* done = new PJRT_Event();
  const bool must_finish_now = a->host_buffer_semantics == PJRT_HostBufferSemantics_kImmutableOnlyDuringCall || !dense;
  if (must_finish_now) {
    // pageable memory has been staged when cudaMemcpyAsync returns; pinned memory is read by DMA later, so wait
    cudaPointerAttributes pa{};
    bool pinned = cudaPointerGetAttributes(&pa, a->data) == cudaSuccess && pa.type == cudaMemoryTypeHost;
    cudaGetLastError();
    if (pinned || !dense) cudaStreamSynchronize(dev->h2d);
    done->set(PJRT_Error_Code_OK, "");
  } else {
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, dev->h2d);
    a->client->post({ev, dev->cuda_ordinal, done, nullptr});
  }
  a->done_with_host_buffer = done;
  a->buffer = b;
  return nullptr;
}

static PJRT_Error* Client_CreateUninitializedBuffer(PJRT_Client_CreateUninitializedBuffer_Args* a) {
  PJRT_Device* dev;
  B2X_RETURN_IF_ERROR(resolve_device(a->client, a->device, a->memory, &dev));
  DType dt = from_pjrt_type(a->shape_element_type);
  if (dt == DType::INVALID) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "buffer element type is not supported");
  TensorType t;
  t.dtype = dt;
  t.dims.assign(a->shape_dims, a->shape_dims + a->shape_num_dims);
  PJRT_Buffer* b;
  B2X_RETURN_IF_ERROR(alloc_buffer(dev, t, dev->compute, &b));
  a->buffer = b;
  return nullptr;
}

static PJRT_Error* Client_CreateViewOfDeviceBuffer(PJRT_Client_CreateViewOfDeviceBuffer_Args* a) {
  PJRT_Device* dev;
  B2X_RETURN_IF_ERROR(resolve_device(a->client, a->device, a->memory, &dev));
  DType dt = from_pjrt_type(a->element_type);
  if (dt == DType::INVALID) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "buffer element type is not supported");
  PJRT_Buffer* b = new PJRT_Buffer();
  b->client = a->client; b->device = dev;
  b->type.dtype = dt;
  b->type.dims.assign(a->dims, a->dims + a->num_dims);
  b->dims = b->type.dims;
  b->pjrt_type = a->element_type;
  b->bytes = (size_t)b->type.byte_size();
  for (int i = b->type.rank() - 1; i >= 0; i--) b->minor_to_major.push_back(i);
  b->ptr = a->device_buffer_ptr;
  b->owns = false;
  if (a->on_delete_callback) {
    auto cb = a->on_delete_callback; void* p = a->device_buffer_ptr; void* arg = a->on_delete_callback_arg;
    b->on_delete = [cb, p, arg] { cb(p, arg); };
  }
  if (a->stream) {  // work already queued on the producer's stream must finish before this buffer is read
    cudaSetDevice(dev->cuda_ordinal);
    cudaEventCreateWithFlags(&b->ready, cudaEventDisableTiming);
    cudaEventRecord(b->ready, (cudaStream_t)a->stream);
  }
  a->buffer = b;
  return nullptr;
}

static PJRT_Error* Client_CreateErrorBuffer(PJRT_Client_CreateErrorBuffer_Args* a) {
  PJRT_Device* dev;
  B2X_RETURN_IF_ERROR(resolve_device(a->client, nullptr, a->memory, &dev));
  PJRT_Buffer* b = new PJRT_Buffer();
  b->client = a->client; b->device = dev;
  b->type.dtype = from_pjrt_type(a->shape_element_type);
  b->type.dims.assign(a->shape_dims, a->shape_dims + a->shape_num_dims);
  b->dims = b->type.dims;
  b->pjrt_type = a->shape_element_type;
  b->owns = false;
  b->err_code = a->error_code;
  b->err_msg = a->error_message ? std::string(a->error_message, a->error_message_size) : std::string();
  for (int i = b->type.rank() - 1; i >= 0; i--) b->minor_to_major.push_back(i);
  a->buffer = b;
  return nullptr;
}

static PJRT_Error* Buffer_Destroy(PJRT_Buffer_Destroy_Args* a) {
  if (!a->buffer) return nullptr;
  {
    std::lock_guard<std::mutex> lk(a->buffer->mu);
    release_buffer_memory(a->buffer);
    if (a->buffer->ready) { cudaEventDestroy(a->buffer->ready); a->buffer->ready = nullptr; }
  }
  delete a->buffer;
  return nullptr;
}
static PJRT_Error* Buffer_Delete(PJRT_Buffer_Delete_Args* a) {
  std::lock_guard<std::mutex> lk(a->buffer->mu);
  release_buffer_memory(a->buffer);
  a->buffer->deleted = true;
  return nullptr;
}
static PJRT_Error* Buffer_IsDeleted(PJRT_Buffer_IsDeleted_Args* a) { a->is_deleted = a->buffer->deleted; return nullptr; }
static PJRT_Error* Buffer_ElementType(PJRT_Buffer_ElementType_Args* a) { a->type = a->buffer->pjrt_type; return nullptr; }
static PJRT_Error* Buffer_Dimensions(PJRT_Buffer_Dimensions_Args* a) { a->dims = a->buffer->dims.data(); a->num_dims = a->buffer->dims.size(); return nullptr; }
static PJRT_Error* Buffer_UnpaddedDimensions(PJRT_Buffer_UnpaddedDimensions_Args* a) {
  a->unpadded_dims = a->buffer->dims.data(); a->num_dims = a->buffer->dims.size(); return nullptr;
}
static PJRT_Error* Buffer_DynamicDimensionIndices(PJRT_Buffer_DynamicDimensionIndices_Args* a) { a->dynamic_dim_indices = nullptr; a->num_dynamic_dims = 0; return nullptr; }
static PJRT_Error* Buffer_GetMemoryLayout(PJRT_Buffer_GetMemoryLayout_Args* a) {
  // dense row-major: minor_to_major = {n-1, ..., 0} (crates/ryft-pjrt/src/extensions/layouts.rs:832-835)
  memset(&a->layout, 0, sizeof(a->layout));
  a->layout.struct_size = sizeof(a->layout);
  a->layout.type = PJRT_Buffer_MemoryLayout_Type_Tiled;
  a->layout.tiled.struct_size = sizeof(a->layout.tiled);
  a->layout.tiled.minor_to_major = a->buffer->minor_to_major.data();
  a->layout.tiled.minor_to_major_size = a->buffer->minor_to_major.size();
  return nullptr;
}
static PJRT_Error* Buffer_OnDeviceSizeInBytes(PJRT_Buffer_OnDeviceSizeInBytes_Args* a) { a->on_device_size_in_bytes = a->buffer->bytes; return nullptr; }
static PJRT_Error* Buffer_Device(PJRT_Buffer_Device_Args* a) { a->device = a->buffer->device; return nullptr; }
static PJRT_Error* Buffer_Memory(PJRT_Buffer_Memory_Args* a) { a->memory = a->buffer->device->memory; return nullptr; }
static PJRT_Error* Buffer_IsOnCpu(PJRT_Buffer_IsOnCpu_Args* a) { a->is_on_cpu = false; return nullptr; }

static PJRT_Error* check_live(PJRT_Buffer* b) {
  if (b->deleted || (!b->ptr && b->err_code == PJRT_Error_Code_OK && b->bytes > 0))
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the buffer has been deleted or donated");
  if (b->err_code != PJRT_Error_Code_OK) return make_error(b->err_code, b->err_msg);
  return nullptr;
}

static PJRT_Error* Buffer_ReadyEvent(PJRT_Buffer_ReadyEvent_Args* a) {
  PJRT_Buffer* b = a->buffer;
  std::lock_guard<std::mutex> lk(b->mu);
  PJRT_Event* ev = new PJRT_Event();
  if (b->pending) {
    std::lock_guard<std::mutex> dl(b->pending->mu);
    if (!b->pending->done) { ev->ref(); b->pending->waiters.push_back(ev); a->event = ev; return nullptr; }
  }
  if (b->err_code != PJRT_Error_Code_OK) { ev->set(b->err_code, b->err_msg); a->event = ev; return nullptr; }
  if (b->deleted) { delete ev; return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the buffer has been deleted"); }
  if (!b->ready) { ev->set(PJRT_Error_Code_OK, ""); a->event = ev; return nullptr; }
  // wait for the definition event on a side stream so that later re-records do not matter
  cudaSetDevice(b->device->cuda_ordinal);
  cudaEvent_t e2;
  cudaEventCreateWithFlags(&e2, cudaEventDisableTiming);
  cudaStreamWaitEvent(b->device->d2h, b->ready, 0);
  cudaEventRecord(e2, b->device->d2h);
  b->client->post({e2, b->device->cuda_ordinal, ev, nullptr});
  a->event = ev;
  return nullptr;
}

static PJRT_Error* copy_to_host(PJRT_Buffer* b, void* dst, size_t offset, size_t size, PJRT_Event** event) {
  await_definition(b);
  PJRT_Device* d = b->device;
  B2X_CUDA(cudaSetDevice(d->cuda_ordinal));
  if (b->ready) B2X_CUDA(cudaStreamWaitEvent(d->d2h, b->ready, 0));
  // Small reads (a loss, a metric) go through a pinned staging block and reach `dst` on the poller thread when the copy
  // has finished: the call returns at once even though `dst` is ordinary pageable memory, so a training loop can
  // enqueue its next step before the current one is done.  Larger reads are dominated by the transfer itself.
  void* staging = nullptr;
  if (size && size <= PJRT_Device::kStagingBlock) {
    std::lock_guard<std::mutex> sl(d->staging_mu);
    if (!d->staging_free.empty()) { staging = d->staging_free.back(); d->staging_free.pop_back(); }
  }
  if (size && size <= PJRT_Device::kStagingBlock && !staging) {
    if (cudaHostAlloc(&staging, PJRT_Device::kStagingBlock, cudaHostAllocDefault) != cudaSuccess) { cudaGetLastError(); staging = nullptr; }
  }
  if (size) B2X_CUDA(cudaMemcpyAsync(staging ? staging : dst, (const char*)b->ptr + offset, size, cudaMemcpyDeviceToHost, d->d2h));
  cudaEvent_t ev, keep;
  B2X_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  B2X_CUDA(cudaEventRecord(ev, d->d2h));
  B2X_CUDA(cudaEventCreateWithFlags(&keep, cudaEventDisableTiming));
  B2X_CUDA(cudaEventRecord(keep, d->d2h));
  // drop read markers that have completed, then remember this one so that freeing the buffer waits for the copy
  for (auto it = b->pending_reads.begin(); it != b->pending_reads.end();) {
    if (cudaEventQuery(*it) == cudaSuccess) { cudaEventDestroy(*it); it = b->pending_reads.erase(it); } else ++it;
  }
  b->pending_reads.push_back(keep);
  PJRT_Event* pe = new PJRT_Event();
  PJRT_Device* dev = d;
  b->client->post({ev, d->cuda_ordinal, pe, [dev, staging, dst, size](PJRT_Error_Code* code, std::string* msg) {
                     if (staging) {
                       if (*code == PJRT_Error_Code_OK) memcpy(dst, staging, size);
                       std::lock_guard<std::mutex> sl(dev->staging_mu);
                       dev->staging_free.push_back(staging);
                     }
                     report_expired_wait(dev, code, msg);
                   }});
  *event = pe;
  return nullptr;
}

static PJRT_Error* Buffer_ToHostBuffer(PJRT_Buffer_ToHostBuffer_Args* a) {
  PJRT_Buffer* b = a->src;
  std::lock_guard<std::mutex> lk(b->mu);
  B2X_RETURN_IF_ERROR(check_live(b));
  if (!a->dst) { a->dst_size = b->bytes; a->event = nullptr; return nullptr; }
  if (a->dst_size < b->bytes) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the destination holds " + std::to_string(a->dst_size) + " bytes but the buffer needs " + std::to_string(b->bytes));
  return copy_to_host(b, a->dst, 0, b->bytes, &a->event);
}
static PJRT_Error* Buffer_CopyRawToHost(PJRT_Buffer_CopyRawToHost_Args* a) {
  PJRT_Buffer* b = a->buffer;
  std::lock_guard<std::mutex> lk(b->mu);
  B2X_RETURN_IF_ERROR(check_live(b));
  if (a->offset < 0 || a->transfer_size < 0 || (size_t)(a->offset + a->transfer_size) > b->bytes)
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "raw copy of " + std::to_string(a->transfer_size) + " bytes at offset " + std::to_string(a->offset) +
                                                            " exceeds the buffer size of " + std::to_string(b->bytes) + " bytes");
  return copy_to_host(b, a->dst, (size_t)a->offset, (size_t)a->transfer_size, &a->event);
}

static PJRT_Error* copy_to_device_impl(PJRT_Buffer* b, PJRT_Device* dst_dev, PJRT_Buffer** out) {
  std::lock_guard<std::mutex> lk(b->mu);
  B2X_RETURN_IF_ERROR(check_live(b));
  if (!dst_dev->addressable) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "copies to devices of other processes are not supported");
  await_definition(b);
  PJRT_Buffer* nb;
  B2X_RETURN_IF_ERROR(alloc_buffer(dst_dev, b->type, dst_dev->compute, &nb));
  cudaSetDevice(dst_dev->cuda_ordinal);
  if (b->ready) cudaStreamWaitEvent(dst_dev->compute, b->ready, 0);
  cudaError_t e = cudaSuccess;
  if (b->bytes) {
    if (dst_dev == b->device) e = cudaMemcpyAsync(nb->ptr, b->ptr, b->bytes, cudaMemcpyDeviceToDevice, dst_dev->compute);
    else e = cudaMemcpyPeerAsync(nb->ptr, dst_dev->cuda_ordinal, b->ptr, b->device->cuda_ordinal, b->bytes, dst_dev->compute);
  }
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&nb->ready, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventRecord(nb->ready, dst_dev->compute);
  if (e != cudaSuccess) { release_buffer_memory(nb); delete nb; return cuda_error(e, "device to device copy"); }
  // the source must outlive the copy: remember the read on the source buffer
  cudaEvent_t keep;
  cudaEventCreateWithFlags(&keep, cudaEventDisableTiming);
  cudaEventRecord(keep, dst_dev->compute);
  b->pending_reads.push_back(keep);
  *out = nb;
  return nullptr;
}
static PJRT_Error* Buffer_CopyToDevice(PJRT_Buffer_CopyToDevice_Args* a) { return copy_to_device_impl(a->buffer, a->dst_device, &a->dst_buffer); }
static PJRT_Error* Buffer_CopyToMemory(PJRT_Buffer_CopyToMemory_Args* a) { return copy_to_device_impl(a->buffer, a->dst_memory->device, &a->dst_buffer); }
static PJRT_Error* Buffer_UnsafePointer(PJRT_Buffer_UnsafePointer_Args* a) { a->buffer_pointer = (uintptr_t)a->buffer->ptr; return nullptr; }
static PJRT_Error* Buffer_OpaqueDeviceMemoryDataPointer(PJRT_Buffer_OpaqueDeviceMemoryDataPointer_Args* a) { a->device_memory_ptr = a->buffer->ptr; return nullptr; }
static PJRT_Error* Buffer_IncRef(PJRT_Buffer_IncreaseExternalReferenceCount_Args* a) { a->buffer->ext_refs++; return nullptr; }
static PJRT_Error* Buffer_DecRef(PJRT_Buffer_DecreaseExternalReferenceCount_Args* a) {
  if (a->buffer->ext_refs.load() <= 0) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "the external reference count is already zero");
  a->buffer->ext_refs--;
  return nullptr;
}
static PJRT_Error* Buffer_Bitcast(PJRT_Buffer_Bitcast_Args*) { return make_error(PJRT_Error_Code_UNIMPLEMENTED, "PJRT_Buffer_Bitcast is not implemented"); }

// ---- compile / executables ----------------------------------------------------------------------------------------------

static int step_kernel_launches(const Step& s);
static uint64_t fnv1a(const std::string& s, uint64_t h = 1469598103934665603ull) {
  for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
  return h;
}

static PJRT_Error* build_core(PJRT_Client* client, const std::string& code, const std::string& options, std::shared_ptr<b2x_ExecutableCore>* out) {
  CompileOptions co;
  std::string perr;
  if (!parse_compile_options(options.data(), options.size(), &co, &perr)) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, perr);
  auto core = std::make_shared<b2x_ExecutableCore>();
  try {
    std::unique_ptr<Module> mod = parse_module(code);
    PlanOptions po;
    po.num_replicas = (int)co.num_replicas;
    po.num_partitions = (int)co.num_partitions;
    po.precision = co.precision;
    if (const char* g = getenv("B2X_GEMM")) po.allow_tensor_core = strcmp(g, "simt") != 0;
    if (const char* f = getenv("B2X_FUSED_ATTENTION")) po.allow_fused_attention = strcmp(f, "0") != 0;
    if (const char* f = getenv("B2X_EPILOGUE_FUSION")) po.allow_epilogue_fusion = strcmp(f, "0") != 0;
    if (const char* f = getenv("B2X_PRECISE_MATH")) po.precise_math = strcmp(f, "0") != 0;
    if (co.use_spmd_partitioning && co.num_partitions > 1)
      return make_error(PJRT_Error_Code_UNIMPLEMENTED, "automatic SPMD partitioning is not supported; express the collectives in the program");
    core->plans.push_back(build_plan(*mod, po, 0));
    if (core->plans[0].uses_replica_id)
      for (int r = 1; r < po.num_replicas; r++) core->plans.push_back(build_plan(*mod, po, r));
    core->name = mod->name;
    if (getenv("B2X_LOG")) fprintf(stderr, "%s", core->plans[0].dump().c_str());
  } catch (const CompileError& e) {
    return make_error((PJRT_Error_Code)e.code, e.what());
  } catch (const std::exception& e) {
    return make_error(PJRT_Error_Code_INTERNAL, std::string("compile failed: ") + e.what());
  }
  core->source = code;
  core->compile_options = options;
  core->num_replicas = (int)co.num_replicas;
  core->num_partitions = (int)co.num_partitions;
  const int n = core->num_replicas;
  if (co.has_device_assignment && !co.da_devices.empty()) {
    if ((int64_t)co.da_devices.size() != co.num_partitions) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "device assignment does not match partition_count");
    for (int r = 0; r < n; r++) {
      if ((int)co.da_devices[0].size() != n) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "device assignment does not match replica_count");
      core->device_assignment.push_back((int)co.da_devices[0][r]);
    }
  } else if (n == 1 && co.device_ordinal >= 0) {
    core->device_assignment.push_back((int)co.device_ordinal);
  } else {
    if (n > (int)client->devices.size())
      return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "replica_count = " + std::to_string(n) + " but the client has only " + std::to_string(client->devices.size()) + " devices");
    // default assignment: replica r on device r; a single-replica program of a process that cannot address device 0
    // (one process per GPU) runs on that process's own first device
    for (int r = 0; r < n; r++) {
      PJRT_Device* d = client->devices[r];
      if (n == 1 && !d->addressable && !client->addressable_devices.empty()) d = client->addressable_devices[0];
      core->device_assignment.push_back(d->desc.id);
    }
  }
  for (int id : core->device_assignment)
    if (id < 0 || id >= (int)client->devices.size()) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "device assignment names device " + std::to_string(id) + " which does not exist");
  const Plan& p = core->plans[0];
  static const char kDevice[] = "device";
  for (auto& o : p.outputs) {
    core->out_types.push_back(to_pjrt_type(o.type.dtype));
    core->out_ranks.push_back(o.type.dims.size());
    for (auto d : o.type.dims) core->out_dims_flat.push_back(d);
    core->out_kinds.push_back(kDevice); core->out_kind_sizes.push_back(6);
  }
  for (size_t i = 0; i < p.arg_types.size(); i++) { core->param_kinds.push_back(kDevice); core->param_kind_sizes.push_back(6); }
  char fp[40];
  snprintf(fp, sizeof(fp), "%016llx", (unsigned long long)fnv1a(options, fnv1a(code)));
  core->fingerprint = fp;
  core->cost_names = {"flops", "bytes accessed", "kernel launches"};
  core->cost_props.resize(3);
  for (int i = 0; i < 3; i++) {
    memset(&core->cost_props[i], 0, sizeof(PJRT_NamedValue));
    core->cost_props[i].struct_size = sizeof(PJRT_NamedValue);
    core->cost_props[i].name = core->cost_names[i].data(); core->cost_props[i].name_size = core->cost_names[i].size();
    core->cost_props[i].type = PJRT_NamedValue_kFloat; core->cost_props[i].value_size = 1;
  }
  core->cost_props[0].float_value = (float)p.total_flops;
  core->cost_props[1].float_value = (float)p.total_bytes;
  {
    int launches = 0;
    for (auto& st : p.steps) launches += step_kernel_launches(st);
    core->cost_props[2].float_value = (float)launches;
  }
  *out = core;
  return nullptr;
}

static PJRT_Error* load_core(PJRT_Client* client, std::shared_ptr<b2x_ExecutableCore> core, PJRT_LoadedExecutable** out) {
  std::unique_ptr<PJRT_LoadedExecutable> le(new PJRT_LoadedExecutable());
  le->client = client;
  le->core = core;
  for (int r = 0; r < core->num_replicas; r++) {
    PJRT_Device* d = client->devices[core->device_assignment[r]];
    if (!d->addressable) continue;
    le->addressable.push_back(d);
    le->logical_ids.push_back({r, 0});
  }
  if (le->addressable.empty()) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "none of the assigned devices is addressable from this process");
  le->per_device.resize(le->addressable.size());
  *out = le.release();
  return nullptr;
}

static PJRT_Error* Client_Compile(PJRT_Client_Compile_Args* a) {
  B2X_CHECK_ARG(a->program && a->program->code, "the program is null");
  std::string format(a->program->format ? a->program->format : "", a->program->format_size);
  if (format != "mlir")
    return make_error(PJRT_Error_Code_UNIMPLEMENTED, "program format '" + format + "' is not supported; this plugin compiles StableHLO passed as 'mlir'");
  std::string code(a->program->code, a->program->code_size);
  std::string options(a->compile_options ? a->compile_options : "", a->compile_options_size);
  std::shared_ptr<b2x_ExecutableCore> core;
  B2X_RETURN_IF_ERROR(build_core(a->client, code, options, &core));
  return load_core(a->client, core, &a->executable);
}

// Serialized form: "B2XE1\n" + u64 options size + options + MLIR text.  Loading re-plans from the text.
static std::string serialize_core(const b2x_ExecutableCore& c) {
  std::string s = "B2XE1\n";
  uint64_t n = c.compile_options.size();
  s.append((const char*)&n, 8);
  s += c.compile_options;
  s += c.source;
  return s;
}
static PJRT_Error* Executable_DeserializeAndLoad(PJRT_Executable_DeserializeAndLoad_Args* a) {
  std::string s(a->serialized_executable, a->serialized_executable_size);
  if (s.size() < 14 || s.compare(0, 6, "B2XE1\n") != 0) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "not an executable serialized by this plugin");
  uint64_t n;
  memcpy(&n, s.data() + 6, 8);
  if (14 + n > s.size()) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "truncated serialized executable");
  std::string options = s.substr(14, n), code = s.substr(14 + n);
  if (a->overridden_serialized_compile_options && a->overridden_serialized_compile_options_size)
    options.assign(a->overridden_serialized_compile_options, a->overridden_serialized_compile_options_size);
  std::shared_ptr<b2x_ExecutableCore> core;
  B2X_RETURN_IF_ERROR(build_core(a->client, code, options, &core));
  return load_core(a->client, core, &a->loaded_executable);
}
static PJRT_Error* Client_Load(PJRT_Client_Load_Args* a) { return load_core(a->client, a->executable->core, &a->loaded_executable); }

static PJRT_Error* Executable_Destroy(PJRT_Executable_Destroy_Args* a) { delete a->executable; return nullptr; }
static PJRT_Error* Executable_Name(PJRT_Executable_Name_Args* a) {
  a->executable_name = a->executable->core->name.data(); a->executable_name_size = a->executable->core->name.size(); return nullptr;
}
static PJRT_Error* Executable_NumReplicas(PJRT_Executable_NumReplicas_Args* a) { a->num_replicas = (size_t)a->executable->core->num_replicas; return nullptr; }
static PJRT_Error* Executable_NumPartitions(PJRT_Executable_NumPartitions_Args* a) { a->num_partitions = (size_t)a->executable->core->num_partitions; return nullptr; }
static PJRT_Error* Executable_NumOutputs(PJRT_Executable_NumOutputs_Args* a) { a->num_outputs = a->executable->core->out_types.size(); return nullptr; }
static PJRT_Error* Executable_SizeOfGeneratedCodeInBytes(PJRT_Executable_SizeOfGeneratedCodeInBytes_Args* a) {
  int64_t n = 0;
  for (auto& s : a->executable->core->plans[0].steps) n += (int64_t)sizeof(B2xVmInstr) * s.vm.prog.n_instr;
  a->size_in_bytes = n;
  return nullptr;
}
static PJRT_Error* Executable_GetCostAnalysis(PJRT_Executable_GetCostAnalysis_Args* a) {
  a->properties = a->executable->core->cost_props.data(); a->num_properties = a->executable->core->cost_props.size(); return nullptr;
}
static PJRT_Error* Executable_OutputMemoryKinds(PJRT_Executable_OutputMemoryKinds_Args* a) {
  auto& c = *a->executable->core;
  a->num_outputs = c.out_kinds.size(); a->memory_kinds = c.out_kinds.data(); a->memory_kind_sizes = c.out_kind_sizes.data(); return nullptr;
}
static PJRT_Error* Executable_ParameterMemoryKinds(PJRT_Executable_ParameterMemoryKinds_Args* a) {
  auto& c = *a->executable->core;
  a->num_parameters = c.param_kinds.size(); a->memory_kinds = c.param_kinds.data(); a->memory_kind_sizes = c.param_kind_sizes.data(); return nullptr;
}
static PJRT_Error* Executable_OptimizedProgram(PJRT_Executable_OptimizedProgram_Args* a) {
  // two-call protocol: code == NULL => report the size; otherwise copy the MLIR text
  const std::string& src = a->executable->core->source;
  static const char kFormat[] = "mlir";
  a->program->format = kFormat; a->program->format_size = 4;
  if (!a->program->code) { a->program->code_size = src.size(); return nullptr; }
  if (a->program->code_size < src.size()) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the program buffer is too small");
  memcpy(a->program->code, src.data(), src.size());
  a->program->code_size = src.size();
  return nullptr;
}
struct SerializedBlob { std::string bytes; };
static void delete_blob_exec(PJRT_SerializedExecutable* p) { delete (SerializedBlob*)p; }
static void delete_blob_opts(PJRT_SerializedCompileOptions* p) { delete (SerializedBlob*)p; }
static void delete_blob_da(PJRT_DeviceAssignmentSerialized* p) { delete (SerializedBlob*)p; }
static PJRT_Error* Executable_Serialize(PJRT_Executable_Serialize_Args* a) {
  SerializedBlob* b = new SerializedBlob{serialize_core(*a->executable->core)};
  a->serialized_bytes = b->bytes.data(); a->serialized_bytes_size = b->bytes.size();
  a->serialized_executable = (PJRT_SerializedExecutable*)b; a->serialized_executable_deleter = delete_blob_exec;
  return nullptr;
}
static PJRT_Error* Executable_GetCompileOptions(PJRT_Executable_GetCompileOptions_Args* a) {
  SerializedBlob* b = new SerializedBlob{a->executable->core->compile_options};
  a->serialized_bytes = b->bytes.data(); a->serialized_bytes_size = b->bytes.size();
  a->serialized_compile_options = (PJRT_SerializedCompileOptions*)b; a->serialized_compile_options_deleter = delete_blob_opts;
  return nullptr;
}
static PJRT_Error* Executable_OutputElementTypes(PJRT_Executable_OutputElementTypes_Args* a) {
  a->output_types = a->executable->core->out_types.data(); a->num_output_types = a->executable->core->out_types.size(); return nullptr;
}
static PJRT_Error* Executable_OutputDimensions(PJRT_Executable_OutputDimensions_Args* a) {
  auto& c = *a->executable->core;
  a->num_outputs = c.out_ranks.size(); a->dims = c.out_dims_flat.data(); a->dim_sizes = c.out_ranks.data(); return nullptr;
}
static PJRT_Error* Executable_Fingerprint(PJRT_Executable_Fingerprint_Args* a) {
  a->executable_fingerprint = a->executable->core->fingerprint.data(); a->executable_fingerprint_size = a->executable->core->fingerprint.size(); return nullptr;
}
static PJRT_Error* Executable_GetCompiledMemoryStats(PJRT_Executable_GetCompiledMemoryStats_Args* a) {
  const Plan& p = a->executable->core->plans[0];
  int64_t args = 0, outs = 0;
  for (auto& t : p.arg_types) args += t.byte_size();
  for (auto& o : p.outputs) outs += o.type.byte_size();
  a->generated_code_size_in_bytes = 0; a->argument_size_in_bytes = args; a->output_size_in_bytes = outs; a->alias_size_in_bytes = 0;
  a->temp_size_in_bytes = p.arena_bytes;
  a->host_generated_code_size_in_bytes = a->host_argument_size_in_bytes = a->host_output_size_in_bytes = a->host_alias_size_in_bytes = a->host_temp_size_in_bytes = 0;
  a->peak_memory_in_bytes = args + outs + p.arena_bytes; a->total_size_in_bytes = args + outs + p.arena_bytes;
  a->total_allocation_bytes = p.arena_bytes; a->indefinite_allocations = 0; a->peak_unpadded_heap_bytes = 0;
  return nullptr;
}

static PJRT_Error* LoadedExecutable_Destroy(PJRT_LoadedExecutable_Destroy_Args* a) { delete a->executable; return nullptr; }
static PJRT_Error* LoadedExecutable_GetExecutable(PJRT_LoadedExecutable_GetExecutable_Args* a) {
  a->executable = new PJRT_Executable{a->loaded_executable->core};
  return nullptr;
}
static PJRT_Error* LoadedExecutable_AddressableDevices(PJRT_LoadedExecutable_AddressableDevices_Args* a) {
  a->addressable_devices = a->executable->addressable.data(); a->num_addressable_devices = a->executable->addressable.size(); return nullptr;
}
static PJRT_Error* LoadedExecutable_AddressableDeviceLogicalIds(PJRT_LoadedExecutable_AddressableDeviceLogicalIds_Args* a) {
  a->addressable_device_logical_ids = a->executable->logical_ids.data(); a->num_addressable_device_logical_ids = a->executable->logical_ids.size(); return nullptr;
}
static PJRT_Error* LoadedExecutable_GetDeviceAssignment(PJRT_LoadedExecutable_GetDeviceAssignment_Args* a) {
  auto& c = *a->executable->core;
  SerializedBlob* b = new SerializedBlob{encode_device_assignment(c.num_replicas, 1, c.device_assignment)};
  a->serialized_bytes = b->bytes.data(); a->serialized_bytes_size = b->bytes.size();
  a->serialized_device_assignment = (PJRT_DeviceAssignmentSerialized*)b; a->serialized_device_assignment_deleter = delete_blob_da;
  return nullptr;
}
static PJRT_Error* LoadedExecutable_Delete(PJRT_LoadedExecutable_Delete_Args* a) { a->executable->deleted = true; return nullptr; }
static PJRT_Error* LoadedExecutable_IsDeleted(PJRT_LoadedExecutable_IsDeleted_Args* a) { a->is_deleted = a->executable->deleted; return nullptr; }
static PJRT_Error* LoadedExecutable_Fingerprint(PJRT_LoadedExecutable_Fingerprint_Args* a) {
  a->executable_fingerprint = a->executable->core->fingerprint.data(); a->executable_fingerprint_size = a->executable->core->fingerprint.size(); return nullptr;
}
static PJRT_Error* ExecuteContext_Create(PJRT_ExecuteContext_Create_Args* a) { a->context = new PJRT_ExecuteContext(); return nullptr; }
static PJRT_Error* ExecuteContext_Destroy(PJRT_ExecuteContext_Destroy_Args* a) { delete a->context; return nullptr; }

// ---- execute ------------------------------------------------------------------------------------------------------------

static PJRT_Error* prepare_device_state(PJRT_LoadedExecutable* le, int li) {
  PJRT_LoadedExecutable::PerDevice& pd = le->per_device[li];
  PJRT_Device* dev = le->addressable[li];
  const Plan& plan = le->core->plans[0];
  B2X_CUDA(cudaSetDevice(dev->cuda_ordinal));
  if (!pd.fork) B2X_CUDA(cudaEventCreateWithFlags(&pd.fork, cudaEventDisableTiming));
  while ((int)pd.coll_done.size() < plan.num_collectives) {
    cudaEvent_t e;
    B2X_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    pd.coll_done.push_back(e);
  }
  if (!pd.arena && plan.arena_bytes > 0) {
    cudaError_t e = cudaMalloc(&pd.arena, (size_t)plan.arena_bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return make_error(PJRT_Error_Code_RESOURCE_EXHAUSTED, "could not allocate " + std::to_string(plan.arena_bytes) + " bytes of device memory for intermediates: " + cudaGetErrorString(e));
    }
    pd.arena_bytes = (size_t)plan.arena_bytes;
    track_alloc(dev, plan.arena_bytes);
  }
  if (!pd.consts && !plan.const_pool.empty()) {
    B2X_CUDA(cudaMalloc(&pd.consts, plan.const_pool.size()));
    B2X_CUDA(cudaMemcpy(pd.consts, plan.const_pool.data(), plan.const_pool.size(), cudaMemcpyHostToDevice));
  }
  return nullptr;
}

static PJRT_Error* LoadedExecutable_Execute(PJRT_LoadedExecutable_Execute_Args* a) {
  PJRT_LoadedExecutable* le = a->executable;
  B2X_CHECK_ARG(le, "the executable is null");
  if (le->deleted) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the executable has been deleted");
  const Plan& plan0 = le->core->plans[0];
  const size_t n_args = plan0.arg_types.size(), n_outs = plan0.outputs.size();
  // which local devices take part
  std::vector<int> locals;
  if (a->execute_device) {
    for (size_t i = 0; i < le->addressable.size(); i++) if (le->addressable[i] == a->execute_device) locals.push_back((int)i);
    B2X_CHECK_ARG(!locals.empty(), "execute_device is not one of the executable's addressable devices");
    B2X_CHECK_ARG(a->num_devices == 1, "num_devices must be 1 when execute_device is given");
  } else {
    if (a->num_devices != le->addressable.size())
      return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "Execute was given argument lists for " + std::to_string(a->num_devices) + " devices but the executable runs on " +
                                                              std::to_string(le->addressable.size()) + " addressable devices");
    for (size_t i = 0; i < le->addressable.size(); i++) locals.push_back((int)i);
  }
  if (a->num_args != n_args)
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the executable takes " + std::to_string(n_args) + " arguments but " + std::to_string(a->num_args) + " were passed");
  const int launch_id = a->options ? a->options->launch_id : 0;

  std::lock_guard<std::mutex> lk(le->mu);
  // validate arguments
  for (size_t k = 0; k < locals.size(); k++) {
    PJRT_Device* dev = le->addressable[locals[k]];
    for (size_t i = 0; i < n_args; i++) {
      PJRT_Buffer* b = a->argument_lists[k][i];
      B2X_CHECK_ARG(b, "argument " + std::to_string(i) + " is null");
      B2X_RETURN_IF_ERROR(check_live(b));
      if (b->device != dev)
        return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "argument " + std::to_string(i) + " lives on device " + std::to_string(b->device->desc.id) + " but replica " +
                                                                std::to_string(le->logical_ids[locals[k]].replica) + " runs on device " + std::to_string(dev->desc.id));
      if (b->type != plan0.arg_types[i])
        return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "argument " + std::to_string(i) + " has type " + b->type.str() + " but the program expects " + plan0.arg_types[i].str());
    }
  }
  // communicators for every replica group the plan uses (collective across processes: all of them execute the same plan)
  for (auto& s : plan0.steps) {
    if (s.coll_id < 0) continue;
    for (auto& g : s.replica_groups) {
      if (g.size() < 2) continue;
      std::vector<int> group;
      for (auto r : g) group.push_back(le->core->device_assignment[(size_t)r]);
      B2X_RETURN_IF_ERROR(le->client->nccl->ensure(group));
    }
  }

  struct PerLaunch { std::vector<void*> args, outs; std::vector<PJRT_Buffer*> out_bufs; PJRT_Error* err = nullptr; };
  std::vector<PerLaunch> launches(locals.size());
  for (size_t k = 0; k < locals.size(); k++) {
    const int li = locals[k];
    PJRT_Device* dev = le->addressable[li];
    PerLaunch& L = launches[k];
    if ((L.err = prepare_device_state(le, li))) break;
    cudaSetDevice(dev->cuda_ordinal);
    for (size_t i = 0; i < n_args; i++) {
      PJRT_Buffer* b = a->argument_lists[k][i];
      await_definition(b);
      if (b->ready) cudaStreamWaitEvent(dev->compute, b->ready, 0);
      L.args.push_back(b->ptr);
    }
    for (size_t o = 0; o < n_outs; o++) {
      PJRT_Buffer* ob = nullptr;
      if ((L.err = alloc_buffer(dev, plan0.outputs[o].type, dev->compute, &ob))) break;
      L.out_bufs.push_back(ob);
      L.outs.push_back(ob->ptr);
    }
    if (L.err) break;
  }
  PJRT_Error* first_err = nullptr;
  for (auto& L : launches) if (L.err && !first_err) first_err = L.err;

  // A launch that was poisoned fails on the host, before anything is enqueued.  Replicas of one execution meet in
  // collectives, so if any local replica is poisoned none of them may start: the others are aborted as well, which
  // keeps every GPU out of a collective that could never complete.
  if (!first_err) {
    int poisoned_k = -1;
    for (size_t k = 0; k < locals.size(); k++) {
      PJRT_Device* dev = le->addressable[locals[k]];
      std::lock_guard<std::mutex> pl(dev->poison_mu);
      auto it = dev->poisoned.find(launch_id);
      if (it != dev->poisoned.end()) {
        launches[k].err = make_error(it->second.first, it->second.second);
        dev->poisoned.erase(it);
        if (poisoned_k < 0) poisoned_k = (int)k;
      }
    }
    if (poisoned_k >= 0) {
      for (size_t k = 0; k < locals.size(); k++)
        if (!launches[k].err)
          launches[k].err = make_error(PJRT_Error_Code_ABORTED, "not launched: replica " + std::to_string(le->logical_ids[locals[poisoned_k]].replica) +
                                                                    " of this execution failed before launch (" + launches[poisoned_k].err->message + ")");
      first_err = launches[poisoned_k].err;
    }
  }
  if (!first_err) {
    std::unique_lock<std::mutex> coll_order;
    if (plan0.num_collectives > 0) coll_order = std::unique_lock<std::mutex>(le->client->collective_enqueue_mu);
    auto run_one = [&](size_t k) {
      const int li = locals[k];
      PJRT_Device* dev = le->addressable[li];
      PerLaunch& L = launches[k];
      std::lock_guard<std::mutex> dl(dev->launch_mu);
      L.err = run_plan(le, li, le->logical_ids[li].replica, L.args, L.outs);
    };
    if (locals.size() == 1) run_one(0);
    else {
      std::vector<std::thread> ts;
      for (size_t k = 0; k < locals.size(); k++) ts.emplace_back(run_one, k);
      for (auto& t : ts) t.join();
    }
    for (auto& L : launches) if (L.err && !first_err) first_err = L.err;
  }

  // completion events and output handles; a failed launch still fills every slot so that the caller can clean up
  for (size_t k = 0; k < locals.size(); k++) {
    PJRT_Device* dev = le->addressable[locals[k]];
    PerLaunch& L = launches[k];
    cudaSetDevice(dev->cuda_ordinal);
    const bool failed = L.err != nullptr;
    // Collectives that the compute stream does not wait for still belong to this execution: its outputs and its
    // completion event are recorded on the communication stream, behind everything the compute stream has queued.
    cudaStream_t done_stream = dev->compute;
    if (!failed && le->core->plans[0].has_detached_collectives) {
      cudaEvent_t join;
      cudaEventCreateWithFlags(&join, cudaEventDisableTiming);
      cudaEventRecord(join, dev->compute);
      cudaStreamWaitEvent(dev->comm, join, 0);
      cudaEventDestroy(join);
      done_stream = dev->comm;
    }
    for (size_t o = 0; o < n_outs; o++) {
      PJRT_Buffer* ob = o < L.out_bufs.size() ? L.out_bufs[o] : nullptr;
      if (!ob) {
        ob = new PJRT_Buffer();
        ob->client = le->client; ob->device = dev; ob->type = plan0.outputs[o].type; ob->dims = ob->type.dims;
        ob->pjrt_type = to_pjrt_type(ob->type.dtype); ob->owns = false;
      }
      if (failed) { ob->err_code = L.err->code; ob->err_msg = L.err->message; }
      else {
        // an output that no detached collective writes is final when the compute stream gets here (a loss can be read back
        // while the gradients' all-reduce is still running behind the next step)
        const bool on_comm = done_stream != dev->compute && (o >= plan0.out_in_detached.size() || plan0.out_in_detached[o]);
        cudaEventCreateWithFlags(&ob->ready, cudaEventDisableTiming);
        cudaEventRecord(ob->ready, on_comm ? done_stream : dev->compute);
      }
      if (a->output_lists && a->output_lists[k]) a->output_lists[k][o] = ob;
    }
    // Inputs are read by the enqueued kernels: their memory must not be reused before those finish.  Memory the plugin
    // owns is freed in compute-stream order, which covers every reader on that stream; a view of foreign memory needs
    // an event, and so does an argument that a detached collective reads or writes, because that happens on the
    // communication stream, which the compute stream never waits for.  (Only those: freeing a buffer with such an event
    // makes the compute stream wait for the collective, which then no longer runs behind the next step.)
    if (!failed) {
      for (size_t i = 0; i < n_args; i++) {
        PJRT_Buffer* b = a->argument_lists[k][i];
        const bool comm_readers = done_stream != dev->compute && (i >= plan0.arg_in_detached.size() || plan0.arg_in_detached[i]);
        if (!b->owns || comm_readers) {
          cudaEvent_t keep;
          cudaEventCreateWithFlags(&keep, cudaEventDisableTiming);
          cudaEventRecord(keep, comm_readers ? done_stream : dev->compute);
          std::lock_guard<std::mutex> bl(b->mu);
          // a buffer that is an argument step after step would otherwise collect one event per execution
          size_t kept = 0;
          for (auto ev : b->pending_reads) {
            if (cudaEventQuery(ev) == cudaSuccess) cudaEventDestroy(ev); else b->pending_reads[kept++] = ev;
          }
          b->pending_reads.resize(kept);
          b->pending_reads.push_back(keep);
        }
      }
    }
    if (a->device_complete_events) {
      PJRT_Event* ev = new PJRT_Event();
      if (failed) ev->set(L.err->code, L.err->message);
      else {
        cudaEvent_t ce;
        cudaEventCreateWithFlags(&ce, cudaEventDisableTiming);
        cudaEventRecord(ce, done_stream);
        PJRT_Device* d = dev;
        le->client->post({ce, dev->cuda_ordinal, ev, [d](PJRT_Error_Code* code, std::string* msg) {
                            report_expired_wait(d, code, msg);
                          }});
      }
      a->device_complete_events[k] = ev;
    }
  }
  le->client->executions++;
  // errors of individual launches are reported through the events and output buffers; the call itself fails only when
  // nothing could be set up
  PJRT_Error* ret = nullptr;
  for (auto& L : launches) {
    if (!L.err) continue;
    if (!a->device_complete_events && !ret) ret = L.err; else delete L.err;
  }
  return ret;
}

// ---- extensions -----------------------------------------------------------------------------------------------------------

static PJRT_Error* Ext_GetStream(PJRT_Get_Stream_For_External_Ready_Events_Args* a) {
  B2X_CHECK_ARG(a->device && a->device->addressable, "the device is not addressable");
  a->stream = (intptr_t)a->device->compute;
  return nullptr;
}
static PJRT_Error* Ext_WaitStream(PJRT_Wait_Until_Buffer_Ready_On_Stream_Args* a) {
  PJRT_Buffer* b = a->buffer;
  std::lock_guard<std::mutex> lk(b->mu);
  B2X_RETURN_IF_ERROR(check_live(b));
  await_definition(b);
  B2X_CUDA(cudaSetDevice(b->device->cuda_ordinal));
  if (b->ready) B2X_CUDA(cudaStreamWaitEvent((cudaStream_t)a->stream, b->ready, 0));
  return nullptr;
}

static int step_kernel_launches(const Step& s) {
  switch (s.kind) {
    case StepKind::ELEMENTWISE: return 1;
    case StepKind::WIDE: return 1;
    case StepKind::REDUCE: return s.wide ? 1 : reduce_launches(s.rA, s.rR, s.rB);
    case StepKind::GEMM: return s.g_split_f32 ? 2 : 1;
    case StepKind::ATTENTION: return 1;
    default: return 0;
  }
}

static PJRT_Error* Ext_StepTiming(B2X_StepTiming_Args* a) {
  PJRT_LoadedExecutable* le = a->executable;
  B2X_CHECK_ARG(le && a->device_index < le->per_device.size(), "bad executable or device index");
  std::lock_guard<std::mutex> lk(le->mu);
  PJRT_LoadedExecutable::PerDevice& pd = le->per_device[a->device_index];
  const Plan& plan = le->core->plans[0];
  if (le->step_labels.empty()) {
    for (auto& s : plan.steps) {
      const char* kind = s.kind == StepKind::GEMM ? (s.g_tensor_core ? "gemm_tc " : "gemm_simt ") : s.kind == StepKind::REDUCE ? "reduce " :
                         s.kind == StepKind::ELEMENTWISE ? "elementwise " : s.kind == StepKind::ATTENTION ? "attention " :
                         s.kind == StepKind::COPY ? "copy " : s.kind == StepKind::WIDE ? "wide " : "collective ";
      le->step_labels.push_back(std::string(kind) + s.label);
      le->step_flops.push_back(s.flops);
      le->step_bytes.push_back(s.bytes);
      le->step_launches.push_back(step_kernel_launches(s));
    }
    for (auto& l : le->step_labels) le->step_label_ptrs.push_back(l.c_str());
  }
  if (a->enable >= 0) pd.timing = a->enable != 0;
  a->num_steps = plan.steps.size();
  a->labels = le->step_label_ptrs.data();
  a->flops = le->step_flops.data();
  a->bytes = le->step_bytes.data();
  a->kernel_launches = le->step_launches.data();
  a->num_executions = 0;
  pd.step_ms.assign(plan.steps.size(), 0.f);
  if (a->collect) {
    B2X_CUDA(cudaSetDevice(le->addressable[a->device_index]->cuda_ordinal));
    for (auto& exec : pd.timed) {
      for (size_t i = 0; i < exec.size() && i < pd.step_ms.size(); i++) {
        float ms = 0.f;
        cudaError_t e = cudaEventSynchronize(exec[i].second);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, exec[i].first, exec[i].second);
        if (e != cudaSuccess) return cuda_error(e, "reading step timing events");
        pd.step_ms[i] += ms;
        cudaEventDestroy(exec[i].first);
        cudaEventDestroy(exec[i].second);
      }
      a->num_executions++;
    }
    pd.timed.clear();
  }
  a->step_ms = pd.step_ms.data();
  if (a->struct_size >= offsetof(B2X_StepTiming_Args, replay_host_ms) + sizeof(float) && a->replay > 0) {
    a->replay_ms = 0.f;
    a->replay_host_ms = 0.f;
    B2X_CHECK_ARG(plan.num_collectives == 0, "replay is for plans without collectives");
    B2X_CHECK_ARG(!pd.last_outs.empty() || !pd.last_args.empty(), "replay needs an execution launched while step timing was enabled");
    PJRT_Device* dev = le->addressable[a->device_index];
    std::lock_guard<std::mutex> dl(dev->launch_mu);
    B2X_CUDA(cudaSetDevice(dev->cuda_ordinal));
    const bool was = pd.timing;
    pd.timing = false;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    B2X_CUDA(cudaEventCreate(&e0));
    B2X_CUDA(cudaEventCreate(&e1));
    PJRT_Error* err = nullptr;
    cudaEventRecord(e0, dev->compute);
    const auto h0 = std::chrono::steady_clock::now();
    for (int i = 0; i < a->replay && !err; i++) err = run_plan(le, (int)a->device_index, le->logical_ids[a->device_index].replica, pd.last_args, pd.last_outs);
    a->replay_host_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - h0).count();
    cudaEventRecord(e1, dev->compute);
    cudaError_t e = cudaEventSynchronize(e1);
    if (e == cudaSuccess && !err) e = cudaEventElapsedTime(&a->replay_ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    pd.timing = was;
    if (err) return err;
    if (e != cudaSuccess) return cuda_error(e, "timing the replayed plan");
  }
  return nullptr;
}

// ---- asynchronous host-to-device transfer manager --------------------------------------------------------------------
// crates/ryft-pjrt/src/transfers.rs:39-349.  Buffers are allocated up front and handed out at any time; each carries a
// pending definition that completes when its last chunk (or a literal) has been enqueued on the transfer stream, or
// when an error is set on it.

struct PJRT_AsyncHostToDeviceTransferManager {
  PJRT_Client* client = nullptr;
  PJRT_Device* device = nullptr;
  struct Slot { PJRT_Buffer* buffer = nullptr; bool retrieved = false; bool finished = false; };
  std::vector<Slot> slots;
  std::mutex mu;
};

// Completes a buffer's pending definition: `code` OK means its contents are whatever the transfer stream holds now.
static void finish_definition(PJRT_Buffer* b, PJRT_Error_Code code, const std::string& msg) {
  std::shared_ptr<b2x_Definition> d = b->pending;
  if (!d) return;
  PJRT_Device* dev = b->device;
  cudaSetDevice(dev->cuda_ordinal);
  if (code == PJRT_Error_Code_OK) {
    cudaEventCreateWithFlags(&b->ready, cudaEventDisableTiming);
    cudaEventRecord(b->ready, dev->h2d);
  } else {
    b->err_code = code;
    b->err_msg = msg;
  }
  std::vector<PJRT_Event*> waiters;
  {
    std::lock_guard<std::mutex> lk(d->mu);
    d->done = true;
    waiters.swap(d->waiters);
  }
  d->cv.notify_all();
  for (PJRT_Event* ev : waiters) {
    if (code != PJRT_Error_Code_OK) { ev->set(code, msg); ev->unref(); continue; }
    cudaEvent_t e2;
    cudaEventCreateWithFlags(&e2, cudaEventDisableTiming);
    cudaEventRecord(e2, dev->h2d);
    b->client->post({e2, dev->cuda_ordinal, ev, nullptr});
    ev->unref();                                              // the waiter list's reference
  }
}

static PJRT_Error* Client_CreateBuffersForAsyncHostToDevice(PJRT_Client_CreateBuffersForAsyncHostToDevice_Args* a) {
  PJRT_Device* dev;
  B2X_RETURN_IF_ERROR(resolve_device(a->client, nullptr, a->memory, &dev));
  auto tm = std::make_unique<PJRT_AsyncHostToDeviceTransferManager>();
  tm->client = a->client;
  tm->device = dev;
  for (size_t i = 0; i < a->num_shape_specs; i++) {
    const PJRT_ShapeSpec& sp = a->shape_specs[i];
    TensorType t;
    t.dtype = from_pjrt_type(sp.element_type);
    PJRT_Error* err = nullptr;
    if (t.dtype == DType::INVALID) err = make_error(PJRT_Error_Code_UNIMPLEMENTED, "buffer element type " + std::to_string(sp.element_type) + " is not supported");
    t.dims.assign(sp.dims, sp.dims + sp.num_dims);
    for (auto d : t.dims) if (!err && d < 0) err = make_error(PJRT_Error_Code_INVALID_ARGUMENT, "negative dimension");
    PJRT_Buffer* b = nullptr;
    if (!err) err = alloc_buffer(dev, t, dev->h2d, &b);
    if (err) {
      for (auto& s : tm->slots) { s.buffer->pending.reset(); release_buffer_memory(s.buffer); delete s.buffer; }
      return err;
    }
    b->pending = std::make_shared<b2x_Definition>();
    tm->slots.push_back({b, false, false});
  }
  a->transfer_manager = tm.release();
  return nullptr;
}
static PJRT_Error* check_slot(PJRT_AsyncHostToDeviceTransferManager* tm, int index) {
  if (!tm) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null transfer manager");
  if (index < 0 || (size_t)index >= tm->slots.size())
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "buffer index " + std::to_string(index) + " is out of range for a transfer manager with " +
                                                            std::to_string(tm->slots.size()) + " buffers");
  return nullptr;
}
static PJRT_Error* TransferManager_Device(PJRT_AsyncHostToDeviceTransferManager_Device_Args* a) {
  if (!a->transfer_manager) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null transfer manager");
  a->device_out = a->transfer_manager->device;
  return nullptr;
}
static PJRT_Error* TransferManager_BufferCount(PJRT_AsyncHostToDeviceTransferManager_BufferCount_Args* a) {
  if (!a->transfer_manager) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null transfer manager");
  a->buffer_count = a->transfer_manager->slots.size();
  return nullptr;
}
static PJRT_Error* TransferManager_BufferSize(PJRT_AsyncHostToDeviceTransferManager_BufferSize_Args* a) {
  B2X_RETURN_IF_ERROR(check_slot(a->transfer_manager, a->buffer_index));
  a->buffer_size = a->transfer_manager->slots[a->buffer_index].buffer->bytes;
  return nullptr;
}
static PJRT_Error* TransferManager_RetrieveBuffer(PJRT_AsyncHostToDeviceTransferManager_RetrieveBuffer_Args* a) {
  B2X_RETURN_IF_ERROR(check_slot(a->transfer_manager, a->buffer_index));
  std::lock_guard<std::mutex> lk(a->transfer_manager->mu);
  auto& s = a->transfer_manager->slots[a->buffer_index];
  if (s.retrieved) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "buffer " + std::to_string(a->buffer_index) + " has already been retrieved");
  s.retrieved = true;
  a->buffer_out = s.buffer;
  return nullptr;
}
// Enqueues one copy into slot `index`; `last` completes the buffer.  Host memory must stay valid until `done` fires.
static PJRT_Error* transfer_into(PJRT_AsyncHostToDeviceTransferManager* tm, int index, const void* data, int64_t offset, int64_t size, bool last,
                                 PJRT_Event** done) {
  B2X_RETURN_IF_ERROR(check_slot(tm, index));
  std::lock_guard<std::mutex> lk(tm->mu);
  auto& s = tm->slots[index];
  if (s.finished) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "buffer " + std::to_string(index) + " has already received its last transfer");
  PJRT_Buffer* b = s.buffer;
  if (offset < 0 || size < 0 || (uint64_t)offset + (uint64_t)size > b->bytes)
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "transfer of " + std::to_string(size) + " bytes at offset " + std::to_string(offset) +
                                                            " exceeds the buffer size of " + std::to_string(b->bytes) + " bytes");
  PJRT_Device* dev = tm->device;
  B2X_CUDA(cudaSetDevice(dev->cuda_ordinal));
  if (size) B2X_CUDA(cudaMemcpyAsync((char*)b->ptr + offset, data, (size_t)size, cudaMemcpyHostToDevice, dev->h2d));
  PJRT_Event* ev = new PJRT_Event();
  cudaEvent_t ce;
  cudaEventCreateWithFlags(&ce, cudaEventDisableTiming);
  cudaEventRecord(ce, dev->h2d);
  tm->client->post({ce, dev->cuda_ordinal, ev, nullptr});
  *done = ev;
  if (last) { s.finished = true; finish_definition(b, PJRT_Error_Code_OK, ""); }
  return nullptr;
}
static PJRT_Error* TransferManager_TransferData(PJRT_AsyncHostToDeviceTransferManager_TransferData_Args* a) {
  return transfer_into(a->transfer_manager, a->buffer_index, a->data, a->offset, a->transfer_size, a->is_last_transfer, &a->done_with_h2d_transfer);
}
static PJRT_Error* TransferManager_TransferLiteral(PJRT_AsyncHostToDeviceTransferManager_TransferLiteral_Args* a) {
  B2X_RETURN_IF_ERROR(check_slot(a->transfer_manager, a->buffer_index));
  PJRT_Buffer* b = a->transfer_manager->slots[a->buffer_index].buffer;
  // the literal must have the buffer's own shape and element type; it is the buffer's only and last transfer
  if (from_pjrt_type(a->shape_element_type) != b->type.dtype || a->shape_num_dims != b->dims.size() ||
      !std::equal(b->dims.begin(), b->dims.end(), a->shape_dims))
    return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the literal's shape does not match buffer " + std::to_string(a->buffer_index));
  return transfer_into(a->transfer_manager, a->buffer_index, a->data, 0, (int64_t)b->bytes, true, &a->done_with_h2d_transfer);
}
static PJRT_Error* TransferManager_SetBufferError(PJRT_AsyncHostToDeviceTransferManager_SetBufferError_Args* a) {
  B2X_RETURN_IF_ERROR(check_slot(a->transfer_manager, a->buffer_index));
  std::lock_guard<std::mutex> lk(a->transfer_manager->mu);
  auto& s = a->transfer_manager->slots[a->buffer_index];
  if (s.finished) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "buffer " + std::to_string(a->buffer_index) + " is already complete");
  s.finished = true;
  finish_definition(s.buffer, a->error_code == PJRT_Error_Code_OK ? PJRT_Error_Code_INTERNAL : a->error_code,
                    std::string(a->error_message ? a->error_message : "", a->error_message_size));
  return nullptr;
}
static PJRT_Error* TransferManager_AddMetadata(PJRT_AsyncHostToDeviceTransferManager_AddMetadata_Args* a) {
  if (!a->transfer_manager) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null transfer manager");
  return nullptr;   // metadata only annotates profiler traces in XLA; there is nothing to attach it to here
}
static PJRT_Error* TransferManager_Destroy(PJRT_AsyncHostToDeviceTransferManager_Destroy_Args* a) {
  PJRT_AsyncHostToDeviceTransferManager* tm = a->transfer_manager;
  if (!tm) return nullptr;
  for (auto& s : tm->slots) {
    // a buffer that never got its last transfer becomes an error buffer, so that nobody waits for it forever
    if (!s.finished) finish_definition(s.buffer, PJRT_Error_Code_ABORTED, "the transfer manager was destroyed before the buffer's last transfer");
    if (!s.retrieved) { release_buffer_memory(s.buffer); delete s.buffer; }
  }
  delete tm;
  return nullptr;
}

// ---- layouts extension ------------------------------------------------------------------------------------------------
// crates/ryft-pjrt/src/extensions/layouts.rs: default layout of a buffer / executable parameter / result.

static PJRT_Layouts_MemoryLayout descending_layout(size_t rank) {
  PJRT_Layouts_MemoryLayout l;
  for (size_t i = 0; i < rank; i++) l.minor_to_major.push_back((int64_t)(rank - 1 - i));
  return l;
}
static PJRT_Error* Layouts_Destroy(PJRT_Layouts_MemoryLayout_Destroy_Args* a) {
  delete a->layout;
  return nullptr;
}
static void Layouts_DeleteSerialized(PJRT_Layouts_SerializedLayout* s) { delete s; }
static PJRT_Error* Layouts_Serialize(PJRT_Layouts_MemoryLayout_Serialize_Args* a) {
  if (!a->layout) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null layout");
  auto* s = new PJRT_Layouts_SerializedLayout();
  s->text = "{";
  for (size_t i = 0; i < a->layout->minor_to_major.size(); i++) s->text += (i ? "," : "") + std::to_string(a->layout->minor_to_major[i]);
  s->text += "}";
  a->serialized_bytes = s->text.data();
  a->serialized_bytes_size = s->text.size();
  a->serialized_layout = s;
  a->serialized_layout_deleter = Layouts_DeleteSerialized;
  return nullptr;
}
static PJRT_Error* Layouts_ClientDefault(PJRT_Layouts_PJRT_Client_GetDefaultLayout_Args* a) {
  if (from_pjrt_type(a->element_type) == DType::INVALID) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "unsupported element type");
  a->layout = new PJRT_Layouts_MemoryLayout(descending_layout(a->num_dims));
  return nullptr;
}
static PJRT_Error* Layouts_BufferLayout(PJRT_Layouts_PJRT_Buffer_MemoryLayout_Args* a) {
  if (!a->buffer) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null buffer");
  a->layout = new PJRT_Layouts_MemoryLayout(descending_layout(a->buffer->dims.size()));
  return nullptr;
}
static void fill_executable_layouts(b2x_ExecutableCore& c) {
  if (!c.param_layout_ptrs.empty() || !c.out_layout_ptrs.empty() || c.plans.empty()) return;
  const b2x::Plan& p = c.plans[0];
  for (auto& t : p.arg_types) c.param_layouts.push_back(descending_layout(t.dims.size()));
  for (size_t r : c.out_ranks) c.out_layouts.push_back(descending_layout(r));
  for (auto& l : c.param_layouts) c.param_layout_ptrs.push_back(&l);
  for (auto& l : c.out_layouts) c.out_layout_ptrs.push_back(&l);
}
static std::mutex g_layouts_mu;
static PJRT_Error* Layouts_ExecutableOutputs(PJRT_Layouts_PJRT_Executable_GetOutputLayouts_Args* a) {
  std::lock_guard<std::mutex> lk(g_layouts_mu);
  fill_executable_layouts(*a->executable->core);
  a->num_outputs = a->executable->core->out_layout_ptrs.size();
  a->layouts = a->executable->core->out_layout_ptrs.data();
  return nullptr;
}
static PJRT_Error* Layouts_ExecutableParameters(PJRT_Layouts_PJRT_Executable_GetParameterLayouts_Args* a) {
  std::lock_guard<std::mutex> lk(g_layouts_mu);
  fill_executable_layouts(*a->executable->core);
  a->num_parameters = a->executable->core->param_layout_ptrs.size();
  a->layouts = a->executable->core->param_layout_ptrs.data();
  return nullptr;
}

// ---- memory-descriptions extension ------------------------------------------------------------------------------------
struct PJRT_MemoryDescription { const char* kind; size_t kind_size; int kind_id; };
static const PJRT_MemoryDescription kDeviceMemoryDescription = {"device", 6, kDeviceMemoryKindId};
static const PJRT_MemoryDescription* const kMemoryDescriptions[1] = {&kDeviceMemoryDescription};
static PJRT_Error* MemDesc_ForDevice(PJRT_DeviceDescription_MemoryDescriptions_Args* a) {
  if (!a->device_description) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null device description");
  a->memory_descriptions = kMemoryDescriptions;
  a->num_memory_descriptions = 1;
  a->default_memory_index = 0;
  return nullptr;
}
static PJRT_Error* MemDesc_Kind(PJRT_MemoryDescription_Kind_Args* a) {
  if (!a->memory_description) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null memory description");
  a->kind = a->memory_description->kind;
  a->kind_size = a->memory_description->kind_size;
  a->kind_id = a->memory_description->kind_id;
  return nullptr;
}

// ---- ABI-version extension -----------------------------------------------------------------------------------------------
// A version is (platform id, serialization generation, SM architecture).  The runtime reads executables of its own
// generation or older, built for its own architecture.
static constexpr uint64_t kSerializationGeneration = 1;  // the "B2XE1" container written by serialize_core
static constexpr uint64_t kSmArchitecture = 100;
struct AbiVersionValue { uint64_t platform = B2X_ABI_PLATFORM_ID, generation = kSerializationGeneration, sm = kSmArchitecture; };
struct PJRT_RuntimeAbiVersion { AbiVersionValue v; };
struct PJRT_ExecutableAbiVersion { AbiVersionValue v; };
static void abi_put_varint(std::string* s, uint64_t v) { while (v >= 0x80) { s->push_back((char)(v | 0x80)); v >>= 7; } s->push_back((char)v); }
static bool abi_get_varint(const unsigned char*& p, const unsigned char* end, uint64_t* out) {
  uint64_t v = 0;
  for (int shift = 0; shift < 64 && p < end; shift += 7) {
    unsigned char b = *p++;
    v |= (uint64_t)(b & 0x7f) << shift;
    if (!(b & 0x80)) { *out = v; return true; }
  }
  return false;
}
static std::string abi_to_proto(const AbiVersionValue& v) {
  std::string payload, s;
  abi_put_varint(&payload, v.generation); abi_put_varint(&payload, v.sm);
  abi_put_varint(&s, (1 << 3) | 0); abi_put_varint(&s, v.platform);
  abi_put_varint(&s, (2 << 3) | 2); abi_put_varint(&s, payload.size()); s += payload;
  return s;
}
static PJRT_Error* abi_from_proto(const char* data, size_t size, AbiVersionValue* out) {
  if (!data && size) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null ABI version proto");
  const unsigned char* p = (const unsigned char*)data; const unsigned char* end = p + size;
  AbiVersionValue v; v.platform = 0; bool have_payload = false;
  while (p < end) {
    uint64_t tag, n;
    if (!abi_get_varint(p, end, &tag)) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "malformed ABI version proto");
    int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (wire == 0) {
      if (!abi_get_varint(p, end, &n)) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "malformed ABI version proto");
      if (field == 1) v.platform = n;
    } else if (wire == 2) {
      if (!abi_get_varint(p, end, &n) || n > (uint64_t)(end - p)) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "malformed ABI version proto");
      if (field == 2) {
        const unsigned char* q = p; const unsigned char* qe = p + n;
        if (!abi_get_varint(q, qe, &v.generation) || !abi_get_varint(q, qe, &v.sm) || q != qe)
          return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the ABI version payload was not written by this plugin");
        have_payload = true;
      }
      p += n;
    } else if (wire == 1) { if (end - p < 8) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "malformed ABI version proto"); p += 8; }
    else if (wire == 5) { if (end - p < 4) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "malformed ABI version proto"); p += 4; }
    else return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "malformed ABI version proto");
  }
  if (v.platform != B2X_ABI_PLATFORM_ID) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the ABI version belongs to another platform");
  if (!have_payload) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "the ABI version proto has no version payload");
  *out = v;
  return nullptr;
}
static PJRT_Error* abi_check(const AbiVersionValue& runtime, const AbiVersionValue& other, bool other_is_executable) {
  if (runtime.platform != other.platform) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "ABI versions of different platforms");
  if (runtime.sm != other.sm)
    return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "built for SM " + std::to_string(other.sm) + ", this runtime drives SM " + std::to_string(runtime.sm));
  if (other_is_executable ? other.generation > runtime.generation : other.generation != runtime.generation)
    return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "serialization generation " + std::to_string(other.generation) +
                                                               " does not fit this runtime's generation " + std::to_string(runtime.generation));
  return nullptr;
}
static void delete_blob_proto(PJRT_SerializedProto* p) { delete (SerializedBlob*)p; }
template <typename Args> static PJRT_Error* abi_emit_proto(Args* a) {
  if (!a->abi_version) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null ABI version");
  SerializedBlob* b = new SerializedBlob{abi_to_proto(a->abi_version->v)};
  a->serialized_proto = b->bytes.data(); a->serialized_proto_size = b->bytes.size();
  a->serialized_proto_holder = (PJRT_SerializedProto*)b; a->serialized_proto_deleter = delete_blob_proto;
  return nullptr;
}
static PJRT_Error* Abi_ClientRuntime(PJRT_Client_RuntimeAbiVersion_Args* a) {
  if (!a->client) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null client");
  a->abi_version = new PJRT_RuntimeAbiVersion(); return nullptr;
}
static PJRT_Error* Abi_Executable(PJRT_Executable_GetAbiVersion_Args* a) {
  if (!a->executable) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null executable");
  a->abi_version = new PJRT_ExecutableAbiVersion(); return nullptr;
}
static PJRT_Error* Abi_RuntimeDestroy(PJRT_RuntimeAbiVersion_Destroy_Args* a) { delete a->abi_version; return nullptr; }
static PJRT_Error* Abi_ExecutableDestroy(PJRT_ExecutableAbiVersion_Destroy_Args* a) { delete a->abi_version; return nullptr; }
static PJRT_Error* Abi_RuntimeWithRuntime(PJRT_RuntimeAbiVersion_IsCompatibleWithRuntime_Args* a) {
  if (!a->abi_version || !a->other_abi_version) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null ABI version");
  return abi_check(a->abi_version->v, a->other_abi_version->v, false);
}
static PJRT_Error* Abi_RuntimeWithExecutable(PJRT_RuntimeAbiVersion_IsCompatibleWithExecutable_Args* a) {
  if (!a->abi_version || !a->executable_abi_version) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null ABI version");
  return abi_check(a->abi_version->v, a->executable_abi_version->v, true);
}
static PJRT_Error* Abi_RuntimeToProto(PJRT_RuntimeAbiVersion_ToProto_Args* a) { return abi_emit_proto(a); }
static PJRT_Error* Abi_ExecutableToProto(PJRT_ExecutableAbiVersion_ToProto_Args* a) { return abi_emit_proto(a); }
static PJRT_Error* Abi_RuntimePlatform(PJRT_RuntimeAbiVersion_PlatformId_Args* a) {
  if (!a->abi_version) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null ABI version");
  a->platform_id = a->abi_version->v.platform; return nullptr;
}
static PJRT_Error* Abi_ExecutablePlatform(PJRT_ExecutableAbiVersion_PlatformId_Args* a) {
  if (!a->abi_version) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "null ABI version");
  a->platform_id = a->abi_version->v.platform; return nullptr;
}
static PJRT_Error* Abi_RuntimeFromProto(PJRT_RuntimeAbiVersion_FromProto_Args* a) {
  AbiVersionValue v;
  B2X_RETURN_IF_ERROR(abi_from_proto(a->serialized_proto, a->serialized_proto_size, &v));
  a->abi_version = new PJRT_RuntimeAbiVersion{v}; return nullptr;
}
static PJRT_Error* Abi_ExecutableFromProto(PJRT_ExecutableAbiVersion_FromProto_Args* a) {
  AbiVersionValue v;
  B2X_RETURN_IF_ERROR(abi_from_proto(a->serialized_proto, a->serialized_proto_size, &v));
  a->abi_version = new PJRT_ExecutableAbiVersion{v}; return nullptr;
}

// ---- table ----------------------------------------------------------------------------------------------------------------

static PJRT_Api make_api() {
  static PJRT_Stream_Extension stream_ext;
  static B2X_StepTiming_Extension timing_ext;
  static PJRT_Layouts_Extension layouts_ext;
  static PJRT_MemoryDescriptions_Extension memdesc_ext;
  static PJRT_AbiVersion_Extension abi_ext;
  memset(&abi_ext, 0, sizeof(abi_ext));
  abi_ext.base.struct_size = sizeof(abi_ext);
  abi_ext.base.extension_type = PJRT_Extension_Type_AbiVersion;
  abi_ext.base.next = nullptr;
  abi_ext.PJRT_Client_RuntimeAbiVersion = Abi_ClientRuntime;
  abi_ext.PJRT_Executable_GetAbiVersion = Abi_Executable;
  abi_ext.PJRT_RuntimeAbiVersion_Destroy = Abi_RuntimeDestroy;
  abi_ext.PJRT_RuntimeAbiVersion_IsCompatibleWithRuntime = Abi_RuntimeWithRuntime;
  abi_ext.PJRT_RuntimeAbiVersion_IsCompatibleWithExecutable = Abi_RuntimeWithExecutable;
  abi_ext.PJRT_RuntimeAbiVersion_ToProto = Abi_RuntimeToProto;
  abi_ext.PJRT_RuntimeAbiVersion_PlatformId = Abi_RuntimePlatform;
  abi_ext.PJRT_ExecutableAbiVersion_Destroy = Abi_ExecutableDestroy;
  abi_ext.PJRT_ExecutableAbiVersion_ToProto = Abi_ExecutableToProto;
  abi_ext.PJRT_ExecutableAbiVersion_PlatformId = Abi_ExecutablePlatform;
  abi_ext.PJRT_RuntimeAbiVersion_FromProto = Abi_RuntimeFromProto;
  abi_ext.PJRT_ExecutableAbiVersion_FromProto = Abi_ExecutableFromProto;
  memset(&memdesc_ext, 0, sizeof(memdesc_ext));
  memdesc_ext.base.struct_size = sizeof(memdesc_ext);
  memdesc_ext.base.extension_type = PJRT_Extension_Type_MemoryDescriptions;
  memdesc_ext.base.next = &abi_ext.base;
  memdesc_ext.PJRT_DeviceDescription_MemoryDescriptions = MemDesc_ForDevice;
  memdesc_ext.PJRT_MemoryDescription_Kind = MemDesc_Kind;
  memset(&layouts_ext, 0, sizeof(layouts_ext));
  layouts_ext.base.struct_size = sizeof(layouts_ext);
  layouts_ext.base.extension_type = PJRT_Extension_Type_Layouts;
  layouts_ext.base.next = &memdesc_ext.base;
  layouts_ext.PJRT_Layouts_MemoryLayout_Destroy = Layouts_Destroy;
  layouts_ext.PJRT_Layouts_MemoryLayout_Serialize = Layouts_Serialize;
  layouts_ext.PJRT_Layouts_PJRT_Client_GetDefaultLayout = Layouts_ClientDefault;
  layouts_ext.PJRT_Layouts_PJRT_Buffer_MemoryLayout = Layouts_BufferLayout;
  layouts_ext.PJRT_Layouts_PJRT_Executable_GetOutputLayouts = Layouts_ExecutableOutputs;
  layouts_ext.PJRT_Layouts_PJRT_Executable_GetParameterLayouts = Layouts_ExecutableParameters;
  memset(&stream_ext, 0, sizeof(stream_ext));
  memset(&timing_ext, 0, sizeof(timing_ext));
  timing_ext.base.struct_size = sizeof(timing_ext);
  timing_ext.base.extension_type = B2X_Extension_Type_StepTiming;
  timing_ext.base.next = &layouts_ext.base;
  timing_ext.step_timing = Ext_StepTiming;
  stream_ext.base.struct_size = sizeof(stream_ext);
  stream_ext.base.extension_type = PJRT_Extension_Type_Stream;
  stream_ext.base.next = &timing_ext.base;
  stream_ext.get_stream = Ext_GetStream;
  stream_ext.wait_stream = Ext_WaitStream;
  PJRT_Api api;
  memset(&api, 0, sizeof(api));
  api.struct_size = sizeof(PJRT_Api);
  api.extension_start = &stream_ext.base;
  api.pjrt_api_version.struct_size = sizeof(PJRT_Api_Version);
  api.pjrt_api_version.major_version = PJRT_API_MAJOR;
  api.pjrt_api_version.minor_version = PJRT_API_MINOR;
#define B2X_SET(name, fn) api.PJRT_##name = fn
  B2X_SET(Error_Destroy, Error_Destroy); B2X_SET(Error_Message, Error_Message); B2X_SET(Error_GetCode, Error_GetCode);
  B2X_SET(Error_ForEachPayload, Error_ForEachPayload);
  B2X_SET(Plugin_Initialize, Plugin_Initialize); B2X_SET(Plugin_Attributes, Plugin_Attributes);
  B2X_SET(Event_Create, Event_Create); B2X_SET(Event_Set, Event_Set); B2X_SET(Event_Destroy, Event_Destroy);
  B2X_SET(Event_IsReady, Event_IsReady); B2X_SET(Event_Error, Event_Error); B2X_SET(Event_Await, Event_Await); B2X_SET(Event_OnReady, Event_OnReady);
  B2X_SET(Client_Create, Client_Create); B2X_SET(Client_Destroy, Client_Destroy); B2X_SET(Client_PlatformName, Client_PlatformName);
  B2X_SET(Client_ProcessIndex, Client_ProcessIndex); B2X_SET(Client_PlatformVersion, Client_PlatformVersion);
  B2X_SET(Client_Devices, Client_Devices); B2X_SET(Client_AddressableDevices, Client_AddressableDevices);
  B2X_SET(Client_LookupDevice, Client_LookupDevice); B2X_SET(Client_LookupAddressableDevice, Client_LookupAddressableDevice);
  B2X_SET(Client_AddressableMemories, Client_AddressableMemories); B2X_SET(Client_Compile, Client_Compile);
  B2X_SET(Client_DefaultDeviceAssignment, Client_DefaultDeviceAssignment); B2X_SET(Client_BufferFromHostBuffer, Client_BufferFromHostBuffer);
  B2X_SET(Client_UpdateGlobalProcessInfo, Client_UpdateGlobalProcessInfo); B2X_SET(Client_DmaMap, Client_DmaMap); B2X_SET(Client_DmaUnmap, Client_DmaUnmap);
  B2X_SET(Client_CreateBuffersForAsyncHostToDevice, Client_CreateBuffersForAsyncHostToDevice);
  B2X_SET(AsyncHostToDeviceTransferManager_Device, TransferManager_Device); B2X_SET(AsyncHostToDeviceTransferManager_BufferCount, TransferManager_BufferCount);
  B2X_SET(AsyncHostToDeviceTransferManager_BufferSize, TransferManager_BufferSize);
  B2X_SET(AsyncHostToDeviceTransferManager_RetrieveBuffer, TransferManager_RetrieveBuffer);
  B2X_SET(AsyncHostToDeviceTransferManager_TransferData, TransferManager_TransferData);
  B2X_SET(AsyncHostToDeviceTransferManager_TransferLiteral, TransferManager_TransferLiteral);
  B2X_SET(AsyncHostToDeviceTransferManager_SetBufferError, TransferManager_SetBufferError);
  B2X_SET(AsyncHostToDeviceTransferManager_AddMetadata, TransferManager_AddMetadata);
  B2X_SET(AsyncHostToDeviceTransferManager_Destroy, TransferManager_Destroy);
  B2X_SET(Client_CreateUninitializedBuffer, Client_CreateUninitializedBuffer); B2X_SET(Client_CreateViewOfDeviceBuffer, Client_CreateViewOfDeviceBuffer);
  B2X_SET(Client_CreateErrorBuffer, Client_CreateErrorBuffer); B2X_SET(Client_Load, Client_Load);
  B2X_SET(DeviceDescription_Id, DeviceDescription_Id); B2X_SET(DeviceDescription_ProcessIndex, DeviceDescription_ProcessIndex);
  B2X_SET(DeviceDescription_Attributes, DeviceDescription_Attributes); B2X_SET(DeviceDescription_Kind, DeviceDescription_Kind);
  B2X_SET(DeviceDescription_DebugString, DeviceDescription_DebugString); B2X_SET(DeviceDescription_ToString, DeviceDescription_ToString);
  B2X_SET(Device_GetDescription, Device_GetDescription); B2X_SET(Device_IsAddressable, Device_IsAddressable);
  B2X_SET(Device_LocalHardwareId, Device_LocalHardwareId); B2X_SET(Device_AddressableMemories, Device_AddressableMemories);
  B2X_SET(Device_DefaultMemory, Device_DefaultMemory); B2X_SET(Device_MemoryStats, Device_MemoryStats);
  B2X_SET(Device_GetAttributes, Device_GetAttributes); B2X_SET(Device_PoisonExecution, Device_PoisonExecution);
  B2X_SET(Memory_Id, Memory_Id); B2X_SET(Memory_Kind, Memory_Kind); B2X_SET(Memory_Kind_Id, Memory_Kind_Id);
  B2X_SET(Memory_DebugString, Memory_DebugString); B2X_SET(Memory_ToString, Memory_ToString); B2X_SET(Memory_AddressableByDevices, Memory_AddressableByDevices);
  B2X_SET(Executable_Destroy, Executable_Destroy); B2X_SET(Executable_Name, Executable_Name); B2X_SET(Executable_NumReplicas, Executable_NumReplicas);
  B2X_SET(Executable_NumPartitions, Executable_NumPartitions); B2X_SET(Executable_NumOutputs, Executable_NumOutputs);
  B2X_SET(Executable_SizeOfGeneratedCodeInBytes, Executable_SizeOfGeneratedCodeInBytes); B2X_SET(Executable_GetCostAnalysis, Executable_GetCostAnalysis);
  B2X_SET(Executable_OutputMemoryKinds, Executable_OutputMemoryKinds); B2X_SET(Executable_ParameterMemoryKinds, Executable_ParameterMemoryKinds);
  B2X_SET(Executable_OptimizedProgram, Executable_OptimizedProgram); B2X_SET(Executable_Serialize, Executable_Serialize);
  B2X_SET(Executable_GetCompileOptions, Executable_GetCompileOptions); B2X_SET(Executable_OutputElementTypes, Executable_OutputElementTypes);
  B2X_SET(Executable_OutputDimensions, Executable_OutputDimensions); B2X_SET(Executable_Fingerprint, Executable_Fingerprint);
  B2X_SET(Executable_GetCompiledMemoryStats, Executable_GetCompiledMemoryStats); B2X_SET(Executable_DeserializeAndLoad, Executable_DeserializeAndLoad);
  B2X_SET(LoadedExecutable_Destroy, LoadedExecutable_Destroy); B2X_SET(LoadedExecutable_GetExecutable, LoadedExecutable_GetExecutable);
  B2X_SET(LoadedExecutable_AddressableDevices, LoadedExecutable_AddressableDevices);
  B2X_SET(LoadedExecutable_AddressableDeviceLogicalIds, LoadedExecutable_AddressableDeviceLogicalIds);
  B2X_SET(LoadedExecutable_GetDeviceAssignment, LoadedExecutable_GetDeviceAssignment);
  B2X_SET(LoadedExecutable_Delete, LoadedExecutable_Delete); B2X_SET(LoadedExecutable_IsDeleted, LoadedExecutable_IsDeleted);
  B2X_SET(LoadedExecutable_Execute, LoadedExecutable_Execute); B2X_SET(LoadedExecutable_Fingerprint, LoadedExecutable_Fingerprint);
  B2X_SET(ExecuteContext_Create, ExecuteContext_Create); B2X_SET(ExecuteContext_Destroy, ExecuteContext_Destroy);
  B2X_SET(Buffer_Destroy, Buffer_Destroy); B2X_SET(Buffer_ElementType, Buffer_ElementType); B2X_SET(Buffer_Dimensions, Buffer_Dimensions);
  B2X_SET(Buffer_UnpaddedDimensions, Buffer_UnpaddedDimensions); B2X_SET(Buffer_DynamicDimensionIndices, Buffer_DynamicDimensionIndices);
  B2X_SET(Buffer_GetMemoryLayout, Buffer_GetMemoryLayout); B2X_SET(Buffer_OnDeviceSizeInBytes, Buffer_OnDeviceSizeInBytes);
  B2X_SET(Buffer_Device, Buffer_Device); B2X_SET(Buffer_Memory, Buffer_Memory); B2X_SET(Buffer_Delete, Buffer_Delete);
  B2X_SET(Buffer_IsDeleted, Buffer_IsDeleted); B2X_SET(Buffer_CopyToDevice, Buffer_CopyToDevice); B2X_SET(Buffer_CopyToMemory, Buffer_CopyToMemory);
  B2X_SET(Buffer_ToHostBuffer, Buffer_ToHostBuffer); B2X_SET(Buffer_CopyRawToHost, Buffer_CopyRawToHost); B2X_SET(Buffer_IsOnCpu, Buffer_IsOnCpu);
  B2X_SET(Buffer_ReadyEvent, Buffer_ReadyEvent); B2X_SET(Buffer_UnsafePointer, Buffer_UnsafePointer);
  B2X_SET(Buffer_IncreaseExternalReferenceCount, Buffer_IncRef); B2X_SET(Buffer_DecreaseExternalReferenceCount, Buffer_DecRef);
  B2X_SET(Buffer_OpaqueDeviceMemoryDataPointer, Buffer_OpaqueDeviceMemoryDataPointer); B2X_SET(Buffer_Bitcast, Buffer_Bitcast);
#undef B2X_SET
  return api;
}

extern "C" __attribute__((visibility("default"))) const PJRT_Api* GetPjrtApi(void) {
  static const PJRT_Api api = make_api();
  return &api;
}
