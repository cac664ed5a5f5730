// Runtime objects behind the opaque PJRT handles (layouts of the handles' users: include/b2x_pjrt_c_api.h).
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../../include/b2x_pjrt_c_api.h"
#include "plan.h"

struct PJRT_Error {
  PJRT_Error_Code code;
  std::string message;
};

namespace b2x {
PJRT_Error* make_error(PJRT_Error_Code code, const std::string& msg);
PJRT_Error* cuda_error(cudaError_t e, const char* what);
#define B2X_CUDA(expr)                                                      \
  do {                                                                      \
    cudaError_t _e = (expr);                                                \
    if (_e != cudaSuccess) return ::b2x::cuda_error(_e, #expr);             \
  } while (0)
#define B2X_RETURN_IF_ERROR(expr)             \
  do {                                        \
    PJRT_Error* _err = (expr);                \
    if (_err) return _err;                    \
  } while (0)
}  // namespace b2x

// Host-visible completion object.  Thread-safe; callbacks run exactly once, on the thread that completes the event
// or immediately on the registering thread if it is already complete (reference expectations:
// crates/ryft-pjrt/src/events.rs:89-144, tests :566-648).
struct PJRT_Event {
  std::mutex mu;
  std::condition_variable cv;
  bool ready = false;
  PJRT_Error_Code code = PJRT_Error_Code_OK;
  std::string message;
  std::vector<std::pair<PJRT_Event_OnReadyCallback, void*>> callbacks;
  std::atomic<int> refs{1};  // the handle owner + internal holders (poller queue)

  void set(PJRT_Error_Code c, const std::string& msg);
  void ref() { refs.fetch_add(1); }
  void unref() { if (refs.fetch_sub(1) == 1) delete this; }
};

struct PJRT_Client;

struct PJRT_DeviceDescription {
  int id = 0;             // global device id
  int process_index = 0;
  int local_hardware_id = -1;
  std::string kind, debug_string, to_string;
  std::vector<PJRT_NamedValue> attributes;
  std::vector<std::string> attr_names;
  std::vector<std::vector<int64_t>> attr_lists;
  std::vector<std::string> attr_strings;
};

struct PJRT_Memory {
  int id = 0;
  std::string kind = "device", debug_string, to_string;
  PJRT_Device* device = nullptr;
  std::vector<PJRT_Device*> devices;
};

struct PJRT_Device {
  PJRT_Client* client = nullptr;
  PJRT_DeviceDescription desc;
  bool addressable = false;
  int cuda_ordinal = -1;
  cudaStream_t compute = nullptr, h2d = nullptr, d2h = nullptr, comm = nullptr;
  PJRT_Memory* memory = nullptr;
  std::vector<PJRT_Memory*> memories;
  int32_t* status_host = nullptr;  // pinned, mapped: kernels write a non-zero code when a bounded wait expires
  int32_t* status_dev = nullptr;
  std::atomic<int64_t> bytes_in_use{0}, peak_bytes{0}, num_allocs{0};
  std::mutex poison_mu;
  std::map<int, std::pair<PJRT_Error_Code, std::string>> poisoned;  // launch_id -> error
  std::mutex launch_mu;  // serialises enqueues of whole executions on this device
  // Pinned staging blocks for small device-to-host reads: a copy into pageable host memory makes cudaMemcpyAsync wait
  // for the stream, so the caller would sit out the whole step it is reading a scalar from.
  std::mutex staging_mu;
  std::vector<void*> staging_free;   // blocks of kStagingBlock bytes
  static constexpr size_t kStagingBlock = 64 << 10;
  // Device blocks of destroyed host-upload buffers, kept with the event behind their last use.  A training loop uploads a
  // buffer of the same size every step from a stream of its own; the stream-ordered pool can hand a block freed on the
  // compute stream to that stream only once the free has retired, and otherwise grows (milliseconds, in the middle of a
  // run).  An upload first looks here for a block of its size whose event has completed.
  struct RecycledBlock { void* ptr; size_t bytes; cudaEvent_t last_use; };
  std::mutex recycle_mu;
  std::vector<RecycledBlock> recycled;
  static constexpr size_t kMaxRecycled = 8;
  static constexpr size_t kMinRecycledBytes = 1 << 20;
  static constexpr size_t kMaxRecycledBytes = 1ull << 30;
};

// Definition of a buffer that is filled after it was created (asynchronous host-to-device transfers): consumers that
// need the contents block until the last chunk has been enqueued (or an error set); ready events register as waiters.
struct b2x_Definition {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::vector<struct PJRT_Event*> waiters;
};

struct PJRT_Buffer {
  std::shared_ptr<b2x_Definition> pending;   // null for buffers that are defined when they are created
  PJRT_Client* client = nullptr;
  PJRT_Device* device = nullptr;
  b2x::TensorType type;
  std::vector<int64_t> dims;
  void* ptr = nullptr;
  size_t bytes = 0;
  bool owns = true;           // false for views of foreign device memory
  bool from_host = false;     // created by a host-to-device upload: its block is recycled for the next upload of that size
  bool deleted = false;
  std::function<void()> on_delete;
  cudaEvent_t ready = nullptr;      // recorded on the producing stream
  PJRT_Event* definition_error = nullptr;  // set for error buffers
  PJRT_Error_Code err_code = PJRT_Error_Code_OK;
  std::string err_msg;
  std::vector<cudaEvent_t> pending_reads;  // D2H copies still in flight on the d2h stream
  std::mutex mu;
  std::atomic<int> ext_refs{0};
  std::vector<int64_t> minor_to_major;
  PJRT_Buffer_Type pjrt_type = PJRT_Buffer_Type_INVALID;
};

struct PJRT_Layouts_MemoryLayout {
  std::vector<int64_t> minor_to_major;   // always {rank-1, ..., 0}: every buffer is dense, major to minor
};
struct PJRT_Layouts_SerializedLayout {
  std::string text;                      // rendered form, e.g. "{2,1,0}"
};

struct PJRT_Executable {
  std::shared_ptr<struct b2x_ExecutableCore> core;
};

namespace b2x { struct NcclComms; }

struct b2x_ExecutableCore {
  std::string name;
  std::string source;               // MLIR text as compiled
  std::string compile_options;      // serialized CompileOptionsProto as received
  std::string fingerprint;
  std::vector<b2x::Plan> plans;     // one per replica when the module reads replica_id, else a single shared plan
  int num_replicas = 1, num_partitions = 1;
  std::vector<int> device_assignment;  // replica -> global device id
  std::vector<PJRT_Buffer_Type> out_types;
  std::vector<int64_t> out_dims_flat;
  std::vector<size_t> out_ranks;
  std::vector<const char*> out_kinds, param_kinds;
  std::vector<size_t> out_kind_sizes, param_kind_sizes;
  std::vector<PJRT_Layouts_MemoryLayout> param_layouts, out_layouts;        // lent out by the layouts extension
  std::vector<PJRT_Layouts_MemoryLayout*> param_layout_ptrs, out_layout_ptrs;
  std::vector<PJRT_NamedValue> cost_props;
  std::vector<std::string> cost_names;
  const b2x::Plan& plan_for(int replica) const { return plans.size() == 1 ? plans[0] : plans[replica]; }
};

struct PJRT_LoadedExecutable {
  PJRT_Client* client = nullptr;
  std::shared_ptr<b2x_ExecutableCore> core;
  std::vector<PJRT_Device*> addressable;          // local devices taking part, in replica order
  std::vector<PJRT_LogicalDeviceIds> logical_ids;
  bool deleted = false;
  struct PerDevice {
    void* arena = nullptr;
    size_t arena_bytes = 0;
    void* consts = nullptr;
    std::vector<cudaEvent_t> coll_done;   // one per collective step
    cudaEvent_t fork = nullptr;
    // step timing (B2X_StepTiming_Extension)
    bool timing = false;
    std::vector<std::vector<std::pair<cudaEvent_t, cudaEvent_t>>> timed;  // [execution][step]
    std::vector<float> step_ms;
    std::vector<void*> last_args, last_outs;   // of the last execution launched while timing was on (for replay)
  };
  std::vector<std::string> step_labels;
  std::vector<const char*> step_label_ptrs;
  std::vector<double> step_flops, step_bytes;
  std::vector<int> step_launches;
  std::vector<PerDevice> per_device;
  std::mutex mu;
  ~PJRT_LoadedExecutable();
};

struct PJRT_ExecuteContext { int unused = 0; };

struct PJRT_Client {
  std::string platform_name = "cuda", platform_version;
  int process_index = 0, num_processes = 1;
  std::vector<std::unique_ptr<PJRT_Device>> device_storage;
  std::vector<std::unique_ptr<PJRT_Memory>> memory_storage;
  std::vector<PJRT_Device*> devices, addressable_devices;
  std::vector<PJRT_Memory*> addressable_memories;
  // key-value store callbacks for cross-process rendezvous (crates/ryft-pjrt/src/clients.rs:698-825)
  PJRT_KeyValueGetCallback kv_get = nullptr; void* kv_get_arg = nullptr;
  PJRT_KeyValuePutCallback kv_put = nullptr; void* kv_put_arg = nullptr;
  // completion poller: turns cudaEvents into PJRT_Events off the caller's thread
  struct Pending { cudaEvent_t ev; int ordinal; PJRT_Event* event; std::function<void(PJRT_Error_Code*, std::string*)> finish; };
  std::mutex q_mu;
  std::condition_variable q_cv;
  std::deque<Pending> queue;
  bool stop = false;
  std::thread poller;
  std::unique_ptr<b2x::NcclComms> nccl;
  std::atomic<int64_t> executions{0};
  // Held while an execution that contains collectives enqueues on all of its devices: two such executions started from
  // different host threads must reach every device's communicator in the same order, or neither collective completes.
  std::mutex collective_enqueue_mu;
  void post(Pending p);
  ~PJRT_Client();
};

namespace b2x {
PJRT_Buffer_Type to_pjrt_type(DType t);
DType from_pjrt_type(PJRT_Buffer_Type t);

// Parsed subset of CompileOptionsProto (crates/ryft-xla-sys/src/protos.rs:3298-3346, 2391-2417, 2340-2354).
struct CompileOptions {
  int64_t num_replicas = 1, num_partitions = 1, device_ordinal = -1;
  bool has_device_assignment = false;
  int64_t da_replicas = 0, da_computations = 0;
  std::vector<std::vector<int64_t>> da_devices;  // [computation][replica]
  int precision = 0;
  bool use_spmd_partitioning = false;
};
bool parse_compile_options(const char* data, size_t size, CompileOptions* out, std::string* err);
std::string encode_device_assignment(int replicas, int computations, const std::vector<int>& replica_major_ids);

// Executes `plan` for one replica on `dev` (enqueue only).  args/outs are device pointers.
PJRT_Error* run_plan(PJRT_LoadedExecutable* le, int local_index, int replica, const std::vector<void*>& args,
                     const std::vector<void*>& outs);
}  // namespace b2x
