// NCCL bound at run time (dlopen) so that single-GPU use needs no NCCL at all and a host process that already
// loaded its own libnccl.so.2 shares that copy.  Implements stablehlo.all_reduce / all_gather
// (crates/ryft-mlir/src/dialects/stable_hlo/operations/communication.rs:768-895) for replicas spread over the GPUs
// of this process and, through the PJRT key-value callbacks, of other processes.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

struct PJRT_Client;
struct PJRT_Error;

namespace b2x {

struct NcclApi;

struct NcclComms {
  explicit NcclComms(PJRT_Client* c) : client(c) {}
  ~NcclComms();
  PJRT_Client* client;
  std::mutex mu;
  // group key (sorted global device ids joined by ',') -> communicator per local device ordinal
  std::map<std::string, std::map<int, void*>> comms;
  int generation = 0;

  // Makes sure every local device in `group` (global device ids, in rank order) has a communicator.
  PJRT_Error* ensure(const std::vector<int>& group);
  void* comm_for(const std::vector<int>& group, int global_device_id);

  PJRT_Error* all_reduce(void* comm, const void* src, void* dst, size_t count, int dtype /*b2x::DType*/, int monoid, cudaStream_t s);
  PJRT_Error* all_gather(void* comm, const void* src, void* dst, size_t count, int dtype, cudaStream_t s);
};

}  // namespace b2x
