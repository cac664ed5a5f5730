#include "nccl_dyn.h"

#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>

#include "objects.h"

namespace b2x {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string load_error;
};

static NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (auto n : names) { api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (api.lib) break; }
    if (!api.lib) { api.load_error = std::string("could not load libnccl.so.2: ") + dlerror(); return; }
#define B2X_SYM(field, name) *(void**)(&api.field) = dlsym(api.lib, name); if (!api.field) api.load_error = std::string("libnccl lacks ") + name;
    B2X_SYM(GetUniqueId, "ncclGetUniqueId")
    B2X_SYM(CommInitRank, "ncclCommInitRank")
    B2X_SYM(CommInitAll, "ncclCommInitAll")
    B2X_SYM(CommDestroy, "ncclCommDestroy")
    B2X_SYM(CommAbort, "ncclCommAbort")
    B2X_SYM(AllReduce, "ncclAllReduce")
    B2X_SYM(AllGather, "ncclAllGather")
    B2X_SYM(GroupStart, "ncclGroupStart")
    B2X_SYM(GroupEnd, "ncclGroupEnd")
    B2X_SYM(GetErrorString, "ncclGetErrorString")
#undef B2X_SYM
  });
  return &api;
}

static PJRT_Error* nccl_err(ncclResult_t r, const char* what) {
  NcclApi* a = nccl_api();
  return make_error(PJRT_Error_Code_INTERNAL, std::string("NCCL error in ") + what + ": " + (a->GetErrorString ? a->GetErrorString(r) : "?"));
}
#define B2X_NCCL(expr) do { ncclResult_t _r = (expr); if (_r != ncclSuccess) return nccl_err(_r, #expr); } while (0)

static std::string group_key(const std::vector<int>& group) {
  std::string k;
  for (auto g : group) { k += std::to_string(g); k += ','; }
  return k;
}

NcclComms::~NcclComms() {
  NcclApi* a = nccl_api();
  if (!a->CommDestroy) return;
  for (auto& kv : comms) for (auto& c : kv.second) if (c.second) a->CommDestroy((ncclComm_t)c.second);
}

void* NcclComms::comm_for(const std::vector<int>& group, int global_id) {
  std::lock_guard<std::mutex> lk(mu);
  auto it = comms.find(group_key(group));
  if (it == comms.end()) return nullptr;
  auto jt = it->second.find(global_id);
  return jt == it->second.end() ? nullptr : jt->second;
}

PJRT_Error* NcclComms::ensure(const std::vector<int>& group) {
  std::lock_guard<std::mutex> lk(mu);
  const std::string key = group_key(group);
  if (comms.count(key)) return nullptr;
  NcclApi* a = nccl_api();
  if (!a->lib || !a->load_error.empty()) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "collectives need NCCL: " + a->load_error);
  const int n = (int)group.size();
  std::vector<int> local_ranks, local_ordinals;
  for (int r = 0; r < n; r++) {
    int gid = group[r];
    if (gid < 0 || gid >= (int)client->devices.size()) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "replica group names device " + std::to_string(gid) + " which does not exist");
    PJRT_Device* d = client->devices[gid];
    if (d->addressable) { local_ranks.push_back(r); local_ordinals.push_back(d->cuda_ordinal); }
  }
  std::map<int, void*> out;
  if ((int)local_ranks.size() == n) {
    std::vector<ncclComm_t> cs(n);
    B2X_NCCL(a->CommInitAll(cs.data(), n, local_ordinals.data()));
    for (int r = 0; r < n; r++) out[group[r]] = cs[r];
  } else {
    if (local_ranks.empty()) { comms[key] = out; return nullptr; }
    if (!client->kv_get || !client->kv_put)
      return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "a replica group spans several processes but the client was created without key-value store callbacks");
    ncclUniqueId id;
    const std::string kv_key = "b2x/nccl/" + key + "/" + std::to_string(generation);
    const bool leader = client->devices[group[0]]->addressable;
    if (leader) {
      B2X_NCCL(a->GetUniqueId(&id));
      static const char* hex = "0123456789abcdef";
      std::string v;
      for (size_t i = 0; i < sizeof(id); i++) { unsigned char c = ((unsigned char*)&id)[i]; v.push_back(hex[c >> 4]); v.push_back(hex[c & 15]); }
      PJRT_KeyValuePutCallback_Args pa{};
      pa.struct_size = sizeof(pa);
      pa.key = kv_key.data(); pa.key_size = kv_key.size();
      pa.value = v.data(); pa.value_size = v.size();
      pa.user_arg = client->kv_put_arg;
      if (PJRT_Error* e = client->kv_put(&pa)) return e;
    } else {
      PJRT_KeyValueGetCallback_Args ga{};
      ga.struct_size = sizeof(ga);
      ga.key = kv_key.data(); ga.key_size = kv_key.size();
      ga.timeout_in_ms = 120000;
      ga.user_arg = client->kv_get_arg;
      if (PJRT_Error* e = client->kv_get(&ga)) return e;
      if (!ga.value || ga.value_size != 2 * sizeof(id)) return make_error(PJRT_Error_Code_INTERNAL, "bad NCCL id in the key-value store");
      auto nib = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
      for (size_t i = 0; i < sizeof(id); i++) ((unsigned char*)&id)[i] = (unsigned char)((nib(ga.value[2 * i]) << 4) | nib(ga.value[2 * i + 1]));
      if (ga.value_deleter_callback) ga.value_deleter_callback(ga.value);
    }
    std::vector<ncclComm_t> cs(local_ranks.size());
    B2X_NCCL(a->GroupStart());
    for (size_t i = 0; i < local_ranks.size(); i++) {
      cudaSetDevice(local_ordinals[i]);
      ncclResult_t r = a->CommInitRank(&cs[i], n, id, local_ranks[i]);
      if (r != ncclSuccess) { a->GroupEnd(); return nccl_err(r, "ncclCommInitRank"); }
    }
    B2X_NCCL(a->GroupEnd());
    for (size_t i = 0; i < local_ranks.size(); i++) out[group[local_ranks[i]]] = cs[i];
  }
  generation++;
  comms[key] = out;
  return nullptr;
}

static bool nccl_type(int dtype, ncclDataType_t* t) {
  switch ((DType)dtype) {
    case DType::S8: *t = ncclInt8; return true;
    case DType::U8: case DType::PRED: *t = ncclUint8; return true;
    case DType::S32: *t = ncclInt32; return true;
    case DType::U32: *t = ncclUint32; return true;
    case DType::S64: *t = ncclInt64; return true;
    case DType::U64: *t = ncclUint64; return true;
    case DType::F16: *t = ncclFloat16; return true;
    case DType::F32: *t = ncclFloat32; return true;
    case DType::F64: *t = ncclFloat64; return true;
    case DType::BF16: *t = ncclBfloat16; return true;
    default: return false;
  }
}

PJRT_Error* NcclComms::all_reduce(void* comm, const void* src, void* dst, size_t count, int dtype, int monoid, cudaStream_t s) {
  NcclApi* a = nccl_api();
  ncclDataType_t t;
  if (!nccl_type(dtype, &t)) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "all_reduce over this element type");
  ncclRedOp_t op;
  switch ((Monoid)monoid) {
    case Monoid::ADD: op = ncclSum; break;
    case Monoid::MUL: op = ncclProd; break;
    case Monoid::MAX: op = ncclMax; break;
    case Monoid::MIN: op = ncclMin; break;
    case Monoid::OR: if ((DType)dtype == DType::PRED) { op = ncclMax; break; }  // fallthrough
    case Monoid::AND: if ((DType)dtype == DType::PRED) { op = ncclMin; break; }  // fallthrough
    default: return make_error(PJRT_Error_Code_UNIMPLEMENTED, "all_reduce with this reduction body");
  }
  B2X_NCCL(a->AllReduce(src, dst, count, t, op, (ncclComm_t)comm, s));
  return nullptr;
}

PJRT_Error* NcclComms::all_gather(void* comm, const void* src, void* dst, size_t count, int dtype, cudaStream_t s) {
  NcclApi* a = nccl_api();
  ncclDataType_t t;
  if (!nccl_type(dtype, &t)) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "all_gather over this element type");
  B2X_NCCL(a->AllGather(src, dst, count, t, (ncclComm_t)comm, s));
  return nullptr;
}

}  // namespace b2x
