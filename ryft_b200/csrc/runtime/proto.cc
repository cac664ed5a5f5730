// Minimal protobuf wire reader/writer for the messages that cross the PJRT boundary.
//
// CompileOptionsProto (crates/ryft-xla-sys/src/protos.rs:3298-3346): field 3 = ExecutableBuildOptions, field 10 =
// matrix_unit_operand_precision.  ExecutableBuildOptions (protos.rs:2391-2417): 1 = device_ordinal, 4 =
// num_replicas, 5 = num_partitions, 6 = use_spmd_partitioning, 9 = DeviceAssignment.  DeviceAssignmentProto
// (protos.rs:2340-2354): 1 = replica_count, 2 = computation_count, 3 = repeated ComputationDevice
// { 1 = repeated replica_device_ids }.  Unknown fields are skipped.
#include <cstring>

#include "objects.h"

namespace b2x {
namespace {
struct Reader {
  const uint8_t* p; const uint8_t* end; bool ok = true;
  bool done() const { return p >= end; }
  uint64_t varint() {
    uint64_t v = 0; int shift = 0;
    while (p < end && shift < 64) { uint8_t b = *p++; v |= (uint64_t)(b & 0x7f) << shift; if (!(b & 0x80)) return v; shift += 7; }
    ok = false; return 0;
  }
  Reader sub() {
    uint64_t n = varint();
    if (!ok || n > (uint64_t)(end - p)) { ok = false; return Reader{p, p}; }
    Reader r{p, p + n}; p += n; return r;
  }
  void skip(int wire) {
    switch (wire) {
      case 0: varint(); break;
      case 1: if (end - p < 8) ok = false; else p += 8; break;
      case 2: sub(); break;
      case 5: if (end - p < 4) ok = false; else p += 4; break;
      default: ok = false;
    }
  }
};

void read_ints(Reader& r, int wire, std::vector<int64_t>* out) {
  if (wire == 2) { Reader s = r.sub(); while (s.ok && !s.done()) out->push_back((int64_t)s.varint()); if (!s.ok) r.ok = false; }
  else out->push_back((int64_t)r.varint());
}

void parse_device_assignment(Reader r, CompileOptions* o) {
  o->has_device_assignment = true;
  while (r.ok && !r.done()) {
    uint64_t tag = r.varint(); int f = (int)(tag >> 3), w = (int)(tag & 7);
    if (f == 1 && w == 0) o->da_replicas = (int64_t)r.varint();
    else if (f == 2 && w == 0) o->da_computations = (int64_t)r.varint();
    else if (f == 3 && w == 2) {
      Reader c = r.sub();
      std::vector<int64_t> ids;
      while (c.ok && !c.done()) {
        uint64_t t2 = c.varint(); int f2 = (int)(t2 >> 3), w2 = (int)(t2 & 7);
        if (f2 == 1) read_ints(c, w2, &ids); else c.skip(w2);
      }
      o->da_devices.push_back(ids);
    } else r.skip(w);
  }
}

void parse_build_options(Reader r, CompileOptions* o) {
  while (r.ok && !r.done()) {
    uint64_t tag = r.varint(); int f = (int)(tag >> 3), w = (int)(tag & 7);
    if (f == 1 && w == 0) o->device_ordinal = (int64_t)r.varint();
    else if (f == 4 && w == 0) o->num_replicas = (int64_t)r.varint();
    else if (f == 5 && w == 0) o->num_partitions = (int64_t)r.varint();
    else if (f == 6 && w == 0) o->use_spmd_partitioning = r.varint() != 0;
    else if (f == 9 && w == 2) parse_device_assignment(r.sub(), o);
    else r.skip(w);
  }
}

void put_varint(std::string* s, uint64_t v) { while (v >= 0x80) { s->push_back((char)(v | 0x80)); v >>= 7; } s->push_back((char)v); }
}  // namespace

bool parse_compile_options(const char* data, size_t size, CompileOptions* out, std::string* err) {
  Reader r{(const uint8_t*)data, (const uint8_t*)data + size};
  while (r.ok && !r.done()) {
    uint64_t tag = r.varint(); int f = (int)(tag >> 3), w = (int)(tag & 7);
    if (f == 3 && w == 2) parse_build_options(r.sub(), out);
    else if (f == 10 && w == 0) out->precision = (int)r.varint();
    else r.skip(w);
  }
  if (!r.ok) { *err = "malformed CompileOptionsProto"; return false; }
  if (out->num_replicas <= 0) out->num_replicas = 1;   // proto default 0 means "unset"
  if (out->num_partitions <= 0) out->num_partitions = 1;
  return true;
}

std::string encode_device_assignment(int replicas, int computations, const std::vector<int>& ids) {
  std::string s;
  put_varint(&s, (1 << 3) | 0); put_varint(&s, (uint64_t)replicas);
  put_varint(&s, (2 << 3) | 0); put_varint(&s, (uint64_t)computations);
  for (int c = 0; c < computations; c++) {
    std::string packed;
    for (int r = 0; r < replicas; r++) put_varint(&packed, (uint64_t)ids[(size_t)r * computations + c]);
    std::string comp;
    put_varint(&comp, (1 << 3) | 2); put_varint(&comp, packed.size()); comp += packed;
    put_varint(&s, (3 << 3) | 2); put_varint(&s, comp.size()); s += comp;
  }
  return s;
}
}  // namespace b2x
