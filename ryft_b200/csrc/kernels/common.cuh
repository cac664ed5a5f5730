// Shared launch helpers for the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdlib>
#include <stdint.h>

namespace b2x {
extern std::atomic<int64_t> g_launch_count;
inline void count_launch(int n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }
constexpr int kNumSms = 148;  // B200: 2 dies x 74 SMs
// B2X_VM_STATIC=0 makes every fused-elementwise program run through the interpreter, also those that have a build-time
// specialised form (for measuring what the specialisation is worth, and for testing the interpreter on the same programs).
inline bool vm_static_enabled() {
  const char* e = getenv("B2X_VM_STATIC");
  return !(e && e[0] == '0');
}
}  // namespace b2x
