// Shared launch helpers for the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <stdint.h>

namespace b2x {
extern std::atomic<int64_t> g_launch_count;
inline void count_launch(int n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }
constexpr int kNumSms = 148;  // B200: 2 dies x 74 SMs
}  // namespace b2x
