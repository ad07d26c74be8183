// Process-wide count of kernel launches made by this library (read by benchmarks
// to report how many of its own kernels ran inside a timed region).
#pragma once
#include <atomic>
#include <stdint.h>

namespace esgd {
extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
}  // namespace esgd
