// Process-wide count of kernels launched by this library (reported by benchmarks so a
// silent library or CPU fallback would show up as zero).
#pragma once
#include <atomic>
#include <stdint.h>

namespace onn
{
extern std::atomic<uint64_t> g_launch_count;
inline void count_launch(int n = 1) { g_launch_count.fetch_add((uint64_t)n, std::memory_order_relaxed); }
}
