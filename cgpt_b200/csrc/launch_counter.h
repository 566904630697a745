// Host-side count of kernel launches issued by this library (reported by cgpt_b200_launch_count()).
#pragma once
#include <atomic>
#include <cstdint>

namespace cgpt {
extern std::atomic<std::uint64_t> g_launch_count;
inline void count_launch(std::uint64_t n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }
}  // namespace cgpt
