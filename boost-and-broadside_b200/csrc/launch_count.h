// Process-wide count of kernel launches issued by this library (read by bnb_launch_count).
#pragma once
#include <atomic>

namespace bnb {
extern std::atomic<unsigned long long> g_launches;
inline void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace bnb
