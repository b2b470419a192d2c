#include <atomic>

#include "../common/launch_count.h"

static std::atomic<long long> g_launches{0};

extern "C" void eredu_count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long eredu_launch_count() { return g_launches.load(std::memory_order_relaxed); }
