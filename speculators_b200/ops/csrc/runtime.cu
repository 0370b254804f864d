// Host-side bookkeeping shared by every launcher: a process-wide count of kernel
// launches issued by this library (the launchers call count_launch once per
// kernel they enqueue, whether the stream is executing or being captured).
#include <atomic>
#include <stdint.h>

namespace sb200 {

static std::atomic<int64_t> g_launches{0};

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

}  // namespace sb200
