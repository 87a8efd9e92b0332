// Library-wide state: the thread-local error text and the version tag.
#include <atomic>

#include "common.cuh"

namespace smore {
unsigned long long launches();
char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
static std::atomic<unsigned long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
unsigned long long launches() { return g_launches.load(std::memory_order_relaxed); }
}  // namespace smore

extern "C" {
const char* smore_last_error(void) { return smore::last_error_buffer(); }
const char* smore_version(void) { return "smore_b200 sm_100a"; }
unsigned long long smore_kernel_launch_count(void) { return smore::launches(); }
}
