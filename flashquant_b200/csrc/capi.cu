// Library-wide pieces of the C ABI: version and the per-thread error text.
#include <atomic>

#include "fq_common.cuh"

namespace fq {
char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace fq

extern "C" int fq_version(void) { return 100; }

extern "C" const char* fq_last_error_string(void) { return fq::last_error_buffer(); }

extern "C" uint64_t fq_launch_count(void) {
  return fq::g_launches.load(std::memory_order_relaxed);
}
