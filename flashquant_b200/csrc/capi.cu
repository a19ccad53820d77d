// Library-wide pieces of the C ABI: version and the per-thread error text.
#include <atomic>

#include "fq_common.cuh"

namespace fq {
char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
static std::atomic<uint64_t> g_launches{0};
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
// 200 ms by default: two orders of magnitude beyond the longest decode launch, short enough
// for a stuck launch to give the GPU back promptly.
static std::atomic<uint64_t> g_wait_limit_ns{200000000ull};
// bumped by every process-wide setter: a recorded sequence of launches (the graph of the packed
// host step) is only replayed while the settings it was recorded under still hold
static std::atomic<uint64_t> g_settings_epoch{0};
uint64_t settings_epoch() { return g_settings_epoch.load(std::memory_order_relaxed); }
void settings_changed() { g_settings_epoch.fetch_add(1, std::memory_order_relaxed); }
uint64_t device_wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
}  // namespace fq

extern "C" int fq_version(void) { return 100; }

extern "C" const char* fq_last_error_string(void) { return fq::last_error_buffer(); }

extern "C" uint64_t fq_launch_count(void) {
  return fq::g_launches.load(std::memory_order_relaxed);
}

extern "C" void fq_set_device_wait_limit_ns(uint64_t nanoseconds) {
  fq::g_wait_limit_ns.store(nanoseconds ? nanoseconds : 1, std::memory_order_relaxed);
  fq::settings_changed();
}

extern "C" uint64_t fq_get_device_wait_limit_ns(void) { return fq::device_wait_limit_ns(); }
