// Library-level entry points: version and per-thread error message.
#include <string>

#include "kvq_common.cuh"

namespace kvq {
static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}
}  // namespace kvq

extern "C" __attribute__((visibility("default"))) int kvq_version(void) { return 100; }

extern "C" __attribute__((visibility("default"))) const char* kvq_last_error(void) { return kvq::g_last_error.c_str(); }
