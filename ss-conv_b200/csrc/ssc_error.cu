// Error reporting and identification entry points.
#include <stdarg.h>

#include "ssc_common.cuh"

namespace ssc {
char *error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace ssc

extern "C" int ssc_version(void) { return 100; }
extern "C" const char *ssc_last_error(void) { return ssc::error_buffer(); }
extern "C" int ssc_has_tcgen05(void) { return 1; }
