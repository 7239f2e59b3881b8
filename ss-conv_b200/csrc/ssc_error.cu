// Error reporting and identification entry points.
#include <stdarg.h>

#include "ssc_common.cuh"

namespace ssc {
unsigned long long launches();
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
static unsigned long long g_launches = 0;
void note_launches(int n) { __atomic_fetch_add(&g_launches, (unsigned long long)n, __ATOMIC_RELAXED); }
unsigned long long launches() { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }
}  // namespace ssc

extern "C" int ssc_version(void) { return 100; }
extern "C" const char *ssc_last_error(void) { return ssc::error_buffer(); }
extern "C" int ssc_has_tcgen05(void) { return 1; }
extern "C" unsigned long long ssc_kernel_launches(void) { return ssc::launches(); }
