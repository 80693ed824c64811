// Per-thread text of the last failed call.
#include <stdarg.h>

#include "common.cuh"

namespace ftk {
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
}  // namespace ftk

extern "C" const char* ftk_last_error(void) { return ftk::g_error; }
