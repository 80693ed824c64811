// Per-thread text of the last failed call.
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"

namespace ftk {
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("FTK_PDL");
    on = !(v && v[0] == '0');
  }
  return on != 0;
}
}  // namespace ftk

extern "C" const char* ftk_last_error(void) { return ftk::g_error; }
