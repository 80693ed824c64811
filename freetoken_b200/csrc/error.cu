// Per-thread text of the last failed call.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace ftk {
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// Which form of a kernel each launch took (tile sizes, tensor-core or CUDA-core path, short or
// segmented sort ...), counted by name, so that a test or a measurement can say what a step ran.
struct VariantCount {
  const char* name;
  long long count;
};
static VariantCount g_variants[128];
static int g_n_variants = 0;
static std::mutex g_variant_mutex;

void note_variant(const char* name) {
  std::lock_guard<std::mutex> lock(g_variant_mutex);
  for (int i = 0; i < g_n_variants; ++i)
    if (g_variants[i].name == name || strcmp(g_variants[i].name, name) == 0) {
      ++g_variants[i].count;
      return;
    }
  if (g_n_variants < 128) g_variants[g_n_variants++] = {name, 1};
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

// "name<TAB>count" lines of every kernel variant launched since the last reset, into buf (NUL-terminated,
// cut at cap); returns the number of bytes the whole text needs.
extern "C" int ftk_variant_counts(char* buf, int cap, int reset) {
  std::lock_guard<std::mutex> lock(ftk::g_variant_mutex);
  int need = 0;
  for (int i = 0; i < ftk::g_n_variants; ++i) {
    char line[160];
    const int n = snprintf(line, sizeof(line), "%s\t%lld\n", ftk::g_variants[i].name, ftk::g_variants[i].count);
    if (buf && need + n < cap) memcpy(buf + need, line, n);
    need += n;
  }
  if (buf && cap > 0) buf[need < cap ? need : cap - 1] = 0;
  if (reset) ftk::g_n_variants = 0;
  return need + 1;
}
