// Log bridge: native code formats a line and hands it to the registered callback (the Python logger); without a
// callback lines go to stderr.  Reference: kernels/src/runtime/log.cpp.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "blaze/runtime.h"

static blz_log_fn g_fn = nullptr;
static std::mutex g_mu;

extern "C" void blz_log_set(blz_log_fn fn) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_fn = fn;
}

extern "C" void blz_log(int level, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_fn) g_fn(level, buf);
  else fprintf(stderr, "[blaze native %d] %s\n", level, buf);
}
