// Diagnostics of the C ABI: version, status strings, last-error message.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace {
std::mutex g_err_mutex;
char g_err[512] = "";
}  // namespace

namespace {
std::atomic<int> g_reserved_sms{0};
std::atomic<int> g_cta_pairs{-1};  // -1: chosen per shape, 0: never, 1: always
}  // namespace

namespace sc {
int reserved_sms() { return g_reserved_sms.load(std::memory_order_relaxed); }
int cta_pairs_mode() { return g_cta_pairs.load(std::memory_order_relaxed); }

int fail(int status, const char* fmt, ...) {
  std::lock_guard<std::mutex> lock(g_err_mutex);
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}
}  // namespace sc

extern "C" int sc_version(void) { return 100; }

extern "C" int sc_set_reserved_sms(int n) {
  SC_REQUIRE(n >= 0 && n <= 64, "sc_set_reserved_sms: %d outside [0, 64]", n);
  g_reserved_sms.store(n, std::memory_order_relaxed);
  return SC_OK;
}

extern "C" int sc_set_cta_pairs(int on) {
  g_cta_pairs.store(on < 0 ? -1 : (on != 0 ? 1 : 0), std::memory_order_relaxed);
  return SC_OK;
}

extern "C" size_t sc_last_error(char* buf, size_t cap) {
  std::lock_guard<std::mutex> lock(g_err_mutex);
  size_t n = strlen(g_err);
  if (buf && cap) {
    size_t c = n < cap - 1 ? n : cap - 1;
    memcpy(buf, g_err, c);
    buf[c] = 0;
  }
  return n;
}

extern "C" const char* sc_status_string(int status) {
  switch (status) {
    case SC_OK: return "ok";
    case SC_ERR_INVALID: return "invalid argument";
    case SC_ERR_UNSUPPORTED: return "unsupported";
    case SC_ERR_WORKSPACE: return "workspace too small";
    case SC_ERR_CUDA: return "CUDA error";
    case SC_ERR_TIMEOUT: return "device-side wait timed out";
    case SC_ERR_TOO_LARGE: return "size beyond the entry point's maximum";
    default: return "unknown status";
  }
}
