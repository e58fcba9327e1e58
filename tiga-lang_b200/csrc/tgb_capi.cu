// Status strings, error text and version of libtiga_b200.
#include <cstring>

#include "tgb_common.cuh"

namespace tgb {

static thread_local char g_error[512] = "";
std::atomic<int64_t> g_launches{0};

void set_error(const char *format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(g_error, sizeof(g_error), format, args);
  va_end(args);
}

}  // namespace tgb

extern "C" {

const char *tgb_status_string(int32_t status) {
  switch (status) {
    case TGB_STATUS_OK: return "ok";
    case TGB_STATUS_INVALID_ARGUMENT: return "invalid argument";
    case TGB_STATUS_UNSUPPORTED: return "unsupported";
    case TGB_STATUS_OUT_OF_MEMORY: return "out of memory";
    case TGB_STATUS_INTERNAL: return "internal error";
    default: return "unknown status";
  }
}

const char *tgb_last_error(void) { return tgb::g_error; }

const char *tgb_version(void) { return "tiga-b200 0.1.0 (sm_100a)"; }

int64_t tgb_launch_count(void) { return tgb::g_launches.load(); }

}  // extern "C"
