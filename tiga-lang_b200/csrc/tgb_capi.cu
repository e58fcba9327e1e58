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

namespace tgb {
namespace {
// one int32 from device memory to pinned (device-mapped) host memory, by a store from an SM: unlike a
// copy-engine transfer it does not queue behind a bulk device-to-host copy that another stream has in
// flight, so mirroring a status word never stalls the stream that launches it
__global__ void k_mirror_word(const int32_t *__restrict__ word, int32_t *__restrict__ host_word) {
  *reinterpret_cast<volatile int32_t *>(host_word) = *word;
  __threadfence_system();
}
}  // namespace
}  // namespace tgb

extern "C" {

int32_t tgb_mirror_word(const void *device_word, void *pinned_host_word, uint64_t stream) {
  if (!device_word || !pinned_host_word) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  tgb::k_mirror_word<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const int32_t *>(device_word), static_cast<int32_t *>(pinned_host_word));
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

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
