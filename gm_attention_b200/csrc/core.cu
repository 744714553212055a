// Library identity and the per-thread error message of libgmb200.
#include "common.cuh"

namespace gmb {

char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(error_buffer(), 512, fmt, args);
  va_end(args);
  return code;
}

}  // namespace gmb

extern "C" int gm_abi_version(void) { return 3; }
extern "C" const char* gm_last_error(void) { return gmb::error_buffer(); }
