#include "../errors.h"

#include <cstdarg>
#include <cstdio>

#include "../../../include/fqb.h"

namespace fqb {
namespace {
thread_local char g_msg[512] = "";
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(g_msg, sizeof g_msg, fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace fqb

extern "C" {

const char* fqb_last_error(void) { return fqb::g_msg; }

const char* fqb_strerror(int code) {
  switch (code) {
    case FQB_OK: return "ok";
    case FQB_ERR_INVALID: return "invalid argument";
    case FQB_ERR_SHAPE: return "unsupported shape";
    case FQB_ERR_CUDA: return "CUDA call failed";
    case FQB_ERR_WORKSPACE: return "scratch too small";
    case FQB_ERR_TIMEOUT: return "bounded wait inside a kernel ran out";
    case FQB_ERR_INDEX: return "index out of range on the device";
    case FQB_ERR_NOMEM: return "block pool exhausted";
    case FQB_ERR_STATE: return "allocator state error";
    default: return "unknown error";
  }
}

}  // extern "C"
