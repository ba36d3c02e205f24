// Status / error reporting of the C ABI (include/flashqla_b200.h).
#include <stdarg.h>

#include "common.cuh"

namespace qla {
namespace {
thread_local char g_last_error[512] = "";
}

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}
}  // namespace qla

extern "C" QLA_API const char* qla_status_string(int code) {
  switch (code) {
    case QLA_OK: return "ok";
    case QLA_ERR_INVALID_ARG: return "invalid argument";
    case QLA_ERR_UNSUPPORTED: return "unsupported configuration";
    case QLA_ERR_CUDA: return "CUDA call failed";
    case QLA_ERR_WORKSPACE: return "workspace missing or too small";
    case QLA_ERR_DEVICE: return "device reported a fault";
    default: return "unknown status";
  }
}

extern "C" QLA_API const char* qla_last_error(void) { return qla::g_last_error; }

extern "C" QLA_API int qla_abi_version(void) { return QLA_ABI_VERSION; }
