// Version and status-string entry points of the C ABI.
#include "common.cuh"

extern "C" int trx_version(void) { return TRX_ABI_VERSION; }

extern "C" const char* trx_status_string(int code) {
  switch (code) {
    case TRX_OK: return "ok";
    case TRX_ERR_NULL_POINTER: return "a required pointer is NULL";
    case TRX_ERR_DTYPE: return "unsupported dtype code";
    case TRX_ERR_SHAPE: return "invalid or inconsistent sizes";
    case TRX_ERR_ALIGNMENT: return "pointer or stride not aligned as required";
    case TRX_ERR_STRIDE: return "stride smaller than the extent it spans";
    case TRX_ERR_UNSUPPORTED: return "request not supported by this build";
    case TRX_ERR_CUDA: return "CUDA reported an error at launch";
    case TRX_ERR_DEVICE_STATUS: return "a kernel recorded a bounded-wait timeout";
    case TRX_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status code";
  }
}
