// ABI bookkeeping: version and error strings.
#include "common.cuh"

extern "C" int hb200_abi_version(void) { return HB200_ABI_VERSION; }

extern "C" const char* hb200_error_string(int code) {
  switch (code) {
    case HB200_OK: return "ok";
    case HB200_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, bad size or alignment)";
    case HB200_ERR_UNSUPPORTED: return "request outside the built kernel variants";
    case HB200_ERR_CUDA: return "CUDA runtime call failed";
    case HB200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case HB200_ERR_WORKSPACE: return "workspace missing or too small";
    case HB200_ERR_SCRATCH_LIMIT:
      return "shape exceeds the 8 MiB built-in scratch (at most 8 activation rows and K <= 65536 always fit); "
             "use the entry point that takes a caller workspace";
    default: return "unknown error code";
  }
}
