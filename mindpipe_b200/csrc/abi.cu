// Library-level entry points: version, status strings, last CUDA error.
#include "common.cuh"

namespace mp {
thread_local int g_last_cuda_error = 0;
}

extern "C" int mp_abi_version(void) { return 1; }

extern "C" int mp_last_cuda_error(void) { return mp::g_last_cuda_error; }

extern "C" const char* mp_status_string(int status) {
  switch (status) {
    case MP_OK: return "ok";
    case MP_ERR_INVALID_ARG: return "invalid argument (null pointer or non-positive size)";
    case MP_ERR_UNSUPPORTED: return "shape not supported by this kernel";
    case MP_ERR_ALIGNMENT: return "pointer or pitch not aligned as required";
    case MP_ERR_WORKSPACE: return "workspace missing or too small";
    case MP_ERR_CUDA: return "CUDA call failed";
    case MP_ERR_DEVICE: return "device-side bounded wait gave up";
    default: return "unknown status";
  }
}
