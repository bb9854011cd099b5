// Library-level entry points: ABI version, error strings, device queries.
#include "common.cuh"

extern "C" int q3_abi_version(void) { return 1; }

extern "C" const char* q3_error_string(int code) {
  switch (code) {
    case Q3_OK: return "ok";
    case Q3_ERR_ARG: return "null pointer or non-positive size";
    case Q3_ERR_SHAPE: return "unsupported shape";
    case Q3_ERR_DTYPE: return "unsupported element type";
    case Q3_ERR_WORKSPACE: return "workspace missing or too small";
    case Q3_ERR_ALIGN: return "unsupported pointer or stride alignment";
    case Q3_ERR_DRIVER: return "required CUDA driver entry point unavailable";
    case Q3_ERR_LIMIT: return "size beyond the fixed scratch capacity of this no-allocation entry point";
    case Q3_ERR_TMAP: return "TMA tensor-map description rejected by the driver";
    default: break;
  }
  if (code <= Q3_ERR_CUDA) return cudaGetErrorString((cudaError_t)(Q3_ERR_CUDA - code));
  return "unknown error";
}

extern "C" int q3_device_sm_count(void) { return q3::sm_count(); }
