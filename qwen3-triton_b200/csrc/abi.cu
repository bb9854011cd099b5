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

// ---------------------------------------------------------------------------------------------------------
// Status word for kernels whose entry points carry no status argument (the bulk-copy ring kernels of
// norm_ring.cu): one int per device in global memory, flagged with the Q3_STATUS_* bits.
static __device__ int g_async_status;

namespace q3 {
int* async_status() {
  static int* ptr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_async_status) == cudaSuccess) ptr[dev] = static_cast<int*>(p);
  }
  return ptr[dev];
}
}  // namespace q3

extern "C" int q3_async_status(int clear, int* value) {
  if (!value) return Q3_ERR_ARG;
  int* p = q3::async_status();
  if (!p) return Q3_ERR_DRIVER;
  cudaError_t e = cudaMemcpy(value, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  if (clear && *value) {
    e = cudaMemset(p, 0, sizeof(int));
    if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  }
  return Q3_OK;
}
