// Shared device/host helpers for the q3b200 C-ABI library (sm_100a only).
//
// Conventions used by every entry point in this library:
//   * raw device pointers + int64 sizes + an explicit cudaStream_t; no torch types;
//   * return value 0 on success, a negative Q3_ERR_* code when the host-side
//     validation rejects the call (nothing is launched in that case);
//   * range violations seen on the device (token id / label out of range, a
//     bounded wait that ran out) are OR-ed into an int32 device status word
//     supplied by the caller; kernels never trap or assert.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/q3b200.h"

namespace q3 {

// ---------------------------------------------------------------- host side
inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the current device only, so a kernel's "already
// configured" note is kept per device. One DeviceFlags object (a function-local static) per kernel instantiation.
struct DeviceFlags { bool done[64]; };

template <typename K> inline int ensure_dynamic_smem(K kern, int bytes, DeviceFlags* flags) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev >= 0 && flags->done[dev]) return Q3_OK;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  if (dev >= 0) flags->done[dev] = true;
  return Q3_OK;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? Q3_OK : Q3_ERR_CUDA - (int)e;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int dtype_size(int dt) { return dt == Q3_F32 ? 4 : 2; }

// Dispatch a generic lambda on the element type named by a Q3 dtype code.
#define Q3_DISPATCH_FLOAT(DT, T, ...)                                  \
  switch (DT) {                                                        \
    case Q3_F32: { using T = float; __VA_ARGS__; break; }              \
    case Q3_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }     \
    case Q3_F16: { using T = __half; __VA_ARGS__; break; }             \
    default: return Q3_ERR_DTYPE;                                      \
  }

// -------------------------------------------------------------- device side
#ifdef __CUDACC__

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// 16-byte vector of T viewed as floats. N = 4 (fp32) or 8 (bf16 / fp16).
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T, int N> struct VecIO;

template <typename T> struct VecIO<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = to_f32<T>(*p); }
  static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { *p = from_f32<T>(v[0]); }
};

template <> struct VecIO<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};

template <> struct VecIO<float, 8> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

template <> struct VecIO<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 t;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = t;
  }
};

template <> struct VecIO<__nv_bfloat16, 4> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 2; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 t;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 2; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

template <> struct VecIO<__half, 4> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int i = 0; i < 2; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[4]) {
    uint2 t;
    __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
    for (int i = 0; i < 2; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

template <> struct VecIO<__half, 8> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 t;
    __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = t;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a group of G consecutive lanes (G a power of two <= 32).
template <int G> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum; `scratch` holds >= 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nwarp; ++i) t += scratch[i];  // same order in every thread: deterministic
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = scratch[0];
  for (int i = 1; i < nwarp; ++i) t = fmaxf(t, scratch[i]);
  return t;
}

__device__ __forceinline__ void flag_status(int* status, int bit) {
  if (status != nullptr) atomicOr(status, bit);
}

#endif  // __CUDACC__
// Row of a multi-tensor table that owns block `blk`: the last row whose `first_block` column is <= blk (the column is
// non-decreasing). Every thread walks the same few table entries, which stay in L1 after the first CTA of an SM.
__device__ __forceinline__ int64_t find_owner(const int64_t* __restrict__ meta, int64_t rows, int stride, int col,
                                              int64_t blk) {
  int64_t lo = 0, hi = rows;
  while (lo + 1 < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (meta[mid * stride + col] <= blk) lo = mid; else hi = mid;
  }
  return lo;
}

}  // namespace q3
