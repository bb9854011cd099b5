// Bandwidth-bound elementwise kernels: residual add, dtype cast, SwiGLU forward/backward,
// position ids. All are persistent grid-stride kernels over 16-byte vectors with a scalar
// tail, fp32 math and one rounding on store.
//
// Replaces, in the reference: qwen3_triton/kernels/residual.py:7-11 (_add),
// kernels/attention.py:10-18 (_cast / cast_tensor), kernels/activation.py:7-20 and
// kernels/math_precision.py:67-81 (SwiGLU fwd/bwd), qwen3_triton/_model.py:30-32 (_positions).
#include "common.cuh"

namespace q3 {

constexpr int kEwThreads = 256;

inline int ew_grid(int64_t nvec) {
  int64_t blocks = cdiv(nvec, kEwThreads);
  int64_t cap = (int64_t)sm_count() * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T, int V>
__global__ void __launch_bounds__(kEwThreads) add_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                         T* __restrict__ out, int64_t n) {
  const int64_t nvec = n / V;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float x[V], y[V];
    VecIO<T, V>::load(a + i * V, x);
    VecIO<T, V>::load(b + i * V, y);
#pragma unroll
    for (int j = 0; j < V; ++j) x[j] += y[j];
    VecIO<T, V>::store(out + i * V, x);
  }
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * V + threadIdx.x; i < n; i += blockDim.x)
      out[i] = from_f32<T>(to_f32<T>(a[i]) + to_f32<T>(b[i]));
  }
}

template <typename S, typename D>
__global__ void __launch_bounds__(kEwThreads) cast_kernel(const S* __restrict__ x, D* __restrict__ y, int64_t n,
                                                          bool vec_ok) {
  // 8 elements per thread per iteration when both sides are 16-byte aligned.
  constexpr int V = 8;
  const int64_t nvec = vec_ok ? n / V : 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float v[V];
    if constexpr (sizeof(S) == 4) {
      float a4[4], b4[4];
      VecIO<S, 4>::load(x + i * V, a4);
      VecIO<S, 4>::load(x + i * V + 4, b4);
#pragma unroll
      for (int j = 0; j < 4; ++j) { v[j] = a4[j]; v[4 + j] = b4[j]; }
    } else {
      VecIO<S, 8>::load(x + i * V, v);
    }
    if constexpr (sizeof(D) == 4) {
      float a4[4], b4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) { a4[j] = v[j]; b4[j] = v[4 + j]; }
      VecIO<D, 4>::store(y + i * V, a4);
      VecIO<D, 4>::store(y + i * V + 4, b4);
    } else {
      VecIO<D, 8>::store(y + i * V, v);
    }
  }
  for (int64_t i = nvec * V + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = from_f32<D>(to_f32<S>(x[i]));
}

__device__ __forceinline__ float sigmoidf_(float g) { return __fdividef(1.f, 1.f + __expf(-g)); }

template <typename T, int V>
__global__ void __launch_bounds__(kEwThreads) swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u,
                                                                T* __restrict__ y, int64_t n) {
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  // two independent vectors per iteration: twice the bytes in flight per thread
  for (; i + stride < nvec; i += 2 * stride) {
    float a0[V], b0[V], a1[V], b1[V];
    VecIO<T, V>::load(g + i * V, a0);
    VecIO<T, V>::load(u + i * V, b0);
    VecIO<T, V>::load(g + (i + stride) * V, a1);
    VecIO<T, V>::load(u + (i + stride) * V, b1);
#pragma unroll
    for (int j = 0; j < V; ++j) { a0[j] = a0[j] * sigmoidf_(a0[j]) * b0[j]; a1[j] = a1[j] * sigmoidf_(a1[j]) * b1[j]; }
    VecIO<T, V>::store(y + i * V, a0);
    VecIO<T, V>::store(y + (i + stride) * V, a1);
  }
  for (; i < nvec; i += stride) {
    float a[V], b[V];
    VecIO<T, V>::load(g + i * V, a);
    VecIO<T, V>::load(u + i * V, b);
#pragma unroll
    for (int j = 0; j < V; ++j) a[j] = a[j] * sigmoidf_(a[j]) * b[j];
    VecIO<T, V>::store(y + i * V, a);
  }
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * V + threadIdx.x; i < n; i += blockDim.x) {
      float a = to_f32<T>(g[i]);
      y[i] = from_f32<T>(a * sigmoidf_(a) * to_f32<T>(u[i]));
    }
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kEwThreads) swiglu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ u,
                                                                const T* __restrict__ dy, T* __restrict__ dg,
                                                                T* __restrict__ du, int64_t n) {
  const int64_t nvec = n / V;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float a[V], b[V], c[V], o1[V], o2[V];
    VecIO<T, V>::load(g + i * V, a);
    VecIO<T, V>::load(u + i * V, b);
    VecIO<T, V>::load(dy + i * V, c);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float s = sigmoidf_(a[j]);
      o1[j] = c[j] * b[j] * s * (1.f + a[j] * (1.f - s));  // d/dg [g*sigmoid(g)] = s*(1+g*(1-s))
      o2[j] = c[j] * a[j] * s;
    }
    VecIO<T, V>::store(dg + i * V, o1);
    VecIO<T, V>::store(du + i * V, o2);
  }
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * V + threadIdx.x; i < n; i += blockDim.x) {
      const float a = to_f32<T>(g[i]), b = to_f32<T>(u[i]), c = to_f32<T>(dy[i]);
      const float s = sigmoidf_(a);
      dg[i] = from_f32<T>(c * b * s * (1.f + a * (1.f - s)));
      du[i] = from_f32<T>(c * a * s);
    }
  }
}

__global__ void positions_kernel(int64_t* pos, int64_t n, int64_t seq) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    pos[i] = i % seq;
}

template <typename S>
int cast_from(const S* x, void* y, int dst, int64_t n, bool vec_ok, cudaStream_t st) {
  const int grid = ew_grid(cdiv(n, 8));
  switch (dst) {
    case Q3_F32: cast_kernel<S, float><<<grid, kEwThreads, 0, st>>>(x, (float*)y, n, vec_ok); break;
    case Q3_BF16: cast_kernel<S, __nv_bfloat16><<<grid, kEwThreads, 0, st>>>(x, (__nv_bfloat16*)y, n, vec_ok); break;
    case Q3_F16: cast_kernel<S, __half><<<grid, kEwThreads, 0, st>>>(x, (__half*)y, n, vec_ok); break;
    default: return Q3_ERR_DTYPE;
  }
  return launch_status();
}

}  // namespace q3

using namespace q3;

extern "C" int q3_residual_add(const void* a, const void* b, void* out, int64_t n, int dtype, q3_stream_t stream) {
  if (!a || !b || !out || n < 1) return Q3_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = aligned16(a) && aligned16(b) && aligned16(out);
  Q3_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    if (vec) add_kernel<T, V><<<ew_grid(cdiv(n, V)), kEwThreads, 0, st>>>((const T*)a, (const T*)b, (T*)out, n);
    else add_kernel<T, 1><<<ew_grid(n), kEwThreads, 0, st>>>((const T*)a, (const T*)b, (T*)out, n);
  });
  return launch_status();
}

extern "C" int q3_cast(const void* x, int src_dtype, void* y, int dst_dtype, int64_t n, q3_stream_t stream) {
  if (!x || !y || n < 1) return Q3_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  // The 8-wide path reads 16 or 32 bytes and writes 16 or 32 bytes per thread.
  const bool vec = aligned16(x) && aligned16(y);
  switch (src_dtype) {
    case Q3_F32: return cast_from<float>((const float*)x, y, dst_dtype, n, vec, st);
    case Q3_BF16: return cast_from<__nv_bfloat16>((const __nv_bfloat16*)x, y, dst_dtype, n, vec, st);
    case Q3_F16: return cast_from<__half>((const __half*)x, y, dst_dtype, n, vec, st);
    default: return Q3_ERR_DTYPE;
  }
}

extern "C" int q3_swiglu_fwd(const void* gate, const void* up, void* y, int64_t n, int dtype, q3_stream_t stream) {
  if (!gate || !up || !y || n < 1) return Q3_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = aligned16(gate) && aligned16(up) && aligned16(y);
  Q3_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    if (vec) swiglu_fwd_kernel<T, V><<<ew_grid(cdiv(n, V)), kEwThreads, 0, st>>>((const T*)gate, (const T*)up, (T*)y, n);
    else swiglu_fwd_kernel<T, 1><<<ew_grid(n), kEwThreads, 0, st>>>((const T*)gate, (const T*)up, (T*)y, n);
  });
  return launch_status();
}

extern "C" int q3_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, int64_t n,
                             int dtype, q3_stream_t stream) {
  if (!gate || !up || !dy || !dgate || !dup || n < 1) return Q3_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = aligned16(gate) && aligned16(up) && aligned16(dy) && aligned16(dgate) && aligned16(dup);
  Q3_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    if (vec)
      swiglu_bwd_kernel<T, V><<<ew_grid(cdiv(n, V)), kEwThreads, 0, st>>>((const T*)gate, (const T*)up, (const T*)dy,
                                                                          (T*)dgate, (T*)dup, n);
    else
      swiglu_bwd_kernel<T, 1><<<ew_grid(n), kEwThreads, 0, st>>>((const T*)gate, (const T*)up, (const T*)dy,
                                                                 (T*)dgate, (T*)dup, n);
  });
  return launch_status();
}

extern "C" int q3_positions(int64_t* pos, int64_t n, int64_t seq, q3_stream_t stream) {
  if (!pos || n < 1 || seq < 1) return Q3_ERR_ARG;
  positions_kernel<<<ew_grid(n), kEwThreads, 0, (cudaStream_t)stream>>>(pos, n, seq);
  return launch_status();
}
