// Token embedding: vectorised row gather, and a dense deterministic weight gradient.
//
// Backward: dW is zero-filled, then one warp per position t decides whether t is the first
// occurrence of its token id (ballot scan over earlier positions). The first occurrence owns the
// token: it walks the later positions in ascending order and accumulates the matching dy rows in
// fp32 registers, then writes the row once. One writer per row, fixed summation order, no float
// atomics, no T^2 masks: the id scan is T/32 ballots per warp.
//
// Replaces, in the reference: qwen3_triton/kernels/embedding.py:13-46 (_lookup/_zero/_backward).
#include "common.cuh"

namespace q3 {

template <typename T, typename I, int V>
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const I* __restrict__ ids, const T* __restrict__ w,
                                                            T* __restrict__ y, int64_t tokens, int64_t H, int64_t vocab,
                                                            int* status) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t nvec = H / V;
  for (int64_t t = blockIdx.x * (int64_t)warps + (threadIdx.x >> 5); t < tokens; t += (int64_t)gridDim.x * warps) {
    const int64_t id = (int64_t)ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && lane == 0) flag_status(status, Q3_STATUS_ID_RANGE);
    const T* src = w + (ok ? id : 0) * H;
    T* dst = y + t * H;
    for (int64_t i = lane; i < nvec; i += 32) {
      float v[V];
      if (ok) VecIO<T, V>::load(src + i * V, v);
      else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = 0.f;
      }
      VecIO<T, V>::store(dst + i * V, v);
    }
    for (int64_t i = nvec * V + lane; i < H; i += 32) dst[i] = ok ? src[i] : from_f32<T>(0.f);
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const I* __restrict__ ids, const T* __restrict__ dy,
                                                            T* __restrict__ dw, int64_t tokens, int64_t H,
                                                            int64_t vocab, int col_tile) {
  // grid.x: warp-sized groups of positions; grid.y: column tiles of `col_tile` elements (32 lanes x k).
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * (int64_t)warps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int64_t id = (int64_t)ids[t];
  if (id < 0 || id >= vocab) return;
  // first occurrence?
  for (int64_t base = 0; base < t; base += 32) {
    const int64_t u = base + lane;
    const bool hit = u < t && (int64_t)ids[u] == id;
    if (__ballot_sync(0xffffffffu, hit)) return;
  }
  const int64_t c0 = (int64_t)blockIdx.y * col_tile;
  constexpr int MAXC = 8;  // col_tile <= 32 * MAXC
  float acc[MAXC];
#pragma unroll
  for (int k = 0; k < MAXC; ++k) {
    const int64_t c = c0 + lane + 32 * k;
    acc[k] = (32 * k < col_tile && c < H) ? to_f32<T>(dy[t * H + c]) : 0.f;
  }
  for (int64_t base = t + 1; base < tokens; base += 32) {
    const int64_t u = base + lane;
    const bool hit = u < tokens && (int64_t)ids[u] == id;
    unsigned mask = __ballot_sync(0xffffffffu, hit);
    while (mask) {
      const int b = __ffs(mask) - 1;
      mask &= mask - 1;
      const int64_t src = base + b;
#pragma unroll
      for (int k = 0; k < MAXC; ++k) {
        const int64_t c = c0 + lane + 32 * k;
        if (32 * k < col_tile && c < H) acc[k] += to_f32<T>(dy[src * H + c]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < MAXC; ++k) {
    const int64_t c = c0 + lane + 32 * k;
    if (32 * k < col_tile && c < H) dw[id * H + c] = from_f32<T>(acc[k]);
  }
}

}  // namespace q3

using namespace q3;

extern "C" int q3_embedding_fwd(const void* ids, int ids_are_int64, const void* weight, void* y, int64_t tokens,
                                int64_t H, int64_t vocab, int dtype, int* status, q3_stream_t stream) {
  if (!ids || !weight || !y) return Q3_ERR_ARG;
  if (tokens < 1 || H < 1 || vocab < 1) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  int64_t g = cdiv(tokens, 8), cap = (int64_t)sm_count() * 8;
  const int grid = (int)(g > cap ? cap : g);
  Q3_DISPATCH_FLOAT(dtype, T, {
    constexpr int VF = Vec16<T>::N;
    const bool vec = aligned16(weight) && aligned16(y) && (H % VF == 0);
    if (ids_are_int64) {
      if (vec) embedding_fwd_kernel<T, int64_t, VF><<<grid, 256, 0, st>>>((const int64_t*)ids, (const T*)weight, (T*)y, tokens, H, vocab, status);
      else embedding_fwd_kernel<T, int64_t, 1><<<grid, 256, 0, st>>>((const int64_t*)ids, (const T*)weight, (T*)y, tokens, H, vocab, status);
    } else {
      if (vec) embedding_fwd_kernel<T, int32_t, VF><<<grid, 256, 0, st>>>((const int32_t*)ids, (const T*)weight, (T*)y, tokens, H, vocab, status);
      else embedding_fwd_kernel<T, int32_t, 1><<<grid, 256, 0, st>>>((const int32_t*)ids, (const T*)weight, (T*)y, tokens, H, vocab, status);
    }
  });
  return launch_status();
}

extern "C" int q3_embedding_bwd(const void* ids, int ids_are_int64, const void* dy, void* dweight, int64_t tokens,
                                int64_t H, int64_t vocab, int dtype, q3_stream_t stream) {
  if (!ids || !dy || !dweight) return Q3_ERR_ARG;
  if (tokens < 1 || H < 1 || vocab < 1) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t bytes = (size_t)vocab * (size_t)H * (size_t)dtype_size(dtype);
  cudaError_t e = cudaMemsetAsync(dweight, 0, bytes, st);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  const int col_tile = 256;
  dim3 grid((unsigned)cdiv(tokens, 8), (unsigned)cdiv(H, col_tile));
  Q3_DISPATCH_FLOAT(dtype, T, {
    if (ids_are_int64) embedding_bwd_kernel<T, int64_t><<<grid, 256, 0, st>>>((const int64_t*)ids, (const T*)dy, (T*)dweight, tokens, H, vocab, col_tile);
    else embedding_bwd_kernel<T, int32_t><<<grid, 256, 0, st>>>((const int32_t*)ids, (const T*)dy, (T*)dweight, tokens, H, vocab, col_tile);
  });
  return launch_status();
}
