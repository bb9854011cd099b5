// Token embedding: vectorised row gather, and a dense deterministic weight gradient; both also for one
// contiguous shard of the vocabulary (rows [row_lo, row_lo + rows) of the table, fp32 master storage), which is
// what a vocabulary-parallel embedding needs.
//
// Backward: dW is zero-filled. A first kernel links equal token ids into chains: one warp per position scans
// forward for the next position with the same id (ballots, stops at the first hit) and marks that position as
// "has a predecessor". A second kernel gives every chain head (position without predecessor) the row of its
// id: it walks the chain in ascending position order, accumulates the dy rows in fp32 registers and writes the
// row once. One writer per row, fixed summation order, no float atomics; the id scan runs once, not once per
// column tile.
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

// Shard gather: rows of `w` (type TW, fp32 master or 16-bit) are table rows [row_lo, row_lo + rows); a token
// whose id falls outside gets a zero row (another rank owns it). Ids outside [0, vocab) flag Q3_STATUS_ID_RANGE.
template <typename TW, typename TO, typename I>
__global__ void __launch_bounds__(256) embedding_shard_fwd_kernel(const I* __restrict__ ids, const TW* __restrict__ w,
                                                                  TO* __restrict__ y, int64_t tokens, int64_t H,
                                                                  int64_t vocab, int64_t row_lo, int64_t rows,
                                                                  int* status) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t nvec = H / 8;   // H % 8 == 0 checked on the host
  for (int64_t t = blockIdx.x * (int64_t)warps + (threadIdx.x >> 5); t < tokens; t += (int64_t)gridDim.x * warps) {
    const int64_t id = (int64_t)ids[t];
    if ((id < 0 || id >= vocab) && lane == 0) flag_status(status, Q3_STATUS_ID_RANGE);
    const bool own = id >= row_lo && id < row_lo + rows;
    const TW* src = w + (own ? id - row_lo : 0) * H;
    TO* dst = y + t * H;
    for (int64_t i = lane; i < nvec; i += 32) {
      float v[8];
      if (own) VecIO<TW, 8>::load(src + i * 8, v);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
      }
      VecIO<TO, 8>::store(dst + i * 8, v);
    }
  }
}

// next[t] = next position after t with the same id (-1 if none); has_prev[next[t]] = 1. Positions whose id is
// outside [row_lo, row_lo + rows) take no part. has_prev must be zero on entry.
template <typename I>
__global__ void __launch_bounds__(256) embedding_chain_kernel(const I* __restrict__ ids, int* __restrict__ next,
                                                              int* __restrict__ has_prev, int64_t tokens,
                                                              int64_t row_lo, int64_t rows) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * (int64_t)warps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int64_t id = (int64_t)ids[t];
  int found = -1;
  if (id >= row_lo && id < row_lo + rows) {
    for (int64_t base = t + 1; base < tokens; base += 32) {
      const int64_t u = base + lane;
      const unsigned mask = __ballot_sync(0xffffffffu, u < tokens && (int64_t)ids[u] == id);
      if (mask) { found = (int)(base + __ffs(mask) - 1); break; }
    }
  }
  if (lane == 0) {
    next[t] = found;
    if (found >= 0) has_prev[found] = 1;
  }
}

// One warp per (position, 256-column tile): chain heads sum their chain's dy rows and write the row, scaled.
template <typename T, typename TO, typename I>
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const I* __restrict__ ids, const T* __restrict__ dy,
                                                            TO* __restrict__ dw, const int* __restrict__ next,
                                                            const int* __restrict__ has_prev, int64_t tokens,
                                                            int64_t H, int64_t row_lo, int64_t rows, float scale) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * (int64_t)warps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int64_t id = (int64_t)ids[t];
  if (id < row_lo || id >= row_lo + rows || has_prev[t]) return;
  const int64_t c0 = (int64_t)blockIdx.y * 256 + lane * 8;
  const bool vec = (H % 8 == 0);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int64_t u = t; u >= 0; u = next[u]) {
    if (vec) {
      if (c0 < H) {
        float v[8];
        VecIO<T, 8>::load(dy + u * H + c0, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += v[k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (c0 + k < H) acc[k] += to_f32<T>(dy[u * H + c0 + k]);
    }
  }
  TO* out = dw + (id - row_lo) * H;
  if (vec) {
    if (c0 < H) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] *= scale;
      VecIO<TO, 8>::store(out + c0, acc);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (c0 + k < H) out[c0 + k] = from_f32<TO>(acc[k] * scale);
  }
}

template <typename I>
static int chain_launch(const void* ids, void* workspace, int64_t workspace_bytes, int64_t tokens, int64_t row_lo,
                        int64_t rows, int** next, int** has_prev, cudaStream_t st) {
  if (tokens > 2147483647LL) return Q3_ERR_LIMIT;
  if (!workspace || workspace_bytes < tokens * 8) return Q3_ERR_WORKSPACE;
  *next = static_cast<int*>(workspace);
  *has_prev = *next + tokens;
  cudaError_t e = cudaMemsetAsync(*has_prev, 0, (size_t)tokens * 4, st);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  embedding_chain_kernel<I><<<(unsigned)cdiv(tokens, 8), 256, 0, st>>>((const I*)ids, *next, *has_prev, tokens, row_lo, rows);
  return Q3_OK;
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

extern "C" int64_t q3_embedding_bwd_workspace_bytes(int64_t tokens) { return tokens < 1 ? 16 : tokens * 8; }

extern "C" int q3_embedding_bwd(const void* ids, int ids_are_int64, const void* dy, void* dweight, void* workspace,
                                int64_t workspace_bytes, int64_t tokens, int64_t H, int64_t vocab, int dtype,
                                q3_stream_t stream) {
  if (!ids || !dy || !dweight) return Q3_ERR_ARG;
  if (tokens < 1 || H < 1 || vocab < 1) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t bytes = (size_t)vocab * (size_t)H * (size_t)dtype_size(dtype);
  cudaError_t e = cudaMemsetAsync(dweight, 0, bytes, st);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  int *next = nullptr, *has_prev = nullptr;
  int rc = ids_are_int64 ? chain_launch<int64_t>(ids, workspace, workspace_bytes, tokens, 0, vocab, &next, &has_prev, st)
                         : chain_launch<int32_t>(ids, workspace, workspace_bytes, tokens, 0, vocab, &next, &has_prev, st);
  if (rc != Q3_OK) return rc;
  if (H % 8 == 0 && !(aligned16(dy) && aligned16(dweight))) return Q3_ERR_ALIGN;   // the 8-wide path needs 16-byte rows
  dim3 grid((unsigned)cdiv(tokens, 8), (unsigned)cdiv(H, 256));
  Q3_DISPATCH_FLOAT(dtype, T, {
    if (ids_are_int64) embedding_bwd_kernel<T, T, int64_t><<<grid, 256, 0, st>>>((const int64_t*)ids, (const T*)dy, (T*)dweight, next, has_prev, tokens, H, 0, vocab, 1.f);
    else embedding_bwd_kernel<T, T, int32_t><<<grid, 256, 0, st>>>((const int32_t*)ids, (const T*)dy, (T*)dweight, next, has_prev, tokens, H, 0, vocab, 1.f);
  });
  return launch_status();
}

// Vocabulary-shard forms. weight_shard [rows, H] in w_dtype (fp32 master or the compute type) holds table rows
// [row_lo, row_lo + rows); y [tokens, H] in y_dtype (bf16 / fp16 / fp32) gets the row or zeros.
extern "C" int q3_embedding_shard_fwd(const void* ids, int ids_are_int64, const void* weight_shard, int w_dtype, void* y,
                                      int y_dtype, int64_t tokens, int64_t H, int64_t vocab, int64_t row_lo,
                                      int64_t rows, int* status, q3_stream_t stream) {
  if (!ids || !weight_shard || !y) return Q3_ERR_ARG;
  if (tokens < 1 || H < 1 || vocab < 1 || rows < 1 || row_lo < 0 || row_lo + rows > vocab) return Q3_ERR_SHAPE;
  if (H % 8 || !aligned16(weight_shard) || !aligned16(y)) return Q3_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  int64_t g = cdiv(tokens, 8), cap = (int64_t)sm_count() * 8;
  const int grid = (int)(g > cap ? cap : g);
#define Q3_ESF(TW, TO)                                                                                                  \
  do {                                                                                                                  \
    if (ids_are_int64) embedding_shard_fwd_kernel<TW, TO, int64_t><<<grid, 256, 0, st>>>((const int64_t*)ids, (const TW*)weight_shard, (TO*)y, tokens, H, vocab, row_lo, rows, status); \
    else embedding_shard_fwd_kernel<TW, TO, int32_t><<<grid, 256, 0, st>>>((const int32_t*)ids, (const TW*)weight_shard, (TO*)y, tokens, H, vocab, row_lo, rows, status); \
  } while (0)
  if (w_dtype == Q3_F32 && y_dtype == Q3_BF16) Q3_ESF(float, __nv_bfloat16);
  else if (w_dtype == Q3_F32 && y_dtype == Q3_F16) Q3_ESF(float, __half);
  else if (w_dtype == Q3_F32 && y_dtype == Q3_F32) Q3_ESF(float, float);
  else if (w_dtype == Q3_BF16 && y_dtype == Q3_BF16) Q3_ESF(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == Q3_F16 && y_dtype == Q3_F16) Q3_ESF(__half, __half);
  else return Q3_ERR_DTYPE;
#undef Q3_ESF
  return launch_status();
}

// dweight_shard [rows, H] fp32 = scale * sum over positions t with ids[t] in [row_lo, row_lo + rows) of dy[t, :]
// (dy in `dtype`), deterministic as q3_embedding_bwd. Workspace as q3_embedding_bwd_workspace_bytes(tokens).
extern "C" int q3_embedding_shard_bwd(const void* ids, int ids_are_int64, const void* dy, int dtype, float* dweight_shard,
                                      void* workspace, int64_t workspace_bytes, int64_t tokens, int64_t H,
                                      int64_t row_lo, int64_t rows, double scale, q3_stream_t stream) {
  if (!ids || !dy || !dweight_shard) return Q3_ERR_ARG;
  if (tokens < 1 || H < 1 || rows < 1 || row_lo < 0) return Q3_ERR_SHAPE;
  if (H % 8 || !aligned16(dy) || !aligned16(dweight_shard)) return Q3_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(dweight_shard, 0, (size_t)rows * (size_t)H * 4, st);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  int *next = nullptr, *has_prev = nullptr;
  int rc = ids_are_int64 ? chain_launch<int64_t>(ids, workspace, workspace_bytes, tokens, row_lo, rows, &next, &has_prev, st)
                         : chain_launch<int32_t>(ids, workspace, workspace_bytes, tokens, row_lo, rows, &next, &has_prev, st);
  if (rc != Q3_OK) return rc;
  dim3 grid((unsigned)cdiv(tokens, 8), (unsigned)cdiv(H, 256));
  Q3_DISPATCH_FLOAT(dtype, T, {
    if (ids_are_int64) embedding_bwd_kernel<T, float, int64_t><<<grid, 256, 0, st>>>((const int64_t*)ids, (const T*)dy, dweight_shard, next, has_prev, tokens, H, row_lo, rows, (float)scale);
    else embedding_bwd_kernel<T, float, int32_t><<<grid, 256, 0, st>>>((const int32_t*)ids, (const T*)dy, dweight_shard, next, has_prev, tokens, H, row_lo, rows, (float)scale);
  });
  return launch_status();
}
