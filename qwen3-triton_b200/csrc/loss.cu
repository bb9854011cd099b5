// Causal (internally shifted) token-mean cross-entropy over materialised logits, and the
// vocabulary-shard-local statistics / gradient kernels of the vocab-parallel head.
//
// Row (b, s) with s < S-1 is scored against labels[b, s+1]; rows are numbered
// row = b*(S-1)+s ("shifted") and physical = b*S+s. Each shifted row is one pass over its V
// logits (online max/sum per thread over 16-byte vectors, block combine), so the logits are read
// from HBM once in forward and once in backward. The mean is a fixed-order single-CTA reduction.
//
// Replaces, in the reference: qwen3_triton/kernels/loss.py:7-44 (_partials/_rows/_mean/_backward)
// and kernels/vocab_ce.py:15-75 (_local_rows/_pack/_finish/_means/_grad/_accum). Semantics follow
// model/qwen_tiny.py:224-227 (shifted F.cross_entropy on fp32 logits, ignore_index=-100).
#include "common.cuh"
#include <math_constants.h>

namespace q3 {

constexpr int kCeThreads = 512;
// The row-statistics kernel ends every row with a block-wide combine during which its CTA has no loads in flight.
// CTAs of 256 threads, four or more resident per SM, reach that point at different times and cover for each other.
constexpr int kCeRowThreads = 256;

struct MaxSum { float m, s; };

__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  MaxSum r;
  r.m = fmaxf(a.m, b.m);
  if (r.m == -CUDART_INF_F) { r.s = 0.f; return r; }
  r.s = a.s * __expf(a.m - r.m) + b.s * __expf(b.m - r.m);
  return r;
}

// Block-wide (max, sumexp) combine in a fixed order; result valid in every thread.
__device__ __forceinline__ MaxSum block_maxsum(MaxSum v, float* smm, float* sms) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other;
    other.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v = combine(v, other);
  }
  __syncthreads();
  if (lane == 0) { smm[warp] = v.m; sms[warp] = v.s; }
  __syncthreads();
  MaxSum t; t.m = smm[0]; t.s = sms[0];
  for (int i = 1; i < nwarp; ++i) { MaxSum o; o.m = smm[i]; o.s = sms[i]; t = combine(t, o); }
  return t;
}

// One CTA per shifted row (grid-stride): lse over the local vocabulary slice and the target logit
// if this slice owns the label (else 0).
template <typename T, int V>
__global__ void __launch_bounds__(kCeRowThreads, 4) ce_rows_kernel(const T* __restrict__ logits,
                                                             const int64_t* __restrict__ labels,
                                                             float* __restrict__ lse, float* __restrict__ target,
                                                             int64_t nrows, int64_t S, int64_t Vn, int64_t start,
                                                             int64_t ignore, int64_t vocab_total, int* status) {
  __shared__ float smm[32], sms[32];
  const int64_t nvec = Vn / V;
  for (int64_t row = blockIdx.x; row < nrows; row += gridDim.x) {
    const int64_t physical = (row / (S - 1)) * S + row % (S - 1);
    const T* x = logits + physical * Vn;
    MaxSum acc; acc.m = -CUDART_INF_F; acc.s = 0.f;
    // four vectors per iteration: the loads are independent of the running (max, sum), so issuing them
    // together keeps 64 B per thread in flight instead of 16 B
    int64_t i = threadIdx.x;
    for (; i + 3 * (int64_t)blockDim.x < nvec; i += 4 * (int64_t)blockDim.x) {
      float v[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u) VecIO<T, V>::load(x + (i + u * (int64_t)blockDim.x) * V, v[u]);
      float vm = v[0][0];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) vm = fmaxf(vm, v[u][j]);
      const float nm = fmaxf(acc.m, vm);
      float s = acc.s * __expf(acc.m - nm);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) s += __expf(v[u][j] - nm);
      acc.m = nm; acc.s = s;
    }
    for (; i < nvec; i += blockDim.x) {
      float v[V];
      VecIO<T, V>::load(x + i * V, v);
      float vm = v[0];
#pragma unroll
      for (int j = 1; j < V; ++j) vm = fmaxf(vm, v[j]);
      const float nm = fmaxf(acc.m, vm);
      float s = acc.s * __expf(acc.m - nm);
#pragma unroll
      for (int j = 0; j < V; ++j) s += __expf(v[j] - nm);
      acc.m = nm; acc.s = s;
    }
    for (int64_t i = nvec * V + threadIdx.x; i < Vn; i += blockDim.x) {
      MaxSum o; o.m = to_f32<T>(x[i]); o.s = 1.f;
      acc = combine(acc, o);
    }
    acc = block_maxsum(acc, smm, sms);
    if (threadIdx.x == 0) {
      const int64_t label = labels[physical + 1];
      float tv = 0.f;
      if (label != ignore) {
        if (label < 0 || label >= vocab_total) flag_status(status, Q3_STATUS_LABEL_RANGE);
        else if (label >= start && label < start + Vn) tv = to_f32<T>(x[label - start]);
      }
      lse[row] = acc.m + logf(acc.s);
      target[row] = tv;
    }
  }
}

// Single CTA: per-row loss, valid-target count and token mean, all in a fixed order.
__global__ void __launch_bounds__(1024) ce_mean_kernel(const float* __restrict__ lse, const float* __restrict__ target,
                                                       const int64_t* __restrict__ labels, float* __restrict__ losses,
                                                       float* __restrict__ loss, int* __restrict__ count, int64_t nrows,
                                                       int64_t S, int64_t ignore, int64_t vocab_total, int* status) {
  __shared__ float sm[32];
  __shared__ int smi[32];
  float total = 0.f;
  int cnt = 0;
  for (int64_t row = threadIdx.x; row < nrows; row += blockDim.x) {
    const int64_t physical = (row / (S - 1)) * S + row % (S - 1);
    const int64_t label = labels[physical + 1];
    const bool valid = label != ignore && label >= 0 && label < vocab_total;
    const float l = valid ? lse[row] - target[row] : 0.f;
    losses[row] = l;
    total += l;
    cnt += valid ? 1 : 0;
  }
  total = block_sum(total, sm);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  __syncthreads();
  if (lane == 0) smi[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = 0;
    for (int i = 0; i < nwarp; ++i) c += smi[i];
    *count = c;
    *loss = total / (float)c;
    if (c == 0) flag_status(status, Q3_STATUS_EMPTY_TARGETS);
  }
}

// dlogits[physical, col] = (exp(x - lse[row]) - [col + start == label]) * up[source] / count[source]
// for scored rows, 0 elsewhere (last position of each sequence, ignored or out-of-range labels).
template <typename T, int V>
__global__ void __launch_bounds__(kCeThreads) ce_grad_kernel(const T* __restrict__ logits,
                                                             const int64_t* __restrict__ labels,
                                                             const float* __restrict__ lse,
                                                             const int* __restrict__ counts,
                                                             const float* __restrict__ ups, T* __restrict__ dz,
                                                             int64_t nphys, int64_t rows_per_rank, int64_t S,
                                                             int64_t Vn, int64_t start, int64_t ignore,
                                                             int64_t vocab_total) {
  const int64_t nvec = Vn / V;
  for (int64_t physical = blockIdx.x; physical < nphys; physical += gridDim.x) {
    const bool scored = (physical % S) < S - 1;
    const int64_t label = scored ? labels[physical + 1] : ignore;
    const bool valid = scored && label != ignore && label >= 0 && label < vocab_total;
    const T* x = logits + physical * Vn;
    T* o = dz + physical * Vn;
    if (!valid) {
      float z[V];
#pragma unroll
      for (int j = 0; j < V; ++j) z[j] = 0.f;
      for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) VecIO<T, V>::store(o + i * V, z);
      for (int64_t i = nvec * V + threadIdx.x; i < Vn; i += blockDim.x) o[i] = from_f32<T>(0.f);
      continue;
    }
    const int64_t source = physical / rows_per_rank;
    const int64_t row = (physical / S) * (S - 1) + physical % S;
    const float l = lse[row];
    const float scale = ups[source] / (float)counts[source];
    const int64_t hot = label - start;  // may fall outside [0, Vn): then no column matches
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
      float v[V];
      VecIO<T, V>::load(x + i * V, v);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = (__expf(v[j] - l) - ((i * V + j) == hot ? 1.f : 0.f)) * scale;
      VecIO<T, V>::store(o + i * V, v);
    }
    for (int64_t i = nvec * V + threadIdx.x; i < Vn; i += blockDim.x)
      o[i] = from_f32<T>((__expf(to_f32<T>(x[i]) - l) - (i == hot ? 1.f : 0.f)) * scale);
  }
}

// pack[0][i] = exp(lse_local[i] - max[i]); pack[1][i] = target[i]
__global__ void vce_pack_kernel(const float* lse_local, const float* maximum, const float* target, float* pack,
                                int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    pack[i] = expf(lse_local[i] - maximum[i]);
    pack[n + i] = target[i];
  }
}

// lse = max + log(sumexp); losses = ignored ? 0 : lse - target
__global__ void vce_finish_kernel(const float* maximum, const float* pack, const int64_t* labels, float* lse,
                                  float* losses, int64_t n, int64_t S, int64_t ignore) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float l = maximum[i] + logf(pack[i]);
    const int64_t physical = (i / (S - 1)) * S + i % (S - 1);
    lse[i] = l;
    losses[i] = labels[physical + 1] == ignore ? 0.f : l - pack[n + i];
  }
}

// One CTA per data rank: count of valid targets and mean loss of that rank's rows (fixed order).
__global__ void __launch_bounds__(1024) vce_means_kernel(const float* losses, const int64_t* labels, int* counts,
                                                         float* means, int64_t rows_per_rank, int64_t S,
                                                         int64_t ignore, int* status) {
  __shared__ float sm[32];
  __shared__ int smi[32];
  const int64_t source = blockIdx.x, n = rows_per_rank / S * (S - 1);
  float total = 0.f;
  int cnt = 0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const int64_t physical = source * rows_per_rank + (i / (S - 1)) * S + i % (S - 1);
    cnt += labels[physical + 1] != ignore ? 1 : 0;
    total += losses[source * n + i];
  }
  total = block_sum(total, sm);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  __syncthreads();
  if (lane == 0) smi[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = 0;
    for (int i = 0; i < nwarp; ++i) c += smi[i];
    counts[source] = c;
    means[source] = total / (float)c;
    if (c == 0) flag_status(status, Q3_STATUS_EMPTY_TARGETS);
  }
}

// out = (first ? 0 : out) + partial * (1/world), fp32 accumulate of a (possibly bf16) partial.
template <typename T>
__global__ void vce_accum_kernel(const T* partial, float* out, int64_t n, float inv_world, int first) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = to_f32<T>(partial[i]) * inv_world;
    out[i] = first ? v : out[i] + v;
  }
}

// labels_eff[b*S+s] = labels[b, s+1] for s < S-1 (out-of-range values flagged and treated as ignored), else ignore
__global__ void shift_labels_kernel(const int64_t* labels, int64_t* eff, int64_t n, int64_t S, int64_t ignore,
                                    int64_t vocab_total, int* status) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t l = ignore;
    if (i % S < S - 1) {
      l = labels[i + 1];
      if (l != ignore && (l < 0 || l >= vocab_total)) { flag_status(status, Q3_STATUS_LABEL_RANGE); l = ignore; }
    }
    eff[i] = l;
  }
}

// lse_local[row] from the per-tile (max, sum exp) partials, combined in tile order
__global__ void lce_combine_kernel(const float* part_max, const float* part_sum, float* lse, int64_t rows, int tiles) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
    float m = part_max[r * tiles], s = part_sum[r * tiles];
    for (int t = 1; t < tiles; ++t) {
      const float pm = part_max[r * tiles + t], ps = part_sum[r * tiles + t];
      const float nm = fmaxf(m, pm);
      s = s * __expf(m - nm) + ps * __expf(pm - nm);
      m = nm;
    }
    lse[r] = m + logf(s);
  }
}

// One CTA per data rank over physical rows: losses, valid-target count, mean (fixed order).
__global__ void __launch_bounds__(1024) lce_finish_kernel(const float* lse, const float* target, const int64_t* eff,
                                                          float* losses, int* counts, float* means,
                                                          int64_t rows_per_rank, int64_t ignore, int* status) {
  __shared__ float sm[32];
  __shared__ int smi[32];
  const int64_t source = blockIdx.x;
  float total = 0.f;
  int cnt = 0;
  for (int64_t i = threadIdx.x; i < rows_per_rank; i += blockDim.x) {
    const int64_t r = source * rows_per_rank + i;
    const bool valid = eff[r] != ignore;
    const float l = valid ? lse[r] - target[r] : 0.f;
    losses[r] = l;
    total += l;
    cnt += valid ? 1 : 0;
  }
  total = block_sum(total, sm);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  __syncthreads();
  if (lane == 0) smi[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = 0;
    for (int i = 0; i < nwarp; ++i) c += smi[i];
    counts[source] = c;
    means[source] = total / (float)c;
    if (c == 0) flag_status(status, Q3_STATUS_EMPTY_TARGETS);
  }
}

__global__ void lce_global_lse_kernel(const float* maximum, const float* pack, float* lse, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    lse[i] = maximum[i] + logf(pack[i]);
}

inline int small_grid(int64_t n, int threads) {
  int64_t g = cdiv(n, threads), cap = (int64_t)sm_count() * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace q3

using namespace q3;

extern "C" int q3_ce_local_rows(const void* logits, const int64_t* labels, float* lse_local, float* target,
                                int64_t physical_rows, int64_t S, int64_t V_local, int64_t vocab_start,
                                int64_t vocab_total, int64_t ignore_index, int dtype, int* status,
                                q3_stream_t stream) {
  if (!logits || !labels || !lse_local || !target) return Q3_ERR_ARG;
  if (physical_rows < 1 || S < 2 || physical_rows % S || V_local < 1) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t nrows = physical_rows / S * (S - 1);
  const int grid = (int)(nrows < (int64_t)sm_count() * 8 ? nrows : (int64_t)sm_count() * 8);
  Q3_DISPATCH_FLOAT(dtype, T, {
    constexpr int VF = Vec16<T>::N;
    // every row start must be 16-byte aligned for the vector path
    const bool vec = aligned16(logits) && (V_local % VF == 0);
    if (vec) ce_rows_kernel<T, VF><<<grid, kCeRowThreads, 0, st>>>((const T*)logits, labels, lse_local, target, nrows, S,
                                                               V_local, vocab_start, ignore_index, vocab_total, status);
    else ce_rows_kernel<T, 1><<<grid, kCeRowThreads, 0, st>>>((const T*)logits, labels, lse_local, target, nrows, S,
                                                          V_local, vocab_start, ignore_index, vocab_total, status);
  });
  return launch_status();
}

extern "C" int q3_ce_fwd(const void* logits, const int64_t* labels, float* lse, float* target, float* losses,
                         float* loss, int* count, int64_t B, int64_t S, int64_t V, int64_t ignore_index, int dtype,
                         int* status, q3_stream_t stream) {
  if (!losses || !loss || !count) return Q3_ERR_ARG;
  if (B < 1) return Q3_ERR_SHAPE;
  int rc = q3_ce_local_rows(logits, labels, lse, target, B * S, S, V, 0, V, ignore_index, dtype, status, stream);
  if (rc != Q3_OK) return rc;
  ce_mean_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(lse, target, labels, losses, loss, count, B * (S - 1), S,
                                                       ignore_index, V, status);
  return launch_status();
}

extern "C" int q3_ce_grad(const void* logits, const int64_t* labels, const float* lse, const int* counts,
                          const float* upstream, void* dlogits, int64_t physical_rows, int64_t rows_per_rank,
                          int64_t S, int64_t V_local, int64_t vocab_start, int64_t vocab_total, int64_t ignore_index,
                          int dtype, q3_stream_t stream) {
  if (!logits || !labels || !lse || !counts || !upstream || !dlogits) return Q3_ERR_ARG;
  if (physical_rows < 1 || S < 2 || physical_rows % S || V_local < 1 || rows_per_rank < 1 ||
      physical_rows % rows_per_rank)
    return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (int)(physical_rows < (int64_t)sm_count() * 4 ? physical_rows : (int64_t)sm_count() * 4);
  Q3_DISPATCH_FLOAT(dtype, T, {
    constexpr int VF = Vec16<T>::N;
    const bool vec = aligned16(logits) && aligned16(dlogits) && (V_local % VF == 0);
    if (vec) ce_grad_kernel<T, VF><<<grid, kCeThreads, 0, st>>>((const T*)logits, labels, lse, counts, upstream,
                                                               (T*)dlogits, physical_rows, rows_per_rank, S, V_local,
                                                               vocab_start, ignore_index, vocab_total);
    else ce_grad_kernel<T, 1><<<grid, kCeThreads, 0, st>>>((const T*)logits, labels, lse, counts, upstream,
                                                          (T*)dlogits, physical_rows, rows_per_rank, S, V_local,
                                                          vocab_start, ignore_index, vocab_total);
  });
  return launch_status();
}

extern "C" int q3_vce_pack(const float* lse_local, const float* maximum, const float* target, float* pack, int64_t n,
                           q3_stream_t stream) {
  if (!lse_local || !maximum || !target || !pack || n < 1) return Q3_ERR_ARG;
  vce_pack_kernel<<<small_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(lse_local, maximum, target, pack, n);
  return launch_status();
}

extern "C" int q3_vce_finish(const float* maximum, const float* pack, const int64_t* labels, float* lse,
                             float* losses, int* counts, float* means, int64_t n, int64_t rows_per_rank, int64_t S,
                             int64_t world, int64_t ignore_index, int* status, q3_stream_t stream) {
  if (!maximum || !pack || !labels || !lse || !losses || !counts || !means) return Q3_ERR_ARG;
  if (n < 1 || S < 2 || world < 1 || rows_per_rank < S || rows_per_rank % S) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  vce_finish_kernel<<<small_grid(n, 256), 256, 0, st>>>(maximum, pack, labels, lse, losses, n, S, ignore_index);
  vce_means_kernel<<<(int)world, 1024, 0, st>>>(losses, labels, counts, means, rows_per_rank, S, ignore_index, status);
  return launch_status();
}

extern "C" int q3_vce_accumulate(const void* partial, int partial_dtype, float* out, int64_t n, int64_t world,
                                 int first, q3_stream_t stream) {
  if (!partial || !out || n < 1 || world < 1) return Q3_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const float iw = 1.f / (float)world;
  Q3_DISPATCH_FLOAT(partial_dtype, T,
                    (vce_accum_kernel<T><<<small_grid(n, 256), 256, 0, st>>>((const T*)partial, out, n, iw, first)));
  return launch_status();
}

extern "C" int q3_shift_labels(const int64_t* labels, int64_t* labels_eff, int64_t rows, int64_t S,
                               int64_t ignore_index, int64_t vocab_total, int* status, q3_stream_t stream) {
  if (!labels || !labels_eff) return Q3_ERR_ARG;
  if (rows < 1 || S < 2 || rows % S) return Q3_ERR_SHAPE;
  shift_labels_kernel<<<small_grid(rows, 256), 256, 0, (cudaStream_t)stream>>>(labels, labels_eff, rows, S, ignore_index,
                                                                            vocab_total, status);
  return launch_status();
}

extern "C" int q3_linear_ce_combine(const float* part_max, const float* part_sum, float* lse_local, int64_t rows,
                                    int64_t tiles, q3_stream_t stream) {
  if (!part_max || !part_sum || !lse_local) return Q3_ERR_ARG;
  if (rows < 1 || tiles < 1) return Q3_ERR_SHAPE;
  lce_combine_kernel<<<small_grid(rows, 128), 128, 0, (cudaStream_t)stream>>>(part_max, part_sum, lse_local, rows, (int)tiles);
  return launch_status();
}

// lse = maximum + log(pack[0]) when the statistics were all-reduced (pass maximum = NULL to use lse_in as is);
// then per data rank: losses, counts, means over physical rows.
extern "C" int q3_linear_ce_finish(const float* maximum, const float* pack, float* lse, const float* target,
                                   const int64_t* labels_eff, float* losses, int* counts, float* means, int64_t rows,
                                   int64_t rows_per_rank, int64_t ignore_index, int* status, q3_stream_t stream) {
  if (!lse || !target || !labels_eff || !losses || !counts || !means) return Q3_ERR_ARG;
  if (rows < 1 || rows_per_rank < 1 || rows % rows_per_rank) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (maximum != nullptr) {
    if (!pack) return Q3_ERR_ARG;
    lce_global_lse_kernel<<<small_grid(rows, 256), 256, 0, st>>>(maximum, pack, lse, rows);
  }
  lce_finish_kernel<<<(int)(rows / rows_per_rank), 1024, 0, st>>>(lse, target, labels_eff, losses, counts, means,
                                                                 rows_per_rank, ignore_index, status);
  return launch_status();
}
