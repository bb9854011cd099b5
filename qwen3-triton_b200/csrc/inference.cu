// Decode-time kernels: positions, KV-cache append, attention over the cache, small-M linear (GEMV) and greedy token
// selection. All of them are bound by HBM traffic (the cache, the weight matrix, the logits), so the work is laid out
// to read each byte once with 16-byte accesses:
//   * attention over the cache runs one CTA per (batch, kv head, chunk of 256 keys) and serves ALL query heads of the
//     group from one pass over that K/V chunk (grouped-query attention: 4 query heads share a kv head in Qwen3, so
//     the cache is read once instead of four times), then a small merge kernel combines the chunks;
//   * the GEMV gives every warp one weight row and streams it once for up to 8 input rows;
//   * the argmax reads the logits once, ties resolved to the lowest index.
//
// Replaces, in the reference: qwen3_triton/inference/kernels.py:12-22 (positions), :25-36 (append), :39-115
// (cached / split-decode attention), :117-148 (GEMV linear), :150-173 (argmax parts + select).
#include "common.cuh"
#include <math_constants.h>

namespace q3 {
namespace inf {

__global__ void positions_kernel(int64_t* __restrict__ pos, int64_t n, int64_t seq, int64_t start) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) pos[i] = start + i % seq;
}

// k, v [B, S, H, D] (token-major, as the projections produce them) -> cache [B, H, C, D] at tokens start .. start+S-1.
// One 16-byte vector per thread; D * sizeof(T) is a multiple of 16.
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ ck, T* __restrict__ cv,
                                 int64_t B, int64_t S, int64_t H, int64_t D, int64_t C, int64_t start) {
  constexpr int W = 16 / (int)sizeof(T);
  const int64_t vec_per_row = D / W, total = B * S * H * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = i % vec_per_row, row = i / vec_per_row;          // row = (b * S + s) * H + h
    const int64_t h = row % H, s = (row / H) % S, b = row / (H * S);
    const int64_t dst = ((b * H + h) * C + start + s) * D + c * W;
    *reinterpret_cast<uint4*>(ck + dst) = *reinterpret_cast<const uint4*>(k + row * D + c * W);
    *reinterpret_cast<uint4*>(cv + dst) = *reinterpret_cast<const uint4*>(v + row * D + c * W);
  }
}

constexpr int kChunk = 256;        // keys per CTA
constexpr int kAttnThreads = 256;  // 8 warps; a warp covers two keys per step (16 lanes per key row)
constexpr int kMaxGroup = 8;       // query heads per kv head served by one CTA

// Partial attention of one query token against one chunk of cached keys, for the G query heads of a kv head.
//   q      [B, S, Hq, D]       cache_k / cache_v [B, Hkv, C, D]
//   part   [B, S, Hq, splits, D] fp32 (normalised within the chunk)   lse [B, S, Hq, splits] fp32 (natural log)
// Key t is visible to query token s iff t <= start + s and t < T = start + S. EPL = D / 16 elements per lane.
template <typename T, int EPL, int G>
__global__ void __launch_bounds__(kAttnThreads)
cache_attention_partial_kernel(const T* __restrict__ q, const T* __restrict__ ck, const T* __restrict__ cv,
                               float* __restrict__ part, float* __restrict__ lse, int64_t S, int64_t Hq, int64_t Hkv,
                               int64_t C, int64_t start, int splits, float scale) {
  constexpr int D = EPL * 16;
  const int split = blockIdx.x, s = blockIdx.y;
  const int64_t bk = blockIdx.z, b = bk / Hkv, kvh = bk % Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  const int64_t visible = start + s + 1;                      // keys 0 .. visible-1
  const int64_t first = (int64_t)split * kChunk;
  int64_t last = first + kChunk;
  if (last > visible) last = visible;

  __shared__ float s_max[8][G], s_sum[8][G];
  __shared__ float s_acc[8][G][D];

  // this lane's slice of the G query vectors, pre-scaled
  float qv[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const T* qp = q + (((b * S + s) * Hq) + kvh * G + g) * D + sub * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[g][e] = to_f32<T>(qp[e]) * scale;
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -CUDART_INF_F; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }
  const T* kbase = ck + (bk * C) * D;
  const T* vbase = cv + (bk * C) * D;
  // warp w takes keys first + 2*w + half, stepping by 16 (8 warps x 2 keys)
  for (int64_t t0 = first + 2 * warp; t0 < last; t0 += 16) {
    const int64_t t = t0 + half;
    const bool live = t < last;
    float kk[EPL], vv[EPL];
    if (live) {
      constexpr int W = (16 / (int)sizeof(T)) < EPL ? (16 / (int)sizeof(T)) : EPL;   // 8- or 16-byte accesses
#pragma unroll
      for (int c = 0; c < EPL / W; ++c) {
        float tmp[W];
        VecIO<T, W>::load(kbase + t * D + sub * EPL + c * W, tmp);
#pragma unroll
        for (int e = 0; e < W; ++e) kk[c * W + e] = tmp[e];
        VecIO<T, W>::load(vbase + t * D + sub * EPL + c * W, tmp);
#pragma unroll
        for (int e = 0; e < W; ++e) vv[c * W + e] = tmp[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) { kk[e] = 0.f; vv[e] = 0.f; }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) dot = fmaf(qv[g][e], kk[e], dot);
      dot = group_sum<16>(dot);                               // the 16 lanes of a key row
      const float sc = live ? dot : -CUDART_INF_F;
      const float nm = fmaxf(m[g], sc);
      if (nm > -CUDART_INF_F) {
        const float alpha = __expf(m[g] - nm);                // m = -inf on the first visible key -> 0
        const float p = live ? __expf(sc - nm) : 0.f;
        l[g] = l[g] * alpha + p;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(acc[g][e], alpha, p * vv[e]);
        m[g] = nm;
      }
    }
  }
  // fold the two half-warps (different keys, same columns), then the 8 warps through shared memory
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float om = __shfl_xor_sync(0xffffffffu, m[g], 16), ol = __shfl_xor_sync(0xffffffffu, l[g], 16);
    const float nm = fmaxf(m[g], om);
    const float a = nm > -CUDART_INF_F ? __expf(m[g] - nm) : 0.f, bsc = nm > -CUDART_INF_F ? __expf(om - nm) : 0.f;
    l[g] = l[g] * a + ol * bsc;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float oa = __shfl_xor_sync(0xffffffffu, acc[g][e], 16);
      acc[g][e] = acc[g][e] * a + oa * bsc;
    }
    m[g] = nm;
    if (lane == 0) { s_max[warp][g] = m[g]; s_sum[warp][g] = l[g]; }
    if (half == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) s_acc[warp][g][sub * EPL + e] = acc[g][e];
    }
  }
  __syncthreads();
  // thread (g, column) combines the 8 warps in warp order: deterministic
  for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
    const int g = idx / D, d = idx % D;
    float nm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 8; ++w) nm = fmaxf(nm, s_max[w][g]);
    float tot = 0.f, val = 0.f;
    if (nm > -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float f = __expf(s_max[w][g] - nm);
        tot += s_sum[w][g] * f;
        val += s_acc[w][g][d] * f;
      }
    }
    const int64_t row = ((b * S + s) * Hq + kvh * G + g) * splits + split;
    part[row * D + d] = tot > 0.f ? val / tot : 0.f;
    if (d == 0) lse[row] = tot > 0.f ? nm + __logf(tot) : -CUDART_INF_F;
  }
}

// out[row, :] = sum_i part[row, i, :] * exp(lse[row, i] - max) / sum_i exp(lse[row, i] - max); one warp per row.
template <typename T>
__global__ void cache_attention_merge_kernel(const float* __restrict__ part, const float* __restrict__ lse,
                                             T* __restrict__ out, int64_t rows, int splits, int D) {
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = -CUDART_INF_F;
  for (int i = 0; i < splits; ++i) mx = fmaxf(mx, lse[row * splits + i]);
  float denom = 0.f;
  for (int i = 0; i < splits; ++i) denom += __expf(lse[row * splits + i] - mx);   // same order in every lane
  for (int d = lane; d < D; d += 32) {
    float val = 0.f;
    for (int i = 0; i < splits; ++i) val += part[(row * splits + i) * D + d] * __expf(lse[row * splits + i] - mx);
    out[row * D + d] = from_f32<T>(val / denom);
  }
}

// y[m, n] = sum_k x[m, k] * w[n, k], M <= 8: a warp owns one n and streams its weight row once, 16 bytes per lane and
// step, against all M input rows (those stay in L1/L2). ACC = float, or double for the `accurate` mode.
template <typename T, typename ACC, int M>
__global__ void __launch_bounds__(256)
gemv_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, int64_t N, int64_t K) {
  constexpr int W = 16 / (int)sizeof(T);
  const int64_t n = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (n >= N) return;
  ACC acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = (ACC)0;
  const T* wr = w + n * K;
  const int64_t kvec = K / W * W;
  for (int64_t k = (int64_t)lane * W; k < kvec; k += 32 * W) {
    float wv[W];
    VecIO<T, W>::load(wr + k, wv);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float xv[W];
      VecIO<T, W>::load(x + m * K + k, xv);
#pragma unroll
      for (int e = 0; e < W; ++e) acc[m] += (ACC)(wv[e] * xv[e]);
    }
  }
  for (int64_t k = kvec + lane; k < K; k += 32) {
    const float wv = to_f32<T>(wr[k]);
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] += (ACC)(wv * to_f32<T>(x[m * K + k]));
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    ACC v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) y[m * N + n] = from_f32<T>((float)v);
  }
}

// Row-wise argmax (lowest index among equal maxima), then the decode bookkeeping of one step: a finished row emits
// `pad`; the token goes to ids[row, position] and next[row]; a row that emits an end-of-sequence id becomes finished.
template <typename T>
__global__ void __launch_bounds__(1024)
select_kernel(const T* __restrict__ logits, int64_t V, int64_t* __restrict__ ids, int64_t ids_stride, int64_t position,
              int64_t* __restrict__ next, uint8_t* __restrict__ done, const int64_t* __restrict__ eos, int n_eos,
              int64_t pad) {
  __shared__ float s_val[32];
  __shared__ int64_t s_idx[32];
  const int64_t row = blockIdx.x;
  const T* x = logits + row * V;
  float best = -CUDART_INF_F;
  int64_t where = INT64_MAX;
  for (int64_t i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = to_f32<T>(x[i]);
    if (v > best || (v == best && i < where)) { best = v; where = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, where, o);
    if (ov > best || (ov == best && oi < where)) { best = ov; where = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = where; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < where)) { best = s_val[w]; where = s_idx[w]; }
    const bool was_done = done[row] != 0;
    const int64_t token = was_done ? pad : (where == INT64_MAX ? 0 : where);
    bool end = false;
    for (int e = 0; e < n_eos; ++e) end |= (token == eos[e]);
    ids[row * ids_stride + position] = token;
    next[row] = token;
    done[row] = (was_done || end) ? 1 : 0;
  }
}

}  // namespace inf
}  // namespace q3

using namespace q3;

extern "C" int q3_inf_positions(int64_t* pos, int64_t batch, int64_t seq, int64_t start, q3_stream_t stream) {
  if (!pos) return Q3_ERR_ARG;
  if (batch < 1 || seq < 1 || start < 0) return Q3_ERR_SHAPE;
  const int64_t n = batch * seq;
  inf::positions_kernel<<<(unsigned)cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>(pos, n, seq, start);
  return launch_status();
}

extern "C" int q3_kv_append(const void* k, const void* v, void* cache_k, void* cache_v, int64_t B, int64_t S, int64_t H,
                            int64_t D, int64_t C, int64_t start, int dtype, q3_stream_t stream) {
  if (!k || !v || !cache_k || !cache_v) return Q3_ERR_ARG;
  if (B < 1 || S < 1 || H < 1 || D < 1 || start < 0 || start + S > C) return Q3_ERR_SHAPE;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  if ((D * dtype_size(dtype)) % 16 || !aligned16(k) || !aligned16(v) || !aligned16(cache_k) || !aligned16(cache_v))
    return Q3_ERR_ALIGN;
  const int64_t vecs = B * S * H * (D * dtype_size(dtype) / 16);
  const int64_t want = cdiv(vecs, 256), cap = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  cudaStream_t st = (cudaStream_t)stream;
  Q3_DISPATCH_FLOAT(dtype, T, (inf::kv_append_kernel<T><<<grid, 256, 0, st>>>((const T*)k, (const T*)v, (T*)cache_k,
                                                                               (T*)cache_v, B, S, H, D, C, start)));
  return launch_status();
}

extern "C" int64_t q3_cache_attention_workspace_bytes(int64_t B, int64_t S, int64_t Hq, int64_t D, int64_t start) {
  if (B < 1 || S < 1 || Hq < 1 || D < 1 || start < 0) return 0;
  const int64_t splits = cdiv(start + S, inf::kChunk);
  return B * S * Hq * splits * (D + 1) * 4;
}

namespace {
template <typename T, int EPL>
int launch_cache_attention(const void* q, const void* ck, const void* cv, void* out, float* part, float* lse, int64_t B,
                           int64_t S, int64_t Hq, int64_t Hkv, int64_t C, int64_t start, float scale, cudaStream_t st) {
  const int G = (int)(Hq / Hkv);
  const int splits = (int)cdiv(start + S, inf::kChunk);
  dim3 grid((unsigned)splits, (unsigned)S, (unsigned)(B * Hkv));
#define Q3_CASE(GG)                                                                                             \
  case GG:                                                                                                      \
    inf::cache_attention_partial_kernel<T, EPL, GG><<<grid, inf::kAttnThreads, 0, st>>>(                        \
        (const T*)q, (const T*)ck, (const T*)cv, part, lse, S, Hq, Hkv, C, start, splits, scale);               \
    break;
  switch (G) {
    Q3_CASE(1) Q3_CASE(2) Q3_CASE(4)
    case 8:
      if constexpr (EPL <= 8) {     // 8 warps x 8 heads x D fp32 of combine space must fit 48 KB
        inf::cache_attention_partial_kernel<T, EPL, 8><<<grid, inf::kAttnThreads, 0, st>>>(
            (const T*)q, (const T*)ck, (const T*)cv, part, lse, S, Hq, Hkv, C, start, splits, scale);
        break;
      }
      return Q3_ERR_SHAPE;
    default: return Q3_ERR_SHAPE;
  }
#undef Q3_CASE
  int rc = launch_status();
  if (rc != Q3_OK) return rc;
  const int64_t rows = B * S * Hq;
  inf::cache_attention_merge_kernel<T><<<(unsigned)cdiv(rows, 8), 256, 0, st>>>(part, lse, (T*)out, rows, splits, EPL * 16);
  return launch_status();
}
}  // namespace

extern "C" int q3_cache_attention(const void* q, const void* cache_k, const void* cache_v, void* out, void* workspace,
                                  int64_t workspace_bytes, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t D,
                                  int64_t C, int64_t start, double scale, int dtype, q3_stream_t stream) {
  if (!q || !cache_k || !cache_v || !out) return Q3_ERR_ARG;
  if (B < 1 || S < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv || start < 0 || start + S > C || S > 65535 || B * Hkv > 65535)
    return Q3_ERR_SHAPE;
  if (D != 64 && D != 128 && D != 256) return Q3_ERR_SHAPE;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  if (!aligned16(q) || !aligned16(cache_k) || !aligned16(cache_v) || !aligned16(out)) return Q3_ERR_ALIGN;
  if (!workspace || workspace_bytes < q3_cache_attention_workspace_bytes(B, S, Hq, D, start)) return Q3_ERR_WORKSPACE;
  const int64_t splits = cdiv(start + S, inf::kChunk);
  float* part = (float*)workspace;
  float* lse = part + B * S * Hq * splits * D;
  cudaStream_t st = (cudaStream_t)stream;
  const float sc = (float)scale;
  Q3_DISPATCH_FLOAT(dtype, T, {
    if (D == 64) return launch_cache_attention<T, 4>(q, cache_k, cache_v, out, part, lse, B, S, Hq, Hkv, C, start, sc, st);
    if (D == 128) return launch_cache_attention<T, 8>(q, cache_k, cache_v, out, part, lse, B, S, Hq, Hkv, C, start, sc, st);
    return launch_cache_attention<T, 16>(q, cache_k, cache_v, out, part, lse, B, S, Hq, Hkv, C, start, sc, st);
  });
  return Q3_OK;
}

extern "C" int q3_gemv(const void* x, const void* weight, void* y, int64_t M, int64_t N, int64_t K, int dtype,
                       int accurate, q3_stream_t stream) {
  if (!x || !weight || !y) return Q3_ERR_ARG;
  if (M < 1 || M > 8 || N < 1 || K < 1) return Q3_ERR_SHAPE;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  if ((K * dtype_size(dtype)) % 16 || !aligned16(x) || !aligned16(weight)) return Q3_ERR_ALIGN;
  const unsigned grid = (unsigned)cdiv(N, 8);
  cudaStream_t st = (cudaStream_t)stream;
#define Q3_GEMV(MM)                                                                                                   \
  case MM:                                                                                                            \
    if (accurate) inf::gemv_kernel<T, double, MM><<<grid, 256, 0, st>>>((const T*)x, (const T*)weight, (T*)y, N, K);   \
    else inf::gemv_kernel<T, float, MM><<<grid, 256, 0, st>>>((const T*)x, (const T*)weight, (T*)y, N, K);             \
    break;
  Q3_DISPATCH_FLOAT(dtype, T, {
    switch ((int)M) { Q3_GEMV(1) Q3_GEMV(2) Q3_GEMV(3) Q3_GEMV(4) Q3_GEMV(5) Q3_GEMV(6) Q3_GEMV(7) Q3_GEMV(8) }
  });
#undef Q3_GEMV
  return launch_status();
}

extern "C" int q3_select_tokens(const void* logits, int64_t B, int64_t V, int64_t* ids, int64_t ids_stride,
                                int64_t position, int64_t* next_token, uint8_t* done, const int64_t* eos_ids, int n_eos,
                                int64_t pad, int dtype, q3_stream_t stream) {
  if (!logits || !ids || !next_token || !done || (n_eos > 0 && !eos_ids)) return Q3_ERR_ARG;
  if (B < 1 || V < 1 || position < 0 || position >= ids_stride || n_eos < 0) return Q3_ERR_SHAPE;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  Q3_DISPATCH_FLOAT(dtype, T, (inf::select_kernel<T><<<(unsigned)B, 1024, 0, st>>>(
                                  (const T*)logits, V, ids, ids_stride, position, next_token, done, eos_ids, n_eos, pad)));
  return launch_status();
}
