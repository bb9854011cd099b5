// Causal grouped-query flash attention on CUDA cores, forward and backward, for any even head
// dimension up to 256 and fp32 / bf16 / fp16 tensors. This is the general-shape path (fp32 models,
// head_dim != 128, sequence tails); the tensor-core kernels take the bf16 head_dim-128 case.
//
// Layout: q [B, Hq, S, D], k/v [B, Hkv, S, D] contiguous; kv head of query head h is h / (Hq/Hkv).
// Tiles of 32 queries x 32 keys; scores are computed one key per lane (no shuffles in the dot
// product), the output / gradient accumulators are kept one head-dim column per lane. Online
// softmax in fp32, log-sum-exp saved as [B, Hq, S] fp32 (natural log). Backward is deterministic:
//   delta = rowsum(dO * O); dQ is query-tile centric; dK/dV are key-tile centric and sum the query
//   heads of a group in registers (no per-query-head partial buffers, no atomics).
//
// Replaces, in the reference: qwen3_triton/kernels/attention_kernels.py:10-253 and
// ops/triton/attention.py:15-133, ops/triton/attention_backward.py:22-162 for those shapes.
// Math follows ops/reference/attention.py:10-54 (forward) and :57-124 (explicit backward).
#include "common.cuh"
#include <math_constants.h>

namespace q3 {

constexpr int kAttThreads = 128;  // 4 warps
constexpr int TQ = 32, TK = 32, RPW = 8;  // 32-query x 32-key tiles, 8 query rows per warp

template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int dst_stride, const T* src, int64_t row0, int64_t rows_total,
                                          int D, int DP) {
  // 32 rows x DP columns, zero-padded beyond D and beyond the sequence end.
  for (int e = threadIdx.x; e < 32 * DP; e += blockDim.x) {
    const int r = e / DP, c = e % DP;
    const int64_t row = row0 + r;
    dst[r * dst_stride + c] = (row < rows_total && c < D) ? to_f32<T>(src[row * D + c]) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(kAttThreads) attn_fwd_simt_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                    const T* __restrict__ v, T* __restrict__ out,
                                                                    float* __restrict__ lse, int Hq, int Hkv, int S,
                                                                    int D, int DP, float scale) {
  extern __shared__ float sm[];
  const int KS = DP + 4;
  float* qs = sm;               // [32][DP]
  float* ks = qs + 32 * DP;     // [32][DP+4]
  float* vs = ks + 32 * KS;     // [32][DP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, bh = blockIdx.y, b = bh / Hq, h = bh % Hq, kvh = h / (Hq / Hkv);
  const T* qp = q + ((int64_t)b * Hq + h) * S * D;
  const T* kp = k + ((int64_t)b * Hkv + kvh) * S * D;
  const T* vp = v + ((int64_t)b * Hkv + kvh) * S * D;
  const int q0 = qt * TQ;
  load_tile<T>(qs, DP, qp, q0, S, D, DP);
  const int NC = DP / 32;
  float m[RPW], l[RPW], o[RPW][8];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    m[r] = -CUDART_INF_F; l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[r][i] = 0.f;
  }
  for (int kt = 0; kt <= qt; ++kt) {
    __syncthreads();
    load_tile<T>(ks, KS, kp, (int64_t)kt * TK, S, D, DP);
    load_tile<T>(vs, DP, vp, (int64_t)kt * TK, S, D, DP);
    __syncthreads();
    const int key = kt * TK + lane;
    float s[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) s[r] = 0.f;
    for (int d = 0; d < DP; d += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(ks + lane * KS + d);
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float4 qq = *reinterpret_cast<const float4*>(qs + (warp * RPW + r) * DP + d);
        s[r] = fmaf(qq.x, kk.x, s[r]); s[r] = fmaf(qq.y, kk.y, s[r]);
        s[r] = fmaf(qq.z, kk.z, s[r]); s[r] = fmaf(qq.w, kk.w, s[r]);
      }
    }
    float p[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int qi = q0 + warp * RPW + r;
      const bool ok = key <= qi && key < S;
      const float sv = ok ? s[r] * scale : -CUDART_INF_F;
      const float mn = fmaxf(m[r], warp_max(sv));
      // every query row sees key 0 in tile 0, so mn is finite from the first tile on
      const float alpha = __expf(m[r] - mn);
      p[r] = ok ? __expf(sv - mn) : 0.f;
      l[r] = l[r] * alpha + warp_sum(p[r]);
      m[r] = mn;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[r][i] *= alpha;
    }
    for (int j = 0; j < TK; ++j) {
      float vv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) vv[i] = i < NC ? vs[j * DP + lane + 32 * i] : 0.f;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float pj = __shfl_sync(0xffffffffu, p[r], j);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[r][i] = fmaf(pj, vv[i], o[r][i]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int qi = q0 + warp * RPW + r;
    if (qi >= S) continue;
    const float inv = 1.f / l[r];
    T* op = out + (((int64_t)b * Hq + h) * S + qi) * D;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;
      if (i < NC && c < D) op[c] = from_f32<T>(o[r][i] * inv);
    }
    if (lane == 0) lse[((int64_t)b * Hq + h) * S + qi] = m[r] + logf(l[r]);
  }
}

// delta[row] = sum_d dO[row][d] * O[row][d]; one warp per row.
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta,
                                  int64_t rows, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float s = 0.f;
  for (int c = lane; c < D; c += 32) s += to_f32<T>(o[row * D + c]) * to_f32<T>(dout[row * D + c]);
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

template <typename T>
__global__ void __launch_bounds__(kAttThreads) attn_dq_simt_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                   const T* __restrict__ v, const T* __restrict__ dout,
                                                                   const float* __restrict__ lse,
                                                                   const float* __restrict__ delta, T* __restrict__ dq,
                                                                   int Hq, int Hkv, int S, int D, int DP, float scale) {
  extern __shared__ float sm[];
  const int KS = DP + 4;
  float* qs = sm;               // [32][DP]
  float* gs = qs + 32 * DP;     // [32][DP]  dO
  float* ks = gs + 32 * DP;     // [32][KS]
  float* vs = ks + 32 * KS;     // [32][KS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, bh = blockIdx.y, b = bh / Hq, h = bh % Hq, kvh = h / (Hq / Hkv);
  const int64_t qoff = ((int64_t)b * Hq + h) * S;
  const T* kp = k + ((int64_t)b * Hkv + kvh) * S * D;
  const T* vp = v + ((int64_t)b * Hkv + kvh) * S * D;
  const int q0 = qt * TQ;
  load_tile<T>(qs, DP, q + qoff * D, q0, S, D, DP);
  load_tile<T>(gs, DP, dout + qoff * D, q0, S, D, DP);
  const int NC = DP / 32;
  float rl[RPW], rd[RPW], acc[RPW][8];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int qi = q0 + warp * RPW + r;
    rl[r] = qi < S ? lse[qoff + qi] : 0.f;
    rd[r] = qi < S ? delta[qoff + qi] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
  }
  for (int kt = 0; kt <= qt; ++kt) {
    __syncthreads();
    load_tile<T>(ks, KS, kp, (int64_t)kt * TK, S, D, DP);
    load_tile<T>(vs, KS, vp, (int64_t)kt * TK, S, D, DP);
    __syncthreads();
    const int key = kt * TK + lane;
    float s[RPW], dp[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) { s[r] = 0.f; dp[r] = 0.f; }
    for (int d = 0; d < DP; d += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(ks + lane * KS + d);
      const float4 vv = *reinterpret_cast<const float4*>(vs + lane * KS + d);
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float4 qq = *reinterpret_cast<const float4*>(qs + (warp * RPW + r) * DP + d);
        const float4 gg = *reinterpret_cast<const float4*>(gs + (warp * RPW + r) * DP + d);
        s[r] = fmaf(qq.x, kk.x, s[r]); s[r] = fmaf(qq.y, kk.y, s[r]);
        s[r] = fmaf(qq.z, kk.z, s[r]); s[r] = fmaf(qq.w, kk.w, s[r]);
        dp[r] = fmaf(gg.x, vv.x, dp[r]); dp[r] = fmaf(gg.y, vv.y, dp[r]);
        dp[r] = fmaf(gg.z, vv.z, dp[r]); dp[r] = fmaf(gg.w, vv.w, dp[r]);
      }
    }
    float ds[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int qi = q0 + warp * RPW + r;
      const bool ok = key <= qi && key < S && qi < S;
      const float p = ok ? __expf(s[r] * scale - rl[r]) : 0.f;
      ds[r] = p * (dp[r] - rd[r]) * scale;
    }
    for (int j = 0; j < TK; ++j) {
      float kk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) kk[i] = i < NC ? ks[j * KS + lane + 32 * i] : 0.f;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float dj = __shfl_sync(0xffffffffu, ds[r], j);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(dj, kk[i], acc[r][i]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int qi = q0 + warp * RPW + r;
    if (qi >= S) continue;
    T* op = dq + (qoff + qi) * D;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;
      if (i < NC && c < D) op[c] = from_f32<T>(acc[r][i]);
    }
  }
}

// One CTA per (32-key tile, batch, kv head). Warp w scores query rows w*8..w*8+7 of each query tile
// (one key per lane) into shared P / dS tiles, then accumulates dV / dK for keys w*8..w*8+7 with one
// head-dim column per lane.
template <typename T>
__global__ void __launch_bounds__(kAttThreads) attn_dkdv_simt_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                     const T* __restrict__ v,
                                                                     const T* __restrict__ dout,
                                                                     const float* __restrict__ lse,
                                                                     const float* __restrict__ delta,
                                                                     T* __restrict__ dk, T* __restrict__ dv, int Hq,
                                                                     int Hkv, int S, int D, int DP, float scale) {
  extern __shared__ float sm[];
  const int KS = DP + 4;
  float* qs = sm;               // [32][DP]
  float* gs = qs + 32 * DP;     // [32][DP]
  float* ks = gs + 32 * DP;     // [32][KS]
  float* vs = ks + 32 * KS;     // [32][KS]
  float* ps = vs + 32 * KS;     // [32][33]
  float* dss = ps + 32 * 33;    // [32][33]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, bk = blockIdx.y, b = bk / Hkv, kvh = bk % Hkv, G = Hq / Hkv;
  const int64_t koff = ((int64_t)b * Hkv + kvh) * S;
  load_tile<T>(ks, KS, k + koff * D, (int64_t)kt * TK, S, D, DP);
  load_tile<T>(vs, KS, v + koff * D, (int64_t)kt * TK, S, D, DP);
  const int NC = DP / 32;
  const int nqt = (S + TQ - 1) / TQ;
  float adk[RPW][8], adv[RPW][8];
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int i = 0; i < 8; ++i) { adk[r][i] = 0.f; adv[r][i] = 0.f; }
  const int key = kt * TK + lane;
  for (int g = 0; g < G; ++g) {
    const int h = kvh * G + g;
    const int64_t qoff = ((int64_t)b * Hq + h) * S;
    for (int qt = kt; qt < nqt; ++qt) {
      const int q0 = qt * TQ;
      __syncthreads();
      load_tile<T>(qs, DP, q + qoff * D, q0, S, D, DP);
      load_tile<T>(gs, DP, dout + qoff * D, q0, S, D, DP);
      __syncthreads();
      float s[RPW], dp[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) { s[r] = 0.f; dp[r] = 0.f; }
      for (int d = 0; d < DP; d += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(ks + lane * KS + d);
        const float4 vv = *reinterpret_cast<const float4*>(vs + lane * KS + d);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const float4 qq = *reinterpret_cast<const float4*>(qs + (warp * RPW + r) * DP + d);
          const float4 gg = *reinterpret_cast<const float4*>(gs + (warp * RPW + r) * DP + d);
          s[r] = fmaf(qq.x, kk.x, s[r]); s[r] = fmaf(qq.y, kk.y, s[r]);
          s[r] = fmaf(qq.z, kk.z, s[r]); s[r] = fmaf(qq.w, kk.w, s[r]);
          dp[r] = fmaf(gg.x, vv.x, dp[r]); dp[r] = fmaf(gg.y, vv.y, dp[r]);
          dp[r] = fmaf(gg.z, vv.z, dp[r]); dp[r] = fmaf(gg.w, vv.w, dp[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const int row = warp * RPW + r, qi = q0 + row;
        const bool ok = key <= qi && key < S && qi < S;
        const float p = ok ? __expf(s[r] * scale - lse[qoff + (qi < S ? qi : 0)]) : 0.f;
        const float dl = qi < S ? delta[qoff + qi] : 0.f;
        ps[row * 33 + lane] = p;
        dss[row * 33 + lane] = p * (dp[r] - dl) * scale;
      }
      __syncthreads();
      for (int row = 0; row < TQ; ++row) {
        float gg[8], qq[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          gg[i] = i < NC ? gs[row * DP + lane + 32 * i] : 0.f;
          qq[i] = i < NC ? qs[row * DP + lane + 32 * i] : 0.f;
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const float pj = ps[row * 33 + warp * RPW + r];
          const float dj = dss[row * 33 + warp * RPW + r];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            adv[r][i] = fmaf(pj, gg[i], adv[r][i]);
            adk[r][i] = fmaf(dj, qq[i], adk[r][i]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int kj = kt * TK + warp * RPW + r;
    if (kj >= S) continue;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;
      if (i < NC && c < D) {
        dk[(koff + kj) * D + c] = from_f32<T>(adk[r][i]);
        dv[(koff + kj) * D + c] = from_f32<T>(adv[r][i]);
      }
    }
  }
}

template <typename K> int set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  }
  return Q3_OK;
}

int attn_fwd_simt(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t Hq,
                  int64_t Hkv, int64_t S, int64_t D, float scale, int dtype, cudaStream_t st) {
  const int DP = (int)cdiv(D, 32) * 32;
  const size_t smem = (size_t)(32 * DP * 2 + 32 * (DP + 4)) * sizeof(float);
  dim3 grid((unsigned)cdiv(S, TQ), (unsigned)(B * Hq));
  Q3_DISPATCH_FLOAT(dtype, T, {
    int rc = set_smem(attn_fwd_simt_kernel<T>, smem);
    if (rc != Q3_OK) return rc;
    attn_fwd_simt_kernel<T><<<grid, kAttThreads, smem, st>>>((const T*)q, (const T*)k, (const T*)v, (T*)out, lse,
                                                             (int)Hq, (int)Hkv, (int)S, (int)D, DP, scale);
  });
  return launch_status();
}

// delta for token-major tensors [B, S, H, D]: input row (b, s, h) -> delta[(b*H + h)*S + s]
template <typename T>
__global__ void attn_delta_bshd_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta,
                                       int64_t rows, int H, int S, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float s = 0.f;
  for (int c = lane; c < D; c += 32) s += to_f32<T>(o[row * D + c]) * to_f32<T>(dout[row * D + c]);
  s = warp_sum(s);
  if (lane == 0) {
    const int64_t h = row % H, bs = row / H, sidx = bs % S, b = bs / S;
    delta[(b * H + h) * S + sidx] = s;
  }
}

int attn_delta_layout(const void* out, const void* dout, float* delta, int64_t B, int64_t H, int64_t S, int64_t D,
                      int layout, int dtype, cudaStream_t st) {
  const int64_t rows = B * H * S;
  if (layout == 0) {
    Q3_DISPATCH_FLOAT(dtype, T, (attn_delta_kernel<T><<<(unsigned)cdiv(rows, 8), 256, 0, st>>>((const T*)out, (const T*)dout, delta, rows, (int)D)));
  } else {
    Q3_DISPATCH_FLOAT(dtype, T, (attn_delta_bshd_kernel<T><<<(unsigned)cdiv(rows, 8), 256, 0, st>>>((const T*)out, (const T*)dout, delta, rows, (int)H, (int)S, (int)D)));
  }
  return launch_status();
}

int attn_delta(const void* out, const void* dout, float* delta, int64_t rows, int64_t D, int dtype, cudaStream_t st) {
  Q3_DISPATCH_FLOAT(dtype, T, (attn_delta_kernel<T><<<(unsigned)cdiv(rows, 8), 256, 0, st>>>((const T*)out, (const T*)dout, delta, rows, (int)D)));
  return launch_status();
}

int attn_bwd_simt(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                  void* dq, void* dk, void* dv, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale,
                  int dtype, cudaStream_t st) {
  const int DP = (int)cdiv(D, 32) * 32;
  const size_t smem_dq = (size_t)(32 * DP * 2 + 32 * (DP + 4) * 2) * sizeof(float);
  const size_t smem_kv = smem_dq + (size_t)(2 * 32 * 33) * sizeof(float);
  dim3 gq((unsigned)cdiv(S, TQ), (unsigned)(B * Hq)), gk((unsigned)cdiv(S, TK), (unsigned)(B * Hkv));
  Q3_DISPATCH_FLOAT(dtype, T, {
    int rc = set_smem(attn_dq_simt_kernel<T>, smem_dq);
    if (rc != Q3_OK) return rc;
    rc = set_smem(attn_dkdv_simt_kernel<T>, smem_kv);
    if (rc != Q3_OK) return rc;
    attn_dq_simt_kernel<T><<<gq, kAttThreads, smem_dq, st>>>((const T*)q, (const T*)k, (const T*)v, (const T*)dout,
                                                             lse, delta, (T*)dq, (int)Hq, (int)Hkv, (int)S, (int)D, DP,
                                                             scale);
    attn_dkdv_simt_kernel<T><<<gk, kAttThreads, smem_kv, st>>>((const T*)q, (const T*)k, (const T*)v, (const T*)dout,
                                                               lse, delta, (T*)dk, (T*)dv, (int)Hq, (int)Hkv, (int)S,
                                                               (int)D, DP, scale);
  });
  return launch_status();
}

}  // namespace q3
