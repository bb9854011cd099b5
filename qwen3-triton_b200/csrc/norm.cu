// Row-wise bandwidth-bound kernels: RMSNorm fwd/bwd, residual-add + RMSNorm fused fwd/bwd,
// per-head RMSNorm + split-half RoPE fwd/bwd, rotary tables and rotary application.
//
// Layout: rows of H (or D) contiguous elements. A row is owned by `tpr` consecutive threads,
// each caching a few 16-byte vectors of the row in registers, so every input byte is read from
// HBM exactly once. fp32 math, one rounding on store. Weight gradients are deterministic:
// each CTA keeps per-column partial sums in registers over all of its rows, combines its row
// slots through shared memory in a fixed order, writes one partial row to the workspace and a
// second kernel sums the partial rows in a fixed order. No atomics.
//
// Replaces, in the reference: qwen3_triton/kernels/norm.py:7-37 (_forward/_backward/_reduce_rows),
// kernels/math_precision.py:16-21 (_hf_norm_forward), kernels/norm_rope.py:12-50 and
// math_precision.py:40-50 (norm+RoPE fwd/bwd), kernels/rotary.py:12-34 (_tables/_apply),
// ops/triton/rms_norm.py, ops/triton/rope.py, ops/triton/fused_qk_norm_rope.py.
// Math follows ops/reference/rms_norm.py:6-13, ops/reference/rope.py:6-55 and
// ops/reference/fused_qk_norm_rope.py:9-80 (fp32 internally, single rounding).
#include "common.cuh"

namespace q3 {

// Wide-row kernels that stage rows through shared memory with bulk copies (norm_ring.cu).
bool rmsnorm_ring_applies(int64_t H, int dtype);
int rmsnorm_bwd_ring_parts(int64_t rows);
int rmsnorm_fwd_ring(const void* x, const void* res, const void* w, void* y, void* res_out, float* inv, int64_t rows,
                     int64_t H, float eps, int dtype, cudaStream_t st);
int rmsnorm_bwd_ring(const void* x, const void* w, const void* dy, const void* dres, const float* inv, void* dx,
                     float* partial, int64_t rows, int64_t H, int dtype, cudaStream_t st);
bool norm_rope_ring_applies(int64_t heads, int64_t D, int dtype);
int norm_rope_bwd_ring_parts(int64_t tokens, int64_t heads, int64_t D, int dtype);
int norm_rope_fwd_ring(const void* x, const void* w, const void* cs, const void* sn, void* y, float* inv,
                       int64_t tokens, int64_t heads, int64_t D, float eps, int dtype, cudaStream_t st);
int norm_rope_bwd_ring(const void* x, const void* w, const void* cs, const void* sn, const void* dy, const float* inv,
                       void* dx, float* partial, int64_t tokens, int64_t heads, int64_t D, int dtype, cudaStream_t st);
void qk_norm_rope_bwd_ring_parts(int64_t tokens, int64_t hq, int64_t hk, int64_t D, int dtype, int* parts_q,
                                 int* parts_k);
int qk_norm_rope_fwd_ring(const void* q, const void* wq, void* yq, float* invq, int64_t hq, const void* k,
                          const void* wk, void* yk, float* invk, int64_t hk, const void* cs, const void* sn,
                          int64_t tokens, int64_t D, float eps, int dtype, cudaStream_t st);
int qk_norm_rope_bwd_ring(const void* q, const void* wq, const void* dyq, void* dq, const float* invq, float* pq,
                          int64_t hq, const void* k, const void* wk, const void* dyk, void* dk, const float* invk,
                          float* pk, int64_t hk, const void* cs, const void* sn, int64_t tokens, int64_t D, int dtype,
                          cudaStream_t st);
template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = Q3_F32; };
template <> struct DtypeOf<__nv_bfloat16> { static constexpr int value = Q3_BF16; };
template <> struct DtypeOf<__half> { static constexpr int value = Q3_F16; };

constexpr int kRowThreads = 256;
constexpr int kPartialRowsPerSm = 4;  // partial dW rows written per SM (workspace bound)

// Sum over the `tpr` threads that own one row. tpr is a power of two; rows never straddle a
// warp when tpr <= 32. For tpr > 32 every thread of the block must call this (it synchronises).
__device__ __forceinline__ float row_sum(float v, int tpr, float* sm) {
  if (tpr <= 32) {
    for (int o = tpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  }
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpr = tpr >> 5;
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  const int first = (warp / wpr) * wpr;
  float t = 0.f;
  for (int i = 0; i < wpr; ++i) t += sm[first + i];
  return t;
}

// Per-thread register cache depth and the widest row group, by vector width. The scalar path
// (odd H or unaligned pointers) may use 1024-thread blocks; the vector paths stay at 256.
template <int V> struct MaxVec {
  static constexpr int N = (V == 8) ? 4 : 8;
  static constexpr int MAX_TPR = (V == 1) ? 1024 : 256;
};

// ------------------------------------------------------------------ RMSNorm forward
template <typename T, int V, bool ADD>
__global__ void __launch_bounds__(MaxVec<V>::MAX_TPR) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                           const T* __restrict__ w, T* __restrict__ y,
                                                           T* __restrict__ res_out, float* __restrict__ inv,
                                                           int64_t rows, int H, float eps, int tpr) {
  constexpr int MV = MaxVec<V>::N;
  __shared__ float sm[32];
  const int rpb = blockDim.x / tpr, rib = threadIdx.x / tpr, t = threadIdx.x % tpr, nvec = H / V;
  for (int64_t base = (int64_t)blockIdx.x * rpb; base < rows; base += (int64_t)gridDim.x * rpb) {
    const int64_t row = base + rib;
    const bool valid = row < rows;
    float c[MV][V];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int v = t + i * tpr;
      if (valid && v < nvec) {
        VecIO<T, V>::load(x + row * H + (int64_t)v * V, c[i]);
        if constexpr (ADD) {
          float r[V];
          VecIO<T, V>::load(res + row * H + (int64_t)v * V, r);
#pragma unroll
          for (int j = 0; j < V; ++j) c[i][j] = to_f32<T>(from_f32<T>(c[i][j] + r[j]));  // the stored value is what is normalised
          VecIO<T, V>::store(res_out + row * H + (int64_t)v * V, c[i]);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) ss += c[i][j] * c[i][j];
      }
    }
    ss = row_sum(ss, tpr, sm);
    const float r = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int v = t + i * tpr;
      if (valid && v < nvec) {
        float ww[V], o[V];
        VecIO<T, V>::load(w + (int64_t)v * V, ww);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = c[i][j] * r * ww[j];
        VecIO<T, V>::store(y + row * H + (int64_t)v * V, o);
      }
    }
    if (valid && t == 0) inv[row] = r;
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = inv * (dy*w - x * inv^2 * mean(dy*w*x)) [+ dres];  dW[c] = sum_rows dy * x * inv.
template <typename T, int V, bool ADD>
__global__ void __launch_bounds__(MaxVec<V>::MAX_TPR) rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           const T* __restrict__ dy, const T* __restrict__ dres,
                                                           const float* __restrict__ inv, T* __restrict__ dx,
                                                           float* __restrict__ partial, int64_t rows, int H, int tpr) {
  constexpr int MV = MaxVec<V>::N;
  extern __shared__ float dsm[];  // [32] reduction scratch, then [rpb][H] combine buffer
  float* sm = dsm;
  float* comb = dsm + 32;
  const int rpb = blockDim.x / tpr, rib = threadIdx.x / tpr, t = threadIdx.x % tpr, nvec = H / V;
  float acc[MV][V];
#pragma unroll
  for (int i = 0; i < MV; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) acc[i][j] = 0.f;

  for (int64_t base = (int64_t)blockIdx.x * rpb; base < rows; base += (int64_t)gridDim.x * rpb) {
    const int64_t row = base + rib;
    const bool valid = row < rows;
    float cx[MV][V], cg[MV][V];
    float s = 0.f;
    const float r = valid ? inv[row] : 0.f;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int v = t + i * tpr;
      if (valid && v < nvec) {
        float ww[V];
        VecIO<T, V>::load(x + row * H + (int64_t)v * V, cx[i]);
        VecIO<T, V>::load(dy + row * H + (int64_t)v * V, cg[i]);
        VecIO<T, V>::load(w + (int64_t)v * V, ww);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          acc[i][j] += cg[i][j] * cx[i][j] * r;
          cg[i][j] *= ww[j];
          s += cg[i][j] * cx[i][j];
        }
      }
    }
    s = row_sum(s, tpr, sm);
    const float coef = s * r * r / (float)H;
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int v = t + i * tpr;
      if (valid && v < nvec) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = (cg[i][j] - cx[i][j] * coef) * r;
        if constexpr (ADD) {
          if (dres != nullptr) {
            float d[V];
            VecIO<T, V>::load(dres + row * H + (int64_t)v * V, d);
#pragma unroll
            for (int j = 0; j < V; ++j) o[j] += d[j];
          }
        }
        VecIO<T, V>::store(dx + row * H + (int64_t)v * V, o);
      }
    }
  }
  // Combine the row slots of this CTA in a fixed order, then write one partial row.
  __syncthreads();
#pragma unroll
  for (int i = 0; i < MV; ++i) {
    const int v = t + i * tpr;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) comb[(int64_t)rib * H + v * V + j] = acc[i][j];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float tsum = 0.f;
    for (int r2 = 0; r2 < rpb; ++r2) tsum += comb[(int64_t)r2 * H + c];
    partial[(int64_t)blockIdx.x * H + c] = tsum;
  }
}

// Sum `parts` partial rows of width H in a fixed order; output in dtype T.
template <typename T>
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                                              int parts, int H) {
  __shared__ float sm[8][33];
  const int col = blockIdx.x * 32 + threadIdx.x;  // blockDim = (32, 8)
  float s = 0.f;
  if (col < H)
    for (int p = threadIdx.y; p < parts; p += 8) s += partial[(int64_t)p * H + col];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && col < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    out[col] = from_f32<T>(t);
  }
}

// ------------------------------------------------------------------ per-head RMSNorm + RoPE
// Row = (token, head) of D elements; each thread owns vector pairs (c, c + D/2).
//   y1 = n1*cos1 - n2*sin1 ; y2 = n2*cos2 + n1*sin2, n = x * inv * w
template <typename T, int V, bool NORM>
__global__ void __launch_bounds__(kRowThreads) norm_rope_fwd_kernel(
    const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ cs, const T* __restrict__ sn,
    T* __restrict__ y, float* __restrict__ inv, int64_t rows, int heads, int64_t seq, int D, float eps, int tpr,
    int layout) {
  constexpr int MP = (V == 1) ? 4 : 1;   // vector paths: one pair per thread (D <= 512); scalar path: up to 4
  const int rpb = blockDim.x / tpr, rib = threadIdx.x / tpr, t = threadIdx.x % tpr, half = D / 2, npair = half / V;
  const int64_t step = (int64_t)gridDim.x * rpb;
  float a[MP][V], b[MP][V], na[MP][V], nb[MP][V];
  auto load_row = [&](int64_t row, float (&a_)[MP][V], float (&b_)[MP][V]) {
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (row < rows && p < npair) {
        VecIO<T, V>::load(x + row * D + (int64_t)p * V, a_[i]);
        VecIO<T, V>::load(x + row * D + half + (int64_t)p * V, b_[i]);
      }
    }
  };
  int64_t base = (int64_t)blockIdx.x * rpb;
  if (base < rows) load_row(base + rib, a, b);
  for (; base < rows; base += step) {
    const int64_t row = base + rib;
    const bool valid = row < rows;
    if (base + step < rows) load_row(base + step + rib, na, nb);   // next row's data in flight during this row's math
    // layout 0: x is [tokens, heads, D]; layout 1: x is [batch, heads, seq, D]
    int64_t token = 0;
    if (valid) token = layout == 0 ? row / heads : (row / ((int64_t)heads * seq)) * seq + row % seq;
    // table and weight loads do not depend on the row statistics: issue them before the reduction
    float c1[MP][V], c2[MP][V], s1[MP][V], s2[MP][V];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (valid && p < npair) {
        VecIO<T, V>::load(cs + token * D + (int64_t)p * V, c1[i]);
        VecIO<T, V>::load(cs + token * D + half + (int64_t)p * V, c2[i]);
        VecIO<T, V>::load(sn + token * D + (int64_t)p * V, s1[i]);
        VecIO<T, V>::load(sn + token * D + half + (int64_t)p * V, s2[i]);
        if constexpr (NORM) {
#pragma unroll
          for (int j = 0; j < V; ++j) ss += a[i][j] * a[i][j] + b[i][j] * b[i][j];
        }
      }
    }
    float r = 1.f;
    if constexpr (NORM) {
      for (int o = tpr >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss / (float)D + eps);
    }
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (valid && p < npair) {
        float o1[V], o2[V];
        if constexpr (NORM) {
          float w1[V], w2[V];
          VecIO<T, V>::load(w + (int64_t)p * V, w1);
          VecIO<T, V>::load(w + half + (int64_t)p * V, w2);
#pragma unroll
          for (int j = 0; j < V; ++j) { a[i][j] *= r * w1[j]; b[i][j] *= r * w2[j]; }
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
          o1[j] = a[i][j] * c1[i][j] - b[i][j] * s1[i][j];
          o2[j] = b[i][j] * c2[i][j] + a[i][j] * s2[i][j];
        }
        VecIO<T, V>::store(y + row * D + (int64_t)p * V, o1);
        VecIO<T, V>::store(y + row * D + half + (int64_t)p * V, o2);
      }
    }
    if constexpr (NORM) {
      if (valid && t == 0) inv[row] = r;
    }
#pragma unroll
    for (int i = 0; i < MP; ++i)
#pragma unroll
      for (int j = 0; j < V; ++j) { a[i][j] = na[i][j]; b[i][j] = nb[i][j]; }
  }
}

// Backward: dn1 = g1*cos1 + g2*sin2 ; dn2 = g2*cos2 - g1*sin1 (transpose of the rotation),
// then the RMSNorm backward of that on x (NORM) or dn itself is the answer (!NORM).
template <typename T, int V, bool NORM>
__global__ void __launch_bounds__(kRowThreads) norm_rope_bwd_kernel(
    const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ cs, const T* __restrict__ sn,
    const T* __restrict__ dy, const float* __restrict__ inv, T* __restrict__ dx, float* __restrict__ partial,
    int64_t rows, int heads, int64_t seq, int D, int tpr, int layout) {
  constexpr int MP = (V == 1) ? 4 : 1;   // vector paths: one pair per thread (D <= 512); scalar path: up to 4
  extern __shared__ float comb[];  // [rpb][D]
  const int rpb = blockDim.x / tpr, rib = threadIdx.x / tpr, t = threadIdx.x % tpr, half = D / 2, npair = half / V;
  float acc1[MP][V], acc2[MP][V];
#pragma unroll
  for (int i = 0; i < MP; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) { acc1[i][j] = 0.f; acc2[i][j] = 0.f; }

  const int64_t step = (int64_t)gridDim.x * rpb;
  float g1[MP][V], g2[MP][V], x1[MP][V], x2[MP][V], ng1[MP][V], ng2[MP][V], nx1[MP][V], nx2[MP][V];
  auto load_row = [&](int64_t row, float (&a1)[MP][V], float (&a2)[MP][V], float (&b1)[MP][V], float (&b2)[MP][V]) {
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (row < rows && p < npair) {
        VecIO<T, V>::load(dy + row * D + (int64_t)p * V, a1[i]);
        VecIO<T, V>::load(dy + row * D + half + (int64_t)p * V, a2[i]);
        if constexpr (NORM) {
          VecIO<T, V>::load(x + row * D + (int64_t)p * V, b1[i]);
          VecIO<T, V>::load(x + row * D + half + (int64_t)p * V, b2[i]);
        }
      }
    }
  };
  int64_t base = (int64_t)blockIdx.x * rpb;
  if (base < rows) load_row(base + rib, g1, g2, x1, x2);
  for (; base < rows; base += step) {
    const int64_t row = base + rib;
    const bool valid = row < rows;
    if (base + step < rows) load_row(base + step + rib, ng1, ng2, nx1, nx2);
    int64_t token = 0;
    if (valid) token = layout == 0 ? row / heads : (row / ((int64_t)heads * seq)) * seq + row % seq;
    float d1[MP][V], d2[MP][V];
    float s = 0.f;
    float r = 1.f;
    if constexpr (NORM) r = valid ? inv[row] : 0.f;
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (valid && p < npair) {
        float c1[V], c2[V], s1[V], s2[V];
        VecIO<T, V>::load(cs + token * D + (int64_t)p * V, c1);
        VecIO<T, V>::load(cs + token * D + half + (int64_t)p * V, c2);
        VecIO<T, V>::load(sn + token * D + (int64_t)p * V, s1);
        VecIO<T, V>::load(sn + token * D + half + (int64_t)p * V, s2);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          d1[i][j] = g1[i][j] * c1[j] + g2[i][j] * s2[j];
          d2[i][j] = g2[i][j] * c2[j] - g1[i][j] * s1[j];
        }
        if constexpr (NORM) {
          float w1[V], w2[V];
          VecIO<T, V>::load(w + (int64_t)p * V, w1);
          VecIO<T, V>::load(w + half + (int64_t)p * V, w2);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            acc1[i][j] += d1[i][j] * x1[i][j] * r;
            acc2[i][j] += d2[i][j] * x2[i][j] * r;
            d1[i][j] *= w1[j];
            d2[i][j] *= w2[j];
            s += d1[i][j] * x1[i][j] + d2[i][j] * x2[i][j];
          }
        }
      }
    }
    float coef = 0.f;
    if constexpr (NORM) {
      for (int o = tpr >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      coef = s * r * r / (float)D;
    }
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (valid && p < npair) {
        if constexpr (NORM) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            d1[i][j] = (d1[i][j] - x1[i][j] * coef) * r;
            d2[i][j] = (d2[i][j] - x2[i][j] * coef) * r;
          }
        }
        VecIO<T, V>::store(dx + row * D + (int64_t)p * V, d1[i]);
        VecIO<T, V>::store(dx + row * D + half + (int64_t)p * V, d2[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < MP; ++i)
#pragma unroll
      for (int j = 0; j < V; ++j) {
        g1[i][j] = ng1[i][j]; g2[i][j] = ng2[i][j];
        if constexpr (NORM) { x1[i][j] = nx1[i][j]; x2[i][j] = nx2[i][j]; }
      }
  }
  if constexpr (NORM) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MP; ++i) {
      const int p = t + i * tpr;
      if (p < npair) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          comb[rib * D + p * V + j] = acc1[i][j];
          comb[rib * D + half + p * V + j] = acc2[i][j];
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float tsum = 0.f;
      for (int r2 = 0; r2 < rpb; ++r2) tsum += comb[r2 * D + c];
      partial[(int64_t)blockIdx.x * D + c] = tsum;
    }
  }
}

// cos/sin tables [tokens, D]: angle = float(pos) * inv_freq[i % (D/2)].
template <typename T, typename P>
__global__ void rope_tables_kernel(const P* __restrict__ pos, const float* __restrict__ freq, T* __restrict__ cs,
                                   T* __restrict__ sn, int64_t tokens, int D) {
  const int half = D / 2;
  const int64_t total = tokens * half;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t tkn = i / half;
    const int f = (int)(i % half);
    const float angle = (float)pos[tkn] * freq[f];
    float s, c;
    sincosf(angle, &s, &c);
    const T cv = from_f32<T>(c), sv = from_f32<T>(s);
    cs[tkn * D + f] = cv; cs[tkn * D + half + f] = cv;
    sn[tkn * D + f] = sv; sn[tkn * D + half + f] = sv;
  }
}

// ------------------------------------------------------------------ host-side planning
inline int pow2ceil(int v) { int p = 1; while (p < v) p <<= 1; return p; }

struct RowPlan { int tpr, block, rpb, grid; };

inline RowPlan plan_rows(int64_t rows, int nvec, int per_thread, int max_per_thread, int max_tpr, int grid_per_sm) {
  RowPlan p;
  p.tpr = pow2ceil((int)cdiv(nvec, per_thread));
  if (p.tpr > max_tpr) p.tpr = max_tpr;
  if (cdiv(nvec, p.tpr) > max_per_thread) { p.tpr = -1; return p; }
  p.block = p.tpr > kRowThreads ? p.tpr : kRowThreads;
  p.rpb = p.block / p.tpr;
  int64_t g = cdiv(rows, p.rpb), cap = (int64_t)sm_count() * grid_per_sm;
  p.grid = (int)(g > cap ? cap : g);
  return p;
}

template <typename T, bool ADD>
int rmsnorm_fwd_launch(const void* x, const void* res, const void* w, void* y, void* res_out, float* inv,
                       int64_t rows, int64_t H, float eps, cudaStream_t st) {
  constexpr int VF = Vec16<T>::N;
  const bool vec = (H % VF == 0) && aligned16(x) && aligned16(w) && aligned16(y) && (!ADD || (aligned16(res) && aligned16(res_out)));
  if (vec && rmsnorm_ring_applies(H, DtypeOf<T>::value))
    return rmsnorm_fwd_ring(x, ADD ? res : nullptr, w, y, res_out, inv, rows, H, eps, DtypeOf<T>::value, st);
  if (vec) {
    RowPlan p = plan_rows(rows, (int)(H / VF), 2, MaxVec<VF>::N, MaxVec<VF>::MAX_TPR, 8);
    if (p.tpr < 0) return Q3_ERR_SHAPE;
    rmsnorm_fwd_kernel<T, VF, ADD><<<p.grid, p.block, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y,
                                                               (T*)res_out, inv, rows, (int)H, eps, p.tpr);
  } else {
    RowPlan p = plan_rows(rows, (int)H, 2, MaxVec<1>::N, MaxVec<1>::MAX_TPR, 8);
    if (p.tpr < 0) return Q3_ERR_SHAPE;
    rmsnorm_fwd_kernel<T, 1, ADD><<<p.grid, p.block, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y,
                                                              (T*)res_out, inv, rows, (int)H, eps, p.tpr);
  }
  return launch_status();
}

template <typename T, bool ADD>
int rmsnorm_bwd_launch(const void* x, const void* w, const void* dy, const void* dres, const float* inv, void* dx,
                       void* dw, float* ws, int64_t ws_bytes, int64_t rows, int64_t H, cudaStream_t st,
                       int max_partial_rows = 1 << 30) {
  constexpr int VF = Vec16<T>::N;
  const bool vec = (H % VF == 0) && aligned16(x) && aligned16(w) && aligned16(dy) && aligned16(dx) &&
                   (!ADD || dres == nullptr || aligned16(dres));
  if (vec && rmsnorm_ring_applies(H, DtypeOf<T>::value) && rmsnorm_bwd_ring_parts(rows) <= max_partial_rows) {
    const int parts = rmsnorm_bwd_ring_parts(rows);
    if (ws == nullptr || ws_bytes < (int64_t)parts * H * 4) return Q3_ERR_WORKSPACE;
    const int rc = rmsnorm_bwd_ring(x, w, dy, ADD ? dres : nullptr, inv, dx, ws, rows, H, DtypeOf<T>::value, st);
    if (rc != Q3_OK) return rc;
    reduce_partials_kernel<T><<<(int)cdiv(H, 32), dim3(32, 8), 0, st>>>(ws, (T*)dw, parts, (int)H);
    return launch_status();
  }
  RowPlan p = vec ? plan_rows(rows, (int)(H / VF), 2, MaxVec<VF>::N, MaxVec<VF>::MAX_TPR, kPartialRowsPerSm)
                  : plan_rows(rows, (int)H, 2, MaxVec<1>::N, MaxVec<1>::MAX_TPR, kPartialRowsPerSm);
  if (p.tpr < 0) return Q3_ERR_SHAPE;
  if (p.grid > max_partial_rows) p.grid = max_partial_rows;
  if (ws == nullptr || ws_bytes < (int64_t)p.grid * H * 4) return Q3_ERR_WORKSPACE;
  const size_t smem = (32 + (size_t)p.rpb * H) * sizeof(float);
  if (vec) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<T, VF, ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rmsnorm_bwd_kernel<T, VF, ADD><<<p.grid, p.block, smem, st>>>((const T*)x, (const T*)w, (const T*)dy,
                                                                  (const T*)dres, inv, (T*)dx, ws, rows, (int)H, p.tpr);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<T, 1, ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rmsnorm_bwd_kernel<T, 1, ADD><<<p.grid, p.block, smem, st>>>((const T*)x, (const T*)w, (const T*)dy,
                                                                 (const T*)dres, inv, (T*)dx, ws, rows, (int)H, p.tpr);
  }
  reduce_partials_kernel<T><<<(int)cdiv(H, 32), dim3(32, 8), 0, st>>>(ws, (T*)dw, p.grid, (int)H);
  return launch_status();
}

template <typename T, bool NORM>
int norm_rope_fwd_launch(const void* x, const void* w, const void* cs, const void* sn, void* y, float* inv,
                         int64_t batch, int64_t seq, int64_t heads, int64_t D, float eps, int layout, cudaStream_t st) {
  constexpr int VF = Vec16<T>::N;
  const int64_t rows = batch * seq * heads, half = D / 2;
  const bool vec = (half % VF == 0) && aligned16(x) && aligned16(cs) && aligned16(sn) && aligned16(y) && (!NORM || aligned16(w));
  if (NORM && vec && layout == 0 && norm_rope_ring_applies(heads, D, DtypeOf<T>::value))
    return norm_rope_fwd_ring(x, w, cs, sn, y, inv, batch * seq, heads, D, eps, DtypeOf<T>::value, st);
  if (vec) {
    RowPlan p = plan_rows(rows, (int)(half / VF), 1, 1, 32, 16);
    if (p.tpr < 0 || p.tpr > 32) return Q3_ERR_SHAPE;
    norm_rope_fwd_kernel<T, VF, NORM><<<p.grid, p.block, 0, st>>>((const T*)x, (const T*)w, (const T*)cs, (const T*)sn,
                                                                  (T*)y, inv, rows, (int)heads, seq, (int)D, eps, p.tpr, layout);
  } else {
    RowPlan p = plan_rows(rows, (int)half, 1, 4, 32, 16);
    if (p.tpr < 0 || p.tpr > 32) return Q3_ERR_SHAPE;
    norm_rope_fwd_kernel<T, 1, NORM><<<p.grid, p.block, 0, st>>>((const T*)x, (const T*)w, (const T*)cs, (const T*)sn,
                                                                 (T*)y, inv, rows, (int)heads, seq, (int)D, eps, p.tpr, layout);
  }
  return launch_status();
}

template <typename T, bool NORM>
int norm_rope_bwd_launch(const void* x, const void* w, const void* cs, const void* sn, const void* dy,
                         const float* inv, void* dx, void* dw, float* ws, int64_t ws_bytes, int64_t batch, int64_t seq,
                         int64_t heads, int64_t D, int layout, cudaStream_t st) {
  constexpr int VF = Vec16<T>::N;
  const int64_t rows = batch * seq * heads, half = D / 2;
  const bool vec = (half % VF == 0) && aligned16(cs) && aligned16(sn) && aligned16(dy) && aligned16(dx) &&
                   (!NORM || (aligned16(x) && aligned16(w)));
  if (NORM && vec && layout == 0 && norm_rope_ring_applies(heads, D, DtypeOf<T>::value)) {
    const int parts = norm_rope_bwd_ring_parts(batch * seq, heads, D, DtypeOf<T>::value);
    if (ws == nullptr || ws_bytes < (int64_t)parts * D * 4) return Q3_ERR_WORKSPACE;
    const int rc = norm_rope_bwd_ring(x, w, cs, sn, dy, inv, dx, ws, batch * seq, heads, D, DtypeOf<T>::value, st);
    if (rc != Q3_OK) return rc;
    reduce_partials_kernel<T><<<(int)cdiv(D, 32), dim3(32, 8), 0, st>>>(ws, (T*)dw, parts, (int)D);
    return launch_status();
  }
  RowPlan p = vec ? plan_rows(rows, (int)(half / VF), 1, 1, 32, kPartialRowsPerSm * 2)
                  : plan_rows(rows, (int)half, 1, 4, 32, kPartialRowsPerSm * 2);
  if (p.tpr < 0 || p.tpr > 32) return Q3_ERR_SHAPE;
  if (NORM && (ws == nullptr || ws_bytes < (int64_t)p.grid * D * 4)) return Q3_ERR_WORKSPACE;
  const size_t smem = NORM ? (size_t)p.rpb * D * sizeof(float) : 0;
  if (vec) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_rope_bwd_kernel<T, VF, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    norm_rope_bwd_kernel<T, VF, NORM><<<p.grid, p.block, smem, st>>>((const T*)x, (const T*)w, (const T*)cs, (const T*)sn,
                                                                     (const T*)dy, inv, (T*)dx, ws, rows, (int)heads, seq,
                                                                     (int)D, p.tpr, layout);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_rope_bwd_kernel<T, 1, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    norm_rope_bwd_kernel<T, 1, NORM><<<p.grid, p.block, smem, st>>>((const T*)x, (const T*)w, (const T*)cs, (const T*)sn,
                                                                    (const T*)dy, inv, (T*)dx, ws, rows, (int)heads, seq,
                                                                    (int)D, p.tpr, layout);
  }
  if (NORM) reduce_partials_kernel<T><<<(int)cdiv(D, 32), dim3(32, 8), 0, st>>>(ws, (T*)dw, p.grid, (int)D);
  return launch_status();
}

}  // namespace q3

using namespace q3;

extern "C" int q3_rmsnorm_fwd(const void* x, const void* weight, void* y, float* inv_rms, int64_t rows, int64_t H,
                              double eps, int dtype, q3_stream_t stream) {
  if (!x || !weight || !y || !inv_rms) return Q3_ERR_ARG;
  if (rows < 1 || H < 1 || H > 8192 || !(eps > 0)) return Q3_ERR_SHAPE;
  Q3_DISPATCH_FLOAT(dtype, T, return (rmsnorm_fwd_launch<T, false>(x, nullptr, weight, y, nullptr, inv_rms, rows, H,
                                                                   (float)eps, (cudaStream_t)stream)));
  return Q3_OK;
}

extern "C" int64_t q3_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t H) {
  (void)rows;
  return (int64_t)sm_count() * kPartialRowsPerSm * 2 * H * 4;
}

extern "C" int q3_rmsnorm_bwd(const void* x, const void* weight, const void* dy, const float* inv_rms, void* dx,
                              void* dweight, void* workspace, int64_t workspace_bytes, int64_t rows, int64_t H,
                              int dtype, q3_stream_t stream) {
  if (!x || !weight || !dy || !inv_rms || !dx || !dweight) return Q3_ERR_ARG;
  if (rows < 1 || H < 1 || H > 8192) return Q3_ERR_SHAPE;
  Q3_DISPATCH_FLOAT(dtype, T, return (rmsnorm_bwd_launch<T, false>(x, weight, dy, nullptr, inv_rms, dx, dweight,
                                                                   (float*)workspace, workspace_bytes, rows, H,
                                                                   (cudaStream_t)stream)));
  return Q3_OK;
}

extern "C" int q3_add_rmsnorm_fwd(const void* x, const void* residual, const void* weight, void* y,
                                  void* residual_out, float* inv_rms, int64_t rows, int64_t H, double eps, int dtype,
                                  q3_stream_t stream) {
  if (!x || !residual || !weight || !y || !residual_out || !inv_rms) return Q3_ERR_ARG;
  if (rows < 1 || H < 1 || H > 8192 || !(eps > 0)) return Q3_ERR_SHAPE;
  Q3_DISPATCH_FLOAT(dtype, T, return (rmsnorm_fwd_launch<T, true>(x, residual, weight, y, residual_out, inv_rms, rows,
                                                                  H, (float)eps, (cudaStream_t)stream)));
  return Q3_OK;
}

extern "C" int q3_add_rmsnorm_bwd(const void* residual_out, const void* weight, const void* dy, const void* dresidual,
                                  const float* inv_rms, void* dx, void* dweight, void* workspace,
                                  int64_t workspace_bytes, int64_t rows, int64_t H, int dtype, q3_stream_t stream) {
  if (!residual_out || !weight || !dy || !inv_rms || !dx || !dweight) return Q3_ERR_ARG;
  if (rows < 1 || H < 1 || H > 8192) return Q3_ERR_SHAPE;
  Q3_DISPATCH_FLOAT(dtype, T, return (rmsnorm_bwd_launch<T, true>(residual_out, weight, dy, dresidual, inv_rms, dx,
                                                                  dweight, (float*)workspace, workspace_bytes, rows, H,
                                                                  (cudaStream_t)stream)));
  return Q3_OK;
}

extern "C" int q3_norm_rope_fwd(const void* x, const void* weight, const void* cos_t, const void* sin_t, void* y,
                                float* inv_rms, int64_t tokens, int64_t heads, int64_t D, double eps, int dtype,
                                q3_stream_t stream) {
  if (!x || !weight || !cos_t || !sin_t || !y || !inv_rms) return Q3_ERR_ARG;
  if (tokens < 1 || heads < 1 || D < 2 || (D & 1) || !(eps > 0)) return Q3_ERR_SHAPE;
  Q3_DISPATCH_FLOAT(dtype, T, return (norm_rope_fwd_launch<T, true>(x, weight, cos_t, sin_t, y, inv_rms, 1, tokens,
                                                                    heads, D, (float)eps, 0, (cudaStream_t)stream)));
  return Q3_OK;
}

extern "C" int64_t q3_norm_rope_bwd_workspace_bytes(int64_t tokens, int64_t heads, int64_t D) {
  (void)tokens; (void)heads;
  return (int64_t)sm_count() * kPartialRowsPerSm * 2 * D * 4;
}

extern "C" int q3_norm_rope_bwd(const void* x, const void* weight, const void* cos_t, const void* sin_t,
                                const void* dy, const float* inv_rms, void* dx, void* dweight, void* workspace,
                                int64_t workspace_bytes, int64_t tokens, int64_t heads, int64_t D, int dtype,
                                q3_stream_t stream) {
  if (!x || !weight || !cos_t || !sin_t || !dy || !inv_rms || !dx || !dweight) return Q3_ERR_ARG;
  if (tokens < 1 || heads < 1 || D < 2 || (D & 1)) return Q3_ERR_SHAPE;
  Q3_DISPATCH_FLOAT(dtype, T, return (norm_rope_bwd_launch<T, true>(x, weight, cos_t, sin_t, dy, inv_rms, dx, dweight,
                                                                    (float*)workspace, workspace_bytes, 1, tokens,
                                                                    heads, D, 0, (cudaStream_t)stream)));
  return Q3_OK;
}

// q [tokens, hq, D] and k [tokens, hk, D] of one layer in one launch (token-major only). Falls back to two launches
// of the single-tensor form where the wide-row kernels do not apply.
extern "C" int q3_qk_norm_rope_fwd(const void* q, const void* k, const void* q_weight, const void* k_weight,
                                   const void* cos_t, const void* sin_t, void* yq, void* yk, float* inv_q, float* inv_k,
                                   int64_t tokens, int64_t hq, int64_t hk, int64_t D, double eps, int dtype,
                                   q3_stream_t stream) {
  if (!q || !k || !q_weight || !k_weight || !cos_t || !sin_t || !yq || !yk || !inv_q || !inv_k) return Q3_ERR_ARG;
  if (tokens < 1 || hq < 1 || hk < 1 || D < 2 || (D & 1) || !(eps > 0)) return Q3_ERR_SHAPE;
  const bool al = aligned16(q) && aligned16(k) && aligned16(q_weight) && aligned16(k_weight) && aligned16(cos_t) &&
                  aligned16(sin_t) && aligned16(yq) && aligned16(yk);
  if (al && norm_rope_ring_applies(hq, D, dtype) && norm_rope_ring_applies(hk, D, dtype))
    return qk_norm_rope_fwd_ring(q, q_weight, yq, inv_q, hq, k, k_weight, yk, inv_k, hk, cos_t, sin_t, tokens, D,
                                 (float)eps, dtype, (cudaStream_t)stream);
  int rc = q3_norm_rope_fwd(q, q_weight, cos_t, sin_t, yq, inv_q, tokens, hq, D, eps, dtype, stream);
  if (rc != Q3_OK) return rc;
  return q3_norm_rope_fwd(k, k_weight, cos_t, sin_t, yk, inv_k, tokens, hk, D, eps, dtype, stream);
}

extern "C" int64_t q3_qk_norm_rope_bwd_workspace_bytes(int64_t tokens, int64_t hq, int64_t hk, int64_t D) {
  return q3_norm_rope_bwd_workspace_bytes(tokens, hq, D) + q3_norm_rope_bwd_workspace_bytes(tokens, hk, D);
}

extern "C" int q3_qk_norm_rope_bwd(const void* q, const void* k, const void* q_weight, const void* k_weight,
                                   const void* cos_t, const void* sin_t, const void* dyq, const void* dyk,
                                   const float* inv_q, const float* inv_k, void* dq, void* dk, void* dq_weight,
                                   void* dk_weight, void* workspace, int64_t workspace_bytes, int64_t tokens,
                                   int64_t hq, int64_t hk, int64_t D, int dtype, q3_stream_t stream) {
  if (!q || !k || !q_weight || !k_weight || !cos_t || !sin_t || !dyq || !dyk || !inv_q || !inv_k || !dq || !dk ||
      !dq_weight || !dk_weight)
    return Q3_ERR_ARG;
  if (tokens < 1 || hq < 1 || hk < 1 || D < 2 || (D & 1)) return Q3_ERR_SHAPE;
  const int64_t wq_bytes = q3_norm_rope_bwd_workspace_bytes(tokens, hq, D);
  if (!workspace || workspace_bytes < q3_qk_norm_rope_bwd_workspace_bytes(tokens, hq, hk, D)) return Q3_ERR_WORKSPACE;
  float* pq = static_cast<float*>(workspace);
  float* pk = reinterpret_cast<float*>(static_cast<char*>(workspace) + wq_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const bool al = aligned16(q) && aligned16(k) && aligned16(q_weight) && aligned16(k_weight) && aligned16(cos_t) &&
                  aligned16(sin_t) && aligned16(dyq) && aligned16(dyk) && aligned16(dq) && aligned16(dk);
  if (al && norm_rope_ring_applies(hq, D, dtype) && norm_rope_ring_applies(hk, D, dtype)) {
    int cq = 0, ck = 0;
    qk_norm_rope_bwd_ring_parts(tokens, hq, hk, D, dtype, &cq, &ck);
    int rc = qk_norm_rope_bwd_ring(q, q_weight, dyq, dq, inv_q, pq, hq, k, k_weight, dyk, dk, inv_k, pk, hk, cos_t,
                                   sin_t, tokens, D, dtype, st);
    if (rc != Q3_OK) return rc;
    if (dtype == Q3_BF16) {
      reduce_partials_kernel<__nv_bfloat16><<<(int)cdiv(D, 32), dim3(32, 8), 0, st>>>(pq, (__nv_bfloat16*)dq_weight, cq, (int)D);
      reduce_partials_kernel<__nv_bfloat16><<<(int)cdiv(D, 32), dim3(32, 8), 0, st>>>(pk, (__nv_bfloat16*)dk_weight, ck, (int)D);
    } else {
      reduce_partials_kernel<__half><<<(int)cdiv(D, 32), dim3(32, 8), 0, st>>>(pq, (__half*)dq_weight, cq, (int)D);
      reduce_partials_kernel<__half><<<(int)cdiv(D, 32), dim3(32, 8), 0, st>>>(pk, (__half*)dk_weight, ck, (int)D);
    }
    return launch_status();
  }
  int rc = q3_norm_rope_bwd(q, q_weight, cos_t, sin_t, dyq, inv_q, dq, dq_weight, pq, wq_bytes, tokens, hq, D, dtype, stream);
  if (rc != Q3_OK) return rc;
  return q3_norm_rope_bwd(k, k_weight, cos_t, sin_t, dyk, inv_k, dk, dk_weight, pk, workspace_bytes - wq_bytes, tokens,
                          hk, D, dtype, stream);
}

extern "C" int q3_rope_apply(const void* x, const void* cos_t, const void* sin_t, void* y, int64_t batch, int64_t seq,
                             int64_t heads, int64_t D, int backward, int layout, int dtype, q3_stream_t stream) {
  if (!x || !cos_t || !sin_t || !y) return Q3_ERR_ARG;
  if (batch < 1 || seq < 1 || heads < 1 || D < 2 || (D & 1) || (layout != 0 && layout != 1)) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (backward) {
    Q3_DISPATCH_FLOAT(dtype, T, return (norm_rope_bwd_launch<T, false>(nullptr, nullptr, cos_t, sin_t, x, nullptr, y,
                                                                       nullptr, nullptr, 0, batch, seq, heads, D,
                                                                       layout, st)));
  } else {
    Q3_DISPATCH_FLOAT(dtype, T, return (norm_rope_fwd_launch<T, false>(x, nullptr, cos_t, sin_t, y, nullptr, batch,
                                                                       seq, heads, D, 0.f, layout, st)));
  }
  return Q3_OK;
}

extern "C" int q3_rope_tables(const void* positions, int positions_are_int64, const float* inv_freq, void* cos_t,
                              void* sin_t, int64_t tokens, int64_t D, int dtype, q3_stream_t stream) {
  if (!positions || !inv_freq || !cos_t || !sin_t) return Q3_ERR_ARG;
  if (tokens < 1 || D < 2 || (D & 1)) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = tokens * (D / 2);
  int64_t g = cdiv(total, 256), cap = (int64_t)sm_count() * 8;
  const int grid = (int)(g > cap ? cap : g);
  Q3_DISPATCH_FLOAT(dtype, T, {
    if (positions_are_int64)
      rope_tables_kernel<T, int64_t><<<grid, 256, 0, st>>>((const int64_t*)positions, inv_freq, (T*)cos_t, (T*)sin_t, tokens, (int)D);
    else
      rope_tables_kernel<T, int32_t><<<grid, 256, 0, st>>>((const int32_t*)positions, inv_freq, (T*)cos_t, (T*)sin_t, tokens, (int)D);
  });
  return launch_status();
}

// ------------------------------------------------------------------ RMSNorm backward without any allocation
// Some callers may not allocate device memory at the point where they need this gradient: code that runs
// inside a memory-pool callback or under an allocator lock, a host that pre-plans every byte of HBM and
// forbids late cudaMalloc, or a real-time loop in which an allocation (and the implicit device
// synchronisation cudaFree can cause) is not acceptable. For them the partial-row scratch of the weight
// gradient lives in this fixed device array instead of a caller workspace. Every GPU that loads the
// library carries the array (16 MiB) until the process exits.
namespace q3 {
constexpr int64_t kNoAllocMaxH = 4096;            // widest row the fixed scratch serves
constexpr int kNoAllocPartialRows = 1024;         // partial weight-gradient rows that fit at that width
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[kNoAllocPartialRows * kNoAllocMaxH];

// The array's name is only a host-side handle; kernels need its device address, which differs per
// device. Resolve it once per device, with that device current.
static int noalloc_scratch(float** out) {
  static float* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  if (dev < 0 || dev >= 64) return Q3_ERR_SHAPE;
  if (cached[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_rmsnorm_bwd_scratch);
    if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return Q3_OK;
}
}  // namespace q3

extern "C" int q3_rmsnorm_bwd_noalloc(const void* x, const void* weight, const void* dy, const float* inv_rms,
                                      void* dx, void* dweight, int64_t rows, int64_t H, int dtype,
                                      q3_stream_t stream) {
  if (!x || !weight || !dy || !inv_rms || !dx || !dweight) return Q3_ERR_ARG;
  if (rows < 1 || H < 1) return Q3_ERR_SHAPE;
  if (H > kNoAllocMaxH) return Q3_ERR_LIMIT;   // beyond the fixed scratch: use q3_rmsnorm_bwd with a workspace
  float* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc != Q3_OK) return rc;
  // The partial rows used by this call are fully overwritten before they are read, so nothing has to be
  // cleared between calls.
  const int max_rows = (int)((kNoAllocPartialRows * kNoAllocMaxH) / H);
  Q3_DISPATCH_FLOAT(dtype, T, return (rmsnorm_bwd_launch<T, false>(x, weight, dy, nullptr, inv_rms, dx, dweight, scratch,
                                                                   (int64_t)kNoAllocPartialRows * kNoAllocMaxH * 4, rows, H,
                                                                   (cudaStream_t)stream, max_rows)));
  return Q3_OK;
}
