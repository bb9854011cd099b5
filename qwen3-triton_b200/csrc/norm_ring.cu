// RMSNorm forward / backward for wide rows (2048 <= H <= 8192 elements of 16 bits), and per-head RMSNorm + RoPE on
// token-major tensors, with the rows staged through a shared-memory ring by bulk asynchronous copies.
//
// The register-resident kernels of norm.cu keep one row per CTA in flight and are limited by occupancy (the
// backward one holds ~100 live floats per thread): 41-61 % of HBM peak at H = 4096. Here a CTA is 8 consumer warps
// plus one producer warp. The producer thread streams whole rows (x, and dy / residual where needed) into a ring
// of `stages` slots with cp.async.bulk, each completing on the slot's mbarrier; consumers wait for a slot, pull
// their 16-byte vectors into registers, hand the slot back (one mbarrier arrival per warp) and then do the
// arithmetic, so up to `stages` rows per CTA are in flight whatever the register count. One named barrier per
// row carries the row reduction; it also votes on the wait results so that an expired wait ends the CTA uniformly
// instead of leaving part of it parked on a barrier.
//
// Replaces, in the reference: qwen3_triton/kernels/norm.py:13-68 (_rms_forward, _rms_backward) and the add+norm
// pair of kernels/residual.py.
#include "tcgen05.cuh"

namespace q3 {

int* async_status();   // abi.cu: device status word for kernels whose entry points carry no status argument

namespace ring {

using namespace q3::tc;

constexpr int kConsumers = 256;
constexpr int kThreads = kConsumers + 32;
constexpr int kMaxStages = 8;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Barrier over the consumer threads only (id 1) that also ANDs a predicate over them.
__device__ __forceinline__ bool consumers_all(bool pred) {
  int r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.s32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.s32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((int)pred), "n"(kConsumers)
      : "memory");
  return r != 0;
}

struct Ring {
  uint32_t full0, empty0;
  volatile int* abort_flag;
  float* red;          // [2][8]
  uint8_t* slots;
  __device__ __forceinline__ uint32_t full(int s) const { return full0 + 8u * s; }
  __device__ __forceinline__ uint32_t empty(int s) const { return empty0 + 8u * s; }
};

// Shared memory: [stages][slot_bytes] | full[kMaxStages] | empty[kMaxStages] | abort | red[16]
__device__ __forceinline__ Ring ring_setup(uint8_t* smem, int stages, size_t slot_bytes) {
  Ring r;
  r.slots = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * slot_bytes);
  r.full0 = smem_u32(bars);
  r.empty0 = r.full0 + 8u * kMaxStages;
  int* tail = reinterpret_cast<int*>(bars + 2 * kMaxStages);
  r.abort_flag = tail;
  r.red = reinterpret_cast<float*>(tail + 4);
  if (threadIdx.x == 0) {
    *r.abort_flag = 0;
    for (int s = 0; s < stages; ++s) { mbar_init(r.full(s), 1); mbar_init(r.empty(s), kConsumers / 32); }
    fence_barrier_init();
  }
  __syncthreads();
  return r;
}

__host__ __device__ inline size_t ring_smem_bytes(int stages, size_t slot_bytes) {
  return (size_t)stages * slot_bytes + 2 * kMaxStages * 8 + 16 + 16 * 4;
}

// Producer: one thread. `n_in` row sources; row r of source i starts at src[i] + r * row_bytes.
template <int NIN>
__device__ __forceinline__ void produce(const Ring& rg, const uint8_t* const (&src)[NIN], int n_in, int64_t rows,
                                        uint32_t row_bytes, int stages, size_t slot_bytes) {
  uint32_t k = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++k) {
    const int s = k % stages;
    const uint32_t ph = (k / stages) & 1u;
    if (!mbar_wait(rg.empty(s), ph ^ 1u, rg.abort_flag)) break;
    mbar_expect_tx(rg.full(s), row_bytes * n_in);
    const uint32_t dst = smem_u32(rg.slots + (size_t)s * slot_bytes);
#pragma unroll
    for (int i = 0; i < NIN; ++i)
      if (i < n_in) bulk_load(dst + i * row_bytes, src[i] + (size_t)row * row_bytes, row_bytes, rg.full(s));
  }
  // Do not leave while copies may still be landing in this CTA's shared memory.
  const uint32_t pending = k < (uint32_t)stages ? k : (uint32_t)stages;
  for (uint32_t j = k - pending; j < k; ++j) mbar_wait_drain(rg.full(j % stages), (j / stages) & 1u);
}

// ------------------------------------------------------------------ forward
// y = x * rsqrt(mean(x^2) + eps) * w; ADD: x := round(x + res) first, also stored to res_out.
template <typename T, int MV, bool ADD>
__global__ void __launch_bounds__(kThreads, MV <= 2 ? 2 : 1)
rmsnorm_fwd_ring_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w, T* __restrict__ y,
                        T* __restrict__ res_out, float* __restrict__ inv, int64_t rows, int H, float eps, int stages,
                        int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t row_bytes = (uint32_t)H * sizeof(T);
  const size_t slot_bytes = (size_t)row_bytes * (ADD ? 2 : 1);
  const Ring rg = ring_setup(smem, stages, slot_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kConsumers / 32) {
    if (lane == 0) {
      const uint8_t* const src[2] = {reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(res)};
      produce<2>(rg, src, ADD ? 2 : 1, rows, row_bytes, stages, slot_bytes);
    }
  } else {
    const int t = threadIdx.x, nvec = H / 8;
    float ww[MV][8];
#pragma unroll
    for (int i = 0; i < MV; ++i)
      if (t + i * kConsumers < nvec) VecIO<T, 8>::load(w + (size_t)(t + i * kConsumers) * 8, ww[i]);
    uint32_t k = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++k) {
      const int s = k % stages;
      const bool ok = mbar_wait(rg.full(s), (k / stages) & 1u, rg.abort_flag);
      const T* sx = reinterpret_cast<const T*>(rg.slots + (size_t)s * slot_bytes);
      float c[MV][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < MV; ++i) {
        const int v = t + i * kConsumers;
        if (v < nvec) {
          VecIO<T, 8>::load(sx + (size_t)v * 8, c[i]);
          if constexpr (ADD) {
            float r[8];
            VecIO<T, 8>::load(sx + H + (size_t)v * 8, r);
#pragma unroll
            for (int j = 0; j < 8; ++j) c[i][j] = to_f32<T>(from_f32<T>(c[i][j] + r[j]));   // the stored value is what is normalised
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += c[i][j] * c[i][j];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(rg.empty(s));
      ss = warp_sum(ss);
      float* red = rg.red + (k & 1u) * 8;
      if (lane == 0) red[warp] = ss;
      if (!consumers_all(ok)) break;
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < kConsumers / 32; ++i) tot += red[i];
      const float r = rsqrtf(tot / (float)H + eps);
#pragma unroll
      for (int i = 0; i < MV; ++i) {
        const int v = t + i * kConsumers;
        if (v < nvec) {
          if constexpr (ADD) VecIO<T, 8>::store(res_out + (size_t)row * H + (size_t)v * 8, c[i]);
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = c[i][j] * r * ww[i][j];
          VecIO<T, 8>::store(y + (size_t)row * H + (size_t)v * 8, o);
        }
      }
      if (t == 0) inv[row] = r;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *rg.abort_flag) flag_status(status, Q3_STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ backward
// dx = inv * (dy*w - x * inv^2 * mean(dy*w*x)) [+ dres];  partial[cta][c] = sum over the CTA's rows of dy * x * inv.
template <typename T, int MV>
__global__ void __launch_bounds__(kThreads, MV <= 2 ? 2 : 1)
rmsnorm_bwd_ring_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                        const T* __restrict__ dres, const float* __restrict__ inv, T* __restrict__ dx,
                        float* __restrict__ partial, int64_t rows, int H, int stages, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t row_bytes = (uint32_t)H * sizeof(T);
  const int n_in = dres != nullptr ? 3 : 2;
  const size_t slot_bytes = (size_t)row_bytes * n_in;
  const Ring rg = ring_setup(smem, stages, slot_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kConsumers / 32) {
    if (lane == 0) {
      const uint8_t* const src[3] = {reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(dy),
                                     reinterpret_cast<const uint8_t*>(dres)};
      produce<3>(rg, src, n_in, rows, row_bytes, stages, slot_bytes);
    }
  } else {
    const int t = threadIdx.x, nvec = H / 8;
    float ww[MV][8], acc[MV][8];
#pragma unroll
    for (int i = 0; i < MV; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { acc[i][j] = 0.f; ww[i][j] = 0.f; }
      if (t + i * kConsumers < nvec) VecIO<T, 8>::load(w + (size_t)(t + i * kConsumers) * 8, ww[i]);
    }
    uint32_t k = 0;
    float r_next = blockIdx.x < rows ? inv[blockIdx.x] : 0.f;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++k) {
      const float r = r_next;
      if (row + gridDim.x < rows) r_next = inv[row + gridDim.x];
      const int s = k % stages;
      const bool ok = mbar_wait(rg.full(s), (k / stages) & 1u, rg.abort_flag);
      const T* sx = reinterpret_cast<const T*>(rg.slots + (size_t)s * slot_bytes);
      float cx[MV][8], cg[MV][8];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < MV; ++i) {
        const int v = t + i * kConsumers;
        if (v < nvec) {
          VecIO<T, 8>::load(sx + (size_t)v * 8, cx[i]);
          VecIO<T, 8>::load(sx + H + (size_t)v * 8, cg[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < MV; ++i) {
        if (t + i * kConsumers < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[i][j] += cg[i][j] * cx[i][j] * r;
            cg[i][j] *= ww[i][j];
            sum += cg[i][j] * cx[i][j];
          }
        }
      }
      sum = warp_sum(sum);
      float* red = rg.red + (k & 1u) * 8;
      if (lane == 0) red[warp] = sum;
      if (!consumers_all(ok)) break;
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < kConsumers / 32; ++i) tot += red[i];
      const float coef = tot * r * r / (float)H;
#pragma unroll
      for (int i = 0; i < MV; ++i) {
        const int v = t + i * kConsumers;
        if (v < nvec) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (cg[i][j] - cx[i][j] * coef) * r;
          if (n_in == 3) {   // the upstream residual gradient is still in the slot
            float d[8];
            VecIO<T, 8>::load(sx + 2 * (size_t)H + (size_t)v * 8, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += d[j];
          }
          VecIO<T, 8>::store(dx + (size_t)row * H + (size_t)v * 8, o);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(rg.empty(s));
    }
    // every consumer writes its columns of this CTA's partial row (zeros if the CTA had no rows)
#pragma unroll
    for (int i = 0; i < MV; ++i) {
      const int v = t + i * kConsumers;
      if (v < nvec) {
        float* dst = partial + (size_t)blockIdx.x * H + (size_t)v * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *rg.abort_flag) flag_status(status, Q3_STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ per-head RMSNorm + RoPE, token-major rows
// x is [tokens, heads, D]; cos/sin are [tokens, D]. A slot holds `tps` consecutive tokens: their heads*D input
// elements (one contiguous copy), for backward the same span of dy, and their cos and sin rows. The 256 consumers
// form 256/tpr groups of tpr = D/16 lanes; group g owns row g of the slot (token g / heads, head g % heads) and
// each lane the vector pair (p, p + D/2). Reductions stay inside a group (shuffles), so consumers need no
// CTA-wide barrier; warps leave the loop on their own if a wait expires.
struct RopeGeom {
  int tpr;        // lanes per (token, head) row = D / 16
  int tps;        // tokens per slot
  uint32_t x_bytes, t_bytes;   // bytes of one token's heads*D elements, of one token's D table elements
};

template <typename T, bool BWD>
__device__ __forceinline__ void rope_produce(const Ring& rg, const RopeGeom& g, const T* x, const T* dy, const T* cs,
                                             const T* sn, int64_t tokens, int stages, size_t slot_bytes, int cta,
                                             int ncta) {
  uint32_t k = 0;
  const int64_t groups = (tokens + g.tps - 1) / g.tps;
  const uint32_t x_slot = g.x_bytes * g.tps, t_slot = g.t_bytes * g.tps;
  for (int64_t tg = cta; tg < groups; tg += ncta, ++k) {
    const int s = k % stages;
    if (!mbar_wait(rg.empty(s), ((k / stages) & 1u) ^ 1u, rg.abort_flag)) break;
    const int64_t tok0 = tg * g.tps;
    const uint32_t n = (uint32_t)((tokens - tok0) < g.tps ? (tokens - tok0) : g.tps);
    const uint32_t xb = g.x_bytes * n, tb = g.t_bytes * n;
    mbar_expect_tx(rg.full(s), (BWD ? 2 : 1) * xb + 2 * tb);
    const uint32_t dst = smem_u32(rg.slots + (size_t)s * slot_bytes);
    const uint8_t* xs = reinterpret_cast<const uint8_t*>(x) + (size_t)tok0 * g.x_bytes;
    bulk_load(dst, xs, xb, rg.full(s));
    uint32_t off = x_slot;
    if (BWD) {
      bulk_load(dst + off, reinterpret_cast<const uint8_t*>(dy) + (size_t)tok0 * g.x_bytes, xb, rg.full(s));
      off += x_slot;
    }
    bulk_load(dst + off, reinterpret_cast<const uint8_t*>(cs) + (size_t)tok0 * g.t_bytes, tb, rg.full(s));
    bulk_load(dst + off + t_slot, reinterpret_cast<const uint8_t*>(sn) + (size_t)tok0 * g.t_bytes, tb, rg.full(s));
  }
  const uint32_t pending = k < (uint32_t)stages ? k : (uint32_t)stages;
  for (uint32_t j = k - pending; j < k; ++j) mbar_wait_drain(rg.full(j % stages), (j / stages) & 1u);
}

// One tensor's share of a launch: q and k of a layer go through one grid, CTAs [0, ncta) of the first job and
// [ncta_a, ncta_a + ncta_b) of the second (ncta = 0: no second tensor).
template <typename T> struct RopeJob {
  const T* x;        // [tokens, heads, D]
  const T* w;        // [D]
  const T* dy;       // backward only
  T* y;              // forward: output; backward: dx
  float* inv;        // [tokens * heads]; forward writes, backward reads
  float* partial;    // backward: [ncta][D]
  int heads, stages, ncta;
  RopeGeom g;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
norm_rope_fwd_ring_kernel(const RopeJob<T> ja, const RopeJob<T> jb, const T* __restrict__ cs, const T* __restrict__ sn,
                          int64_t tokens, int D, float eps, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const bool second = (int)blockIdx.x >= ja.ncta;
  const RopeJob<T>& job = second ? jb : ja;
  const int cta = second ? (int)blockIdx.x - ja.ncta : (int)blockIdx.x, ncta = job.ncta;
  const RopeGeom g = job.g;
  const int heads = job.heads, stages = job.stages;
  const T* __restrict__ x = job.x;
  const T* __restrict__ w = job.w;
  T* __restrict__ y = job.y;
  float* __restrict__ inv = job.inv;
  const size_t slot_bytes = (size_t)g.tps * (g.x_bytes + 2 * g.t_bytes);
  const Ring rg = ring_setup(smem, stages, slot_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kConsumers / 32) {
    if (lane == 0) rope_produce<T, false>(rg, g, x, nullptr, cs, sn, tokens, stages, slot_bytes, cta, ncta);
  } else {
    const int half = D / 2, grp = threadIdx.x / g.tpr, p = threadIdx.x % g.tpr;
    const int ltok = grp / heads, head = grp - ltok * heads;     // this lane's row inside a slot
    float w1[8], w2[8];
    VecIO<T, 8>::load(w + p * 8, w1);
    VecIO<T, 8>::load(w + half + p * 8, w2);
    const int64_t groups = (tokens + g.tps - 1) / g.tps;
    uint32_t k = 0;
    for (int64_t tg = cta; tg < groups; tg += ncta, ++k) {
      const int s = k % stages;
      bool ok = mbar_wait(rg.full(s), (k / stages) & 1u, rg.abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int64_t token = tg * g.tps + ltok;
      const bool valid = token < tokens;
      const T* sx = reinterpret_cast<const T*>(rg.slots + (size_t)s * slot_bytes);
      const T* row = sx + (size_t)grp * D;
      const T* scs = sx + (size_t)g.tps * heads * D + (size_t)ltok * D;
      const T* ssn = scs + (size_t)g.tps * D;
      float a[8], b[8], c1[8], c2[8], s1[8], s2[8];
      if (valid) {
        VecIO<T, 8>::load(row + p * 8, a);
        VecIO<T, 8>::load(row + half + p * 8, b);
        VecIO<T, 8>::load(scs + p * 8, c1);
        VecIO<T, 8>::load(scs + half + p * 8, c2);
        VecIO<T, 8>::load(ssn + p * 8, s1);
        VecIO<T, 8>::load(ssn + half + p * 8, s2);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = b[j] = c1[j] = c2[j] = s1[j] = s2[j] = 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(rg.empty(s));
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += a[j] * a[j] + b[j] * b[j];
      for (int o = g.tpr >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss / (float)D + eps);
      if (valid) {
        float o1[8], o2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float na = a[j] * r * w1[j], nb = b[j] * r * w2[j];
          o1[j] = na * c1[j] - nb * s1[j];
          o2[j] = nb * c2[j] + na * s2[j];
        }
        T* out = y + ((size_t)token * heads + head) * D;
        VecIO<T, 8>::store(out + p * 8, o1);
        VecIO<T, 8>::store(out + half + p * 8, o2);
        if (p == 0) inv[(size_t)token * heads + head] = r;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *rg.abort_flag) flag_status(status, Q3_STATUS_WAIT_TIMEOUT);
}

// Backward: dn1 = g1*cos1 + g2*sin2 ; dn2 = g2*cos2 - g1*sin1, then the RMSNorm backward of dn on x.
// partial[cta][c] = sum over the CTA's rows of dn[c] * x[c] * inv, combined over the CTA's groups in a fixed order.
template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
norm_rope_bwd_ring_kernel(const RopeJob<T> ja, const RopeJob<T> jb, const T* __restrict__ cs, const T* __restrict__ sn,
                          int64_t tokens, int D, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const bool second = (int)blockIdx.x >= ja.ncta;
  const RopeJob<T>& job = second ? jb : ja;
  const int cta = second ? (int)blockIdx.x - ja.ncta : (int)blockIdx.x, ncta = job.ncta;
  const RopeGeom g = job.g;
  const int heads = job.heads, stages = job.stages;
  const T* __restrict__ x = job.x;
  const T* __restrict__ w = job.w;
  const T* __restrict__ dy = job.dy;
  T* __restrict__ dx = job.y;
  const float* __restrict__ inv = job.inv;
  float* __restrict__ partial = job.partial;
  const size_t slot_bytes = (size_t)g.tps * (2 * g.x_bytes + 2 * g.t_bytes);
  const Ring rg = ring_setup(smem, stages, slot_bytes);
  float* comb = reinterpret_cast<float*>(smem + ring_smem_bytes(stages, slot_bytes));   // [groups][D], 16-byte aligned
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kConsumers / 32) {
    if (lane == 0) rope_produce<T, true>(rg, g, x, dy, cs, sn, tokens, stages, slot_bytes, cta, ncta);
  } else {
    const int half = D / 2, grp = threadIdx.x / g.tpr, p = threadIdx.x % g.tpr;
    const int ltok = grp / heads, head = grp - ltok * heads;
    float w1[8], w2[8], acc1[8], acc2[8];
    VecIO<T, 8>::load(w + p * 8, w1);
    VecIO<T, 8>::load(w + half + p * 8, w2);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc1[j] = acc2[j] = 0.f;
    const int64_t groups = (tokens + g.tps - 1) / g.tps;
    uint32_t k = 0;
    auto inv_of = [&](int64_t tg) {
      const int64_t token = tg * g.tps + ltok;
      return (tg < groups && token < tokens) ? inv[(size_t)token * heads + head] : 0.f;
    };
    float r_next = inv_of(cta);
    for (int64_t tg = cta; tg < groups; tg += ncta, ++k) {
      const float r = r_next;
      r_next = inv_of(tg + ncta);
      const int s = k % stages;
      bool ok = mbar_wait(rg.full(s), (k / stages) & 1u, rg.abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int64_t token = tg * g.tps + ltok;
      const bool valid = token < tokens;
      const T* sx = reinterpret_cast<const T*>(rg.slots + (size_t)s * slot_bytes);
      const size_t span = (size_t)g.tps * heads * D;
      const T* xrow = sx + (size_t)grp * D;
      const T* grow = sx + span + (size_t)grp * D;
      const T* scs = sx + 2 * span + (size_t)ltok * D;
      const T* ssn = scs + (size_t)g.tps * D;
      // rotate the gradient first so that the tables and dy are dead before x is read: fewer live registers
      float x1[8], x2[8], d1[8], d2[8];
      if (valid) {
        float g1[8], g2[8], c[8], sv[8];
        VecIO<T, 8>::load(grow + p * 8, g1);
        VecIO<T, 8>::load(grow + half + p * 8, g2);
        VecIO<T, 8>::load(scs + p * 8, c);
        VecIO<T, 8>::load(ssn + half + p * 8, sv);
#pragma unroll
        for (int j = 0; j < 8; ++j) d1[j] = g1[j] * c[j] + g2[j] * sv[j];
        VecIO<T, 8>::load(scs + half + p * 8, c);
        VecIO<T, 8>::load(ssn + p * 8, sv);
#pragma unroll
        for (int j = 0; j < 8; ++j) d2[j] = g2[j] * c[j] - g1[j] * sv[j];
        VecIO<T, 8>::load(xrow + p * 8, x1);
        VecIO<T, 8>::load(xrow + half + p * 8, x2);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x1[j] = x2[j] = d1[j] = d2[j] = 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(rg.empty(s));
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc1[j] += d1[j] * x1[j] * r;
        acc2[j] += d2[j] * x2[j] * r;
        d1[j] *= w1[j];
        d2[j] *= w2[j];
        sum += d1[j] * x1[j] + d2[j] * x2[j];
      }
      for (int o = g.tpr >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float coef = sum * r * r / (float)D;
      if (valid) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          d1[j] = (d1[j] - x1[j] * coef) * r;
          d2[j] = (d2[j] - x2[j] * coef) * r;
        }
        T* out = dx + ((size_t)token * heads + head) * D;
        VecIO<T, 8>::store(out + p * 8, d1);
        VecIO<T, 8>::store(out + half + p * 8, d2);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      comb[(size_t)grp * D + p * 8 + j] = acc1[j];
      comb[(size_t)grp * D + half + p * 8 + j] = acc2[j];
    }
  }
  __syncthreads();
  const int ngroups = kConsumers / g.tpr;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float tsum = 0.f;
    for (int r2 = 0; r2 < ngroups; ++r2) tsum += comb[(size_t)r2 * D + c];
    partial[(size_t)cta * D + c] = tsum;
  }
  if (threadIdx.x == 0 && *rg.abort_flag) flag_status(status, Q3_STATUS_WAIT_TIMEOUT);
}

inline int pick_stages(size_t slot_bytes) {
  // two CTAs per SM, ~100 KB of ring each; at least 2 slots
  int s = (int)((100 * 1024) / slot_bytes);
  return s < 2 ? 2 : (s > kMaxStages ? kMaxStages : s);
}

template <typename K> inline int allow_smem(K kern, size_t bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_CUDA - (int)e;
}

}  // namespace ring

// True if the ring kernels serve this row width and element type.
bool rmsnorm_ring_applies(int64_t H, int dtype) {
  return (dtype == Q3_BF16 || dtype == Q3_F16) && H >= 2048 && H <= 8192 && H % 8 == 0;
}

// Number of partial weight-gradient rows the backward ring kernel writes (its grid size).
int rmsnorm_bwd_ring_parts(int64_t rows) {
  const int64_t cap = (int64_t)sm_count() * 2;
  return (int)(rows < cap ? rows : cap);
}

template <typename T>
static int fwd_ring_t(const void* x, const void* res, const void* w, void* y, void* res_out, float* inv, int64_t rows,
                      int64_t H, float eps, cudaStream_t st) {
  using namespace ring;
  const bool add = res != nullptr;
  const size_t slot = (size_t)H * sizeof(T) * (add ? 2 : 1);
  const int stages = pick_stages(slot);
  const size_t smem = ring_smem_bytes(stages, slot);
  const int64_t cap = (int64_t)sm_count() * 2;
  const int grid = (int)(rows < cap ? rows : cap);
  int* status = async_status();
  int rc;
#define Q3_FWD(MV, ADD)                                                                                          \
  do {                                                                                                           \
    auto kern = rmsnorm_fwd_ring_kernel<T, MV, ADD>;                                                             \
    if ((rc = allow_smem(kern, smem)) != Q3_OK) return rc;                                                       \
    kern<<<grid, kThreads, smem, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)res_out, inv, rows,   \
                                       (int)H, eps, stages, status);                                             \
  } while (0)
  if (H <= 4096) { if (add) Q3_FWD(2, true); else Q3_FWD(2, false); }
  else { if (add) Q3_FWD(4, true); else Q3_FWD(4, false); }
#undef Q3_FWD
  return launch_status();
}

int rmsnorm_fwd_ring(const void* x, const void* res, const void* w, void* y, void* res_out, float* inv, int64_t rows,
                     int64_t H, float eps, int dtype, cudaStream_t st) {
  return dtype == Q3_BF16 ? fwd_ring_t<__nv_bfloat16>(x, res, w, y, res_out, inv, rows, H, eps, st)
                          : fwd_ring_t<__half>(x, res, w, y, res_out, inv, rows, H, eps, st);
}

template <typename T>
static int bwd_ring_t(const void* x, const void* w, const void* dy, const void* dres, const float* inv, void* dx,
                      float* partial, int64_t rows, int64_t H, cudaStream_t st) {
  using namespace ring;
  const size_t slot = (size_t)H * sizeof(T) * (dres ? 3 : 2);
  const int stages = pick_stages(slot);
  const size_t smem = ring_smem_bytes(stages, slot);
  const int grid = rmsnorm_bwd_ring_parts(rows);
  int* status = async_status();
  int rc;
#define Q3_BWD(MV)                                                                                               \
  do {                                                                                                           \
    auto kern = rmsnorm_bwd_ring_kernel<T, MV>;                                                                  \
    if ((rc = allow_smem(kern, smem)) != Q3_OK) return rc;                                                       \
    kern<<<grid, kThreads, smem, st>>>((const T*)x, (const T*)w, (const T*)dy, (const T*)dres, inv, (T*)dx,      \
                                       partial, rows, (int)H, stages, status);                                   \
  } while (0)
  if (H <= 4096) Q3_BWD(2); else Q3_BWD(4);
#undef Q3_BWD
  return launch_status();
}

int rmsnorm_bwd_ring(const void* x, const void* w, const void* dy, const void* dres, const float* inv, void* dx,
                     float* partial, int64_t rows, int64_t H, int dtype, cudaStream_t st) {
  return dtype == Q3_BF16 ? bwd_ring_t<__nv_bfloat16>(x, w, dy, dres, inv, dx, partial, rows, H, st)
                          : bwd_ring_t<__half>(x, w, dy, dres, inv, dx, partial, rows, H, st);
}


// Geometry of the token-major norm+RoPE ring kernels, or tpr = 0 if they do not serve this shape: D a multiple of 16
// up to 512 (16, 32, 64 ... lanes per row must divide a warp), and heads dividing the 256 / (D/16) rows of a slot.
static ring::RopeGeom rope_geom(int64_t heads, int64_t D, int dtype) {
  ring::RopeGeom g{0, 0, 0, 0};
  if (dtype != Q3_BF16 && dtype != Q3_F16) return g;
  if (D % 16 != 0 || D > 512) return g;
  const int tpr = (int)(D / 16);
  if (tpr & (tpr - 1)) return g;
  const int rows = ring::kConsumers / tpr;
  if (heads > rows || rows % heads != 0) return g;
  g.tpr = tpr;
  g.tps = (int)(rows / heads);
  g.x_bytes = (uint32_t)(heads * D * 2);
  g.t_bytes = (uint32_t)(D * 2);
  return g;
}

bool norm_rope_ring_applies(int64_t heads, int64_t D, int dtype) { return rope_geom(heads, D, dtype).tpr != 0; }

// CTAs given to a tensor: all two-per-SM slots when it is alone, its share by bytes when q and k go together.
static int rope_ctas(int64_t tokens, const ring::RopeGeom& g, int64_t cap) {
  const int64_t groups = (tokens + g.tps - 1) / g.tps;
  return (int)(groups < cap ? groups : (cap < 1 ? 1 : cap));
}

int norm_rope_bwd_ring_parts(int64_t tokens, int64_t heads, int64_t D, int dtype) {
  return rope_ctas(tokens, rope_geom(heads, D, dtype), (int64_t)sm_count() * 2);
}

// Number of partial rows each tensor of a fused q+k backward writes: q first, then k.
void qk_norm_rope_bwd_ring_parts(int64_t tokens, int64_t hq, int64_t hk, int64_t D, int dtype, int* parts_q,
                                 int* parts_k) {
  const int64_t cap = (int64_t)sm_count() * 2;
  int64_t cq = cap * hq / (hq + hk);
  if (cq < 1) cq = 1;
  if (cq > cap - 1) cq = cap - 1;
  *parts_q = rope_ctas(tokens, rope_geom(hq, D, dtype), cq);
  *parts_k = rope_ctas(tokens, rope_geom(hk, D, dtype), cap - cq);
}

template <typename T>
static ring::RopeJob<T> make_job(const void* x, const void* w, const void* dy, void* y, float* inv, float* partial,
                                 int64_t heads, int64_t D, int dtype, int ncta, bool bwd, size_t* smem) {
  using namespace ring;
  RopeJob<T> j{};
  j.x = (const T*)x; j.w = (const T*)w; j.dy = (const T*)dy; j.y = (T*)y; j.inv = inv; j.partial = partial;
  j.heads = (int)heads; j.ncta = ncta;
  *smem = 0;
  if (ncta == 0) return j;
  j.g = rope_geom(heads, D, dtype);
  const size_t slot = (size_t)j.g.tps * ((bwd ? 2 : 1) * j.g.x_bytes + 2 * j.g.t_bytes);
  const size_t comb = bwd ? (size_t)(kConsumers / j.g.tpr) * D * sizeof(float) : 0;
  int stages = (int)((100 * 1024 - comb) / slot);
  j.stages = stages < 2 ? 2 : (stages > kMaxStages ? kMaxStages : stages);
  *smem = ring_smem_bytes(j.stages, slot) + comb;
  return j;
}

template <typename T>
static int rope_fwd_launch(const void* xa, const void* wa, void* ya, float* inva, int64_t ha, int ca, const void* xb,
                           const void* wb, void* yb, float* invb, int64_t hb, int cb, const void* cs, const void* sn,
                           int64_t tokens, int64_t D, float eps, int dtype, cudaStream_t st) {
  using namespace ring;
  size_t sa, sb;
  const RopeJob<T> ja = make_job<T>(xa, wa, nullptr, ya, inva, nullptr, ha, D, dtype, ca, false, &sa);
  const RopeJob<T> jb = make_job<T>(xb, wb, nullptr, yb, invb, nullptr, hb, D, dtype, cb, false, &sb);
  const size_t smem = sa > sb ? sa : sb;
  auto kern = norm_rope_fwd_ring_kernel<T>;
  int rc = allow_smem(kern, smem);
  if (rc != Q3_OK) return rc;
  kern<<<ca + cb, kThreads, smem, st>>>(ja, jb, (const T*)cs, (const T*)sn, tokens, (int)D, eps, async_status());
  return launch_status();
}

template <typename T>
static int rope_bwd_launch(const void* xa, const void* wa, const void* dya, void* dxa, const float* inva, float* pa,
                           int64_t ha, int ca, const void* xb, const void* wb, const void* dyb, void* dxb,
                           const float* invb, float* pb, int64_t hb, int cb, const void* cs, const void* sn,
                           int64_t tokens, int64_t D, int dtype, cudaStream_t st) {
  using namespace ring;
  size_t sa, sb;
  const RopeJob<T> ja = make_job<T>(xa, wa, dya, dxa, const_cast<float*>(inva), pa, ha, D, dtype, ca, true, &sa);
  const RopeJob<T> jb = make_job<T>(xb, wb, dyb, dxb, const_cast<float*>(invb), pb, hb, D, dtype, cb, true, &sb);
  const size_t smem = sa > sb ? sa : sb;
  auto kern = norm_rope_bwd_ring_kernel<T>;
  int rc = allow_smem(kern, smem);
  if (rc != Q3_OK) return rc;
  kern<<<ca + cb, kThreads, smem, st>>>(ja, jb, (const T*)cs, (const T*)sn, tokens, (int)D, async_status());
  return launch_status();
}

int norm_rope_fwd_ring(const void* x, const void* w, const void* cs, const void* sn, void* y, float* inv,
                       int64_t tokens, int64_t heads, int64_t D, float eps, int dtype, cudaStream_t st) {
  const int c = rope_ctas(tokens, rope_geom(heads, D, dtype), (int64_t)sm_count() * 2);
  return dtype == Q3_BF16
             ? rope_fwd_launch<__nv_bfloat16>(x, w, y, inv, heads, c, nullptr, nullptr, nullptr, nullptr, 0, 0, cs, sn, tokens, D, eps, dtype, st)
             : rope_fwd_launch<__half>(x, w, y, inv, heads, c, nullptr, nullptr, nullptr, nullptr, 0, 0, cs, sn, tokens, D, eps, dtype, st);
}

int norm_rope_bwd_ring(const void* x, const void* w, const void* cs, const void* sn, const void* dy, const float* inv,
                       void* dx, float* partial, int64_t tokens, int64_t heads, int64_t D, int dtype,
                       cudaStream_t st) {
  const int c = norm_rope_bwd_ring_parts(tokens, heads, D, dtype);
  return dtype == Q3_BF16
             ? rope_bwd_launch<__nv_bfloat16>(x, w, dy, dx, inv, partial, heads, c, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, cs, sn, tokens, D, dtype, st)
             : rope_bwd_launch<__half>(x, w, dy, dx, inv, partial, heads, c, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, cs, sn, tokens, D, dtype, st);
}

// q and k of one layer in one launch.
int qk_norm_rope_fwd_ring(const void* q, const void* wq, void* yq, float* invq, int64_t hq, const void* k,
                          const void* wk, void* yk, float* invk, int64_t hk, const void* cs, const void* sn,
                          int64_t tokens, int64_t D, float eps, int dtype, cudaStream_t st) {
  int cq, ck;
  qk_norm_rope_bwd_ring_parts(tokens, hq, hk, D, dtype, &cq, &ck);
  return dtype == Q3_BF16
             ? rope_fwd_launch<__nv_bfloat16>(q, wq, yq, invq, hq, cq, k, wk, yk, invk, hk, ck, cs, sn, tokens, D, eps, dtype, st)
             : rope_fwd_launch<__half>(q, wq, yq, invq, hq, cq, k, wk, yk, invk, hk, ck, cs, sn, tokens, D, eps, dtype, st);
}

int qk_norm_rope_bwd_ring(const void* q, const void* wq, const void* dyq, void* dq, const float* invq, float* pq,
                          int64_t hq, const void* k, const void* wk, const void* dyk, void* dk, const float* invk,
                          float* pk, int64_t hk, const void* cs, const void* sn, int64_t tokens, int64_t D, int dtype,
                          cudaStream_t st) {
  int cq, ck;
  qk_norm_rope_bwd_ring_parts(tokens, hq, hk, D, dtype, &cq, &ck);
  return dtype == Q3_BF16
             ? rope_bwd_launch<__nv_bfloat16>(q, wq, dyq, dq, invq, pq, hq, cq, k, wk, dyk, dk, invk, pk, hk, ck, cs, sn, tokens, D, dtype, st)
             : rope_bwd_launch<__half>(q, wq, dyq, dq, invq, pq, hq, cq, k, wk, dyk, dk, invk, pk, hk, ck, cs, sn, tokens, D, dtype, st);
}

}  // namespace q3
