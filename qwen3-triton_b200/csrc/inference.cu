// Decode-time kernels: positions, KV-cache append, attention over the cache, small-M linear (GEMV) and greedy token
// selection. All of them are bound by HBM traffic (the cache, the weight matrix, the logits), so the work is laid out
// to read each byte once, with 16-byte accesses and enough of them in flight:
//   * attention over the cache runs one CTA per (batch, kv head, chunk of keys) and serves ALL query heads of the
//     group from one pass over that K/V chunk (grouped-query attention: 4 query heads share a kv head in Qwen3, so
//     the cache is read once instead of four times); the chunk is staged in shared memory with asynchronous copies,
//     and a small merge kernel combines the chunks by their log-sum-exp;
//   * the GEMV gives every warp a few weight rows and streams them once for up to 8 input rows;
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

constexpr int kAttnThreads = 256;  // 8 warps; a warp covers two keys per step (16 lanes per key row)
constexpr int kTileBytes = 32768;  // one K (or V) chunk in shared memory
// keys per CTA: as many rows of D elements as fit 32 KB (128 keys at head_dim 128 in bf16)
__host__ __device__ constexpr int chunk_keys(int D, int elem_bytes) { return kTileBytes / (D * elem_bytes); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Partial attention of one query token against one chunk of cached keys, for the G query heads of a kv head.
//   q      [B, S, Hq, D]       cache_k / cache_v [B, Hkv, C, D]
//   part   [B, S, Hq, splits, D] fp32 (normalised within the chunk)   lse [B, S, Hq, splits] fp32 (natural log)
// Key t is visible to query token s iff t <= start + s. EPL = D / 16 elements per lane.
// The CTA first brings the live part of its K and V chunk into shared memory with 16-byte asynchronous copies (up to
// 64 KB in flight per CTA, two CTAs per SM: enough outstanding bytes to keep HBM busy), then its warps walk the keys
// from there.
template <typename T, int EPL, int G>
__global__ void __launch_bounds__(kAttnThreads, 2)
cache_attention_partial_kernel(const T* __restrict__ q, const T* __restrict__ ck, const T* __restrict__ cv,
                               float* __restrict__ part, float* __restrict__ lse, int64_t S, int64_t Hq, int64_t Hkv,
                               int64_t C, int64_t start, int splits, float scale) {
  constexpr int D = EPL * 16;
  constexpr int CHUNK = chunk_keys(D, (int)sizeof(T));
  extern __shared__ __align__(128) uint8_t smem[];
  const T* ks = reinterpret_cast<const T*>(smem);
  const T* vs = reinterpret_cast<const T*>(smem + kTileBytes);
  const int split = blockIdx.x, s = blockIdx.y;
  const int64_t bk = blockIdx.z, b = bk / Hkv, kvh = bk % Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  const int64_t visible = start + s + 1;                      // keys 0 .. visible-1
  const int64_t first = (int64_t)split * CHUNK;
  int64_t last = first + CHUNK;
  if (last > visible) last = visible;
  const int live_keys = last > first ? (int)(last - first) : 0;

  {   // the live part of the chunk is one contiguous range of the cache
    const uint8_t* kg = reinterpret_cast<const uint8_t*>(ck + (bk * C + first) * D);
    const uint8_t* vg = reinterpret_cast<const uint8_t*>(cv + (bk * C + first) * D);
    const int nbytes = live_keys * D * (int)sizeof(T);
    for (int off = threadIdx.x * 16; off < nbytes; off += kAttnThreads * 16) {
      cp_async16(smem + off, kg + off);
      cp_async16(smem + kTileBytes + off, vg + off);
    }
  }
  // this lane's slice of the G query vectors, pre-scaled (overlaps the copies)
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
  cp_async_wait_all();
  __syncthreads();
  // warp w takes keys 2*w + half, stepping by 16 (8 warps x 2 keys)
  for (int t0 = 2 * warp; t0 < live_keys; t0 += 16) {
    const int t = t0 + half;
    const bool live = t < live_keys;
    float kk[EPL], vv[EPL];
    if (live) {
      constexpr int W = (16 / (int)sizeof(T)) < EPL ? (16 / (int)sizeof(T)) : EPL;   // 8- or 16-byte accesses
#pragma unroll
      for (int c = 0; c < EPL / W; ++c) {
        float tmp[W];
        VecIO<T, W>::load(ks + t * D + sub * EPL + c * W, tmp);
#pragma unroll
        for (int e = 0; e < W; ++e) kk[c * W + e] = tmp[e];
        VecIO<T, W>::load(vs + t * D + sub * EPL + c * W, tmp);
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
  __syncthreads();                                             // every warp is done with the tiles: reuse them
  float* s_acc = reinterpret_cast<float*>(smem);               // [8 warps][G][D], at most 32 KB
  float* s_max = reinterpret_cast<float*>(smem + kTileBytes);  // [8][G]
  float* s_sum = s_max + 8 * G;
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
    if (lane == 0) { s_max[warp * G + g] = m[g]; s_sum[warp * G + g] = l[g]; }
    if (half == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) s_acc[(warp * G + g) * D + sub * EPL + e] = acc[g][e];
    }
  }
  __syncthreads();
  // thread (g, column) combines the 8 warps in warp order: deterministic
  for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
    const int g = idx / D, d = idx % D;
    float nm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 8; ++w) nm = fmaxf(nm, s_max[w * G + g]);
    float tot = 0.f, val = 0.f;
    if (nm > -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float f = __expf(s_max[w * G + g] - nm);
        tot += s_sum[w * G + g] * f;
        val += s_acc[(w * G + g) * D + d] * f;
      }
    }
    const int64_t row = ((b * S + s) * Hq + kvh * G + g) * splits + split;
    part[row * D + d] = tot > 0.f ? val / tot : 0.f;
    if (d == 0) lse[row] = tot > 0.f ? nm + __logf(tot) : -CUDART_INF_F;
  }
}

// ---- the same partial attention on the tensor cores (16-bit types, head_dim 128) ------------------------------------
// The CUDA-core kernel above spends ~90 instructions per key on a 4-head group and is issue-bound at a quarter of the
// HBM rate. Here the G query heads of a group are the rows of a 16-row MMA tile (rows G..15 are zero), so one
// mma.sync m16n8k16 per 8 keys and 16 head-dim values does the score work of all heads at once, and a second one per
// 8 output columns the value work: about 150 instructions per warp for its 16 keys. Each of the 8 warps takes 16 of
// the chunk's 128 keys, so there is no running rescale inside a warp; the warps are merged as in the kernel above.
// K and V rows (256 bytes) are stored with their 16-byte pieces XOR-swizzled by (key & 7), which makes the
// ldmatrix reads - eight rows 256 bytes apart - conflict-free.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T> __device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0;   // rows 8..15 of the A tile are zero
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_16816<__half>(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
// all 16 rows of the A tile in use
template <typename T> __device__ __forceinline__ void mma_16816_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_16816_full<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_16816_full<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One CTA walks `chunks_per_cta` consecutive 128-key chunks through two shared-memory stages: the copies of the next
// chunk are in flight while the tensor cores work on the current one. Every warp keeps a running (max, sum, output)
// for its 16 keys of each chunk and rescales when the maximum moves.
template <typename T, int G>
__global__ void __launch_bounds__(kAttnThreads, 1)
cache_attention_partial_mma_kernel(const T* __restrict__ q, const T* __restrict__ ck, const T* __restrict__ cv,
                                   float* __restrict__ part, float* __restrict__ lse, int64_t S, int64_t Hq, int64_t Hkv,
                                   int64_t C, int64_t start, int splits, int chunks_per_cta, float scale) {
  constexpr int D = 128, CHUNK = 128, ROW = 256;               // ROW: bytes per key row
  constexpr int STAGE = 2 * kTileBytes;                        // K tile + V tile
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_u = (uint32_t)__cvta_generic_to_shared(smem);
  const int split = blockIdx.x, s = blockIdx.y;
  const int64_t bk = blockIdx.z, b = bk / Hkv, kvh = bk % Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t visible = start + s + 1;
  const int64_t cta_first = (int64_t)split * chunks_per_cta * CHUNK;
  int nchunks = 0;
  if (cta_first < visible) {
    const int64_t span = visible - cta_first;
    nchunks = (int)((span + CHUNK - 1) / CHUNK);
    if (nchunks > chunks_per_cta) nchunks = chunks_per_cta;
  }
  const uint8_t* kg = reinterpret_cast<const uint8_t*>(ck + (bk * C + cta_first) * D);
  const uint8_t* vg = reinterpret_cast<const uint8_t*>(cv + (bk * C + cta_first) * D);

  // 16-byte pieces of the live rows, swizzled; V rows past the live range are zeroed (0 * garbage must stay 0)
  auto load_chunk = [&](int i) {
    uint8_t* stage = smem + (i & 1) * STAGE;
    const int64_t left = visible - (cta_first + (int64_t)i * CHUNK);
    const int live = left < CHUNK ? (int)left : CHUNK;
    const uint8_t* ksrc = kg + (int64_t)i * kTileBytes;
    const uint8_t* vsrc = vg + (int64_t)i * kTileBytes;
    for (int piece = threadIdx.x; piece < CHUNK * 16; piece += kAttnThreads) {
      const int key = piece >> 4, c = piece & 15;
      const int dst = key * ROW + ((c ^ (key & 7)) << 4);
      if (key < live) {
        cp_async16(stage + dst, ksrc + piece * 16);
        cp_async16(stage + kTileBytes + dst, vsrc + piece * 16);
      } else {
        *reinterpret_cast<uint4*>(stage + kTileBytes + dst) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_commit();
  };
  if (nchunks > 0) load_chunk(0);

  // A fragments of Q: row g = lane / 4 (zero for g >= G), two head-dim values at 16*k + 2*(lane % 4) (+8)
  const int g = lane >> 2, pair = (lane & 3) * 2;
  uint32_t qa[8][2];
  {
    const T* qp = q + (((b * S + s) * Hq) + kvh * G + (g < G ? g : 0)) * D;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      qa[k][0] = g < G ? *reinterpret_cast<const uint32_t*>(qp + 16 * k + pair) : 0u;
      qa[k][1] = g < G ? *reinterpret_cast<const uint32_t*>(qp + 16 * k + 8 + pair) : 0u;
    }
  }
  const int kbase = warp * 16;                                  // this warp's keys within every chunk
  float m_w = -CUDART_INF_F, l_w = 0.f;
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  for (int i = 0; i < nchunks; ++i) {
    if (i + 1 < nchunks) { load_chunk(i + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint32_t ks = smem_u + (i & 1) * STAGE, vs = ks + kTileBytes;
    const int64_t left = visible - (cta_first + (int64_t)i * CHUNK);
    const int live_keys = left < CHUNK ? (int)left : CHUNK;
    if (kbase < live_keys) {
      // S[16 x 16 keys] = Q K^T: per 16 head-dim values one ldmatrix.x4 (keys 0-7 / 8-15 x two 8-value pieces), two MMAs
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int key = kbase + (lane & 7) + ((lane >> 4) << 3), sub = (lane >> 3) & 1;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint32_t r[4];
          ldmatrix_x4(r, ks + key * ROW + (((2 * k + sub) ^ (key & 7)) << 4));
          mma_16816<T>(sc[0], qa[k][0], qa[k][1], r[0], r[1]);
          mma_16816<T>(sc[1], qa[k][0], qa[k][1], r[2], r[3]);
        }
      }
      // this thread: row g, keys kbase + 8*nt + pair + {0, 1}
      float p[2][2];
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool live = kbase + 8 * nt + pair + e < live_keys;
          p[nt][e] = live ? sc[nt][e] * scale : -CUDART_INF_F;
          mx = fmaxf(mx, p[nt][e]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));       // the four lanes of a row; finite: key kbase is live
      const float nm = fmaxf(m_w, mx);
      const float alpha = __expf(m_w - nm);                      // 0 on the first chunk (m_w = -inf)
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[nt][e] = __expf(p[nt][e] - nm);
          sum += p[nt][e];
        }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_w = l_w * alpha + sum;
      m_w = nm;
      if (i > 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] *= alpha; o[j][1] *= alpha; }
      }
      // O[16 x 128] += P V: P's accumulator layout is the A-fragment layout of the next product
      const uint32_t pa0 = pack_pair<T>(p[0][0], p[0][1]), pa2 = pack_pair<T>(p[1][0], p[1][1]);
      {
        const int key = kbase + (lane & 7) + (((lane >> 3) & 1) << 3), sub = lane >> 4;
#pragma unroll
        for (int j = 0; j < 8; ++j) {                            // two 8-column output tiles per ldmatrix
          uint32_t r[4];
          ldmatrix_x4_trans(r, vs + key * ROW + (((2 * j + sub) ^ (key & 7)) << 4));
          mma_16816<T>(o[2 * j], pa0, pa2, r[0], r[1]);
          mma_16816<T>(o[2 * j + 1], pa0, pa2, r[2], r[3]);
        }
      }
    }
    __syncthreads();                                             // this stage may be overwritten two chunks later
  }
  float* s_acc = reinterpret_cast<float*>(smem);               // [8 warps][G][128]: at most 32 KB of stage 0
  float* s_max = reinterpret_cast<float*>(smem + kTileBytes);  // [8][G]
  float* s_sum = s_max + 8 * G;
  if (g < G) {
    if ((lane & 3) == 0) { s_max[warp * G + g] = m_w; s_sum[warp * G + g] = l_w; }
#pragma unroll
    for (int j = 0; j < 16; ++j)
      *reinterpret_cast<float2*>(s_acc + (warp * G + g) * D + 8 * j + pair) = make_float2(o[j][0], o[j][1]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
    const int gg = idx / D, d = idx % D;
    float nm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 8; ++w) nm = fmaxf(nm, s_max[w * G + gg]);
    float tot = 0.f, val = 0.f;
    if (nm > -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float f = __expf(s_max[w * G + gg] - nm);         // exp(-inf) = 0 for a warp without live keys
        tot += s_sum[w * G + gg] * f;
        val += s_acc[(w * G + gg) * D + d] * f;
      }
    }
    const int64_t row = ((b * S + s) * Hq + kvh * G + gg) * splits + split;
    part[row * D + d] = tot > 0.f ? val / tot : 0.f;
    if (d == 0) lse[row] = tot > 0.f ? nm + __logf(tot) : -CUDART_INF_F;
  }
}

// ---- small-M linear on the tensor cores (16-bit types) ------------------------------------------------------------
// y[m, n] = sum_k x[m, k] w[n, k], M <= 8: 16 weight rows are the rows of an MMA tile and the M input rows its 8
// columns, so the arithmetic costs two instructions per 16 x 32 block of weights and the kernel is a pure stream.
// The contraction index may be permuted freely as long as both operands agree: lane (g, t) loads 16 contiguous bytes
// w[n0 + g][k0 + 8t .. 8t+7] (and the same for row g + 8) and x[g][k0 + 8t .. 8t+7]; the four register pairs of each
// load feed the (2t, 2t+1) and (2t+8, 2t+9) slots of two MMAs. The 4 warps of a CTA split K and add up in shared
// memory (fixed order), which quadruples the bytes in flight per weight row.
template <typename T, int UNROLL>
__global__ void __launch_bounds__(128)
gemv_mma_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, int64_t M, int64_t N, int64_t K) {
  __shared__ float red[4][16][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t n0 = (int64_t)blockIdx.x * 16;
  const int64_t ra = n0 + g < N ? n0 + g : N - 1, rb = n0 + g + 8 < N ? n0 + g + 8 : N - 1;   // clamped: rows past N are not stored
  const T* wa = w + ra * K + 8 * t;
  const T* wb = w + rb * K + 8 * t;
  const T* xr = x + (int64_t)(g < M ? g : 0) * K + 8 * t;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int64_t steps = K / 32;                                  // K % 32 == 0
  for (int64_t st = warp * UNROLL; st < steps; st += 4 * UNROLL) {
    uint4 a[UNROLL], c[UNROLL], xv[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const bool in = st + u < steps;
      const int64_t k0 = (st + u) * 32;
      a[u] = in ? __ldcs(reinterpret_cast<const uint4*>(wa + k0)) : make_uint4(0u, 0u, 0u, 0u);
      c[u] = in ? __ldcs(reinterpret_cast<const uint4*>(wb + k0)) : make_uint4(0u, 0u, 0u, 0u);
      xv[u] = (in && g < M) ? *reinterpret_cast<const uint4*>(xr + k0) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      mma_16816_full<T>(acc, a[u].x, c[u].x, a[u].y, c[u].y, xv[u].x, xv[u].y);
      mma_16816_full<T>(acc, a[u].z, c[u].z, a[u].w, c[u].w, xv[u].z, xv[u].w);
    }
  }
  // accumulator: (row g, cols 2t, 2t+1), (row g + 8, same cols); columns are the input rows m
  red[warp][g][2 * t] = acc[0]; red[warp][g][2 * t + 1] = acc[1];
  red[warp][g + 8][2 * t] = acc[2]; red[warp][g + 8][2 * t + 1] = acc[3];
  __syncthreads();
  const int r = threadIdx.x >> 3, m = threadIdx.x & 7;         // 128 threads = 16 rows x 8 columns
  if (n0 + r < N && m < M)
    y[(int64_t)m * N + n0 + r] = from_f32<T>((red[0][r][m] + red[1][r][m]) + (red[2][r][m] + red[3][r][m]));
}

// out[row, :] = sum_i part[row, i, :] * w_i, w_i = exp(lse[row, i] - max) / sum_j exp(lse[row, j] - max); one warp per
// row. The lanes first share out the chunks to find the maximum and the weights (kept in registers, 32 chunks per
// round), then every lane owns CPL = D / 32 consecutive columns and adds the chunks up in order - independent,
// unrolled vector loads rather than one dependent load after another.
template <typename T, int CPL>
__global__ void __launch_bounds__(128)
cache_attention_merge_kernel(const float* __restrict__ part, const float* __restrict__ lse, T* __restrict__ out,
                             int64_t rows, int splits) {
  constexpr int D = CPL * 32;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* l = lse + row * splits;
  float mx = -CUDART_INF_F;
  for (int i = lane; i < splits; i += 32) mx = fmaxf(mx, l[i]);
  mx = warp_max(mx);
  float denom = 0.f;
  for (int i = lane; i < splits; i += 32) denom += __expf(l[i] - mx);
  denom = warp_sum(denom);                       // xor-butterfly: the same value, bit for bit, in every lane
  const float inv = 1.f / denom;
  float acc[CPL];
#pragma unroll
  for (int c = 0; c < CPL; ++c) acc[c] = 0.f;
  const float* p = part + row * splits * D + lane * CPL;
  for (int base = 0; base < splits; base += 32) {
    const float mine = base + lane < splits ? __expf(l[base + lane] - mx) * inv : 0.f;
    const int n = splits - base < 32 ? splits - base : 32;
#pragma unroll 8
    for (int i = 0; i < n; ++i) {
      const float w = __shfl_sync(0xffffffffu, mine, i);
      float v[CPL];
      if constexpr (CPL >= 4) {
#pragma unroll
        for (int c = 0; c < CPL; c += 4) {
          const float4 t = *reinterpret_cast<const float4*>(p + (int64_t)(base + i) * D + c);
          v[c] = t.x; v[c + 1] = t.y; v[c + 2] = t.z; v[c + 3] = t.w;
        }
      } else {
        const float2 t = *reinterpret_cast<const float2*>(p + (int64_t)(base + i) * D);
        v[0] = t.x; v[1] = t.y;
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) acc[c] = fmaf(v[c], w, acc[c]);
    }
  }
  T* o = out + row * D + lane * CPL;
#pragma unroll
  for (int c = 0; c < CPL; ++c) o[c] = from_f32<T>(acc[c]);
}

// 16 bytes of T as floats through a streaming load: weight rows are read exactly once and must not evict the
// input rows from L1.
template <typename T> __device__ __forceinline__ void load_stream16(const T* p, float (&v)[16 / sizeof(T)]);
template <> __device__ __forceinline__ void load_stream16<float>(const float* p, float (&v)[4]) {
  const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load_stream16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load_stream16<__half>(const __half* p, float (&v)[8]) {
  const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}

// y[m, n] = sum_k x[m, k] * w[n, k], M <= 8. A warp owns R consecutive weight rows and walks K in chunks of 32
// 16-byte vectors. Per chunk it issues, before any arithmetic, R streaming loads of weights (R independent 512-byte
// requests in flight per warp; the matrix is read exactly once and bypasses L1) and the M loads of its slice of the
// input rows (which stay in L1). ACC = float, or double for the `accurate` mode (products in fp32, as the
// reference accumulates them).
template <typename T, typename ACC, int M, int R>
__global__ void __launch_bounds__(128)
gemv_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, int64_t N, int64_t K) {
  constexpr int W = 16 / (int)sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t n0 = (blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5)) * R;
  if (n0 >= N) return;
  ACC acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = (ACC)0;
  for (int64_t k = (int64_t)lane * W; k < K; k += 32 * W) {       // K is a multiple of W: a vector is all in or all out
    float wv[R][W], xv[M][W];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (n0 + r < N) load_stream16<T>(w + (n0 + r) * K + k, wv[r]);
      else {
#pragma unroll
        for (int e = 0; e < W; ++e) wv[r][e] = 0.f;
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) VecIO<T, W>::load(x + m * K + k, xv[m]);
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int e = 0; e < W; ++e) acc[r][m] += (ACC)(wv[r][e] * xv[m][e]);
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      ACC v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && n0 + r < N) y[m * N + n0 + r] = from_f32<T>((float)v);
    }
}

// Greedy selection in two stages. Stage 1: every row is cut into `parts` slices, one CTA each, which reduce their
// slice to (maximum, lowest index holding it). Stage 2: one warp per row reduces the slices the same way and does
// the bookkeeping of a decode step: a finished row emits `pad`; the token goes to ids[row, position] and next[row];
// a row that emits an end-of-sequence id becomes finished.
__device__ __forceinline__ void better(float& best, int64_t& where, float v, int64_t i) {
  if (v > best || (v == best && i < where)) { best = v; where = i; }
}

template <typename T>
__global__ void __launch_bounds__(256)
argmax_parts_kernel(const T* __restrict__ logits, int64_t V, int parts, float* __restrict__ pval, int64_t* __restrict__ pidx) {
  __shared__ float s_val[8];
  __shared__ int64_t s_idx[8];
  const int64_t row = blockIdx.y;
  const int part = blockIdx.x;
  const int64_t per = (V + parts - 1) / parts, lo = part * per, hi = lo + per < V ? lo + per : V;
  const T* x = logits + row * V;
  float best = -CUDART_INF_F;
  int64_t where = INT64_MAX;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) better(best, where, to_f32<T>(x[i]), i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    better(best, where, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, where, o));
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = where; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) better(best, where, s_val[w], s_idx[w]);
    pval[row * parts + part] = best;
    pidx[row * parts + part] = where;
  }
}

__global__ void select_kernel(const float* __restrict__ pval, const int64_t* __restrict__ pidx, int parts,
                              int64_t* __restrict__ ids, int64_t ids_stride, int64_t position, int64_t* __restrict__ next,
                              uint8_t* __restrict__ done, const int64_t* __restrict__ eos, int n_eos, int64_t pad,
                              int64_t rows) {
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float best = -CUDART_INF_F;
  int64_t where = INT64_MAX;
  for (int i = lane; i < parts; i += 32) better(best, where, pval[row * parts + i], pidx[row * parts + i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    better(best, where, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, where, o));
  if (lane == 0) {
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

static int64_t cache_attention_splits(int64_t total, int64_t D, int dtype) {
  return cdiv(total, inf::chunk_keys((int)D, dtype_size(dtype)));
}

extern "C" int64_t q3_cache_attention_workspace_bytes(int64_t B, int64_t S, int64_t Hq, int64_t D, int64_t start,
                                                      int dtype) {
  if (B < 1 || S < 1 || Hq < 1 || D < 1 || start < 0 || dtype < Q3_F32 || dtype > Q3_F16) return 0;
  return B * S * Hq * cache_attention_splits(start + S, D, dtype) * (D + 1) * 4;
}

namespace {
template <typename T, int EPL, int G>
int launch_partial(dim3 grid, const void* q, const void* ck, const void* cv, float* part, float* lse, int64_t S, int64_t Hq,
                   int64_t Hkv, int64_t C, int64_t start, int splits, float scale, cudaStream_t st) {
  auto kern = inf::cache_attention_partial_kernel<T, EPL, G>;
  static DeviceFlags configured = {};
  const int smem = 2 * inf::kTileBytes;
  if (int rc = ensure_dynamic_smem(kern, smem, &configured); rc != Q3_OK) return rc;
  kern<<<grid, inf::kAttnThreads, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, part, lse, S, Hq, Hkv, C, start,
                                              splits, scale);
  return launch_status();
}

template <typename T, int G>
int launch_partial_mma(dim3 grid, const void* q, const void* ck, const void* cv, float* part, float* lse, int64_t S,
                       int64_t Hq, int64_t Hkv, int64_t C, int64_t start, int splits, int chunks_per_cta, float scale,
                       cudaStream_t st) {
  auto kern = inf::cache_attention_partial_mma_kernel<T, G>;
  static DeviceFlags configured = {};
  const int smem = 4 * inf::kTileBytes;                        // two stages of (K tile, V tile)
  if (int rc = ensure_dynamic_smem(kern, smem, &configured); rc != Q3_OK) return rc;
  kern<<<grid, inf::kAttnThreads, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, part, lse, S, Hq, Hkv, C, start,
                                              splits, chunks_per_cta, scale);
  return launch_status();
}

// Process-wide switch for tests and tuning: 0 = tensor cores where they apply (default), 1 = CUDA cores always.
int g_cache_attention_path = 0;

template <typename T, int EPL>
int launch_cache_attention(const void* q, const void* ck, const void* cv, void* out, float* part, float* lse, int64_t B,
                           int64_t S, int64_t Hq, int64_t Hkv, int64_t C, int64_t start, float scale, cudaStream_t st) {
  const int G = (int)(Hq / Hkv);
  const int splits = (int)cdiv(start + S, inf::chunk_keys(EPL * 16, (int)sizeof(T)));
  dim3 grid((unsigned)splits, (unsigned)S, (unsigned)(B * Hkv));
  int rc = Q3_ERR_SHAPE;
  if constexpr (EPL == 8 && sizeof(T) == 2) {
    if (g_cache_attention_path == 0) {
      // chunks per CTA: as many as keep at least four CTAs per SM in the grid (fewer, larger partial results to merge
      // and copies that overlap the arithmetic inside a CTA); the workspace is sized for one chunk per CTA
      const int64_t chunks = cdiv(start + S, 128), base = B * Hkv * S;
      int cpc = 8;
      while (cpc > 1 && base * cdiv(chunks, cpc) < 4 * (int64_t)sm_count()) cpc >>= 1;
      const int nsplit = (int)cdiv(chunks, cpc);
      dim3 grid2((unsigned)nsplit, (unsigned)S, (unsigned)(B * Hkv));
      if (G == 1) rc = launch_partial_mma<T, 1>(grid2, q, ck, cv, part, lse, S, Hq, Hkv, C, start, nsplit, cpc, scale, st);
      else if (G == 2) rc = launch_partial_mma<T, 2>(grid2, q, ck, cv, part, lse, S, Hq, Hkv, C, start, nsplit, cpc, scale, st);
      else if (G == 4) rc = launch_partial_mma<T, 4>(grid2, q, ck, cv, part, lse, S, Hq, Hkv, C, start, nsplit, cpc, scale, st);
      else if (G == 8) rc = launch_partial_mma<T, 8>(grid2, q, ck, cv, part, lse, S, Hq, Hkv, C, start, nsplit, cpc, scale, st);
      if (rc != Q3_OK) return rc;
      const int64_t rows2 = B * S * Hq;
      inf::cache_attention_merge_kernel<T, EPL / 2><<<(unsigned)cdiv(rows2, 4), 128, 0, st>>>(part, lse, (T*)out, rows2, nsplit);
      return launch_status();
    }
  }
  if (G == 1) rc = launch_partial<T, EPL, 1>(grid, q, ck, cv, part, lse, S, Hq, Hkv, C, start, splits, scale, st);
  else if (G == 2) rc = launch_partial<T, EPL, 2>(grid, q, ck, cv, part, lse, S, Hq, Hkv, C, start, splits, scale, st);
  else if (G == 4) rc = launch_partial<T, EPL, 4>(grid, q, ck, cv, part, lse, S, Hq, Hkv, C, start, splits, scale, st);
  else if (G == 8) {
    // 8 warps x 8 heads x D fp32 of combine space must fit the 32 KB tile it reuses
    if constexpr (EPL <= 8) rc = launch_partial<T, EPL, 8>(grid, q, ck, cv, part, lse, S, Hq, Hkv, C, start, splits, scale, st);
  }
  if (rc != Q3_OK) return rc;
  const int64_t rows = B * S * Hq;
  inf::cache_attention_merge_kernel<T, EPL / 2><<<(unsigned)cdiv(rows, 4), 128, 0, st>>>(part, lse, (T*)out, rows, splits);
  return launch_status();
}
}  // namespace

// 0: tensor-core kernel for 16-bit caches at head_dim 128 (default); 1: CUDA-core kernel for everything. Returns the
// previous setting; any other argument only queries.
extern "C" int q3_cache_attention_path(int path) {
  const int old = g_cache_attention_path;
  if (path == 0 || path == 1) g_cache_attention_path = path;
  return old;
}

extern "C" int q3_cache_attention(const void* q, const void* cache_k, const void* cache_v, void* out, void* workspace,
                                  int64_t workspace_bytes, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t D,
                                  int64_t C, int64_t start, double scale, int dtype, q3_stream_t stream) {
  if (!q || !cache_k || !cache_v || !out) return Q3_ERR_ARG;
  if (B < 1 || S < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv || start < 0 || start + S > C || S > 65535 || B * Hkv > 65535)
    return Q3_ERR_SHAPE;
  if (D != 64 && D != 128 && D != 256) return Q3_ERR_SHAPE;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  if (!aligned16(q) || !aligned16(cache_k) || !aligned16(cache_v) || !aligned16(out)) return Q3_ERR_ALIGN;
  if (!workspace || workspace_bytes < q3_cache_attention_workspace_bytes(B, S, Hq, D, start, dtype)) return Q3_ERR_WORKSPACE;
  const int64_t splits = cache_attention_splits(start + S, D, dtype);
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
  cudaStream_t st = (cudaStream_t)stream;
  if (!accurate && dtype != Q3_F32 && K % 32 == 0 && aligned16(x) && aligned16(weight)) {
    const unsigned grid = (unsigned)cdiv(N, 16);
    if (dtype == Q3_BF16) inf::gemv_mma_kernel<__nv_bfloat16, 4><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, (__nv_bfloat16*)y, M, N, K);
    else inf::gemv_mma_kernel<__half, 4><<<grid, 128, 0, st>>>((const __half*)x, (const __half*)weight, (__half*)y, M, N, K);
    return launch_status();
  }
  // 4 warps per CTA; 8 weight rows per warp for up to two input rows, 4 beyond (register budget: R x M accumulators)
#define Q3_GEMV(MM)                                                                                                     \
  case MM: {                                                                                                            \
    constexpr int R = MM <= 2 ? 8 : 4;                                                                                  \
    const unsigned grid = (unsigned)cdiv(N, 4 * R);                                                                     \
    if (accurate) inf::gemv_kernel<T, double, MM, R><<<grid, 128, 0, st>>>((const T*)x, (const T*)weight, (T*)y, N, K); \
    else inf::gemv_kernel<T, float, MM, R><<<grid, 128, 0, st>>>((const T*)x, (const T*)weight, (T*)y, N, K);           \
    break;                                                                                                              \
  }
  Q3_DISPATCH_FLOAT(dtype, T, {
    switch ((int)M) { Q3_GEMV(1) Q3_GEMV(2) Q3_GEMV(3) Q3_GEMV(4) Q3_GEMV(5) Q3_GEMV(6) Q3_GEMV(7) Q3_GEMV(8) }
  });
#undef Q3_GEMV
  return launch_status();
}

static int select_parts(int64_t V) { return (int)(cdiv(V, 4096) < 64 ? cdiv(V, 4096) : 64); }

extern "C" int64_t q3_select_tokens_workspace_bytes(int64_t B, int64_t V) {
  if (B < 1 || V < 1) return 0;
  return B * select_parts(V) * 12;
}

extern "C" int q3_select_tokens(const void* logits, int64_t B, int64_t V, int64_t* ids, int64_t ids_stride,
                                int64_t position, int64_t* next_token, uint8_t* done, const int64_t* eos_ids, int n_eos,
                                int64_t pad, void* workspace, int64_t workspace_bytes, int dtype, q3_stream_t stream) {
  if (!logits || !ids || !next_token || !done || (n_eos > 0 && !eos_ids)) return Q3_ERR_ARG;
  if (B < 1 || B > 65535 || V < 1 || position < 0 || position >= ids_stride || n_eos < 0) return Q3_ERR_SHAPE;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  if (!workspace || workspace_bytes < q3_select_tokens_workspace_bytes(B, V) ||
      (reinterpret_cast<uintptr_t>(workspace) & 7u))
    return Q3_ERR_WORKSPACE;
  const int parts = select_parts(V);
  int64_t* pidx = (int64_t*)workspace;                       // 8-byte entries first: keeps them aligned
  float* pval = (float*)(pidx + B * parts);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)parts, (unsigned)B);
  Q3_DISPATCH_FLOAT(dtype, T, (inf::argmax_parts_kernel<T><<<grid, 256, 0, st>>>((const T*)logits, V, parts, pval, pidx)));
  int rc = launch_status();
  if (rc != Q3_OK) return rc;
  inf::select_kernel<<<(unsigned)cdiv(B, 4), 128, 0, st>>>(pval, pidx, parts, ids, ids_stride, position, next_token, done,
                                                            eos_ids, n_eos, pad, B);
  return launch_status();
}
