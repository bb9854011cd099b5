// Causal grouped-query flash attention on the tcgen05 tensor cores, head_dim 128, bf16 / fp16.
//
// Layout: q/out/dout/dq [B, Hq, S, 128], k/v/dk/dv [B, Hkv, S, 128], lse/delta [B, Hq, S] fp32.
// Every operand tile is brought in by TMA (3-D maps [B*H, S, 128], so rows past the sequence end read
// as zero) into 128-byte-swizzled shared memory as two 64-column halves; the same K (or V, Q, dO) tile
// serves as a K-major operand (contraction over head_dim) and as an MN-major operand (contraction over
// its rows) through two descriptor views, so no tile is ever transposed or loaded twice.
//
// Forward (one CTA per 128-query tile of one (batch, query head); 192 threads):
//   warp 0  : TMA producer - Q once, then a 2-stage ring of K tiles and of V tiles (128 keys each)
//   warp 1  : MMA issuer   - S_j = Q K_j^T into one of two TMEM score buffers, then O_j = P_j V_j into one
//             of two TMEM output buffers; S_{j+1} is issued before P_j is ready, so the score GEMM
//             overlaps the softmax
//   warps 2-5: softmax     - one query row per thread: tcgen05.ld the scores, online max / exp2 / sum in
//             fp32, write P_j (bf16) into swizzled shared memory for the second GEMM, fold O_{j-1} from
//             TMEM into the fp32 register accumulator while the tensor core works on tile j
// Backward is two deterministic kernels:
//   dQ    (one CTA per 128-query tile): S = Q K^T, dP = dO V^T, dS = P*(dP - delta) -> smem, dQ += dS K
//         accumulated in TMEM over the key tiles.
//   dK/dV (one CTA per 128-key tile of one (batch, kv head)): loops over the query heads of the group
//         and over 64-query sub-tiles at or below the diagonal; S^T = K Q^T, dP^T = V dO^T, then
//         dV += P^T dO and dK += dS^T Q accumulate in TMEM across the whole group - the per-query-head
//         partial buffers and the reduction kernel of the reference do not exist here.
//
// Replaces, in the reference: qwen3_triton/kernels/attention_precision.py:15-143 (the kernels the 8B
// graph uses) and kernels/attention_kernels.py:10-253. Math: ops/reference/attention.py:10-124.
#include "tcgen05.cuh"
#include <math_constants.h>
#include <algorithm>

namespace q3 {
namespace tc {

constexpr int AD = 128;           // head dim
constexpr int TILE = 128;         // query rows / keys per tile
constexpr int HALF_BYTES = TILE * 128;       // one 64-column half of a 128-row tile (16 KB)
constexpr int TILE_BYTES = 2 * HALF_BYTES;   // 32 KB
constexpr int kAttnThreads = 320;   // dK/dV kernel: warp 0 TMA, warp 1 MMA, warps 2..9 compute (two threads per tile row)
constexpr int kComputeThreads = 256;   // of the dK/dV kernel
// The dQ kernel has no reduction along a row, so its rows are cut four ways (16 compute warps, one 32-column chunk of
// the score tile per thread): twice the warps to hide tensor-memory load latency, half the registers per thread.
constexpr int kDqComputeThreads = 512;
constexpr int kDqThreads = 64 + kDqComputeThreads;
// The forward kernel also runs four threads per row (32 score and 32 output columns each); the row maximum and the
// row sum cross the four through shared memory and a 128-thread hardware barrier.
constexpr int kFwdComputeThreads = 512;
constexpr int kFwdThreads = 64 + kFwdComputeThreads;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnParams {
  void* out;
  float* lse;
  int Hq, Hkv, S;
  int64_t q_ss, q_hs, q_bs;  // element strides of q/out over (sequence, head, batch)
  float scale_log2;  // softmax scale * log2(e)
  uint32_t idesc_qk; // A K-major, B K-major, N = 128
  uint32_t idesc_pv; // A K-major, B MN-major, N = 128
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Write 32 consecutive elements (columns c0..c0+31 of row `row`) of a [128 x 128] K-major tile held as
// two 64-column halves with the 128-byte swizzle (16-byte chunk index XOR row%8).
template <typename T>
__device__ __forceinline__ void store_swizzled32(uint8_t* tile, int row, int c0, const float (&v)[32]) {
  uint8_t* half = tile + (c0 >> 6) * HALF_BYTES + row * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 w;
    w.x = pack2<T>(v[8 * j + 0], v[8 * j + 1]);
    w.y = pack2<T>(v[8 * j + 2], v[8 * j + 3]);
    w.z = pack2<T>(v[8 * j + 4], v[8 * j + 5]);
    w.w = pack2<T>(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(half + (((chunk0 + j) ^ (row & 7)) << 4)) = w;
  }
}

// 8 MMAs (k = 16 each) covering a contraction of 128 over two 64-wide halves, both operands K-major.
__device__ __forceinline__ void mma_kk_128(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, uint32_t idesc,
                                           bool accumulate_first) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
    mma_f16_ss(d_tmem, make_smem_desc(a_smem + off, 0, 1024), make_smem_desc(b_smem + off, 0, 1024), idesc,
               (accumulate_first || k) ? 1u : 0u);
  }
}
// A K-major [128 x kk] (kk = 16 * ksteps, halves of 64), B MN-major: rows = contraction index, 128 columns
// as two 64-wide atoms HALF_BYTES apart.
__device__ __forceinline__ void mma_kmn(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, uint32_t idesc,
                                        int ksteps, uint32_t a_half_bytes, bool accumulate_first) {
  for (int k = 0; k < ksteps; ++k) {
    const uint32_t a_off = (k >> 2) * a_half_bytes + (k & 3) * 32;
    const uint32_t b_off = k * (16 * 128);
    mma_f16_ss(d_tmem, make_smem_desc(a_smem + a_off, 0, 1024), make_smem_desc(b_smem + b_off, HALF_BYTES, 1024),
               idesc, (accumulate_first || k) ? 1u : 0u);
  }
}

// Barrier over the four compute warps that share a TMEM lane quarter (128 threads, hardware barrier 1 + quarter),
// ANDing a predicate over them. All four warps must reach every call: no early exit between two calls.
__device__ __forceinline__ bool row_group_all(int quarter, bool pred) {
  int r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.s32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, 128, q;\n\t"
      "selp.s32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((int)pred), "r"(quarter + 1)
      : "memory");
  return r != 0;
}

template <typename T>
__global__ void __launch_bounds__(kFwdThreads, 1)   // 18 warps: 5 on one scheduler, whose 16 K registers cap a thread at 96
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  // [Q 32K][K0 32K][K1 32K][V0 32K][V1 32K][P 32K][barriers]
  const uint32_t q_s = base, k_s = base + TILE_BYTES, v_s = base + 3 * TILE_BYTES, p_s = base + 5 * TILE_BYTES;
  uint8_t* p_ptr = smem + 5 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int s) { return bar0 + 8u * (9 + s); };
  auto o_full = [&](int s) { return bar0 + 8u * (11 + s); };
  const uint32_t p_full = bar0 + 8u * 13, done_bar = bar0 + 8u * 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xmax = reinterpret_cast<float*>(bars + 18);   // [2 tiles in flight + 1][4 column quarters][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + TILE - 1) / TILE;
  // grid = (batch * heads, query tiles): blocks start in x-major order, so every head's heaviest (last) query tile
  // starts before any lighter one - longest work first over the whole grid, not per head
  const int qt = nq - 1 - (int)blockIdx.y;
  const int bh = blockIdx.x, b = bh / p.Hq, h = bh % p.Hq, kvh = h / (p.Hq / p.Hkv);
  const int bkv = b * p.Hkv + kvh;
  const int ntiles = qt + 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 13; ++i) mbar_init(bar0 + 8u * i, 1);
    mbar_init(p_full, kFwdComputeThreads / 32);   // one arrival per compute warp
    mbar_init(done_bar, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;  // columns: S0 0..127, S1 128..255, O0 256..383, O1 384..511

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_4d(q_s, &tmQ, 0, qt * TILE, bh % p.Hq, bh / p.Hq, q_full);
      tma_load_4d(q_s + HALF_BYTES, &tmQ, 64, qt * TILE, bh % p.Hq, bh / p.Hq, q_full);
      int issued = 0;
      for (int j = 0; j < ntiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(k_empty(s), ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(k_full(s), TILE_BYTES);
        tma_load_4d(k_s + s * TILE_BYTES, &tmK, 0, j * TILE, bkv % p.Hkv, bkv / p.Hkv, k_full(s));
        tma_load_4d(k_s + s * TILE_BYTES + HALF_BYTES, &tmK, 64, j * TILE, bkv % p.Hkv, bkv / p.Hkv, k_full(s));
        if (!mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { mbar_wait_drain(k_full(s), ph); break; }
        mbar_expect_tx(v_full(s), TILE_BYTES);
        tma_load_4d(v_s + s * TILE_BYTES, &tmV, 0, j * TILE, bkv % p.Hkv, bkv / p.Hkv, v_full(s));
        tma_load_4d(v_s + s * TILE_BYTES + HALF_BYTES, &tmV, 64, j * TILE, bkv % p.Hkv, bkv / p.Hkv, v_full(s));
        issued = j + 1;
      }
      // make sure nothing is still landing in shared memory when the CTA exits
      mbar_wait_drain(q_full, 0);
      for (int j = issued > 2 ? issued - 2 : 0; j < issued; ++j) {
        mbar_wait_drain(k_full(j & 1), (j >> 1) & 1u);
        mbar_wait_drain(v_full(j & 1), (j >> 1) & 1u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(k_full(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_kk_128(tmem + 0, q_s, k_s, p.idesc_qk, false);
        mma_commit(s_full(0));
        mma_commit(k_empty(0));
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (j + 1 < ntiles) {
          const int s1 = (j + 1) & 1;
          if (!mbar_wait(k_full(s1), ((j + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kk_128(tmem + s1 * 128, q_s, k_s + s1 * TILE_BYTES, p.idesc_qk, false);
          mma_commit(s_full(s1));
          mma_commit(k_empty(s1));
        }
        if (!mbar_wait(p_full, j & 1u, abort_flag) || !mbar_wait(v_full(s), ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_kmn(tmem + 256 + s * 128, p_s, v_s + s * TILE_BYTES, p.idesc_pv, 8, HALF_BYTES, false);
        mma_commit(o_full(s));
        mma_commit(v_empty(s));
      }
      mma_commit(done_bar);
      mbar_wait_drain(done_bar, 0);
    }
  } else {
    // ------------------------------------------------------------------ softmax / accumulate / epilogue
    // Four threads per query row: warps 2-5 take score / output columns 0..31, warps 6-9 columns 32..63, and so
    // on. The quarters exchange their row maximum through shared memory once per key tile.
    const int qd = warp & 3;                 // TMEM lane quarter of this warp
    const int ch = (warp - 2) >> 2;          // column quarter
    const int row = qd * 32 + lane;          // query row within the tile
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16);
    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = 0.f;
    float m = -CUDART_INF_F, l = 0.f, alpha_prev = 1.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int s = j & 1;
      if (!mbar_wait(s_full(s), (j >> 1) & 1u, abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      const uint32_t s_addr = lane_addr + s * 128 + ch * 32;
      const bool diag = (j == ntiles - 1);
      // pass 1: maximum of this thread's 32 raw scores (re-read from tensor memory for pass 2: keeping them across
      // the barrier does not fit the 96 registers a thread can have here)
      float mx = -CUDART_INF_F;
      if (ok) {
        uint32_t r[32];
        tmem_ld32(s_addr, r);
        tmem_ld_wait();
        if (!diag) {   // all but the last key tile of a query tile: no causal mask, no per-element compare
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (ch * 32 + i <= row) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      float* xm = xmax + (j & 1) * 512;
      xm[ch * 128 + row] = mx;
      // the partner threads (same row, other column quarters) sit in the warps 4, 8 and 12 away: a 128-thread hardware
      // barrier publishes the four maxima and makes the keep-going decision uniform over them
      ok = row_group_all(qd, ok);
      if (!ok) break;
      mx = fmaxf(fmaxf(m, xm[row]), fmaxf(fmaxf(xm[128 + row], xm[256 + row]), xm[384 + row]));
      const float mc = mx * p.scale_log2;
      const float alpha = fast_exp2(m * p.scale_log2 - mc);  // m = -inf on the first tile -> 0
      // pass 2: probabilities, partial row sum
      float pv[32];
      float sum = 0.f;
      uint32_t r[32];
      tmem_ld32(s_addr, r);
      tmem_ld_wait();
      if (!diag) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          pv[i] = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -mc));
          sum += pv[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -mc));
          pv[i] = (ch * 32 + i <= row) ? e : 0.f;
          sum += pv[i];
        }
      }
      // the P buffer and O_{j-1} are free / ready once the previous PV product has completed
      if (j > 0 && !mbar_wait(o_full((j - 1) & 1), ((j - 1) >> 1) & 1u, abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      if (ok) store_swizzled32<T>(p_ptr, row, ch * 32, pv);
      l = l * alpha + sum;
      m = mx;
      tc_fence_before();
      fence_proxy_async_smem();   // generic-proxy writes of P must be visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);   // the warp's writes are ordered before lane 0's arrival
      // fold this thread's quarter of O_{j-1} into registers while the tensor core computes S_{j+1} and P_j V_j
      if (j > 0 && ok) {
        uint32_t ro[32];
        tmem_ld32(lane_addr + 256 + ((j - 1) & 1) * 128 + ch * 32, ro);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = fmaf(o[i], alpha_prev, __uint_as_float(ro[i]));
      }
      alpha_prev = alpha;
    }
    // combine the four partial row sums (own slot of the exchange buffer, one more round of the barrier)
    xmax[1024 + ch * 128 + row] = l;
    ok = row_group_all(qd, ok);
    if (ok) l = (xmax[1024 + row] + xmax[1024 + 128 + row]) + (xmax[1024 + 256 + row] + xmax[1024 + 384 + row]);
    bool fin = ok && mbar_wait(o_full((ntiles - 1) & 1), ((ntiles - 1) >> 1) & 1u, abort_flag);
    fin = __all_sync(0xffffffffu, fin);
    if (fin) {
      tc_fence_after();
      const float inv = 1.f / l;
      const int qi = qt * TILE + row;
      T* orow = reinterpret_cast<T*>(p.out) + (int64_t)b * p.q_bs + (int64_t)h * p.q_hs + (int64_t)qi * p.q_ss + ch * 32;
      uint32_t ro[32];
      tmem_ld32(lane_addr + 256 + ((ntiles - 1) & 1) * 128 + ch * 32, ro);
      tmem_ld_wait();
      if (qi < p.S) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = g * 8 + e * 2;
            wp[e] = pack2<T>(fmaf(o[i], alpha_prev, __uint_as_float(ro[i])) * inv,
                             fmaf(o[i + 1], alpha_prev, __uint_as_float(ro[i + 1])) * inv);
          }
          *reinterpret_cast<uint4*>(orow + g * 8) = w;
        }
      }
      if (qi < p.S && ch == 0) p.lse[(int64_t)bh * p.S + qi] = (m * p.scale_log2 + log2f(l)) * kLn2;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag) flag_status(p.status, Q3_STATUS_WAIT_TIMEOUT);
}

constexpr int kFwdSmem = 6 * TILE_BYTES + 1024 + 256 + 3 * 4 * 128 * 4;

// ====================================================================================== backward
struct AttnBwdParams {
  const float* lse;
  const float* delta;
  void* dq;
  void* dk;
  void* dv;
  float* part;      // fp32 partial dK/dV [gsplit][2][B*Hkv*S][128] when gsplit > 1
  int gsplit;       // 1: one CTA sums the whole query-head group; G: one CTA per query head + reduce kernel
  int Hq, Hkv, S;
  int64_t q_ss, q_hs, q_bs, k_ss, k_hs, k_bs;  // element strides over (sequence, head, batch)
  float scale, scale_log2;
  uint32_t idesc_kk128;  // A K-major, B K-major, N = 128
  uint32_t idesc_kk64;   // A K-major, B K-major, N = 64
  uint32_t idesc_kmn;    // A K-major, B MN-major, N = 128
  int* status;
};

// Generic helpers with explicit half strides. A/B K-major, contraction 16*ksteps over 64-wide halves.
__device__ __forceinline__ void mma_kk(uint32_t d_tmem, uint32_t a_smem, uint32_t a_half, uint32_t b_smem,
                                       uint32_t b_half, uint32_t idesc, int ksteps, bool accumulate_first) {
  for (int k = 0; k < ksteps; ++k) {
    mma_f16_ss(d_tmem, make_smem_desc(a_smem + (k >> 2) * a_half + (k & 3) * 32, 0, 1024),
               make_smem_desc(b_smem + (k >> 2) * b_half + (k & 3) * 32, 0, 1024), idesc,
               (accumulate_first || k) ? 1u : 0u);
  }
}
// A K-major, B MN-major with `b_lbo` bytes between its 64-wide column atoms; contraction over B's rows.
__device__ __forceinline__ void mma_kmn2(uint32_t d_tmem, uint32_t a_smem, uint32_t a_half, uint32_t b_smem,
                                         uint32_t b_lbo, uint32_t idesc, int ksteps, bool accumulate_first) {
  for (int k = 0; k < ksteps; ++k) {
    mma_f16_ss(d_tmem, make_smem_desc(a_smem + (k >> 2) * a_half + (k & 3) * 32, 0, 1024),
               make_smem_desc(b_smem + k * (16 * 128), b_lbo, 1024), idesc, (accumulate_first || k) ? 1u : 0u);
  }
}

// ------------------------------------------------------------------ dQ: one CTA per 128-query tile
// smem: [Q][dO][K0][K1][V0][V1][dS] 32 KB each. TMEM columns: S double-buffered 0..127 / 128..255, dP 256..383,
// dQ 384..511. The score product of the next key tile is issued before the tensor core waits for dS of the current
// one, so it runs under the exponentials; dP and dQ stay in order behind it.
template <typename T>
__global__ void __launch_bounds__(kDqThreads, 1)
attn_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                  const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, do_s = base + TILE_BYTES, k_s = base + 2 * TILE_BYTES, v_s = base + 4 * TILE_BYTES,
                 ds_s = base + 6 * TILE_BYTES;
  uint8_t* ds_ptr = smem + 6 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * TILE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  const uint32_t dp_full = bar0 + 8u * 9, dq_full = bar0 + 8u * 10, ds_full = bar0 + 8u * 11, done_bar = bar0 + 8u * 12;
  auto s_full = [&](int s) { return bar0 + 8u * (13 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + TILE - 1) / TILE;
  const int qt = nq - 1 - (int)blockIdx.y;   // heaviest query tiles of all heads first
  const int bh = blockIdx.x, b = bh / p.Hq, h = bh % p.Hq, kvh = h / (p.Hq / p.Hkv);
  const int bkv = b * p.Hkv + kvh;
  const int ntiles = qt + 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 11; ++i) mbar_init(bar0 + 8u * i, 1);
    mbar_init(ds_full, kDqComputeThreads / 32);   // one arrival per compute warp
    mbar_init(done_bar, 1);
    mbar_init(s_full(0), 1);
    mbar_init(s_full(1), 1);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      tma_load_4d(q_s, &tmQ, 0, qt * TILE, bh % p.Hq, bh / p.Hq, q_full);
      tma_load_4d(q_s + HALF_BYTES, &tmQ, 64, qt * TILE, bh % p.Hq, bh / p.Hq, q_full);
      tma_load_4d(do_s, &tmDO, 0, qt * TILE, bh % p.Hq, bh / p.Hq, q_full);
      tma_load_4d(do_s + HALF_BYTES, &tmDO, 64, qt * TILE, bh % p.Hq, bh / p.Hq, q_full);
      int issued = 0;
      for (int j = 0; j < ntiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(k_empty(s), ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(k_full(s), TILE_BYTES);
        tma_load_4d(k_s + s * TILE_BYTES, &tmK, 0, j * TILE, bkv % p.Hkv, bkv / p.Hkv, k_full(s));
        tma_load_4d(k_s + s * TILE_BYTES + HALF_BYTES, &tmK, 64, j * TILE, bkv % p.Hkv, bkv / p.Hkv, k_full(s));
        if (!mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { mbar_wait_drain(k_full(s), ph); break; }
        mbar_expect_tx(v_full(s), TILE_BYTES);
        tma_load_4d(v_s + s * TILE_BYTES, &tmV, 0, j * TILE, bkv % p.Hkv, bkv / p.Hkv, v_full(s));
        tma_load_4d(v_s + s * TILE_BYTES + HALF_BYTES, &tmV, 64, j * TILE, bkv % p.Hkv, bkv / p.Hkv, v_full(s));
        issued = j + 1;
      }
      mbar_wait_drain(q_full, 0);
      for (int j = issued > 2 ? issued - 2 : 0; j < issued; ++j) {
        mbar_wait_drain(k_full(j & 1), (j >> 1) & 1u);
        mbar_wait_drain(v_full(j & 1), (j >> 1) & 1u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(k_full(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_kk(tmem + 0, q_s, HALF_BYTES, k_s, HALF_BYTES, p.idesc_kk128, 8, false);                       // S_0
        mma_commit(s_full(0));
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        // dP_j: its buffer is free, the compute warps finished tile j-1 before ds_full(j-1) completed
        if (!mbar_wait(v_full(s), ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_kk(tmem + 256, do_s, HALF_BYTES, v_s + s * TILE_BYTES, HALF_BYTES, p.idesc_kk128, 8, false);  // dP_j
        mma_commit(dp_full);
        mma_commit(v_empty(s));
        // S_{j+1} into the other score buffer (last read for tile j-1): runs while the compute warps work on tile j
        if (j + 1 < ntiles) {
          const int s1 = (j + 1) & 1;
          if (!mbar_wait(k_full(s1), ((j + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kk(tmem + s1 * 128, q_s, HALF_BYTES, k_s + s1 * TILE_BYTES, HALF_BYTES, p.idesc_kk128, 8, false);
          mma_commit(s_full(s1));
        }
        if (!mbar_wait(ds_full, j & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_kmn2(tmem + 384, ds_s, HALF_BYTES, k_s + s * TILE_BYTES, HALF_BYTES, p.idesc_kmn, 8, j > 0);   // dQ += dS K
        mma_commit(k_empty(s));
      }
      if (ok) mma_commit(dq_full);
      mma_commit(done_bar);
      mbar_wait_drain(done_bar, 0);
    }
  } else {
    // four threads per query row: warps 2-5 take key columns 0..31 of each tile, 6-9 columns 32..63, and so on
    const int qd = warp & 3, ch = (warp - 2) >> 2, row = qd * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16);
    const int qi = qt * TILE + row;
    const float lse2 = (qi < p.S ? p.lse[(int64_t)bh * p.S + qi] : 0.f) * kLog2e;
    const float dl = qi < p.S ? p.delta[(int64_t)bh * p.S + qi] : 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      if (!mbar_wait(s_full(j & 1), (j >> 1) & 1u, abort_flag) || !mbar_wait(dp_full, j & 1u, abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (j == ntiles - 1);
      const uint32_t s_addr = lane_addr + (j & 1) * 128;
      {
        const int c = ch;
        uint32_t rs[32], rp[32];
        float ds[32];
        tmem_ld32(s_addr + c * 32, rs);
        tmem_ld32(lane_addr + 256 + c * 32, rp);
        tmem_ld_wait();
        if (!diag && qi < p.S) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            ds[i] = fast_exp2(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2)) * (__uint_as_float(rp[i]) - dl);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pr = fast_exp2(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
            const bool keep = (!diag || c * 32 + i <= row) && qi < p.S;
            ds[i] = keep ? pr * (__uint_as_float(rp[i]) - dl) : 0.f;
          }
        }
        store_swizzled32<T>(ds_ptr, row, c * 32, ds);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);   // the warp's writes are ordered before lane 0's arrival
    }
    bool fin = ok && mbar_wait(dq_full, 0, abort_flag);
    fin = __all_sync(0xffffffffu, fin);
    if (fin) {
      tc_fence_after();
      T* orow = reinterpret_cast<T*>(p.dq) + (int64_t)b * p.q_bs + (int64_t)h * p.q_hs + (int64_t)qi * p.q_ss;
      {
        const int c = ch;
        uint32_t r[32];
        tmem_ld32(lane_addr + 384 + c * 32, r);
        tmem_ld_wait();
        if (qi < p.S) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wp[e] = pack2<T>(__uint_as_float(r[g * 8 + 2 * e]) * p.scale, __uint_as_float(r[g * 8 + 2 * e + 1]) * p.scale);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag) flag_status(p.status, Q3_STATUS_WAIT_TIMEOUT);
}
constexpr int kDqSmem = 7 * TILE_BYTES + 1024 + 256;

// ------------------------------------------------------------------ dK/dV: one CTA per 128-key tile of (b, kv head)
// Work items: (query head g of the group) x (64-query sub-tile i >= 2*kt). Shared memory:
//   [K 32K][V 32K] resident, 3 stages of {Q_i 16K, dO_i 16K}, [P^T 16K][dS^T 16K], lse/delta 2 x 64 floats.
// TMEM columns: S^T buffers 0..63 / 64..127, dP^T buffers 128..191 / 192..255, dK 256..383, dV 384..511.
constexpr int QSUB = 64;
constexpr int SUB_HALF = QSUB * 128;        // 8 KB: one 64-column half of a 64-row tile
constexpr int SUB_BYTES = 2 * SUB_HALF;     // 16 KB
constexpr int KV_STAGES = 3;

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t k_s = base, v_s = base + TILE_BYTES, st_s = base + 2 * TILE_BYTES;
  const uint32_t pt_off = 2 * TILE_BYTES + KV_STAGES * 2 * SUB_BYTES;
  const uint32_t pt_s = base + pt_off, dst_s = pt_s + SUB_BYTES;
  uint8_t* pt_ptr = smem + pt_off;
  uint8_t* dst_ptr = pt_ptr + SUB_BYTES;
  float* stat = reinterpret_cast<float*>(dst_ptr + SUB_BYTES);   // [2 items in flight][lse*log2e 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stat + 4 * QSUB);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t kv_full = bar0;
  auto st_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto st_empty = [&](int s) { return bar0 + 8u * (4 + s); };
  auto sdp_full = [&](int s) { return bar0 + 8u * (7 + s); };
  const uint32_t pds_empty = bar0 + 8u * 9, acc_full = bar0 + 8u * 10, done_bar = bar0 + 8u * 11,
                 pds_full = bar0 + 8u * 12, stat_bar = bar0 + 8u * 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid = (batch * kv heads * group split, key tiles): key tile 0 sees every query and goes first for all heads
  const int gs = p.gsplit > 1 ? p.gsplit : 1;
  const int kt = blockIdx.y, bk = (int)blockIdx.x / gs, zsplit = (int)blockIdx.x % gs;
  const int b = bk / p.Hkv, kvh = bk % p.Hkv, G = p.Hq / p.Hkv;
  const int nsub = (p.S + QSUB - 1) / QSUB, first = kt * (TILE / QSUB);
  const int g0 = p.gsplit > 1 ? zsplit : 0, ng = p.gsplit > 1 ? 1 : G;
  const int per_head = nsub - first, total = ng * per_head;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 12; ++i) mbar_init(bar0 + 8u * i, 1);
    mbar_init(pds_full, kComputeThreads / 32);    // one arrival per compute warp
    mbar_init(stat_bar, kComputeThreads / 32);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_4d(k_s, &tmK, 0, kt * TILE, bk % p.Hkv, bk / p.Hkv, kv_full);
      tma_load_4d(k_s + HALF_BYTES, &tmK, 64, kt * TILE, bk % p.Hkv, bk / p.Hkv, kv_full);
      tma_load_4d(v_s, &tmV, 0, kt * TILE, bk % p.Hkv, bk / p.Hkv, kv_full);
      tma_load_4d(v_s + HALF_BYTES, &tmV, 64, kt * TILE, bk % p.Hkv, bk / p.Hkv, kv_full);
      int issued = 0;
      for (int it = 0; it < total; ++it) {
        const int s = it % KV_STAGES;
        const uint32_t ph = (it / KV_STAGES) & 1u;
        if (!mbar_wait(st_empty(s), ph ^ 1u, abort_flag)) break;
        const int g = g0 + it / per_head, i = first + it % per_head;
        const int bh = (b * p.Hkv + kvh) * G + g;   // query head = kvh * G + g
        const uint32_t dst = st_s + s * 2 * SUB_BYTES;
        mbar_expect_tx(st_full(s), 2 * SUB_BYTES);
        tma_load_4d(dst, &tmQ, 0, i * QSUB, bh % p.Hq, bh / p.Hq, st_full(s));
        tma_load_4d(dst + SUB_HALF, &tmQ, 64, i * QSUB, bh % p.Hq, bh / p.Hq, st_full(s));
        tma_load_4d(dst + SUB_BYTES, &tmDO, 0, i * QSUB, bh % p.Hq, bh / p.Hq, st_full(s));
        tma_load_4d(dst + SUB_BYTES + SUB_HALF, &tmDO, 64, i * QSUB, bh % p.Hq, bh / p.Hq, st_full(s));
        issued = it + 1;
      }
      mbar_wait_drain(kv_full, 0);
      for (int it = issued > KV_STAGES ? issued - KV_STAGES : 0; it < issued; ++it)
        mbar_wait_drain(st_full(it % KV_STAGES), (it / KV_STAGES) & 1u);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(kv_full, 0, abort_flag) && mbar_wait(st_full(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_kk(tmem + 0, k_s, HALF_BYTES, st_s, SUB_HALF, p.idesc_kk64, 8, false);                 // S^T = K Q^T
        mma_kk(tmem + 128, v_s, HALF_BYTES, st_s + SUB_BYTES, SUB_HALF, p.idesc_kk64, 8, false);   // dP^T = V dO^T
        mma_commit(sdp_full(0));
      }
      for (int it = 0; it < total && ok; ++it) {
        const int s = it % KV_STAGES;
        if (it + 1 < total) {
          const int s1 = (it + 1) % KV_STAGES, buf = (it + 1) & 1;
          if (!mbar_wait(st_full(s1), ((it + 1) / KV_STAGES) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st1 = st_s + s1 * 2 * SUB_BYTES;
          mma_kk(tmem + buf * 64, k_s, HALF_BYTES, st1, SUB_HALF, p.idesc_kk64, 8, false);
          mma_kk(tmem + 128 + buf * 64, v_s, HALF_BYTES, st1 + SUB_BYTES, SUB_HALF, p.idesc_kk64, 8, false);
          mma_commit(sdp_full(buf));
        }
        if (!mbar_wait(pds_full, it & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t st0 = st_s + s * 2 * SUB_BYTES;
        mma_kmn2(tmem + 384, pt_s, 0, st0 + SUB_BYTES, SUB_HALF, p.idesc_kmn, 4, it > 0);   // dV += P^T dO
        mma_kmn2(tmem + 256, dst_s, 0, st0, SUB_HALF, p.idesc_kmn, 4, it > 0);             // dK += dS^T Q
        mma_commit(st_empty(s));
        mma_commit(pds_empty);
      }
      if (ok) mma_commit(acc_full);
      mma_commit(done_bar);
      mbar_wait_drain(done_bar, 0);
    }
  } else {
    // two threads per key row: warps 2-5 take query columns 0..31 of each 64-query sub-tile, warps 6-9 32..63
    const int qd = warp & 3, ch = (warp - 2) >> 2, row = qd * 32 + lane;   // key row within the tile
    const int tid = threadIdx.x - 64;                                      // 0..255 among the compute threads
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16);
    const int kj = kt * TILE + row;
    // lse / delta of the 64 queries of an item: threads 0..63 fetch lse, 64..127 delta
    auto load_stat = [&](int it) -> float {
      const int g = g0 + it / per_head, i = first + it % per_head;
      const int bh = (b * p.Hkv + kvh) * G + g;
      const int qi = i * QSUB + (tid & 63);
      if (qi >= p.S) return 0.f;
      return tid < 64 ? p.lse[(int64_t)bh * p.S + qi] * kLog2e : p.delta[(int64_t)bh * p.S + qi];
    };
    float nxt = (tid < 128 && total > 0) ? load_stat(0) : 0.f;
    bool ok = true;
    for (int it = 0; it < total; ++it) {
      const int i = first + it % per_head;
      float* st = stat + (it & 1) * 2 * QSUB;
      if (tid < 128) st[tid] = nxt;
      __syncwarp();
      if (lane == 0) mbar_arrive(stat_bar);   // the warp's writes are ordered before lane 0's arrival
      if (!mbar_wait(stat_bar, it & 1u, abort_flag)) ok = false;
      // the next item's values travel from global memory while this item is processed
      if (it + 1 < total && tid < 128) nxt = load_stat(it + 1);
      if (ok && !mbar_wait(sdp_full(it & 1), (it >> 1) & 1u, abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (i * QSUB < kt * TILE + TILE);   // sub-tile overlaps the diagonal block
      {
        const int c = ch;
        uint32_t rs[32], rp[32];
        float pv[32], dsv[32];
        tmem_ld32(lane_addr + (it & 1) * 64 + c * 32, rs);
        tmem_ld32(lane_addr + 128 + (it & 1) * 64 + c * 32, rp);
        tmem_ld_wait();
        if (!diag && (i + 1) * QSUB <= p.S) {   // sub-tile strictly below the diagonal block and inside the sequence
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            pv[e] = fast_exp2(fmaf(__uint_as_float(rs[e]), p.scale_log2, -st[col]));
            dsv[e] = pv[e] * (__uint_as_float(rp[e]) - st[QSUB + col]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e, qi = i * QSUB + col;
            const float pr = fast_exp2(fmaf(__uint_as_float(rs[e]), p.scale_log2, -st[col]));
            const bool keep = qi < p.S && (!diag || kj <= qi);
            pv[e] = keep ? pr : 0.f;
            dsv[e] = keep ? pr * (__uint_as_float(rp[e]) - st[QSUB + col]) : 0.f;
          }
        }
        // P^T / dS^T of the previous item must have been consumed before they are overwritten; waiting only here
        // lets this item's exponentials run under the previous item's dV / dK products
        if (!mbar_wait(pds_empty, (it & 1u) ^ 1u, abort_flag)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          store_swizzled32<T>(pt_ptr, row, c * 32, pv);
          store_swizzled32<T>(dst_ptr, row, c * 32, dsv);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);   // the warp's writes are ordered before lane 0's arrival
    }
    bool fin = ok && mbar_wait(acc_full, 0, abort_flag);
    fin = __all_sync(0xffffffffu, fin);
    if (fin) {
      tc_fence_after();
      if (p.gsplit > 1) {
        // fp32 partials of this query head; a second kernel sums the group in a fixed order
        const int64_t rows = (int64_t)(gridDim.x / gs) * p.S;
        float* pk = p.part + (((int64_t)zsplit * 2 + 0) * rows + (int64_t)bk * p.S + kj) * AD;
        float* pvp = p.part + (((int64_t)zsplit * 2 + 1) * rows + (int64_t)bk * p.S + kj) * AD;
#pragma unroll 1
        for (int c = 2 * ch; c < 2 * ch + 2; ++c) {
          uint32_t rk[32], rv[32];
          tmem_ld32(lane_addr + 256 + c * 32, rk);
          tmem_ld32(lane_addr + 384 + c * 32, rv);
          tmem_ld_wait();
          if (kj < p.S) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              *reinterpret_cast<uint4*>(pk + c * 32 + g * 4) = make_uint4(rk[g * 4], rk[g * 4 + 1], rk[g * 4 + 2], rk[g * 4 + 3]);
              *reinterpret_cast<uint4*>(pvp + c * 32 + g * 4) = make_uint4(rv[g * 4], rv[g * 4 + 1], rv[g * 4 + 2], rv[g * 4 + 3]);
            }
          }
        }
      } else {
        T* krow = reinterpret_cast<T*>(p.dk) + (int64_t)b * p.k_bs + (int64_t)kvh * p.k_hs + (int64_t)kj * p.k_ss;
        T* vrow = reinterpret_cast<T*>(p.dv) + (int64_t)b * p.k_bs + (int64_t)kvh * p.k_hs + (int64_t)kj * p.k_ss;
#pragma unroll 1
        for (int c = 2 * ch; c < 2 * ch + 2; ++c) {
          uint32_t rk[32], rv[32];
          tmem_ld32(lane_addr + 256 + c * 32, rk);
          tmem_ld32(lane_addr + 384 + c * 32, rv);
          tmem_ld_wait();
          if (kj < p.S) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 wk, wv;
              uint32_t* pk = reinterpret_cast<uint32_t*>(&wk);
              uint32_t* pv2 = reinterpret_cast<uint32_t*>(&wv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                pk[e] = pack2<T>(__uint_as_float(rk[g * 8 + 2 * e]) * p.scale, __uint_as_float(rk[g * 8 + 2 * e + 1]) * p.scale);
                pv2[e] = pack2<T>(__uint_as_float(rv[g * 8 + 2 * e]), __uint_as_float(rv[g * 8 + 2 * e + 1]));
              }
              *reinterpret_cast<uint4*>(krow + c * 32 + g * 8) = wk;
              *reinterpret_cast<uint4*>(vrow + c * 32 + g * 8) = wv;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag) flag_status(p.status, Q3_STATUS_WAIT_TIMEOUT);
}
constexpr int kDkdvSmem = 2 * TILE_BYTES + KV_STAGES * 2 * SUB_BYTES + 2 * SUB_BYTES + 4 * QSUB * 4 + 1024 + 256;

// Sum the per-query-head fp32 partials of dK / dV in head order, scale dK, round once, store with strides.
template <typename T>
__global__ void attn_dkdv_reduce_kernel(const float* __restrict__ part, T* __restrict__ dk, T* __restrict__ dv, int G,
                                        int64_t rows, int Hkv, int S, int64_t k_ss, int64_t k_hs, int64_t k_bs,
                                        float scale) {
  const int64_t total = rows * (AD / 4);
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / (AD / 4);
    const int c = (int)(idx % (AD / 4)) * 4;
    float4 ak = make_float4(0.f, 0.f, 0.f, 0.f), av = ak;
    for (int z = 0; z < G; ++z) {
      const float4 a = *reinterpret_cast<const float4*>(part + (((int64_t)z * 2 + 0) * rows + row) * AD + c);
      const float4 bq = *reinterpret_cast<const float4*>(part + (((int64_t)z * 2 + 1) * rows + row) * AD + c);
      ak.x += a.x; ak.y += a.y; ak.z += a.z; ak.w += a.w;
      av.x += bq.x; av.y += bq.y; av.z += bq.z; av.w += bq.w;
    }
    const int64_t sidx = row % S, bkv = row / S, kvh = bkv % Hkv, b = bkv / Hkv;
    const int64_t off = b * k_bs + kvh * k_hs + sidx * k_ss + c;
    uint2 wk, wv;
    wk.x = pack2<T>(ak.x * scale, ak.y * scale); wk.y = pack2<T>(ak.z * scale, ak.w * scale);
    wv.x = pack2<T>(av.x, av.y); wv.y = pack2<T>(av.z, av.w);
    *reinterpret_cast<uint2*>(dk + off) = wk;
    *reinterpret_cast<uint2*>(dv + off) = wv;
  }
}

template <typename K> int configure_smem(K kern, int bytes, DeviceFlags* done) {
  return ensure_dynamic_smem(kern, bytes, done);
}

}  // namespace tc

bool attn_tc_available() { return true; }

// How the dK/dV kernel covers a query-head group: 0 = by grid size (below), 1 = always one CTA per key tile that
// accumulates the whole group in tensor memory, 2 = always one CTA per query head plus the reduce kernel.
static int g_group_policy = 0;
int attn_bwd_set_group_policy(int policy) {
  const int old = g_group_policy;
  if (policy >= 0 && policy <= 2) g_group_policy = policy;
  return old;
}

// One CTA per query head (plus a reduce kernel) when one CTA per key tile would leave SMs idle.
int attn_bwd_group_split(int64_t B, int64_t Hq, int64_t Hkv, int64_t S) {
  const int64_t G = Hq / Hkv, ctas = B * Hkv * cdiv(S, tc::TILE);
  if (G <= 1 || g_group_policy == 1) return 1;
  if (g_group_policy == 2) return (int)G;
  return ctas < 2 * (int64_t)sm_count() ? (int)G : 1;
}

namespace {
// Element strides over (sequence, head, batch) for layout 0 = [B, H, S, 128] and layout 1 = [B, S, H, 128].
struct Strides { int64_t ss, hs, bs; };
inline Strides strides_for(int layout, int64_t H, int64_t S) {
  if (layout == 0) return {tc::AD, S * tc::AD, H * S * tc::AD};
  return {H * tc::AD, tc::AD, S * H * tc::AD};
}
}  // namespace

int attn_fwd_tc(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t Hq, int64_t Hkv,
                int64_t S, float scale, int dtype, int layout, int* status, cudaStream_t st) {
  using namespace tc;
  const bool bf16 = dtype == Q3_BF16;
  const Strides sq = strides_for(layout, Hq, S), sk = strides_for(layout, Hkv, S);
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_4d(&tmQ, q, bf16, B, Hq, S, AD, sq.ss, sq.hs, sq.bs, 64, TILE);
  if (rc != Q3_OK) return rc;
  rc = make_tmap_4d(&tmK, k, bf16, B, Hkv, S, AD, sk.ss, sk.hs, sk.bs, 64, TILE);
  if (rc != Q3_OK) return rc;
  rc = make_tmap_4d(&tmV, v, bf16, B, Hkv, S, AD, sk.ss, sk.hs, sk.bs, 64, TILE);
  if (rc != Q3_OK) return rc;
  AttnParams p{};
  p.out = out; p.lse = lse; p.Hq = (int)Hq; p.Hkv = (int)Hkv; p.S = (int)S;
  p.q_ss = sq.ss; p.q_hs = sq.hs; p.q_bs = sq.bs;
  p.scale_log2 = scale * kLog2e;
  p.idesc_qk = make_idesc_f16(128, 128, bf16, false, false);
  p.idesc_pv = make_idesc_f16(128, 128, bf16, false, true);
  p.status = status;
  dim3 grid((unsigned)(B * Hq), (unsigned)cdiv(S, TILE));
  if (bf16) {
    static DeviceFlags cfg = {};
    if ((rc = configure_smem(attn_fwd_tc_kernel<__nv_bfloat16>, kFwdSmem, &cfg)) != Q3_OK) return rc;
    attn_fwd_tc_kernel<__nv_bfloat16><<<grid, kFwdThreads, kFwdSmem, st>>>(tmQ, tmK, tmV, p);
  } else {
    static DeviceFlags cfg = {};
    if ((rc = configure_smem(attn_fwd_tc_kernel<__half>, kFwdSmem, &cfg)) != Q3_OK) return rc;
    attn_fwd_tc_kernel<__half><<<grid, kFwdThreads, kFwdSmem, st>>>(tmQ, tmK, tmV, p);
  }
  return launch_status();
}

int attn_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                void* dq, void* dk, void* dv, float* partials, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, float scale,
                int dtype, int layout, int* status, cudaStream_t st) {
  using namespace tc;
  const bool bf16 = dtype == Q3_BF16;
  const Strides sq = strides_for(layout, Hq, S), sk = strides_for(layout, Hkv, S);
  CUtensorMap tmQ, tmK, tmV, tmDO, tmQs, tmDOs;
  int rc;
  if ((rc = make_tmap_4d(&tmQ, q, bf16, B, Hq, S, AD, sq.ss, sq.hs, sq.bs, 64, TILE)) != Q3_OK) return rc;
  if ((rc = make_tmap_4d(&tmDO, dout, bf16, B, Hq, S, AD, sq.ss, sq.hs, sq.bs, 64, TILE)) != Q3_OK) return rc;
  if ((rc = make_tmap_4d(&tmK, k, bf16, B, Hkv, S, AD, sk.ss, sk.hs, sk.bs, 64, TILE)) != Q3_OK) return rc;
  if ((rc = make_tmap_4d(&tmV, v, bf16, B, Hkv, S, AD, sk.ss, sk.hs, sk.bs, 64, TILE)) != Q3_OK) return rc;
  if ((rc = make_tmap_4d(&tmQs, q, bf16, B, Hq, S, AD, sq.ss, sq.hs, sq.bs, 64, QSUB)) != Q3_OK) return rc;
  if ((rc = make_tmap_4d(&tmDOs, dout, bf16, B, Hq, S, AD, sq.ss, sq.hs, sq.bs, 64, QSUB)) != Q3_OK) return rc;
  AttnBwdParams p{};
  p.lse = lse; p.delta = delta; p.dq = dq; p.dk = dk; p.dv = dv;
  p.gsplit = attn_bwd_group_split(B, Hq, Hkv, S);
  p.part = partials;
  if (p.gsplit > 1 && partials == nullptr) return Q3_ERR_WORKSPACE;
  p.Hq = (int)Hq; p.Hkv = (int)Hkv; p.S = (int)S; p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.q_ss = sq.ss; p.q_hs = sq.hs; p.q_bs = sq.bs; p.k_ss = sk.ss; p.k_hs = sk.hs; p.k_bs = sk.bs;
  p.idesc_kk128 = make_idesc_f16(128, 128, bf16, false, false);
  p.idesc_kk64 = make_idesc_f16(128, 64, bf16, false, false);
  p.idesc_kmn = make_idesc_f16(128, 128, bf16, false, true);
  p.status = status;
  dim3 gq((unsigned)(B * Hq), (unsigned)cdiv(S, TILE)), gk((unsigned)(B * Hkv * p.gsplit), (unsigned)cdiv(S, TILE));
  const int64_t kv_rows = B * Hkv * S;
  const int red_grid = (int)std::min<int64_t>(cdiv(kv_rows * (AD / 4), 256), (int64_t)sm_count() * 8);
  if (bf16) {
    static DeviceFlags c1 = {}, c2 = {};
    if ((rc = configure_smem(attn_dq_tc_kernel<__nv_bfloat16>, kDqSmem, &c1)) != Q3_OK) return rc;
    if ((rc = configure_smem(attn_dkdv_tc_kernel<__nv_bfloat16>, kDkdvSmem, &c2)) != Q3_OK) return rc;
    attn_dkdv_tc_kernel<__nv_bfloat16><<<gk, kAttnThreads, kDkdvSmem, st>>>(tmQs, tmK, tmV, tmDOs, p);
    if (p.gsplit > 1)
      attn_dkdv_reduce_kernel<__nv_bfloat16><<<red_grid, 256, 0, st>>>(partials, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, p.gsplit, kv_rows,
                                                                     (int)Hkv, (int)S, sk.ss, sk.hs, sk.bs, scale);
    attn_dq_tc_kernel<__nv_bfloat16><<<gq, kDqThreads, kDqSmem, st>>>(tmQ, tmK, tmV, tmDO, p);
  } else {
    static DeviceFlags c1 = {}, c2 = {};
    if ((rc = configure_smem(attn_dq_tc_kernel<__half>, kDqSmem, &c1)) != Q3_OK) return rc;
    if ((rc = configure_smem(attn_dkdv_tc_kernel<__half>, kDkdvSmem, &c2)) != Q3_OK) return rc;
    attn_dkdv_tc_kernel<__half><<<gk, kAttnThreads, kDkdvSmem, st>>>(tmQs, tmK, tmV, tmDOs, p);
    if (p.gsplit > 1)
      attn_dkdv_reduce_kernel<__half><<<red_grid, 256, 0, st>>>(partials, (__half*)dk, (__half*)dv, p.gsplit, kv_rows, (int)Hkv, (int)S,
                                                              sk.ss, sk.hs, sk.bs, scale);
    attn_dq_tc_kernel<__half><<<gq, kDqThreads, kDqSmem, st>>>(tmQ, tmK, tmV, tmDO, p);
  }
  return launch_status();
}

}  // namespace q3
