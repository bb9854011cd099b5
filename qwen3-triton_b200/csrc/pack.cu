// Multi-tensor strided copy with dtype conversion: the data movement FSDP2 does around its collectives.
//   all-gather copy-in : every local fp32 (or bf16) shard -> its slice of the bf16 all-gather input   (rows = 1)
//   split-copy-out     : all-gather output [world, total] -> per-parameter [world, n_i] tensors          (strided rows)
//   chunk-cat          : bf16 gradients, chunked along dim 0 into `world` pieces (zero-padded) and laid side by
//                        side as fp32 rows of the reduce-scatter input                                   (upcast + pad)
// One launch handles every tensor of an FSDP unit. The grid is persistent (one resident wave) and sweeps the pieces of
// a device table one after another, grid-stride inside a piece, so that at any moment the whole grid reads one
// contiguous window of DRAM; 8 adjacent elements per lane per access, four accesses in flight.
//
// Table: int64 [n][8] = {src, dst, rows, cols, src_row_stride, dst_row_stride, src_valid, vec_ok};
// element (r, c) is read from src[r*src_row_stride + c] if that index is < src_valid, else it is 0.
//
// Replaces, in the reference: qwen3_triton/runtime/ops.py:70-93,116-127,186-202 (_runtime_strided_copy,
// _runtime_chunk_cat_one, copy-in) routed by runtime/dispatch.py:105-119.
#include "common.cuh"

namespace q3 {

constexpr int kPackCols = 8;        // table columns
constexpr int kPackCtasPerSm = 2;   // measured best overall of 2..12 (chunk-cat 5.6 TB/s, split 5.5, copy-in 4.6)

// 8 elements with the streaming (evict-first) cache policy on both sides: these copies move gigabytes that nobody
// re-reads from L2, beside GEMMs whose operand reuse lives in L2. With the default policy the gradient pack of one FSDP
// unit evicted the activations of the weight-gradient GEMM running next to it, which then took 2.6 times as long.
template <typename T> struct Stream8;
template <> struct Stream8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
    __stcs(reinterpret_cast<float4*>(p + 4), make_float4(v[4], v[5], v[6], v[7]));
  }
};
template <> struct Stream8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 t;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    __stcs(reinterpret_cast<uint4*>(p), t);
  }
};
template <> struct Stream8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 t;
    __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    __stcs(reinterpret_cast<uint4*>(p), t);
  }
};

// One lane's share of one vectorised piece. A lane visits vectors first, first + stride, ...; its source and
// destination offsets advance by constant steps with one conditional wrap to the next row, so the loop has no
// division (index arithmetic, not DRAM, limited the divided form to 4.9 TB/s). IDX = unsigned when every offset of the
// piece fits 32 bits; CHECK = false when no vector of the piece reaches past src_valid.
template <typename S, typename D, typename IDX, bool CHECK>
__device__ __forceinline__ void sweep_piece(const S* __restrict__ src, D* __restrict__ dst, int64_t cols64, int64_t ss64,
                                            int64_t ds64, int64_t valid64, int64_t nvec, int64_t first, int64_t stride) {
  const int64_t e0 = first << 3, hop = stride << 3;
  int64_t r0, r_step;
  if (((e0 | hop | cols64) >> 32) == 0) {   // the usual case: 32-bit divisions
    r0 = (unsigned)e0 / (unsigned)cols64;
    r_step = (unsigned)hop / (unsigned)cols64;
  } else {
    r0 = e0 / cols64;
    r_step = hop / cols64;
  }
  const IDX cols = (IDX)cols64, valid = (IDX)valid64;
  IDX c = (IDX)(e0 - r0 * cols64);
  const IDX c_step = (IDX)(hop - r_step * cols64);
  IDX si = (IDX)(r0 * ss64) + c, di = (IDX)(r0 * ds64) + c;
  const IDX step_s = (IDX)(r_step * ss64) + c_step, step_d = (IDX)(r_step * ds64) + c_step;
  const IDX wrap_s = (IDX)(ss64 - cols64), wrap_d = (IDX)(ds64 - cols64);
  auto advance = [&]() {
    c += c_step; si += step_s; di += step_d;
    if (c >= cols) { c -= cols; si += wrap_s; di += wrap_d; }
  };
  auto load = [&](IDX at, float (&v)[8]) {
    if (!CHECK || at + 8 <= valid) {
      Stream8<S>::load(src + at, v);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = at + j < valid ? to_f32<S>(src[at + j]) : 0.f;
    }
  };
  constexpr int U = 4;   // independent accesses in flight per lane
  int64_t left64 = (nvec - first + stride - 1) / stride;   // vectors this lane owns
  int64_t left = left64;
  for (; left >= U; left -= U) {
    float v[U][8];
    IDX d[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      d[u] = di;
      load(si, v[u]);
      advance();
    }
#pragma unroll
    for (int u = 0; u < U; ++u) Stream8<D>::store(dst + d[u], v[u]);
  }
  // Tail one vector at a time: predicating the batch instead (tried both on loads and on stores) cost more
  // registers or serialised the main loop and lost 5-30 % on whole-buffer copies.
  for (; left > 0; --left) {
    float v0[8];
    load(si, v0);
    Stream8<D>::store(dst + di, v0);
    advance();
  }
}

template <typename S, typename D>
__global__ void __launch_bounds__(256) multi_copy_kernel(const int64_t* __restrict__ meta, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  const int64_t first = blockIdx.x * (int64_t)256 + threadIdx.x;
  for (int64_t ent = 0; ent < n; ++ent) {
    const int64_t* e = meta + ent * kPackCols;
    const S* __restrict__ src = reinterpret_cast<const S*>(e[0]);
    D* __restrict__ dst = reinterpret_cast<D*>(e[1]);
    const int64_t rows = e[2], cols = e[3], ss = e[4], ds = e[5], valid = e[6];
    const int64_t total = rows * cols;
    if (e[7]) {
      // cols and both strides are multiples of 8, both bases 16-byte aligned
      const int64_t nvec = total >> 3;
      if (first >= nvec) continue;
      const int64_t reach = (rows - 1) * (ss > ds ? ss : ds) + cols;       // largest offset + 1 on either side
      const bool small = reach < ((int64_t)1 << 32) - 8 && valid < ((int64_t)1 << 32) - 8;   // unsigned offsets: the unused advance past the last vector may wrap
      const bool check = (rows - 1) * ss + cols > valid;
      if (small) {
        if (check) sweep_piece<S, D, unsigned, true>(src, dst, cols, ss, ds, valid, nvec, first, stride);
        else sweep_piece<S, D, unsigned, false>(src, dst, cols, ss, ds, valid, nvec, first, stride);
      } else {
        sweep_piece<S, D, int64_t, true>(src, dst, cols, ss, ds, valid, nvec, first, stride);
      }
    } else {
      for (int64_t i = first; i < total; i += stride) {
        const int64_t r = i / cols, c = i - r * cols;
        const int64_t si = r * ss + c;
        dst[r * ds + c] = from_f32<D>(si < valid ? to_f32<S>(src[si]) : 0.f);
      }
    }
  }
}

}  // namespace q3

using namespace q3;

extern "C" int q3_multi_copy(const int64_t* meta, int64_t n_entries, int64_t total_elements, int src_dtype,
                             int dst_dtype, q3_stream_t stream) {
  if (!meta) return Q3_ERR_ARG;
  if (n_entries < 1 || total_elements < 1) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  // Fewer CTAs for the copies that run beside compute kernels on a side stream were tried (74 and 32 instead of 296):
  // no gain in step time within the run-to-run spread, and a loss once the copy no longer keeps up.
  const int64_t want = cdiv(cdiv(total_elements, 8), 256), cap = (int64_t)sm_count() * kPackCtasPerSm;
  const unsigned g = (unsigned)(want < cap ? want : cap);
#define Q3_MC(S, D) multi_copy_kernel<S, D><<<g, 256, 0, st>>>(meta, n_entries)
  if (src_dtype == Q3_F32 && dst_dtype == Q3_BF16) Q3_MC(float, __nv_bfloat16);
  else if (src_dtype == Q3_BF16 && dst_dtype == Q3_F32) Q3_MC(__nv_bfloat16, float);
  else if (src_dtype == Q3_BF16 && dst_dtype == Q3_BF16) Q3_MC(__nv_bfloat16, __nv_bfloat16);
  else if (src_dtype == Q3_F32 && dst_dtype == Q3_F32) Q3_MC(float, float);
  else if (src_dtype == Q3_F32 && dst_dtype == Q3_F16) Q3_MC(float, __half);
  else if (src_dtype == Q3_F16 && dst_dtype == Q3_F32) Q3_MC(__half, float);
  else if (src_dtype == Q3_F16 && dst_dtype == Q3_F16) Q3_MC(__half, __half);
  else return Q3_ERR_DTYPE;
#undef Q3_MC
  return launch_status();
}
