// Multi-tensor AdamW on fp32 master parameters with fp32 moments: one launch updates every tensor
// of a parameter group. Streaming kernel: 16 B read per element (p, g, m, v) and 12 B written
// (p, m, v), 128-bit vector accesses, one CTA per `block`-element chunk of one tensor.
//
// Table layout (device, int64[rows][7]): {p, g, m, v, step pointers, numel, first_block}.
// Math order: decoupled decay, moments, bias corrections bc1 = 1-b1^t, sqrt(bc2) = sqrt(1-b2^t),
// step_size = lr/bc1, denom = sqrt(v)/sqrt(bc2) + eps; the per-tensor coefficients are computed in fp64, the
// per-element arithmetic in fp32.
//
// Replaces, in the reference: qwen3_triton/runtime/adamw.py:20-30 (_adamw_prepare) and
// runtime/adamw.py:34-61 (_adamw_update).
#include "common.cuh"

namespace q3 {

__global__ void adamw_prepare_kernel(const int64_t* __restrict__ meta, float* __restrict__ coeff, int64_t rows,
                                     double lr, double b1, double b2) {
  const int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float* step_ptr = reinterpret_cast<float*>(meta[r * 7 + 4]);
  const float step = *step_ptr + 1.f;
  *step_ptr = step;
  const float bc1 = (float)(1.0 - pow(b1, (double)step));
  const float bc2 = (float)sqrt(1.0 - pow(b2, (double)step));
  coeff[r * 3 + 0] = bc1;
  coeff[r * 3 + 1] = bc2;
  coeff[r * 3 + 2] = (float)(lr / (double)bc1);
}

// One element. The hyper-parameters arrive as doubles (the host's values) and are rounded to fp32 once per thread; the
// per-element arithmetic is fp32 with fused multiply-adds and IEEE sqrt / division. (An earlier form did the
// per-element arithmetic in fp64: ten fp64 conversions and operations per element made the kernel compute-bound
// at the 1.36 GHz the chip holds under its power cap inside a training step.) Against the fp64 oracle the result
// differs by a few 1e-7 relative, inside the 1e-5 gate.
__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v, double lr, double b1, double b2,
                                          double decay, double eps, float bc2, float size) {
  const float lr_decay = (float)(lr * decay), b1f = (float)b1, omb1 = (float)(1.0 - b1), b2f = (float)b2,
              omb2 = (float)(1.0 - b2), epsf = (float)eps;
  p = fmaf(-lr_decay, p, p);
  m = fmaf(b1f, m, omb1 * g);
  v = fmaf(b2f, v, (omb2 * g) * g);
  const float denom = __fdiv_rn(__fsqrt_rn(v), bc2) + epsf;
  p = p - __fdiv_rn(size * m, denom);
}

__global__ void __launch_bounds__(256) adamw_update_kernel(const int64_t* __restrict__ meta,
                                                           const float* __restrict__ coeff, int64_t rows, double lr,
                                                           double b1, double b2, double decay, double eps,
                                                           int block_elems) {
  // Find the tensor that owns this block: last row whose first_block <= blockIdx.x.
  const int64_t blk = blockIdx.x;
  int64_t lo = 0, hi = rows;
  while (lo + 1 < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (meta[mid * 7 + 6] <= blk) lo = mid; else hi = mid;
  }
  const int64_t r = lo;
  float* __restrict__ p = reinterpret_cast<float*>(meta[r * 7 + 0]);
  const float* __restrict__ g = reinterpret_cast<const float*>(meta[r * 7 + 1]);
  float* __restrict__ m = reinterpret_cast<float*>(meta[r * 7 + 2]);
  float* __restrict__ v = reinterpret_cast<float*>(meta[r * 7 + 3]);
  const int64_t n = meta[r * 7 + 5];
  const int64_t begin = (blk - meta[r * 7 + 6]) * (int64_t)block_elems;
  const int64_t end = begin + block_elems < n ? begin + block_elems : n;
  const float bc2 = coeff[r * 3 + 1], size = coeff[r * 3 + 2];
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
  if (vec) {
    const int64_t vend = begin + ((end - begin) & ~(int64_t)3);
    for (int64_t i = begin + threadIdx.x * 4; i < vend; i += blockDim.x * 4) {
      float4 pp = *reinterpret_cast<const float4*>(p + i);
      const float4 gg = *reinterpret_cast<const float4*>(g + i);
      float4 mm = *reinterpret_cast<const float4*>(m + i);
      float4 vv = *reinterpret_cast<const float4*>(v + i);
      adamw_one(pp.x, gg.x, mm.x, vv.x, lr, b1, b2, decay, eps, bc2, size);
      adamw_one(pp.y, gg.y, mm.y, vv.y, lr, b1, b2, decay, eps, bc2, size);
      adamw_one(pp.z, gg.z, mm.z, vv.z, lr, b1, b2, decay, eps, bc2, size);
      adamw_one(pp.w, gg.w, mm.w, vv.w, lr, b1, b2, decay, eps, bc2, size);
      *reinterpret_cast<float4*>(p + i) = pp;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
    }
    for (int64_t i = vend + threadIdx.x; i < end; i += blockDim.x) {
      float pp = p[i], mm = m[i], vv = v[i];
      adamw_one(pp, g[i], mm, vv, lr, b1, b2, decay, eps, bc2, size);
      p[i] = pp; m[i] = mm; v[i] = vv;
    }
  } else {
    for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
      float pp = p[i], mm = m[i], vv = v[i];
      adamw_one(pp, g[i], mm, vv, lr, b1, b2, decay, eps, bc2, size);
      p[i] = pp; m[i] = mm; v[i] = vv;
    }
  }
}

// Mixed-precision variant: the gradient may arrive in bf16/fp16 (read directly, no fp32 staging copy) and the
// updated parameter may also be written as a bf16/fp16 working copy, so a single-GPU mixed-precision step needs
// neither a gradient-upcast pass nor a master->working cast pass. Table: int64[rows][9] =
// {p, g_fp32 (or 0), m, v, step, numel, first_block, g_lowp (or 0), p_lowp (or 0)}.
// BOTH: every row has a low-precision gradient and a low-precision copy (the single-GPU mixed-precision step): no
// fp32 gradient pointer, no per-row branches, 48 registers and five CTAs per SM.
template <typename L, bool BOTH>
__global__ void __launch_bounds__(256, BOTH ? 5 : 4) adamw_update_mp_kernel(const int64_t* __restrict__ meta,
                                                              const float* __restrict__ coeff, int64_t rows, double lr,
                                                              double b1, double b2, double decay, double eps,
                                                              int block_elems, int64_t total_blocks) {
  // one block per CTA when the grid covers them all; a smaller grid (an update that runs beside compute kernels and
  // must leave them most of the memory bandwidth) strides over the blocks
  for (int64_t blk = blockIdx.x; blk < total_blocks; blk += gridDim.x) {
  int64_t lo = 0, hi = rows;
  while (lo + 1 < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (meta[mid * 9 + 6] <= blk) lo = mid; else hi = mid;
  }
  const int64_t r = lo;
  float* __restrict__ p = reinterpret_cast<float*>(meta[r * 9 + 0]);
  const float* __restrict__ g32 = BOTH ? nullptr : reinterpret_cast<const float*>(meta[r * 9 + 1]);
  float* __restrict__ m = reinterpret_cast<float*>(meta[r * 9 + 2]);
  float* __restrict__ v = reinterpret_cast<float*>(meta[r * 9 + 3]);
  const L* __restrict__ glo = reinterpret_cast<const L*>(meta[r * 9 + 7]);
  L* __restrict__ plo = reinterpret_cast<L*>(meta[r * 9 + 8]);
  const int64_t n = meta[r * 9 + 5];
  const int64_t begin = (blk - meta[r * 9 + 6]) * (int64_t)block_elems;
  const int64_t end = begin + block_elems < n ? begin + block_elems : n;
  const float bc2 = coeff[r * 3 + 1], size = coeff[r * 3 + 2];
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(g32) | reinterpret_cast<uintptr_t>(glo) |
                         reinterpret_cast<uintptr_t>(plo);
  if ((bits & 15u) == 0) {
    // same shape as the fp32-gradient kernel: 4 elements per thread per iteration, one 16-byte access on each fp32
    // array and one 8-byte access on each 16-bit array
    // 32-bit offsets from the chunk's base pointers keep the loop at 48 registers
    const int vspan = (int)(end - begin) & ~3;
    const int64_t vend = begin + vspan;
    float* __restrict__ pb = p + begin;
    float* __restrict__ mb = m + begin;
    float* __restrict__ vb = v + begin;
    const L* __restrict__ gb = glo + begin;
    L* __restrict__ lb = plo + begin;
    for (int i = threadIdx.x * 4; i < vspan; i += 256 * 4) {
      float pp[4], mm[4], vv[4], gg[4];
      *reinterpret_cast<float4*>(pp) = *reinterpret_cast<const float4*>(pb + i);
      *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(mb + i);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(vb + i);
      if (BOTH || glo != nullptr) VecIO<L, 4>::load(gb + i, gg);
      else *reinterpret_cast<float4*>(gg) = *reinterpret_cast<const float4*>(g32 + begin + i);
#pragma unroll
      for (int e = 0; e < 4; ++e) adamw_one(pp[e], gg[e], mm[e], vv[e], lr, b1, b2, decay, eps, bc2, size);
      *reinterpret_cast<float4*>(pb + i) = *reinterpret_cast<float4*>(pp);
      *reinterpret_cast<float4*>(mb + i) = *reinterpret_cast<float4*>(mm);
      *reinterpret_cast<float4*>(vb + i) = *reinterpret_cast<float4*>(vv);
      if (BOTH || plo != nullptr) VecIO<L, 4>::store(lb + i, pp);
    }
    for (int64_t i = vend + threadIdx.x; i < end; i += blockDim.x) {
      float pp = p[i], mm = m[i], vv = v[i];
      adamw_one(pp, glo ? to_f32<L>(glo[i]) : g32[i], mm, vv, lr, b1, b2, decay, eps, bc2, size);
      p[i] = pp; m[i] = mm; v[i] = vv;
      if (plo) plo[i] = from_f32<L>(pp);
    }
  } else {
    for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
      float pp = p[i], mm = m[i], vv = v[i];
      adamw_one(pp, glo ? to_f32<L>(glo[i]) : g32[i], mm, vv, lr, b1, b2, decay, eps, bc2, size);
      p[i] = pp; m[i] = mm; v[i] = vv;
      if (plo) plo[i] = from_f32<L>(pp);
    }
  }
  }
}

__global__ void adamw_prepare9_kernel(const int64_t* __restrict__ meta, float* __restrict__ coeff, int64_t rows,
                                      double lr, double b1, double b2) {
  const int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float* step_ptr = reinterpret_cast<float*>(meta[r * 9 + 4]);
  const float step = *step_ptr + 1.f;
  *step_ptr = step;
  const float bc1 = (float)(1.0 - pow(b1, (double)step));
  coeff[r * 3 + 0] = bc1;
  coeff[r * 3 + 1] = (float)sqrt(1.0 - pow(b2, (double)step));
  coeff[r * 3 + 2] = (float)(lr / (double)bc1);
}

}  // namespace q3

using namespace q3;

extern "C" int q3_adamw_multi_mp(const int64_t* meta, float* coeff, int64_t n_tensors, int64_t total_blocks,
                                 int block_elems, int lowp_dtype, int all_rows_lowp, double lr, double beta1,
                                 double beta2, double weight_decay, double eps, q3_stream_t stream) {
  if (!meta || !coeff) return Q3_ERR_ARG;
  if (n_tensors < 1 || total_blocks < 1 || total_blocks > 2147483647LL || block_elems < 256 || (block_elems & 7))
    return Q3_ERR_SHAPE;
  if (lowp_dtype != Q3_BF16 && lowp_dtype != Q3_F16) return Q3_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  adamw_prepare9_kernel<<<(int)cdiv(n_tensors, 128), 128, 0, st>>>(meta, coeff, n_tensors, lr, beta1, beta2);
  static const int cap = [] { const char* e = getenv("Q3_ADAMW_CTAS"); return e ? atoi(e) : 0; }();
  const unsigned grid = (unsigned)((cap > 0 && cap < total_blocks) ? cap : total_blocks);
#define Q3_MP(L, BOTH)                                                                                    \
  adamw_update_mp_kernel<L, BOTH><<<grid, 256, 0, st>>>(meta, coeff, n_tensors, lr, beta1, beta2, \
                                                        weight_decay, eps, block_elems, total_blocks)
  if (lowp_dtype == Q3_BF16) { if (all_rows_lowp) Q3_MP(__nv_bfloat16, true); else Q3_MP(__nv_bfloat16, false); }
  else { if (all_rows_lowp) Q3_MP(__half, true); else Q3_MP(__half, false); }
#undef Q3_MP
  return launch_status();
}

extern "C" int q3_adamw_multi(const int64_t* meta, float* coeff, int64_t n_tensors, int64_t total_blocks,
                              int block_elems, double lr, double beta1, double beta2, double weight_decay, double eps,
                              q3_stream_t stream) {
  if (!meta || !coeff) return Q3_ERR_ARG;
  if (n_tensors < 1 || total_blocks < 1 || total_blocks > 2147483647LL || block_elems < 256 || (block_elems & 3))
    return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  adamw_prepare_kernel<<<(int)cdiv(n_tensors, 128), 128, 0, st>>>(meta, coeff, n_tensors, lr, beta1, beta2);
  adamw_update_kernel<<<(unsigned)total_blocks, 256, 0, st>>>(meta, coeff, n_tensors, lr, beta1, beta2, weight_decay,
                                                             eps, block_elems);
  return launch_status();
}
