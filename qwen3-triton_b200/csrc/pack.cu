// Multi-tensor strided copy with dtype conversion: the data movement FSDP2 does around its collectives.
//   all-gather copy-in : every local fp32 (or bf16) shard -> its slice of the bf16 all-gather input   (rows = 1)
//   split-copy-out     : all-gather output [world, total] -> per-parameter [world, n_i] tensors          (strided rows)
//   chunk-cat          : bf16 gradients, chunked along dim 0 into `world` pieces (zero-padded) and laid side by
//                        side as fp32 rows of the reduce-scatter input                                   (upcast + pad)
// One launch handles every tensor of an FSDP unit: a device table describes the 2-D pieces, a CTA takes a
// 16384-element span of one piece (binary search on the table), 16-byte accesses when the piece allows.
//
// Table: int64 [n][9] = {src, dst, rows, cols, src_row_stride, dst_row_stride, src_valid, first_block, vec_ok};
// element (r, c) is read from src[r*src_row_stride + c] if that index is < src_valid, else it is 0.
//
// Replaces, in the reference: qwen3_triton/runtime/ops.py:70-93,116-127,186-202 (_runtime_strided_copy,
// _runtime_chunk_cat_one, copy-in) routed by runtime/dispatch.py:105-119.
#include "common.cuh"

namespace q3 {

constexpr int kPackSpan = 16384;

template <typename S, typename D>
__global__ void __launch_bounds__(256) multi_copy_kernel(const int64_t* __restrict__ meta, int64_t n) {
  const int64_t blk = blockIdx.x;
  const int64_t lo = find_owner(meta, n, 9, 7, blk);
  const int64_t* e = meta + lo * 9;
  const S* __restrict__ src = reinterpret_cast<const S*>(e[0]);
  D* __restrict__ dst = reinterpret_cast<D*>(e[1]);
  const int64_t rows = e[2], cols = e[3], ss = e[4], ds = e[5], valid = e[6];
  const int64_t total = rows * cols;
  const int64_t begin = (blk - e[7]) * kPackSpan;
  const int64_t end = begin + kPackSpan < total ? begin + kPackSpan : total;
  // the row of a span's first element by one 64-bit division; inside the span 32-bit arithmetic on the offset
  const int64_t r0 = begin / cols, c0 = begin - r0 * cols;
  const int span = (int)(end - begin);
  const bool narrow = cols < (int64_t)1 << 31;
  const unsigned ucols = (unsigned)cols;
  auto locate = [&](int off, int64_t& si, int64_t& di) {
    int64_t r, c;
    if (narrow) {
      const unsigned t = (unsigned)c0 + (unsigned)off;   // c0 < 2^31 and off <= 16384
      const unsigned q = t / ucols;
      r = r0 + q;
      c = t - q * ucols;
    } else {
      const int64_t t = c0 + off;
      r = r0 + (t >= cols);
      c = t >= cols ? t - cols : t;
    }
    si = r * ss + c;
    di = r * ds + c;
  };
  if (e[8]) {
    // cols and strides are multiples of 8 and both bases 16-byte aligned: a lane moves 8 adjacent elements per
    // access (one or two 16-byte words), four accesses in flight. Measured faster than 4-element lanes spread a
    // CTA-width apart (chunk-cat 4.6 vs 3.9 TB/s).
    constexpr int VEC = 8;
    constexpr int BATCH = 4;
    for (int base = threadIdx.x * VEC; base < span; base += 256 * VEC * BATCH) {
      float v[BATCH][VEC];
      int64_t di[BATCH];
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int off = base + b * 256 * VEC;
        di[b] = -1;
        if (off < span) {
          int64_t si;
          locate(off, si, di[b]);
          if (si + VEC <= valid) {
            VecIO<S, VEC>::load(src + si, v[b]);
          } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[b][j] = si + j < valid ? to_f32<S>(src[si + j]) : 0.f;
          }
        }
      }
#pragma unroll
      for (int b = 0; b < BATCH; ++b)
        if (di[b] >= 0) VecIO<D, VEC>::store(dst + di[b], v[b]);
    }
  } else {
    for (int off = threadIdx.x; off < span; off += 256) {
      int64_t si, di;
      locate(off, si, di);
      dst[di] = from_f32<D>(si < valid ? to_f32<S>(src[si]) : 0.f);
    }
  }
}

}  // namespace q3

using namespace q3;

extern "C" int64_t q3_multi_copy_span(void) { return kPackSpan; }

extern "C" int q3_multi_copy(const int64_t* meta, int64_t n_entries, int64_t total_blocks, int src_dtype, int dst_dtype,
                             q3_stream_t stream) {
  if (!meta) return Q3_ERR_ARG;
  if (n_entries < 1 || total_blocks < 1 || total_blocks > 2147483647LL) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned g = (unsigned)total_blocks;
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
