// Token-block data path and validation statistics on the device.
//
// The training corpus is a flat array of little-endian uint32 token ids cut into blocks of `seq` tokens; the training
// order visits block ((i + offset) * stride + seed) mod n with a stride coprime to n (a full-period permutation
// without a shuffle buffer). With 180 GB of HBM the whole corpus can live on the GPU, so a batch is one gather
// kernel away: no host-side indexing, no pinned staging, no H2D copy per step.
//
// Replaces, in the reference: training/data.py:9-28 (Blocks.__getitem__: index arithmetic and the uint32 -> int64
// widening) and qwen3_triton/runtime/metrics.py:8-17 (fp64 accumulation of validation loss and token count).
#include "common.cuh"

namespace q3 {

__device__ __forceinline__ int64_t permuted_block(int64_t i, int64_t offset, int64_t stride, int64_t seed, int64_t n) {
  // exact for any int64 arguments: the product is formed in 128 bits, as Python's integers would
  const __int128 v = ((__int128)i + (__int128)offset) * (__int128)stride + (__int128)seed;
  __int128 r = v % (__int128)n;
  if (r < 0) r += n;    // Python's % is non-negative for a positive modulus
  return (int64_t)r;
}

__global__ void block_order_kernel(int64_t* __restrict__ out, int64_t first, int64_t count, int64_t offset,
                                   int64_t stride, int64_t seed, int64_t n, int training) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= count) return;
  out[i] = training ? permuted_block(first + i, offset, stride, seed, n) : first + i;
}

// ids[b, s] = corpus[block[b] * seq + s], widened to int64. One warp per 32 consecutive tokens keeps both the 4-byte
// reads and the 8-byte writes coalesced; a block index outside [0, n) flags the status word and writes zeros.
__global__ void token_blocks_kernel(const uint32_t* __restrict__ corpus, const int64_t* __restrict__ block,
                                    int64_t* __restrict__ ids, int64_t batch, int64_t seq, int64_t n, int* status) {
  const int64_t total = batch * seq;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = t / seq, s = t - b * seq;
    const int64_t blk = block[b];
    if (blk < 0 || blk >= n) {
      if (s == 0) flag_status(status, Q3_STATUS_ID_RANGE);
      ids[t] = 0;
    } else {
      ids[t] = (int64_t)corpus[blk * seq + s];
    }
  }
}

// totals[0] += loss * tokens, totals[1] += tokens, in fp64 without fused multiply-add (the host computes the same
// two roundings); one thread: the accumulator is two doubles.
__global__ void validation_accumulate_kernel(const float* __restrict__ loss, double* __restrict__ totals, double tokens) {
  const double value = (double)loss[0];
  totals[0] = __dadd_rn(totals[0], __dmul_rn(value, tokens));
  totals[1] = __dadd_rn(totals[1], tokens);
}

// totals[0] += sum of losses[b, s] over the shifted rows (b, s < S-1) whose target labels[b, s+1] is not ignore_index,
// totals[1] += their number. fp64, fixed summation order (one CTA, strided partials, tree in shared memory).
__global__ void validation_rows_kernel(const float* __restrict__ losses, const int64_t* __restrict__ labels,
                                       int64_t B, int64_t S, int64_t ignore, double* __restrict__ totals) {
  __shared__ double part[1024];
  __shared__ double cnt[1024];
  double a = 0.0, c = 0.0;
  const int64_t rows = B * (S - 1);
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) {
    const int64_t b = i / (S - 1), s = i - b * (S - 1);
    if (labels[b * S + s + 1] != ignore) { a += (double)losses[i]; c += 1.0; }
  }
  part[threadIdx.x] = a;
  cnt[threadIdx.x] = c;
  __syncthreads();
  for (int w = blockDim.x / 2; w > 0; w >>= 1) {
    if ((int)threadIdx.x < w) { part[threadIdx.x] += part[threadIdx.x + w]; cnt[threadIdx.x] += cnt[threadIdx.x + w]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { totals[0] += part[0]; totals[1] += cnt[0]; }
}

}  // namespace q3

using namespace q3;

extern "C" int q3_block_order(int64_t* out, int64_t first, int64_t count, int64_t offset, int64_t stride, int64_t seed,
                              int64_t n, int training, q3_stream_t stream) {
  if (!out) return Q3_ERR_ARG;
  if (count < 1 || n < 1 || stride < 1) return Q3_ERR_SHAPE;
  block_order_kernel<<<(unsigned)cdiv(count, 256), 256, 0, (cudaStream_t)stream>>>(out, first, count, offset, stride,
                                                                                   seed, n, training);
  return launch_status();
}

extern "C" int q3_token_blocks(const uint32_t* corpus, int64_t corpus_tokens, const int64_t* block, int64_t* ids,
                               int64_t batch, int64_t seq, int* status, q3_stream_t stream) {
  if (!corpus || !block || !ids) return Q3_ERR_ARG;
  if (batch < 1 || seq < 2 || corpus_tokens < seq) return Q3_ERR_SHAPE;
  const int64_t total = batch * seq;
  const int64_t want = cdiv(total, 256), cap = (int64_t)sm_count() * 8;
  token_blocks_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, (cudaStream_t)stream>>>(
      corpus, block, ids, batch, seq, corpus_tokens / seq, status);
  return launch_status();
}

extern "C" int q3_validation_accumulate(const float* loss, double* totals, int64_t tokens, q3_stream_t stream) {
  if (!loss || !totals) return Q3_ERR_ARG;
  if (tokens < 0) return Q3_ERR_SHAPE;
  if (tokens == 0) return Q3_OK;
  validation_accumulate_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(loss, totals, (double)tokens);
  return launch_status();
}

extern "C" int q3_validation_rows(const float* losses, const int64_t* labels, int64_t B, int64_t S,
                                  int64_t ignore_index, double* totals, q3_stream_t stream) {
  if (!losses || !labels || !totals) return Q3_ERR_ARG;
  if (B < 1 || S < 2) return Q3_ERR_SHAPE;
  validation_rows_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(losses, labels, B, S, ignore_index, totals);
  return launch_status();
}
