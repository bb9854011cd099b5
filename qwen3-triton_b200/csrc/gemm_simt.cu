// Generic strided GEMM on CUDA cores: C[M,N] = A[M,K] * B[K,N], any element strides, fp32/bf16/fp16
// inputs, fp32 accumulation, contiguous output in any of the three types. This is the path for
// shapes the tensor-core kernel does not take (fp32 operands, leading dimensions that are not a
// multiple of 16 bytes, misaligned bases) and the on-device cross-check for it in the tests.
// 64x64 output tile per CTA, 16-deep k slices staged through shared memory as fp32, 4x4 register
// micro-tile per thread.
//
// Replaces, in the reference: qwen3_triton/kernels/linear.py:14-42 (_gemm) for those shapes.
#include "common.cuh"

namespace q3 {

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TI* __restrict__ A, int64_t a_sm, int64_t a_sk,
                                                        const TI* __restrict__ B, int64_t b_sk, int64_t b_sn,
                                                        TO* __restrict__ C, int64_t M, int64_t N, int64_t K) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // Pick the thread->element map that walks the unit-stride dimension fastest.
  const bool a_kfast = a_sk <= a_sm, b_nfast = b_sn <= b_sk;
  for (int64_t k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += 256) {
      const int mm = a_kfast ? e / BK : e % BM, kk = a_kfast ? e % BK : e / BM;
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < K) ? to_f32<TI>(A[m * a_sm + k * a_sk]) : 0.f;
    }
    for (int e = tid; e < BN * BK; e += 256) {
      const int nn = b_nfast ? e % BN : e / BK, kk = b_nfast ? e / BN : e % BK;
      const int64_t n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < N && k < K) ? to_f32<TI>(B[k * b_sk + n * b_sn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < N) C[m * N + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

template <typename TI>
int gemm_simt_out(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c,
                  int64_t M, int64_t N, int64_t K, int out_dtype, cudaStream_t st) {
  dim3 grid((unsigned)cdiv(N, 64), (unsigned)cdiv(M, 64));
  switch (out_dtype) {
    case Q3_F32: gemm_simt_kernel<TI, float><<<grid, 256, 0, st>>>((const TI*)a, a_sm, a_sk, (const TI*)b, b_sk, b_sn, (float*)c, M, N, K); break;
    case Q3_BF16: gemm_simt_kernel<TI, __nv_bfloat16><<<grid, 256, 0, st>>>((const TI*)a, a_sm, a_sk, (const TI*)b, b_sk, b_sn, (__nv_bfloat16*)c, M, N, K); break;
    case Q3_F16: gemm_simt_kernel<TI, __half><<<grid, 256, 0, st>>>((const TI*)a, a_sm, a_sk, (const TI*)b, b_sk, b_sn, (__half*)c, M, N, K); break;
    default: return Q3_ERR_DTYPE;
  }
  return launch_status();
}

int gemm_simt(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c,
              int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, cudaStream_t st) {
  if (cdiv(M, 64) > 65535) return Q3_ERR_SHAPE;
  switch (in_dtype) {
    case Q3_F32: return gemm_simt_out<float>(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, out_dtype, st);
    case Q3_BF16: return gemm_simt_out<__nv_bfloat16>(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, out_dtype, st);
    case Q3_F16: return gemm_simt_out<__half>(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, out_dtype, st);
    default: return Q3_ERR_DTYPE;
  }
}

}  // namespace q3
