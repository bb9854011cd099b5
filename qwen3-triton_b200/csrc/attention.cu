// C-ABI entry points of causal grouped-query attention: argument checks and path selection between
// the tensor-core kernels (bf16/fp16, head_dim 128) and the general CUDA-core kernels.
//
// Stand in for reference qwen3_triton/kernels/attention.py:20-50 (_Attention / causal_attention),
// kernels/attention_precision.py:147-182 (_NativePrecision / candidate), ops/triton/attention.py:136-199
// and ops/triton/attention_backward.py:196-236.
#include "common.cuh"

namespace q3 {
int attn_fwd_simt(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t Hq,
                  int64_t Hkv, int64_t S, int64_t D, float scale, int dtype, cudaStream_t st);
int attn_delta(const void* out, const void* dout, float* delta, int64_t rows, int64_t D, int dtype, cudaStream_t st);
int attn_bwd_simt(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                  void* dq, void* dk, void* dv, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale,
                  int dtype, cudaStream_t st);
int attn_fwd_tc(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t Hq, int64_t Hkv,
                int64_t S, float scale, int dtype, int layout, int* status, cudaStream_t st);
int attn_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                void* dq, void* dk, void* dv, float* partials, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, float scale,
                int dtype, int layout, int* status, cudaStream_t st);
int attn_bwd_group_split(int64_t B, int64_t Hq, int64_t Hkv, int64_t S);
int attn_bwd_set_group_policy(int policy);
int attn_delta_layout(const void* out, const void* dout, float* delta, int64_t B, int64_t H, int64_t S, int64_t D,
                      int layout, int dtype, cudaStream_t st);
bool attn_tc_available();

static int check_shape(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D) {
  if (B < 1 || Hq < 1 || Hkv < 1 || S < 1 || D < 2 || D > 256 || (D & 1) || Hq % Hkv) return Q3_ERR_SHAPE;
  if (B * Hq > 65535) return Q3_ERR_SHAPE;
  return Q3_OK;
}
static bool tc_eligible(const void* q, const void* k, const void* v, const void* o, int64_t D, int dtype) {
  return attn_tc_available() && D == 128 && (dtype == Q3_BF16 || dtype == Q3_F16) && aligned16(q) && aligned16(k) &&
         aligned16(v) && aligned16(o);
}
}  // namespace q3

using namespace q3;

// 1 if the tensor-core attention kernels run for these arguments, 0 for the CUDA-core kernels.
extern "C" int q3_attn_path(const void* q, const void* k, const void* v, const void* out, int64_t D, int dtype) {
  return tc_eligible(q, k, v, out, D, dtype) ? 1 : 0;
}

extern "C" int q3_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t Hq,
                           int64_t Hkv, int64_t S, int64_t D, double scale, int dtype, int* status,
                           q3_stream_t stream) {
  if (!q || !k || !v || !out || !lse) return Q3_ERR_ARG;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != Q3_OK) return rc;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (tc_eligible(q, k, v, out, D, dtype)) return attn_fwd_tc(q, k, v, out, lse, B, Hq, Hkv, S, (float)scale, dtype, 0, status, st);
  return attn_fwd_simt(q, k, v, out, lse, B, Hq, Hkv, S, D, (float)scale, dtype, st);
}

// Which of the two dK/dV schedules q3_attn_bwd runs at head_dim 128 for this shape: 1 = one CTA per key tile sums the
// whole query-head group in tensor memory; G = Hq/Hkv = one CTA per query head and a fixed-order reduction.
extern "C" int q3_attn_bwd_group_split(int64_t B, int64_t Hq, int64_t Hkv, int64_t S) {
  if (B < 1 || Hq < 1 || Hkv < 1 || S < 1 || Hq % Hkv) return Q3_ERR_SHAPE;
  return attn_bwd_group_split(B, Hq, Hkv, S);
}

// Tuning / test switch for that choice (process-wide): 0 by grid size (default), 1 always group-accumulate, 2 always
// per-head split. Returns the previous value; other values only query. Change it only while no backward is in flight
// between its workspace query and its launch.
extern "C" int q3_attn_bwd_group_policy(int policy) { return attn_bwd_set_group_policy(policy); }

// delta = rowsum(dO * O) [B,Hq,S] fp32, then (small grids only) per-query-head fp32 partials of dK and dV
static int64_t delta_bytes(int64_t B, int64_t Hq, int64_t S) { return ((B * Hq * S * 4 + 255) / 256) * 256; }

extern "C" int64_t q3_attn_bwd_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D) {
  int64_t bytes = delta_bytes(B, Hq, S);
  if (D == 128 && Hkv > 0 && Hq % Hkv == 0) {
    const int split = attn_bwd_group_split(B, Hq, Hkv, S);
    if (split > 1) bytes += (int64_t)split * 2 * B * Hkv * S * 128 * 4;
  }
  return bytes;
}

extern "C" int q3_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                           const float* lse, void* dq, void* dk, void* dv, void* workspace, int64_t workspace_bytes,
                           int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D, double scale, int dtype,
                           int* status, q3_stream_t stream) {
  if (!q || !k || !v || !out || !dout || !lse || !dq || !dk || !dv) return Q3_ERR_ARG;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != Q3_OK) return rc;
  if (dtype < Q3_F32 || dtype > Q3_F16) return Q3_ERR_DTYPE;
  if (!workspace || workspace_bytes < q3_attn_bwd_workspace_bytes(B, Hq, Hkv, S, D)) return Q3_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  float* delta = (float*)workspace;
  rc = attn_delta(out, dout, delta, B * Hq * S, D, dtype, st);
  if (rc != Q3_OK) return rc;
  if (tc_eligible(q, k, v, dout, D, dtype) && aligned16(dq) && aligned16(dk) && aligned16(dv))
    return attn_bwd_tc(q, k, v, dout, lse, delta, dq, dk, dv, (float*)((char*)workspace + delta_bytes(B, Hq, S)), B, Hq, Hkv,
                       S, (float)scale, dtype, 0, status, st);
  return attn_bwd_simt(q, k, v, dout, lse, delta, dq, dk, dv, B, Hq, Hkv, S, D, (float)scale, dtype, st);
}

// Token-major variants: q/out/dout/dq are [B, S, Hq, 128] and k/v/dk/dv [B, S, Hkv, 128] - the layout the
// q/k/v projections produce and the output projection consumes - so a decoder layer needs no transpose
// copies around attention. Tensor-core path only (bf16/fp16, head_dim 128); lse stays [B, Hq, S].
extern "C" int q3_attn_fwd_bshd(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B,
                                int64_t S, int64_t Hq, int64_t Hkv, int64_t D, double scale, int dtype, int* status,
                                q3_stream_t stream) {
  if (!q || !k || !v || !out || !lse) return Q3_ERR_ARG;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != Q3_OK) return rc;
  if (!tc_eligible(q, k, v, out, D, dtype)) return Q3_ERR_SHAPE;
  return attn_fwd_tc(q, k, v, out, lse, B, Hq, Hkv, S, (float)scale, dtype, 1, status, (cudaStream_t)stream);
}

extern "C" int q3_attn_bwd_bshd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                const float* lse, void* dq, void* dk, void* dv, void* workspace,
                                int64_t workspace_bytes, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t D,
                                double scale, int dtype, int* status, q3_stream_t stream) {
  if (!q || !k || !v || !out || !dout || !lse || !dq || !dk || !dv) return Q3_ERR_ARG;
  int rc = check_shape(B, Hq, Hkv, S, D);
  if (rc != Q3_OK) return rc;
  if (!tc_eligible(q, k, v, dout, D, dtype) || !aligned16(dq) || !aligned16(dk) || !aligned16(dv)) return Q3_ERR_SHAPE;
  if (!workspace || workspace_bytes < q3_attn_bwd_workspace_bytes(B, Hq, Hkv, S, D)) return Q3_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  float* delta = (float*)workspace;
  rc = attn_delta_layout(out, dout, delta, B, Hq, S, D, 1, dtype, st);
  if (rc != Q3_OK) return rc;
  return attn_bwd_tc(q, k, v, dout, lse, delta, dq, dk, dv, (float*)((char*)workspace + delta_bytes(B, Hq, S)), B, Hq, Hkv, S,
                     (float)scale, dtype, 1, status, st);
}
