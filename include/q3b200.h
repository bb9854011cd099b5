/* q3b200 — C ABI of the B200 (sm_100a) training-kernel library behind the qwen3_triton operator API.
 *
 * The reference project (wuyii8941/qwen3-triton) has no FFI: its operators are Python
 * torch.autograd.Function classes that launch Triton kernels. This header is the boundary a
 * binding would target instead: one extern "C" entry per kernel family and direction, taking raw
 * device pointers, int64 sizes, a stream and (where the device can detect a violation) a device
 * status word. Each declaration cites the reference function it stands in for (paths are relative
 * to the reference repository).
 *
 * Common rules
 *   - all pointers are device pointers unless a parameter is documented as host memory;
 *   - tensors are contiguous unless strides are passed explicitly;
 *   - return 0 (Q3_OK) on success; a negative Q3_ERR_* value means the call was rejected on the
 *     host and nothing was launched; values <= Q3_ERR_CUDA encode (Q3_ERR_CUDA - cudaError_t);
 *   - kernels run on `stream`; the library keeps no mutable global state except per-device caches;
 *   - `status` (may be NULL) is an int32 device word; kernels OR Q3_STATUS_* bits into it and never
 *     trap. The caller clears and reads it.
 *   - outputs are fully overwritten; workspaces are caller-allocated, sized by the *_workspace_bytes
 *     query of the same family, and need no initialisation.
 */
#ifndef Q3B200_H_
#define Q3B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* q3_stream_t;

/* element types */
enum { Q3_F32 = 0, Q3_BF16 = 1, Q3_F16 = 2 };

/* return codes */
enum {
  Q3_OK = 0,
  Q3_ERR_ARG = -1,       /* null pointer or non-positive size */
  Q3_ERR_SHAPE = -2,     /* unsupported shape */
  Q3_ERR_DTYPE = -3,     /* unsupported element type */
  Q3_ERR_WORKSPACE = -4, /* workspace missing or too small */
  Q3_ERR_ALIGN = -5,     /* pointer or stride alignment not supported by any path */
  Q3_ERR_DRIVER = -6,    /* a required driver entry point is unavailable */
  Q3_ERR_TMAP = -7,      /* the driver rejected a TMA tensor-map description */
  Q3_ERR_LIMIT = -8,     /* size beyond the fixed capacity of a no-allocation entry point */
  Q3_ERR_CUDA = -1000    /* Q3_ERR_CUDA - cudaError_t */
};

/* device status bits */
enum {
  Q3_STATUS_ID_RANGE = 1,    /* embedding id outside [0, V) */
  Q3_STATUS_LABEL_RANGE = 2, /* label outside [0, V) and not ignore_index */
  Q3_STATUS_WAIT_TIMEOUT = 4,/* a bounded barrier wait inside a kernel gave up */
  Q3_STATUS_EMPTY_TARGETS = 8/* cross-entropy saw no valid target */
};

int q3_abi_version(void);
const char* q3_error_string(int code);
int q3_device_sm_count(void);

/* Device status word of the entry points that take no `status` argument (RMSNorm and norm+RoPE, whose wide-row
 * kernels wait on bulk-copy barriers with a time limit): synchronising read of the Q3_STATUS_* bits flagged on the
 * current device since the last clear. No counterpart in the reference. */
int q3_async_status(int clear, int* value);

/* ---- elementwise --------------------------------------------------------------------------- */

/* out = a + b in fp32, rounded once. Reference: qwen3_triton/kernels/residual.py:7-11,29-30. */
int q3_residual_add(const void* a, const void* b, void* out, int64_t n, int dtype, q3_stream_t stream);

/* y = cast(x). Reference: qwen3_triton/kernels/attention.py:10-18 (cast_tensor). */
int q3_cast(const void* x, int src_dtype, void* y, int dst_dtype, int64_t n, q3_stream_t stream);

/* y = silu(gate) * up. Reference: qwen3_triton/kernels/activation.py:7-11,
 * kernels/math_precision.py:67-71, ops/triton/silu_and_mul.py:111-121; math of ops/reference/swiglu.py:9-21. */
int q3_swiglu_fwd(const void* gate, const void* up, void* y, int64_t n, int dtype, q3_stream_t stream);

/* dgate = dy*up*s*(1+gate*(1-s)), dup = dy*gate*s, s = sigmoid(gate).
 * Reference: qwen3_triton/kernels/activation.py:14-20, kernels/math_precision.py:73-81. */
int q3_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, int64_t n, int dtype,
                  q3_stream_t stream);

/* pos[i] = i % seq (int64). Reference: qwen3_triton/_model.py:30-32 (_positions). */
int q3_positions(int64_t* pos, int64_t n, int64_t seq, q3_stream_t stream);

/* ---- RMSNorm ------------------------------------------------------------------------------- */

/* y = x * rsqrt(mean(x^2) + eps) * weight over rows of H (H <= 8192); inv_rms[rows] fp32 is saved.
 * Reference: qwen3_triton/kernels/norm.py:7-13,39-66; math_precision.py:16-37; ops/triton/rms_norm.py:136-138. */
int q3_rmsnorm_fwd(const void* x, const void* weight, void* y, float* inv_rms, int64_t rows, int64_t H, double eps,
                   int dtype, q3_stream_t stream);

int64_t q3_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t H);

/* dx and a deterministic dweight (per-CTA partial rows in the workspace, summed in fixed order).
 * Reference: qwen3_triton/kernels/norm.py:16-37,53-63. */
int q3_rmsnorm_bwd(const void* x, const void* weight, const void* dy, const float* inv_rms, void* dx, void* dweight,
                   void* workspace, int64_t workspace_bytes, int64_t rows, int64_t H, int dtype, q3_stream_t stream);

/* q3_rmsnorm_bwd for callers that cannot allocate device memory when they need it (inside an allocator or
 * memory-pool callback, in a host that fixes its whole HBM plan up front, in a latency-critical loop that must
 * not risk cudaMalloc/cudaFree): the partial-row scratch is a fixed 16 MiB device array inside the library
 * instead of a caller workspace, and the call allocates nothing. Limit: H <= 4096 (Q3_ERR_LIMIT beyond that).
 * The first call on each device resolves the array's device address and may make the driver load the module
 * that holds the array: make that call during set-up, before the region in which nothing may be allocated
 * and before starting any stream capture. All calls on a device share the array, so calls that overlap on the GPU (different streams)
 * race: serialise them. Same results as q3_rmsnorm_bwd.
 * This entry point has no counterpart in the reference. */
int q3_rmsnorm_bwd_noalloc(const void* x, const void* weight, const void* dy, const float* inv_rms, void* dx,
                           void* dweight, int64_t rows, int64_t H, int dtype, q3_stream_t stream);

/* residual_out = x + residual (rounded to dtype); y = RMSNorm(residual_out) * weight.
 * Fuses reference qwen3_triton/kernels/residual.py:7-11 with kernels/norm.py:7-13 (one pass over HBM). */
int q3_add_rmsnorm_fwd(const void* x, const void* residual, const void* weight, void* y, void* residual_out,
                       float* inv_rms, int64_t rows, int64_t H, double eps, int dtype, q3_stream_t stream);

/* dx = RMSNorm-backward(dy) on residual_out [+ dresidual if not NULL]; the result is the gradient of both
 * x and residual. Fuses reference kernels/norm.py:16-37 with the residual fan-in of residual.py:26-27. */
int q3_add_rmsnorm_bwd(const void* residual_out, const void* weight, const void* dy, const void* dresidual,
                       const float* inv_rms, void* dx, void* dweight, void* workspace, int64_t workspace_bytes,
                       int64_t rows, int64_t H, int dtype, q3_stream_t stream);

/* ---- per-head RMSNorm + RoPE, RoPE ---------------------------------------------------------- */

/* x [tokens, heads, D] -> y = rope(RMSNorm_D(x) * weight); cos/sin [tokens, D] in `dtype`.
 * Split-half rotation: y1 = n1*cos1 - n2*sin1, y2 = n2*cos2 + n1*sin2.
 * Reference: qwen3_triton/kernels/norm_rope.py:12-27,52-71; math_precision.py:40-64;
 * ops/triton/fused_qk_norm_rope.py:263-273; math of ops/reference/fused_qk_norm_rope.py:9-33. */
int q3_norm_rope_fwd(const void* x, const void* weight, const void* cos_t, const void* sin_t, void* y,
                     float* inv_rms, int64_t tokens, int64_t heads, int64_t D, double eps, int dtype,
                     q3_stream_t stream);

int64_t q3_norm_rope_bwd_workspace_bytes(int64_t tokens, int64_t heads, int64_t D);

/* Reference: qwen3_triton/kernels/norm_rope.py:30-50,63-69; ops/reference/fused_qk_norm_rope.py:36-80. */
int q3_norm_rope_bwd(const void* x, const void* weight, const void* cos_t, const void* sin_t, const void* dy,
                     const float* inv_rms, void* dx, void* dweight, void* workspace, int64_t workspace_bytes,
                     int64_t tokens, int64_t heads, int64_t D, int dtype, q3_stream_t stream);

/* q [tokens, hq, D] and k [tokens, hk, D] of one layer through per-head RMSNorm + RoPE in ONE launch (one grid shared
 * out between the two tensors by size); same arithmetic as two q3_norm_rope_* calls, which is also the fallback where
 * the wide-row kernels do not apply. workspace: q3_qk_norm_rope_bwd_workspace_bytes.
 * Reference: ops/triton/fused_qk_norm_rope.py (`_FusedQKNormRoPEFunction`, one kernel for q and k) and the pair of
 * `_norm_rope_forward` / `_norm_rope_backward` launches of qwen3_triton/kernels/norm_rope.py. */
int q3_qk_norm_rope_fwd(const void* q, const void* k, const void* q_weight, const void* k_weight, const void* cos_t,
                        const void* sin_t, void* yq, void* yk, float* inv_q, float* inv_k, int64_t tokens, int64_t hq,
                        int64_t hk, int64_t D, double eps, int dtype, q3_stream_t stream);
int64_t q3_qk_norm_rope_bwd_workspace_bytes(int64_t tokens, int64_t hq, int64_t hk, int64_t D);
int q3_qk_norm_rope_bwd(const void* q, const void* k, const void* q_weight, const void* k_weight, const void* cos_t,
                        const void* sin_t, const void* dyq, const void* dyk, const float* inv_q, const float* inv_k,
                        void* dq, void* dk, void* dq_weight, void* dk_weight, void* workspace, int64_t workspace_bytes,
                        int64_t tokens, int64_t hq, int64_t hk, int64_t D, int dtype, q3_stream_t stream);

/* RoPE (backward != 0: its transpose). layout 0: x [batch, seq, heads, D]; layout 1: x [batch, heads, seq, D];
 * cos/sin [batch, seq, D]. Reference: qwen3_triton/kernels/rotary.py:20-34,47-66; ops/triton/rope.py:164-170;
 * ops/reference/rope.py:13-55. */
int q3_rope_apply(const void* x, const void* cos_t, const void* sin_t, void* y, int64_t batch, int64_t seq,
                  int64_t heads, int64_t D, int backward, int layout, int dtype, q3_stream_t stream);

/* cos/sin [tokens, D] = cos/sin(float(pos) * inv_freq[i % (D/2)]); positions int32 or int64.
 * Reference: qwen3_triton/kernels/rotary.py:12-17,36-45. */
int q3_rope_tables(const void* positions, int positions_are_int64, const float* inv_freq, void* cos_t, void* sin_t,
                   int64_t tokens, int64_t D, int dtype, q3_stream_t stream);

/* ---- embedding ------------------------------------------------------------------------------ */

/* y[t, :] = weight[ids[t], :]; ids int32 or int64; an id outside [0, vocab) yields a zero row and sets
 * Q3_STATUS_ID_RANGE. Reference: qwen3_triton/kernels/embedding.py:13-20,49-66. */
int q3_embedding_fwd(const void* ids, int ids_are_int64, const void* weight, void* y, int64_t tokens, int64_t H,
                     int64_t vocab, int dtype, int* status, q3_stream_t stream);

/* Dense dweight [vocab, H]: zero-filled, then one writer per token id sums its dy rows in position order
 * (deterministic, no float atomics). workspace: q3_embedding_bwd_workspace_bytes(tokens) bytes (two int32 per
 * position: next position with the same id, "has a predecessor").
 * Reference: qwen3_triton/kernels/embedding.py:24-46,68-77. */
int64_t q3_embedding_bwd_workspace_bytes(int64_t tokens);
int q3_embedding_bwd(const void* ids, int ids_are_int64, const void* dy, void* dweight, void* workspace,
                     int64_t workspace_bytes, int64_t tokens, int64_t H, int64_t vocab, int dtype, q3_stream_t stream);

/* One contiguous shard of the table, rows [row_lo, row_lo + rows), stored in w_dtype (fp32 master or the compute type):
 * y[t, :] (y_dtype) = the row of ids[t] if this shard owns it, else zeros, so that the sum over shards is the full
 * lookup; H % 8 == 0. An id outside [0, vocab) sets Q3_STATUS_ID_RANGE. The backward form writes the shard's fp32
 * gradient scale * sum of dy rows over owned positions, zero elsewhere, deterministically.
 * No counterpart in the reference (its embedding is sharded by FSDP and gathered whole). */
int q3_embedding_shard_fwd(const void* ids, int ids_are_int64, const void* weight_shard, int w_dtype, void* y, int y_dtype,
                           int64_t tokens, int64_t H, int64_t vocab, int64_t row_lo, int64_t rows, int* status,
                           q3_stream_t stream);
int q3_embedding_shard_bwd(const void* ids, int ids_are_int64, const void* dy, int dtype, float* dweight_shard,
                           void* workspace, int64_t workspace_bytes, int64_t tokens, int64_t H, int64_t row_lo,
                           int64_t rows, double scale, q3_stream_t stream);

/* ---- cross-entropy over materialised logits ------------------------------------------------- */

/* Causal (internally shifted) token-mean CE: row (b,s), s < S-1, is scored against labels[b,s+1].
 * logits [B,S,V] in `dtype`, labels [B,S] int64. Outputs: lse/target/losses [B*(S-1)] fp32, loss fp32 scalar,
 * count int32 scalar. Reference: qwen3_triton/kernels/loss.py:7-32,46-62. */
int q3_ce_fwd(const void* logits, const int64_t* labels, float* lse, float* target, float* losses, float* loss,
              int* count, int64_t B, int64_t S, int64_t V, int64_t ignore_index, int dtype, int* status,
              q3_stream_t stream);

/* Vocabulary-slice statistics: lse over V_local columns per shifted row and the target logit when the slice
 * [vocab_start, vocab_start+V_local) owns the label (else 0). logits [physical_rows, V_local].
 * Reference: qwen3_triton/kernels/loss.py:7-13 + kernels/vocab_ce.py:15-22,78-87 (local_statistics). */
int q3_ce_local_rows(const void* logits, const int64_t* labels, float* lse_local, float* target,
                     int64_t physical_rows, int64_t S, int64_t V_local, int64_t vocab_start, int64_t vocab_total,
                     int64_t ignore_index, int dtype, int* status, q3_stream_t stream);

/* dlogits = (softmax - onehot) * upstream[source] / counts[source] on scored rows, 0 elsewhere;
 * source = physical_row / rows_per_rank (single GPU: rows_per_rank = physical_rows, one count, one upstream).
 * Reference: qwen3_triton/kernels/loss.py:35-44,64-68 and kernels/vocab_ce.py:57-67,107-112 (logit_gradient). */
int q3_ce_grad(const void* logits, const int64_t* labels, const float* lse, const int* counts, const float* upstream,
               void* dlogits, int64_t physical_rows, int64_t rows_per_rank, int64_t S, int64_t V_local,
               int64_t vocab_start, int64_t vocab_total, int64_t ignore_index, int dtype, q3_stream_t stream);

/* pack[0,:] = exp(lse_local - maximum), pack[1,:] = target. Reference: kernels/vocab_ce.py:26-30,88-91. */
int q3_vce_pack(const float* lse_local, const float* maximum, const float* target, float* pack, int64_t n,
                q3_stream_t stream);

/* lse = maximum + log(pack[0]); losses; per-data-rank counts and means.
 * Reference: kernels/vocab_ce.py:34-53,92-106 (finish_statistics). */
int q3_vce_finish(const float* maximum, const float* pack, const int64_t* labels, float* lse, float* losses,
                  int* counts, float* means, int64_t n, int64_t rows_per_rank, int64_t S, int64_t world,
                  int64_t ignore_index, int* status, q3_stream_t stream);

/* out = (first ? 0 : out) + partial / world, fp32. Reference: kernels/vocab_ce.py:71-75,113-114. */
int q3_vce_accumulate(const void* partial, int partial_dtype, float* out, int64_t n, int64_t world, int first,
                      q3_stream_t stream);

/* ---- AdamW ---------------------------------------------------------------------------------- */

/* Multi-tensor AdamW over fp32 tensors. meta: device int64 [n_tensors][7] =
 * {param, grad, exp_avg, exp_avg_sq, step (fp32 scalar) device addresses, numel, first_block};
 * coeff: device fp32 [n_tensors][3] scratch; total_blocks = sum ceil(numel / block_elems).
 * Increments each step scalar, then updates p, m, v in place.
 * Reference: qwen3_triton/runtime/adamw.py:20-61,118-159. */
int q3_adamw_multi(const int64_t* meta, float* coeff, int64_t n_tensors, int64_t total_blocks, int block_elems,
                   double lr, double beta1, double beta2, double weight_decay, double eps, q3_stream_t stream);

/* Mixed-precision form of q3_adamw_multi for a single-GPU fp32-master / bf16-working setup: table int64 [n][9] =
 * {param fp32, grad fp32 or 0, exp_avg, exp_avg_sq, step, numel, first_block, grad lowp or 0, working-copy lowp or 0}.
 * When the low-precision gradient pointer is set it is read directly (no fp32 staging copy); when the working-copy
 * pointer is set the updated parameter is also written there in `lowp_dtype` (bf16/fp16). Same update math.
 * all_rows_lowp = 1 promises that every row has both low-precision pointers (selects a leaner kernel).
 * Fuses the reference's cast passes (qwen3_triton/runtime/ops.py:53-58,193-202) into runtime/adamw.py:34-61. */
int q3_adamw_multi_mp(const int64_t* meta, float* coeff, int64_t n_tensors, int64_t total_blocks, int block_elems,
                      int lowp_dtype, int all_rows_lowp, double lr, double beta1, double beta2, double weight_decay,
                      double eps, q3_stream_t stream);

/* ---- FSDP pack / unpack -------------------------------------------------------------------------------------- */

/* One launch copies (and converts) every 2-D piece listed in a device table int64 [n][8] =
 * {src, dst, rows, cols, src_row_stride, dst_row_stride, src_valid, vec_ok}: dst[r*dst_row_stride + c] =
 * convert(src[r*src_row_stride + c]) or 0 where the source index is >= src_valid (padding of the last chunk).
 * vec_ok = 1 when cols and both strides are multiples of 8 and both bases are 16-byte aligned. total_elements
 * (sum of rows*cols) only sizes the grid. Covers FSDP2's all_gather_copy_in (fp32 shard -> bf16),
 * split_with_sizes_copy and chunk_cat (bf16 grads -> fp32 reduce-scatter rows).
 * Reference: qwen3_triton/runtime/ops.py:70-93,116-127,186-202 behind runtime/dispatch.py:105-119. */
int q3_multi_copy(const int64_t* meta, int64_t n_entries, int64_t total_elements, int src_dtype, int dst_dtype,
                  q3_stream_t stream);

/* ---- GEMM ----------------------------------------------------------------------------------- */

/* C[M,N] (contiguous, out_dtype) = A * B with A(m,k) at a[m*a_sm + k*a_sk] and B(k,n) at b[k*b_sk + n*b_sn],
 * fp32 accumulation. bf16/fp16 operands whose unit-stride dimension and 16-byte alignment allow TMA run on the
 * tcgen05 tensor cores (forward X*W^T, input gradient dY*W and weight gradient dY^T*X all qualify without a
 * copy); everything else runs on CUDA cores. Reference: qwen3_triton/kernels/linear.py:14-77 (matmul). */
int q3_gemm(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c, int64_t M,
            int64_t N, int64_t K, int in_dtype, int out_dtype, int* status, q3_stream_t stream);

/* 1 if q3_gemm would use the tensor-core kernel for these arguments, else 0. */
int q3_gemm_path(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, const void* c,
                 int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype);

/* G = X*Wg^T, U = X*Wu^T (both rounded to dtype and stored), Y = silu(G)*U; X [M,K], Wg/Wu [N,K], outputs [M,N].
 * Reference: qwen3_triton/kernels/mlp_precision.py:17-52, kernels/mlp.py:14-45, ops/triton/gate_up_swiglu.py:274-288. */
int q3_gate_up_swiglu_fwd(const void* x, const void* w_gate, const void* w_up, void* gate, void* up, void* y,
                          int64_t M, int64_t N, int64_t K, int dtype, int* status, q3_stream_t stream);
int q3_gate_up_path(const void* x, const void* w_gate, const void* w_up, const void* gate, const void* up,
                    const void* y, int64_t M, int64_t N, int64_t K, int dtype);

/* C (fp32, contiguous) += A * B; operands as q3_gemm, tensor-core path only (Q3_ERR_ALIGN otherwise). Used to
 * accumulate the hidden-state gradient of the vocabulary head over vocabulary chunks in fp32, as the reference keeps
 * partial_dx in fp32 (qwen3_triton/training/vocab_parallel.py:76). */
int q3_gemm_acc_f32(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, float* c,
                    int64_t M, int64_t N, int64_t K, int in_dtype, int* status, q3_stream_t stream);

/* C += A * B with C contiguous [M,N] in out_dtype (fp32, or the input type: read, add in fp32, round once). Same
 * operand rules as q3_gemm, tensor-core path only (Q3_ERR_ALIGN otherwise). Used to sum the input gradients of
 * projections that share an input (q/k/v, gate/up) without add kernels; the reference does those sums with its
 * `_add` kernel (qwen3_triton/kernels/residual.py:13-27) after separate `_gemm` launches. */
int q3_gemm_acc(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c,
                int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, int* status, q3_stream_t stream);

/* Linear layers that share their input (q/k/v, gate/up), `count` = 2 or 3 weights W_i [N_i, K], row-major contiguous
 * 16-bit tensors, one persistent launch each instead of `count` GEMMs (+ adds):
 *   fwd   y_i [M, N_i] = x [M, K] * W_i^T
 *   dgrad dx [M, K]    = sum_i dy_i [M, N_i] * W_i          (every N_i a multiple of 64)
 *   wgrad dW_i [N_i,K] = dy_i^T * x
 * `weights`, `ys`, `dys`, `dws` and `n` are HOST arrays of `count` device pointers / sizes, read at launch.
 * Reference: the same `_gemm` launches of qwen3_triton/kernels/linear.py:45-77, one per projection, and `_add`. */
int q3_linear_fwd_grouped(const void* x, const void* const* weights, void* const* ys, const int64_t* n, int count,
                          int64_t M, int64_t K, int dtype, int* status, q3_stream_t stream);
int q3_linear_dgrad_grouped(const void* const* dys, const void* const* weights, void* dx, const int64_t* n, int count,
                            int64_t M, int64_t K, int dtype, int* status, q3_stream_t stream);
int q3_linear_wgrad_grouped(const void* const* dys, const void* x, void* const* dws, const int64_t* n, int count,
                            int64_t M, int64_t K, int dtype, int* status, q3_stream_t stream);

/* Input gradient of down_proj fused with the SwiGLU backward: dY = dM [M,H] * W_down [H,I] is formed tile by tile in
 * tensor memory and turned into dG, dU (from the saved G, U [M,I]) in the epilogue; dY itself is never written.
 * Bit-identical to q3_gemm (dgrad) followed by q3_swiglu_bwd. Reference: `_gemm` (kernels/linear.py:45-77) then
 * `_backward` (kernels/activation.py:22-34). */
int q3_down_dgrad_swiglu_bwd(const void* dm, const void* w_down, const void* gate, const void* up, void* dgate, void* dup,
                             int64_t M, int64_t I, int64_t H, int dtype, int* status, q3_stream_t stream);

/* ---- fused lm_head + cross-entropy (no logits in memory) ---------------------------------------------------
 * The reference materialises the logits [W*r, V/W] and their gradient (qwen3_triton/training/vocab_parallel.py:52,75;
 * kernels/vocab_ce.py:78-112). Here the projection runs on the tensor cores and the softmax statistics / gradient are
 * computed in the GEMM epilogue from tensor memory:
 *   q3_shift_labels      labels_eff[b*S+s] = labels[b,s+1] (s < S-1) else ignore_index   (the shift of kernels/loss.py:9,20)
 *   q3_linear_ce_stats   per (row, 256-column tile): max and sum-exp of the logits rounded to `dtype`; target logit
 *                        where the vocabulary slice [vocab_start, vocab_start+V_local) owns the label
 *   q3_linear_ce_combine lse_local[row] from the tile partials (tiles = q3_linear_ce_tiles(V_local))
 *   q3_linear_ce_finish  optional lse = maximum + log(pack[0]) after the two all-reduces, then per data rank
 *                        losses / counts / means (kernels/vocab_ce.py:34-53 on physical rows)
 *   q3_linear_ce_grad    dZ [M, Vc] of one vocabulary chunk, recomputing that chunk of the logits */
int64_t q3_linear_ce_tiles(int64_t V_local);
int q3_shift_labels(const int64_t* labels, int64_t* labels_eff, int64_t rows, int64_t S, int64_t ignore_index,
                    int64_t vocab_total, int* status, q3_stream_t stream);
int q3_linear_ce_stats(const void* hidden, const void* weight, const int64_t* labels_eff, float* part_max,
                       float* part_sum, float* target, int64_t M, int64_t V_local, int64_t K, int64_t vocab_start,
                       int64_t ignore_index, int dtype, int* status, q3_stream_t stream);
int q3_linear_ce_combine(const float* part_max, const float* part_sum, float* lse_local, int64_t rows, int64_t tiles,
                         q3_stream_t stream);
int q3_linear_ce_finish(const float* maximum, const float* pack, float* lse, const float* target,
                        const int64_t* labels_eff, float* losses, int* counts, float* means, int64_t rows,
                        int64_t rows_per_rank, int64_t ignore_index, int* status, q3_stream_t stream);
int q3_linear_ce_grad(const void* hidden, const void* weight_chunk, const int64_t* labels_eff, const float* lse,
                      const float* upstream, const int* counts, void* dz, int64_t M, int64_t Vc, int64_t K,
                      int64_t vocab_start, int64_t rows_per_rank, int64_t ignore_index, int dtype, int* status,
                      q3_stream_t stream);

/* ---- attention ------------------------------------------------------------------------------ */

/* Causal grouped-query attention. q/out [B,Hq,S,D], k/v [B,Hkv,S,D] contiguous, kv head = q head / (Hq/Hkv);
 * lse [B,Hq,S] fp32 (natural log). D even, <= 256.
 * Reference: qwen3_triton/kernels/attention.py:20-36,49-50; kernels/attention_precision.py:147-158,181-182;
 * ops/triton/attention.py:136-199; math of ops/reference/attention.py:10-54. */
int q3_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t Hq,
                int64_t Hkv, int64_t S, int64_t D, double scale, int dtype, int* status, q3_stream_t stream);

int64_t q3_attn_bwd_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D);

/* dq, dk, dv (dk/dv already summed over the query heads of each group; deterministic).
 * Reference: qwen3_triton/kernels/attention.py:37-47; kernels/attention_precision.py:159-179;
 * ops/triton/attention_backward.py:196-236; math of ops/reference/attention.py:57-124. */
int q3_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                void* dq, void* dk, void* dv, void* workspace, int64_t workspace_bytes, int64_t B, int64_t Hq,
                int64_t Hkv, int64_t S, int64_t D, double scale, int dtype, int* status, q3_stream_t stream);

/* Token-major variants of the two calls above: q/out/dout/dq [B,S,Hq,128], k/v/dk/dv [B,S,Hkv,128] - what the
 * q/k/v projections write and the output projection reads - so no transpose copies surround attention
 * (the reference makes four per layer and direction: qwen3_triton/components.py:29,31). Tensor-core path only:
 * Q3_ERR_SHAPE unless q3_attn_path() is 1. lse stays [B,Hq,S]. */
int q3_attn_fwd_bshd(const void* q, const void* k, const void* v, void* out, float* lse, int64_t B, int64_t S,
                     int64_t Hq, int64_t Hkv, int64_t D, double scale, int dtype, int* status, q3_stream_t stream);
int q3_attn_bwd_bshd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                     void* dq, void* dk, void* dv, void* workspace, int64_t workspace_bytes, int64_t B, int64_t S,
                     int64_t Hq, int64_t Hkv, int64_t D, double scale, int dtype, int* status, q3_stream_t stream);

/* 1 if the tensor-core attention kernels run for these arguments, else 0. */
int q3_attn_path(const void* q, const void* k, const void* v, const void* out, int64_t D, int dtype);

/* The dK/dV pass of q3_attn_bwd at head_dim 128 has two schedules: one CTA per key tile that accumulates the gradients
 * of the whole query-head group in tensor memory (returns 1), or, on grids too small to fill the GPU, one CTA per
 * query head followed by a fixed-order reduction (returns G = Hq/Hkv; the reference always does the latter:
 * qwen3_triton/kernels/attention_precision.py:84-143). q3_attn_bwd_group_split tells which one runs for a shape;
 * q3_attn_bwd_group_policy(0 | 1 | 2) selects by grid size (default) / always the first / always the second,
 * process-wide, and returns the previous setting (any other argument only queries). Both give the same result
 * up to fp32 summation order; the workspace query follows the setting. */
int q3_attn_bwd_group_split(int64_t B, int64_t Hq, int64_t Hkv, int64_t S);
int q3_attn_bwd_group_policy(int policy);

/* How the persistent GEMM kernels (every q3_gemm* / q3_linear* / q3_gate_up* / q3_down_dgrad* entry) hand out their
 * 128-row output tiles: 1 (default) = each CTA draws its next tile from a device counter, 0 = CTA b takes tiles
 * b, b + grid, ... . Drawn tiles keep a launch short when some SMs are held by a kernel of another stream (a
 * collective during a data-parallel step): with the fixed stride the CTAs that start late still own a full share.
 * Returns the previous policy (any other argument only queries); process-wide; results are bit-identical.
 * The first GEMM call on a device allocates and zeroes the counters (32 KB): make it outside stream capture. */
int q3_gemm_tile_schedule(int mode);

/* Where an output has at least two 128-row tiles, the GEMM kernels run as pairs of CTAs (clusters of 2, tcgen05
 * cta_group::2): the pair shares one 256 x 256 tile, each CTA stages its own 128 rows of A and half of B's rows, the
 * MMAs read both CTAs' shared memory. A CTA then brings 32 KB per k-block into shared memory instead of 48 KB for the
 * same tensor work - the single-CTA form is limited by that traffic to about 80 % of the tensor rate. No multicast
 * loads are involved. 1 = pairs (default; tiles then go to the pairs with a fixed stride), 0 = single CTAs everywhere.
 * Returns the previous policy (any other argument only queries); process-wide; results are bit-identical. */
int q3_gemm_cta_pairs(int mode);

/* ---- token-block data path and validation statistics ---------------------------------------- */

/* out[i] = training ? ((first + i + offset) * stride + seed) mod n : first + i, for i in [0, count): the order in
 * which training visits the n blocks of a corpus (stride coprime to n gives a full-period permutation); exact 128-bit
 * integer arithmetic. Reference: training/data.py:26-27 (Blocks.__getitem__ index). */
int q3_block_order(int64_t* out, int64_t first, int64_t count, int64_t offset, int64_t stride, int64_t seed, int64_t n,
                   int training, q3_stream_t stream);

/* ids[b, s] = corpus[block[b] * seq + s] widened to int64, for a corpus of uint32 token ids resident on the device.
 * block [batch] int64 on the device; a block outside [0, corpus_tokens / seq) sets Q3_STATUS_ID_RANGE and yields zeros.
 * Reference: training/data.py:28 (the slice and astype(int64) of Blocks.__getitem__). */
int q3_token_blocks(const uint32_t* corpus, int64_t corpus_tokens, const int64_t* block, int64_t* ids, int64_t batch,
                    int64_t seq, int* status, q3_stream_t stream);

/* totals[0] += loss[0] * tokens; totals[1] += tokens, in fp64 with separate multiply and add (totals: 2 doubles on the
 * device; tokens == 0 launches nothing). Reference: qwen3_triton/runtime/metrics.py:8-17 (accumulate_validation). */
int q3_validation_accumulate(const float* loss, double* totals, int64_t tokens, q3_stream_t stream);

/* totals[0] += sum of losses[b, s] over the shifted rows (s < S-1) whose target labels[b, s+1] != ignore_index,
 * totals[1] += their number; fp64, fixed summation order. losses [B*(S-1)] as written by q3_ce_fwd, labels [B,S].
 * Reference: training/evaluation.py:20-26 (shifted_nll: summed NLL and scored-token count of a batch). */
int q3_validation_rows(const float* losses, const int64_t* labels, int64_t B, int64_t S, int64_t ignore_index,
                       double* totals, q3_stream_t stream);

/* ---- gradient reduce-scatter over peer memory ------------------------------------------------ */

/* A device buffer that other processes on the node can map (plain cudaMalloc + its 64-byte IPC handle), the mapping
 * of a peer's buffer from its handle, and their release. The staging buffers of q3_reduce_scatter_pull are made this
 * way once, at set-up; no counterpart in the reference's Python (its symmetric-memory experiments live in scripts/). */
int q3_peer_alloc(int64_t bytes, void** ptr, void* handle64);
int q3_peer_open(const void* handle64, void** ptr);
int q3_peer_close(void* ptr);
int q3_peer_free(void* ptr);

/* One asynchronous device-to-device copy on `stream` (either pointer may come from q3_peer_open): a copy-engine
 * transfer that occupies no SM. The parameter all-gather of runtime/peer_gather.py issues one per source rank, from
 * the peer's mapped all-gather buffer into this rank's. Reference: qwen3_triton/runtime/collectives.py:88-137. */
int q3_peer_copy(void* dst, const void* src, int64_t bytes, q3_stream_t stream);
/* `count` such copies issued in order on `stream`; dst, src, bytes are HOST arrays. Used to deliver every rank's shard
 * of every parameter of an FSDP unit straight into the parameter's tensor (no rank-major buffer to split afterwards). */
int q3_peer_copy_many(void* const* dst, const void* const* src, const int64_t* bytes, int64_t count,
                      q3_stream_t stream);

/* out[i] = scale * sum_r widen(peers[r][first + i]), i in [0, count): this rank's rows of every rank's 16-bit staging
 * buffer, pulled with plain peer loads, added in fp32 in rank order. `peers` is a HOST array of `world` (2, 4 or 8)
 * device pointers; first % 8 == 0. One kernel replaces the chunk-cat upcast and the fp32 ring reduce-scatter of a
 * gradient bucket; the result equals an fp32 reduce-scatter of the upcast values. Ordering across ranks (staging
 * complete before the pull, not overwritten before every rank has pulled) is the caller's job.
 * Reference: qwen3_triton/runtime/collectives.py:139-203 (reduce_scatter, lossless_bf16) + runtime/ops.py:193-202. */
int q3_reduce_scatter_pull(const void* const* peers, int world, float* out, int64_t first, int64_t count, double scale,
                           int dtype, q3_stream_t stream);

/* ---- decode-time kernels -------------------------------------------------------------------- */

/* pos[b, s] = start + s (int64 [batch, seq]). Reference: qwen3_triton/inference/kernels.py:12-22 (positions). */
int q3_inf_positions(int64_t* pos, int64_t batch, int64_t seq, int64_t start, q3_stream_t stream);

/* Append the new keys / values k, v [B,S,H,D] (token-major) to the caches [B,H,C,D] at tokens start .. start+S-1.
 * D * element size must be a multiple of 16 bytes. Reference: inference/kernels.py:25-36 (append). */
int q3_kv_append(const void* k, const void* v, void* cache_k, void* cache_v, int64_t B, int64_t S, int64_t H, int64_t D,
                 int64_t C, int64_t start, int dtype, q3_stream_t stream);

/* Causal attention of S new query tokens q [B,S,Hq,D] over the cached keys / values [B,Hkv,C,D], which already hold
 * tokens 0 .. start+S-1: query s sees keys t <= start + s. out [B,S,Hq,D]. D in {64,128,256}; Hq/Hkv in {1,2,4,8}.
 * One pass over each chunk of the cache (32 KB of keys: 128 at head_dim 128 in bf16) serves all query heads of a kv
 * head; chunks are merged by their log-sum-exp (fp32 partials in the workspace). Reference: inference/kernels.py:39-115 (cached attention and the
 * split decode path, which this replaces for every S). */
int64_t q3_cache_attention_workspace_bytes(int64_t B, int64_t S, int64_t Hq, int64_t D, int64_t start, int dtype);
/* 16-bit caches at head_dim 128 run the chunk products on the tensor cores (the G query heads of a group are rows of
 * one MMA tile); everything else, or everything after q3_cache_attention_path(1), runs the CUDA-core kernel. The
 * switch is process-wide, returns the previous setting, and only queries for arguments other than 0 / 1. */
int q3_cache_attention_path(int path);
int q3_cache_attention(const void* q, const void* cache_k, const void* cache_v, void* out, void* workspace,
                       int64_t workspace_bytes, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t D, int64_t C,
                       int64_t start, double scale, int dtype, q3_stream_t stream);

/* y [M,N] = x [M,K] * weight[N,K]^T for M <= 8 (decode): the weight matrix is streamed once. fp32 accumulation, or
 * fp64 with accurate != 0. K * element size must be a multiple of 16 bytes.
 * Reference: inference/kernels.py:117-148 (_inference_gemv behind linear(gemv=True)). */
int q3_gemv(const void* x, const void* weight, void* y, int64_t M, int64_t N, int64_t K, int dtype, int accurate,
            q3_stream_t stream);

/* Greedy decode step over logits [B,V]: token = argmax (lowest index among equal maxima), or `pad` for a row that is
 * already done; ids[row, position] = next_token[row] = token; done[row] |= token in eos_ids (n_eos int64 on the
 * device). done is one byte per row; the workspace (8-byte aligned) holds the per-slice maxima of the first stage.
 * Reference: inference/kernels.py:150-173 (argmax parts + select). */
int64_t q3_select_tokens_workspace_bytes(int64_t B, int64_t V);
int q3_select_tokens(const void* logits, int64_t B, int64_t V, int64_t* ids, int64_t ids_stride, int64_t position,
                     int64_t* next_token, uint8_t* done, const int64_t* eos_ids, int n_eos, int64_t pad, void* workspace,
                     int64_t workspace_bytes, int dtype, q3_stream_t stream);

/* ---- self-test ------------------------------------------------------------------------------ */

/* Makes a bounded wait run out on purpose, the harmless way: one CTA waits on a barrier nothing arrives at, with a
 * limit of limit_ns (1 us .. 100 ms). The kernel must come back by itself with Q3_STATUS_WAIT_TIMEOUT OR-ed into
 * *status and outcome[0] = outcome[1] = 0 (both warps gave up: the first by its time limit, the second through the
 * CTA-wide abort flag). The same mbar_wait guards every barrier in the tensor-core and bulk-copy kernels. Stands in
 * for the reference's timed-out barrier check, scripts/check_triton_collectives_v14.py:127-133. */
int q3_selftest_wait_timeout(int64_t limit_ns, int* status, int* outcome, q3_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* Q3B200_H_ */
