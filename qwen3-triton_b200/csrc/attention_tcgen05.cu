// Tensor-core (tcgen05) causal GQA attention for head_dim 128 - placeholder until the kernels land.
#include "tcgen05.cuh"

namespace q3 {
bool attn_tc_available() { return false; }
int attn_fwd_tc(const void*, const void*, const void*, void*, float*, int64_t, int64_t, int64_t, int64_t, float, int,
                int*, cudaStream_t) { return Q3_ERR_SHAPE; }
int attn_bwd_tc(const void*, const void*, const void*, const void*, const float*, const float*, void*, void*, void*,
                int64_t, int64_t, int64_t, int64_t, float, int, int*, cudaStream_t) { return Q3_ERR_SHAPE; }
}  // namespace q3
