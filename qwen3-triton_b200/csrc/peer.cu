// Gradient reduce-scatter as one pull kernel over peer memory (NVLink / NVSwitch), for data-parallel ranks that run as
// one process per GPU on one node.
//
// FSDP2's gradient path is: bf16 gradients -> chunk-cat + upcast into an fp32 staging buffer (6 bytes per element of
// HBM traffic) -> NCCL ring reduce-scatter of the fp32 buffer (every hop reads, adds and writes 4-byte elements, and
// 4 bytes per element cross the links). The gradients are bf16 when they are produced, so nothing is lost by moving
// them as bf16 and widening at the point of accumulation: every rank packs its gradients, still bf16, into a staging
// buffer that its peers can read, and after a barrier each rank pulls ITS rows of every peer's staging buffer with
// plain 16-byte loads, adds them in fp32 in rank order (deterministic, the same sum an fp32 reduce-scatter of the
// upcast values forms) and writes its fp32 shard once. 2 bytes per element cross the links, and HBM sees one bf16
// write (pack), one bf16 read (pull, on the owner's side) and 4/W bytes of result per element.
//
// Only plain peer loads are used: no multicast objects, no TMA from peer memory, and no kernel here waits on a flag
// written by another GPU (ranks synchronise on the host side of the stream, through their collective library).
//
// Replaces, in the reference: the fp32 reduce-scatter behind qwen3_triton/runtime/fsdp.py:26-37 (TritonReduceScatter)
// and runtime/collectives.py:139-203 (reduce_scatter(..., lossless_bf16=...)), together with the chunk-cat upcast of
// runtime/ops.py:193-202.
#include "common.cuh"
#include <string.h>

namespace q3 {

constexpr int kMaxPeers = 16;
struct PeerTable { const void* base[kMaxPeers]; };

// out[i] = scale * sum_r widen(peer_r[first + i]) for i in [0, count): this rank's chunk of every peer's staging
// buffer. T = 16-bit type on the wire. Eight elements (16 bytes) per thread and peer, all peers' loads issued before
// the first add; ranks are added in index order.
template <typename T, int W>
__global__ void __launch_bounds__(256)
reduce_scatter_pull_kernel(const PeerTable peers, float* __restrict__ out, int64_t first, int64_t count, float scale) {
  const int64_t nvec = count / 8;
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    uint4 raw[W];
#pragma unroll
    for (int r = 0; r < W; ++r)
      raw[r] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(peers.base[r]) + first + v * 8));
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int r = 0; r < W; ++r) {
      const T* h = reinterpret_cast<const T*>(&raw[r]);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += to_f32<T>(h[e]);
    }
    // streaming stores as well as loads: a gigabyte-sized shard must not push the neighbouring GEMMs' operands out of L2
    float4* o = reinterpret_cast<float4*>(out + v * 8);
    __stcs(o, make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale));
    __stcs(o + 1, make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale));
  }
  // tail (count not a multiple of 8): the first threads of the grid, one element each
  const int64_t tail = nvec * 8 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (tail < count) {
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < W; ++r) acc += to_f32<T>(reinterpret_cast<const T*>(peers.base[r])[first + tail]);
    out[tail] = acc * scale;
  }
}

template <typename T>
int launch_pull(int world, const PeerTable& t, float* out, int64_t first, int64_t count, float scale, cudaStream_t st) {
  static const int forced = [] { const char* e = getenv("Q3_PULL_CTAS"); return e ? atoi(e) : 0; }();
  const int64_t want = cdiv(count / 8 + 1, 256), cap = forced > 0 ? forced : (int64_t)sm_count() * 4;   // measured on local buffers: 6.1 TB/s at 4 CTAs per SM, 4.9 at 8, 4.8 at 2
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  switch (world) {
    case 2: reduce_scatter_pull_kernel<T, 2><<<grid, 256, 0, st>>>(t, out, first, count, scale); break;
    case 4: reduce_scatter_pull_kernel<T, 4><<<grid, 256, 0, st>>>(t, out, first, count, scale); break;
    case 8: reduce_scatter_pull_kernel<T, 8><<<grid, 256, 0, st>>>(t, out, first, count, scale); break;
    default: return Q3_ERR_SHAPE;
  }
  return launch_status();
}

}  // namespace q3

using namespace q3;

// A device buffer other processes on this node can map: plain cudaMalloc (not a sub-block of a caching allocator,
// which an IPC handle cannot describe) plus its 64-byte handle.
extern "C" int q3_peer_alloc(int64_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes < 1) return Q3_ERR_ARG;
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) { cudaFree(*ptr); *ptr = nullptr; return Q3_ERR_CUDA - (int)e; }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return Q3_OK;
}

extern "C" int q3_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return Q3_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_CUDA - (int)e;
}

extern "C" int q3_peer_close(void* ptr) {
  if (!ptr) return Q3_ERR_ARG;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_CUDA - (int)e;
}

extern "C" int q3_peer_free(void* ptr) {
  if (!ptr) return Q3_ERR_ARG;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_CUDA - (int)e;
}

// One asynchronous device-to-device copy on `stream`; either side may be a pointer mapped with q3_peer_open, and the
// transfer then runs on a copy engine over NVLink without occupying an SM (the all-gather of runtime/peer_gather.py:
// one call per source rank).
extern "C" int q3_peer_copy(void* dst, const void* src, int64_t bytes, q3_stream_t stream) {
  if (!dst || !src) return Q3_ERR_ARG;
  if (bytes < 0) return Q3_ERR_SHAPE;
  if (bytes == 0) return Q3_OK;
  cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
  return e == cudaSuccess ? Q3_OK : Q3_ERR_CUDA - (int)e;
}

// `count` such copies, issued one after the other on `stream` (host arrays of pointers and sizes): the all-gather that
// delivers every rank's shard of every parameter straight into the parameter's own tensor.
extern "C" int q3_peer_copy_many(void* const* dst, const void* const* src, const int64_t* bytes, int64_t count,
                                 q3_stream_t stream) {
  if (!dst || !src || !bytes) return Q3_ERR_ARG;
  if (count < 0) return Q3_ERR_SHAPE;
  for (int64_t i = 0; i < count; ++i) {
    if (bytes[i] < 0) return Q3_ERR_SHAPE;
    if (bytes[i] == 0) continue;
    if (!dst[i] || !src[i]) return Q3_ERR_ARG;
    cudaError_t e = cudaMemcpyAsync(dst[i], src[i], (size_t)bytes[i], cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  }
  return Q3_OK;
}

// out [count] fp32 = scale * sum over ranks r of peers[r][first .. first + count) widened to fp32, added in rank order.
// peers: host array of `world` device pointers (this rank's own staging buffer at index `rank`, the others mapped
// with q3_peer_open), all holding the same [world * count]-element layout in `dtype` (bf16 or fp16). The caller
// makes sure every rank has finished writing its staging buffer (a barrier on the launching stream) and does not let
// any rank overwrite it before all ranks have pulled.
extern "C" int q3_reduce_scatter_pull(const void* const* peers, int world, float* out, int64_t first, int64_t count,
                                      double scale, int dtype, q3_stream_t stream) {
  if (!peers || !out) return Q3_ERR_ARG;
  if ((world != 2 && world != 4 && world != 8) || count < 0 || first < 0) return Q3_ERR_SHAPE;
  if (dtype != Q3_BF16 && dtype != Q3_F16) return Q3_ERR_DTYPE;
  if ((first % 8) || !aligned16(out)) return Q3_ERR_ALIGN;
  if (count == 0) return Q3_OK;
  PeerTable t{};
  for (int r = 0; r < world; ++r) {
    if (!peers[r] || !aligned16(peers[r])) return Q3_ERR_ALIGN;
    t.base[r] = peers[r];
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q3_BF16) return launch_pull<__nv_bfloat16>(world, t, out, first, count, (float)scale, st);
  return launch_pull<__half>(world, t, out, first, count, (float)scale, st);
}
