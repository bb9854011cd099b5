// Dense bf16/fp16 GEMM on the 5th-generation tensor cores (tcgen05) with fp32 accumulators in
// tensor memory, operands staged by TMA into 128-byte-swizzled shared memory.
//
//   C[M,N] = A[M,K] * B[K,N]   (contiguous C in bf16 / fp16 / fp32)
//
// Either operand may be stored with the contraction dimension contiguous ("K-major": A as [M,K]
// row-major, B as [N,K] row-major) or with its outer dimension contiguous ("MN-major": A as [K,M]
// row-major, B as [K,N] row-major). That covers the three products of a linear layer without a
// transpose copy: forward X*W^T (K-major, K-major), input gradient dY*W (K-major, MN-major) and
// weight gradient dY^T*X (MN-major, MN-major).
//
// Kernel structure (persistent, one CTA per SM, 192 threads):
//   warp 0   : TMA producer - fills a ring of {A tile 128x64, B tile BNx64} stages
//   warp 1   : MMA issuer  - one thread issues tcgen05.mma (M=128, N=BN, K=16) x4 per stage into one
//              of two TMEM accumulators, releases stages with tcgen05.commit
//   warps 2-5: epilogue    - tcgen05.ld the finished accumulator (32 lanes per warp), convert and
//              store while the MMA warp already works on the next tile in the other accumulator
// Tiles are visited in grouped-M order so that CTAs running together share operand tiles in L2, and are
// drawn from a device counter, so that a CTA that starts late (its SM held by a kernel of another stream)
// does not own a fixed share of the work.
//
// Where the output has at least two 128-row tiles the kernel runs as CTA pairs (template argument PAIR,
// clusters of 2, tcgen05 cta_group::2): the pair owns a 256x256 tile, each CTA stages its own 128 rows of A
// and half of the B rows and keeps its 128 accumulator rows in its own tensor memory; the rank-0 CTA issues
// M=256 MMAs that read both CTAs' shared memory. Per k-block a CTA then fetches 32 KB instead of 48 KB for the
// same tensor work, which is what limited the single-CTA form to about 80 % tensor-pipe activity.
// Barriers across the pair: loads of both CTAs are counted on rank 0's `full` barrier (armed by rank 0 with
// both CTAs' bytes); rank 0 commits `empty` and `tfull` once to each CTA; the epilogue warps of both CTAs
// release an accumulator on rank 0's `tempty`; rank 0 publishes every tile into both CTAs' tile queues.
// A cluster barrier before the first and after the last cross-CTA signal. All TMA loads are plain per-CTA
// loads: every CTA fetches what it stages itself.
//
// The fused gate/up variant loads W_gate and W_up rows into one 256-row B tile, so one N=256 MMA
// produces gate in accumulator columns [0,128) and up in [128,256); its epilogue stores G, U and
// Y = silu(G)*U.
//
// Replaces, in the reference: qwen3_triton/kernels/linear.py:14-77 (_gemm / matmul),
// kernels/mlp.py:14-32 and kernels/mlp_precision.py:17-35 (_gate_up).
#include "tcgen05.cuh"
#include <atomic>
#include <mutex>
#include <string.h>

namespace q3 {

int gemm_simt(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c,
              int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, cudaStream_t st);

namespace tc {

constexpr int BM = 128, BK = 64, UK = 16;
constexpr int kGemmThreads = 192;
// M-tiles per group of the tile order (see tile_coords): all N-tiles of a group are visited before the next group, so
// the weight operand is streamed from DRAM once per group while the group's activation rows stay in L2.
constexpr int kGroupM = 8, kGroupMWide = 16;

struct GemmParams {
  void* c0;   // C, or G for the gate/up variant, or dG for the SwiGLU-backward variant
  void* c1;   // U, or dU
  void* c2;   // Y
  const void* aux0;   // saved G (SwiGLU backward)
  const void* aux1;   // saved U
  int64_t M, N, K;  // N = output columns (per matrix for gate/up)
  int tiles_m, tiles_n, kblocks;
  int group_m;      // M-tiles per group of the tile order
  uint32_t idesc;
  int a_mn, b_mn;   // operand is MN-major
  int prefetch;     // issue L2 prefetches ahead of the smem ring
  int* status;
  // Tile hand-out. nullptr: CTA b works on tiles b, b + grid, ... (static). Otherwise {next tile, CTAs finished}, both
  // zero at launch: every CTA draws its tiles from the counter, and the last CTA to finish zeroes the pair again.
  int* sched;
  // grouped products that share one operand (seg_mode 0 = plain GEMM):
  //   1: segments along N  - B_i and C_i differ, A shared            (q/k/v projections of one input)
  //   2: segments along K  - A_i and B_i differ, one C               (sum of their input gradients)
  //   3: segments along M  - A_i and C_i differ, B shared            (their weight gradients)
  // seg_end[i] = cumulative count of N tiles / k-blocks / M tiles up to and including segment i.
  int seg_mode;
  int seg_end[3];
  void* seg_c[3];
  int64_t seg_dim[3];   // N_i (mode 1) or M_i (mode 3)
  // cross-entropy epilogues
  const int64_t* labels;   // effective label per row (ignore_index where the row is not scored)
  const float* lse;        // per row (EPI_CE_GRAD)
  const float* ups;        // upstream gradient per data rank
  const int* counts;       // valid-target count per data rank
  int64_t rows_per_rank, vocab_start, ignore;
  float* part_max;         // [M][tiles_n] (EPI_CE_STATS)
  float* part_sum;
  float* target;           // [M], must be zero-filled by the caller
};

struct alignas(64) GemmMaps {
  CUtensorMap a[3];
  CUtensorMap b[3];   // gate/up: b[0] = W_gate, b[1] = W_up
};

__device__ __forceinline__ int seg_of(const GemmParams& p, int idx, int& start) {
  const int seg = (idx >= p.seg_end[0]) + (idx >= p.seg_end[1]);
  start = seg == 0 ? 0 : p.seg_end[seg - 1];
  return seg;
}

// PAIR: two CTAs (a cluster of 2) share one 256 x BN output tile. Each stages its own 128 rows of A and half of the B
// rows, so a CTA moves 32 KB per k-block from L2 into shared memory instead of 48 KB for the same 128 x 256 x 64 of
// MMA work: the single-CTA kernel is bound by that traffic at about 80 % of the tensor rate.
template <int BN, bool PAIR = false> struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;   // rows of the B tile staged by this CTA
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : ((BN == 256) ? 4 : 6);
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};
// Slots of the in-CTA tile queue (producer -> MMA issuer and epilogue warps). The producer runs at most one tile ahead
// of the MMA issuer and the epilogue at most two behind it; the queue's own barriers make any depth correct.
constexpr int kSched = 4;
static_assert((2 * 7 + 6 + 2 * kSched) * 8 + kSched * 4 <= 256, "barrier area");

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

template <typename TO> __device__ __forceinline__ void store_chunk32(TO* dst, const uint32_t (&r)[32], int64_t col0, int64_t N);

template <> __device__ __forceinline__ void store_chunk32<float>(float* dst, const uint32_t (&r)[32], int64_t col0, int64_t N) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (col0 + 4 * j + 4 <= N)
      *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
  }
}
template <> __device__ __forceinline__ void store_chunk32<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&r)[32], int64_t col0, int64_t N) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (col0 + 8 * j + 8 <= N) {
      uint4 v;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
      *reinterpret_cast<uint4*>(dst + 8 * j) = v;
    }
  }
}
template <> __device__ __forceinline__ void store_chunk32<__half>(__half* dst, const uint32_t (&r)[32], int64_t col0, int64_t N) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (col0 + 8 * j + 8 <= N) {
      uint4 v;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
      *reinterpret_cast<uint4*>(dst + 8 * j) = v;
    }
  }
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& mi, int& ni) {
  const int group = group_m * tiles_n;
  const int g = tile / group, first = g * group_m;
  const int height = (tiles_m - first) < group_m ? (tiles_m - first) : group_m;
  const int in = tile - g * group;
  mi = first + in % height;
  ni = in / height;
}

// Epilogues:
//   EPI_STORE    C = A*B (TO = bf16 / fp16 / fp32)
//   EPI_GATE_UP  BN must be 256; B tile = [W_gate rows | W_up rows]; stores G, U and silu(G)*U
//   EPI_ACC_F32  C += A*B, C in fp32 or (read-add-round) in a 16-bit type
//   EPI_CE_STATS A*B are logits that are never stored: per row and N-tile the (max, sum exp) of the logits rounded
//                to TO, and the target logit where the tile owns the row's label
//   EPI_CE_GRAD  stores dZ = (exp(z - lse[row]) - onehot) * upstream[source] / count[source] for the logits z
//   EPI_SWIGLU_BWD  A*B is dY of y = silu(G)*U, rounded to TO as the stored dY would be; stores dG and dU, never dY
enum { EPI_STORE = 0, EPI_GATE_UP = 1, EPI_ACC_F32 = 2, EPI_CE_STATS = 3, EPI_CE_GRAD = 4, EPI_SWIGLU_BWD = 5 };

template <int BN, typename TO, int EPI, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
  constexpr bool GATE_UP = (EPI == EPI_GATE_UP);
  static_assert(!PAIR || BN == 256, "CTA pairs use the 256-column tile");
  using C = Cfg<BN, PAIR>;
  // PAIR: rank 0 of the cluster issues the MMAs and owns the barriers both CTAs report to (full, tempty)
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment keeps the 128-byte swizzle phase identical for TMA and UMMA.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  // barrier slots: full[STAGES], empty[STAGES], tfull[2], tempty[2], done
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + 2 + a); };
  const uint32_t done_bar = bar0 + 8u * (2 * C::STAGES + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // tile queue: sfull[kSched], sempty[kSched], then the tile numbers
  const uint32_t sbar0 = bar0 + 8u * (2 * C::STAGES + 6);
  auto sfull_bar = [&](int i) { return sbar0 + 8u * i; };
  auto sempty_bar = [&](int i) { return sbar0 + 8u * (kSched + i); };
  volatile int* sched_tile = reinterpret_cast<volatile int*>(bars + 2 * C::STAGES + 6 + 2 * kSched);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // PAIR: a tile is 256 rows (two consecutive 128-row tiles, one per CTA); rank 0 decides the pair's next tile and
  // puts it into both CTAs' tile queues
  const int tiles_m_sched = PAIR ? (p.tiles_m + 1) / 2 : p.tiles_m;
  const int group_m_sched = PAIR ? (p.group_m + 1) / 2 : p.group_m;
  const int total_tiles = tiles_m_sched * p.tiles_n;
  const int first_static = PAIR ? (int)cluster_id_x() : (int)blockIdx.x;
  const int stride_static = PAIR ? (int)cluster_count_x() : (int)gridDim.x;
  // this CTA's 128-row tile and the N tile of a scheduled tile
  auto coords_of = [&](int tile, int& mi, int& ni) {
    tile_coords(tile, tiles_m_sched, p.tiles_n, group_m_sched, mi, ni);
    if (PAIR) mi = 2 * mi + (int)rank;
  };
  // Consumer side of the tile queue (MMA issuer: one thread; epilogue: whole warps, lane 0 releases the slot).
  // Returns the tile, -1 after the last one, -2 when a wait gave up.
  // PAIR: every consumer of either CTA releases a slot on rank 0's barrier, where the publisher waits.
  uint32_t taken = 0;
  const uint32_t sempty_lead0 = PAIR ? mapa_u32(sempty_bar(0), 0) : 0u;
  auto next_tile = [&](bool whole_warp) -> int {
    const int slot = taken % kSched;
    const uint32_t ph = (taken / kSched) & 1u;
    ++taken;
    if (PAIR ? !mbar_wait_cluster(sfull_bar(slot), ph, abort_flag) : !mbar_wait(sfull_bar(slot), ph, abort_flag))
      return -2;
    const int t = sched_tile[slot];
    if (whole_warp) __syncwarp();
    if (!whole_warp || lane == 0) {
      if (PAIR) mbar_arrive_cluster(sempty_lead0 + 8u * slot);
      else mbar_arrive(sempty_bar(slot));
    }
    return t;
  };

  // The producer thread draws its first tile before anything else: the counter's round trip to L2 runs beside the
  // barrier set-up, the tensor-memory allocation and the CTA-wide sync below.
  int first_tile = first_static;
  if (threadIdx.x == 0 && p.sched && leader) first_tile = atomicAdd(p.sched, 1);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    // tempty: the four epilogue warps of every CTA that holds rows of the accumulator
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), PAIR ? 8 : 4); }
    mbar_init(done_bar, 1);
    // a slot is released by the MMA thread and the 4 epilogue warps (PAIR: of both CTAs, and rank 1's producer)
    for (int i = 0; i < kSched; ++i) { mbar_init(sfull_bar(i), 1); mbar_init(sempty_bar(i), PAIR ? 11 : 5); }
    fence_barrier_init();
    prefetch_tmap(&maps.a[0]);
    prefetch_tmap(&maps.b[0]);
    if (GATE_UP) prefetch_tmap(&maps.b[1]);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0, published = 0;
      auto publish = [&](int t) -> bool {
        const int slot = published % kSched;
        const uint32_t ph = (published / kSched) & 1u;
        ++published;
        if (!mbar_wait(sempty_bar(slot), ph ^ 1u, abort_flag)) return false;
        sched_tile[slot] = t;
        mbar_arrive(sfull_bar(slot));   // release: the consumers' waits acquire
        if (PAIR) {                     // the same into rank 1's queue
          st_cluster_u32(mapa_u32(smem_u32(const_cast<int*>(&sched_tile[slot])), 1), (uint32_t)t);
          mbar_arrive_cluster(mapa_u32(sfull_bar(slot), 1));
        }
        return true;
      };
      // PAIR, rank 1: the producer is one more reader of the queue rank 0 fills
      int tile = first_tile;
      if (tile >= total_tiles) tile = -1;
      bool ok = true;
      if (leader) ok = publish(tile);
      else { tile = next_tile(false); ok = tile > -2; }
      const bool draw = leader && p.sched != nullptr;
      // PAIR: both CTAs' loads are counted on the rank-0 CTA's full barriers
      const uint32_t full0 = PAIR ? mapa_u32(full_bar(0), 0) : full_bar(0);
      while (ok && tile >= 0) {
        // the next tile is drawn now and needed only after this tile's loads are issued
        int next = draw ? atomicAdd(p.sched, 1) : tile + stride_static;
        int mi, ni;
        coords_of(tile, mi, ni);
        int m0 = mi * BM, n0 = ni * (GATE_UP ? BN / 2 : BN);
        const CUtensorMap* tmA = &maps.a[0];
        const CUtensorMap* tmB = &maps.b[0];
        const CUtensorMap* tmB2 = &maps.b[1];
        if (p.seg_mode == 1) {
          int start;
          const int seg = seg_of(p, ni, start);
          tmB = &maps.b[seg];
          n0 = (ni - start) * BN;
        } else if (p.seg_mode == 3) {
          int start;
          const int seg = seg_of(p, mi, start);
          tmA = &maps.a[seg];
          m0 = (mi - start) * BM;
        }
        // Operands that stream from HBM (weights of the vocabulary head, token-major operands of the weight
        // gradient) see a longer latency than the smem ring covers: pull boxes into L2 kPrefetch k-blocks ahead.
        auto prefetch = [&](int kb) {
          const int k0 = kb * BK;
          if (!p.a_mn) tma_prefetch_2d(tmA, k0, m0);
          else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_prefetch_2d(tmA, m0 + 64 * j, k0);
          }
          if (GATE_UP) { tma_prefetch_2d(tmB, k0, n0); tma_prefetch_2d(tmB2, k0, n0); }
          else if (!p.b_mn) tma_prefetch_2d(tmB, k0, n0);
          else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_prefetch_2d(tmB, n0 + 64 * j, k0);
          }
        };
        constexpr int kPrefetch = C::STAGES + 6;
        if (p.prefetch) {
          for (int kb = 0; kb < kPrefetch && kb < p.kblocks; ++kb) prefetch(kb);
        }
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (p.prefetch && kb + kPrefetch < p.kblocks) prefetch(kb + kPrefetch);
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES, b_dst = a_dst + C::A_BYTES;
          if (!PAIR) mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
          else if (leader) mbar_expect_tx(full_bar(s), 2 * C::STAGE_BYTES);   // this CTA's bytes and the peer's
          int k0 = kb * BK;
          if (p.seg_mode == 2) {   // this k-block belongs to one (A_i, B_i) pair
            int start;
            const int seg = seg_of(p, kb, start);
            tmA = &maps.a[seg];
            tmB = &maps.b[seg];
            k0 = (kb - start) * BK;
          }
          if constexpr (!PAIR) {
            if (!p.a_mn) {
              tma_load_2d(a_dst, tmA, k0, m0, full_bar(s));
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), tmA, m0 + 64 * j, k0, full_bar(s));
            }
            if (GATE_UP) {
              tma_load_2d(b_dst, tmB, k0, n0, full_bar(s));
              tma_load_2d(b_dst + (BN / 2) * 128, tmB2, k0, n0, full_bar(s));
            } else if (!p.b_mn) {
              tma_load_2d(b_dst, tmB, k0, n0, full_bar(s));
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), tmB, n0 + 64 * j, k0, full_bar(s));
            }
          } else {
            // this CTA's 128 rows of A, and its half of the tile's B rows: columns [0,128) of the accumulator come
            // from rank 0's shared memory, [128,256) from rank 1's (gate/up: rank 0 stages W_gate, rank 1 W_up)
            const uint32_t bar = full0 + 8u * s;
            if (!p.a_mn) {
              tma_load_2d_pair(a_dst, tmA, k0, m0, bar);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), tmA, m0 + 64 * j, k0, bar);
            }
            if (GATE_UP) {
              tma_load_2d_pair(b_dst, rank ? tmB2 : tmB, k0, n0, bar);
            } else if (!p.b_mn) {
              tma_load_2d_pair(b_dst, tmB, k0, n0 + (int)rank * C::B_ROWS, bar);
            } else {
#pragma unroll
              for (int j = 0; j < C::B_ROWS / 64; ++j)
                tma_load_2d_pair(b_dst + j * (BK * 128), tmB, n0 + (int)rank * C::B_ROWS + 64 * j, k0, bar);
            }
          }
        }
        if (!ok) break;
        if (leader) {
          if (next >= total_tiles) next = -1;
          ok = publish(next);
          tile = next;
        } else {
          tile = next_tile(false);
          ok = tile > -2;
        }
      }
      if (draw) {
        // This CTA draws no more tiles. The last drawing CTA of the grid to get here leaves the counters zeroed for
        // the next launch.
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == stride_static - 1) {
          p.sched[0] = 0;
          p.sched[1] = 0;
          __threadfence();
        }
      }
      // Do not leave the CTA while bulk copies may still be landing in its shared memory. (PAIR, rank 1: its copies
      // are counted on rank 0's barriers; they have landed once the MMAs that read them are done, which the
      // epilogue of this CTA waits for, and both CTAs meet at the cluster barrier before they leave.)
      const uint32_t pending = (PAIR && !leader) ? 0u : (it < (uint32_t)C::STAGES ? it : (uint32_t)C::STAGES);
      for (uint32_t j = it - pending; j < it; ++j) {
        const int s = j % C::STAGES;
        const uint32_t ph = (j / C::STAGES) & 1u;
        mbar_wait_drain(full_bar(s), ph);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tl = 0;
      bool ok = true;
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 0, b_lbo = p.b_mn ? BK * 128 : 0;
      const uint32_t a_kadv = p.a_mn ? (UK * 128) >> 4 : (UK * 2) >> 4;  // descriptor units of 16 B
      const uint32_t b_kadv = p.b_mn ? (UK * 128) >> 4 : (UK * 2) >> 4;
      // PAIR: completion is reported to the same barrier of both CTAs (one commit each; empty: both producers may
      // refill the stage, tfull: both epilogues may read their rows)
      const uint32_t peer_empty0 = PAIR ? mapa_u32(empty_bar(0), 1) : 0u;
      const uint32_t peer_tfull0 = PAIR ? mapa_u32(tfull_bar(0), 1) : 0u;
      for (int tile = next_tile(false); tile >= 0 && ok; tile = next_tile(false), ++tl) {
        if (PAIR && !leader) continue;    // rank 1 issues nothing; its thread only keeps the tile queue moving
        const int acc = tl & 1;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + s * C::STAGE_BYTES, b_src = a_src + C::A_BYTES;
          const uint64_t adesc = make_smem_desc(a_src, a_lbo, 1024);
          const uint64_t bdesc = make_smem_desc(b_src, b_lbo, 1024);
          if constexpr (PAIR) {
#pragma unroll
            for (int k = 0; k < BK / UK; ++k)
              mma_f16_ss_pair(d_tmem, adesc + (uint64_t)(k * a_kadv), bdesc + (uint64_t)(k * b_kadv), p.idesc,
                              (kb | k) != 0 ? 1u : 0u);
            mma_commit_pair(empty_bar(s));
            mma_commit_pair(peer_empty0 + 8u * s);
          } else {
#pragma unroll
            for (int k = 0; k < BK / UK; ++k)
              mma_f16_ss(d_tmem, adesc + (uint64_t)(k * a_kadv), bdesc + (uint64_t)(k * b_kadv), p.idesc,
                         (kb | k) != 0 ? 1u : 0u);
            mma_commit(empty_bar(s));
          }
        }
        if (ok) {
          if constexpr (PAIR) {
            mma_commit_pair(tfull_bar(acc));
            mma_commit_pair(peer_tfull0 + 8u * acc);
          } else {
            mma_commit(tfull_bar(acc));
          }
        }
      }
      // Everything issued must have completed before tensor memory is released.
      if (!PAIR) {
        mma_commit(done_bar);
        mbar_wait_drain(done_bar, 0);
      } else if (leader) {
        mma_commit_pair(done_bar);
        mbar_wait_drain(done_bar, 0);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tl = 0;
    bool ok = true;
    const uint32_t tempty0 = PAIR ? mapa_u32(tempty_bar(0), 0) : 0u;   // rank 0 collects both CTAs' releases
    for (int tile = next_tile(true); tile >= 0 && ok; tile = next_tile(true), ++tl) {
      int mi, ni;
      coords_of(tile, mi, ni);
      const int acc = tl & 1;
      const uint32_t aph = (tl >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int64_t row = (int64_t)mi * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if constexpr (EPI == EPI_STORE) {
        int64_t n0 = (int64_t)ni * BN, ncols = p.N, mrows = p.M, crow_idx = row;
        TO* cbase = reinterpret_cast<TO*>(p.c0);
        if (p.seg_mode == 1) {
          int start;
          const int seg = seg_of(p, ni, start);
          cbase = reinterpret_cast<TO*>(p.seg_c[seg]);
          ncols = p.seg_dim[seg];
          n0 = (int64_t)(ni - start) * BN;
        } else if (p.seg_mode == 3) {
          int start;
          const int seg = seg_of(p, mi, start);
          cbase = reinterpret_cast<TO*>(p.seg_c[seg]);
          mrows = p.seg_dim[seg];
          crow_idx = (int64_t)(mi - start) * BM + q * 32 + lane;
        }
        TO* crow = cbase + crow_idx * ncols + n0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          if (crow_idx < mrows && n0 + c * 32 < ncols) store_chunk32<TO>(crow + c * 32, r, n0 + c * 32, ncols);
        }
      } else if constexpr (EPI == EPI_ACC_F32) {
        // C += A*B with C in TO (fp32, or a 16-bit type: read, add in fp32, round once)
        const int64_t n0 = (int64_t)ni * BN;
        TO* crow = reinterpret_cast<TO*>(p.c0) + row * p.N + n0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          if (row < p.M && n0 + c * 32 < p.N) {
            constexpr int W = 16 / (int)sizeof(TO);   // elements per 16-byte access
#pragma unroll
            for (int j = 0; j < 32 / W; ++j) {
              if (n0 + c * 32 + W * j + W <= p.N) {
                float old[W];
                VecIO<TO, W>::load(crow + c * 32 + W * j, old);
#pragma unroll
                for (int e = 0; e < W; ++e) r[W * j + e] = __float_as_uint(__uint_as_float(r[W * j + e]) + old[e]);
              }
            }
            store_chunk32<TO>(crow + c * 32, r, n0 + c * 32, p.N);
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
        const int64_t n0 = (int64_t)ni * BN;
        const TO* grow = reinterpret_cast<const TO*>(p.aux0) + row * p.N + n0;
        const TO* urow = reinterpret_cast<const TO*>(p.aux1) + row * p.N + n0;
        TO* dgrow = reinterpret_cast<TO*>(p.c0) + row * p.N + n0;
        TO* durow = reinterpret_cast<TO*>(p.c1) + row * p.N + n0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32], du[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          if (row < p.M && n0 + c * 32 < p.N) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (n0 + c * 32 + 8 * j + 8 <= p.N) {
                float g8[8], u8[8];
                VecIO<TO, 8>::load(grow + c * 32 + 8 * j, g8);
                VecIO<TO, 8>::load(urow + c * 32 + 8 * j, u8);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float dy = to_f32<TO>(from_f32<TO>(__uint_as_float(r[8 * j + e])));   // the dY a separate GEMM would store
                  const float sg = __fdividef(1.f, 1.f + __expf(-g8[e]));
                  r[8 * j + e] = __float_as_uint(dy * u8[e] * sg * (1.f + g8[e] * (1.f - sg)));
                  du[8 * j + e] = __float_as_uint(dy * g8[e] * sg);
                }
              }
            }
            store_chunk32<TO>(dgrow + c * 32, r, n0 + c * 32, p.N);
            store_chunk32<TO>(durow + c * 32, du, n0 + c * 32, p.N);
          }
        }
      } else if constexpr (EPI == EPI_CE_STATS) {
        const int64_t n0 = (int64_t)ni * BN;
        const int64_t label = row < p.M ? p.labels[row] : p.ignore;
        const int64_t hot = label - p.vocab_start - n0;   // column of the label inside this tile, if any
        float mx = -3.0e38f, sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          if (n0 + c * 32 < p.N) {
            float z[32];
            float cm = -3.0e38f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              z[j] = to_f32<TO>(from_f32<TO>(__uint_as_float(r[j])));   // the loss is defined on the rounded logits
              if (n0 + c * 32 + j < p.N) cm = fmaxf(cm, z[j]);
              if (c * 32 + j == hot && label != p.ignore && row < p.M) p.target[row] = z[j];
            }
            const float nm = fmaxf(mx, cm);
            float acc_s = sum * __expf(mx - nm);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c * 32 + j < p.N) acc_s += __expf(z[j] - nm);
            mx = nm; sum = acc_s;
          }
        }
        if (row < p.M) {
          p.part_max[row * p.tiles_n + ni] = mx;
          p.part_sum[row * p.tiles_n + ni] = sum;
        }
      } else if constexpr (EPI == EPI_CE_GRAD) {
        const int64_t n0 = (int64_t)ni * BN;
        TO* crow = reinterpret_cast<TO*>(p.c0) + row * p.N + n0;
        const int64_t label = row < p.M ? p.labels[row] : p.ignore;
        const bool valid = label != p.ignore;
        const int64_t hot = label - p.vocab_start - n0;
        float l = 0.f, scale = 0.f;
        if (valid) {
          const int64_t source = row / p.rows_per_rank;
          l = p.lse[row];
          scale = p.ups[source] / (float)p.counts[source];
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          if (row < p.M && n0 + c * 32 < p.N) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float z = to_f32<TO>(from_f32<TO>(__uint_as_float(r[j])));
              const float g = valid ? (__expf(z - l) - (c * 32 + j == hot ? 1.f : 0.f)) * scale : 0.f;
              r[j] = __float_as_uint(g);
            }
            store_chunk32<TO>(crow + c * 32, r, n0 + c * 32, p.N);
          }
        }
      } else {
        const int64_t n0 = (int64_t)ni * (BN / 2);
        TO* grow = reinterpret_cast<TO*>(p.c0) + row * p.N + n0;
        TO* urow = reinterpret_cast<TO*>(p.c1) + row * p.N + n0;
        TO* yrow = reinterpret_cast<TO*>(p.c2) + row * p.N + n0;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld32(t_row + c * 32, g);
          tmem_ld32(t_row + BN / 2 + c * 32, u);
          tmem_ld_wait();
          if (row < p.M && n0 + c * 32 < p.N) {
            store_chunk32<TO>(grow + c * 32, g, n0 + c * 32, p.N);
            store_chunk32<TO>(urow + c * 32, u, n0 + c * 32, p.N);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              // the saved (rounded) gate/up values define Y, so backward reproduces it exactly
              const float gr = to_f32<TO>(from_f32<TO>(__uint_as_float(g[j])));
              const float ur = to_f32<TO>(from_f32<TO>(__uint_as_float(u[j])));
              g[j] = __float_as_uint(silu_f(gr) * ur);
            }
            store_chunk32<TO>(yrow + c * 32, g, n0 + c * 32, p.N);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(tempty0 + 8u * acc);
        else mbar_arrive(tempty_bar(acc));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA frees tensor memory or leaves while the other may still use the pair
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    else tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) flag_status(p.status, Q3_STATUS_WAIT_TIMEOUT);
}

struct Operand {
  const void* ptr;
  bool mn_major;
  int64_t ld;  // leading dimension in elements
};

// Classify an operand given the strides of its (outer, contraction) dimensions.
inline bool classify(const void* ptr, int64_t s_outer, int64_t s_k, int64_t outer, int64_t k, Operand* o) {
  if (!aligned16(ptr)) return false;
  if (s_k == 1 && (s_outer % 8 == 0 || outer == 1) && s_outer >= k) { *o = {ptr, false, s_outer}; return true; }
  if (s_outer == 1 && (s_k % 8 == 0 || k == 1) && s_k >= outer) { *o = {ptr, true, s_k}; return true; }
  return false;
}

// 16 M-tiles per group when their activation rows (16 x 128 x K 16-bit values) fit comfortably in the 126 MB L2: with
// 16 or 32 M-tiles (2048 / 4096 tokens) that halves the number of times the weights are fetched from DRAM compared
// with groups of 8. Q3_GEMM_GROUP_M overrides (tuning).
inline int pick_group_m(int tiles_m, int64_t K) {
  static const int forced = [] { const char* e = getenv("Q3_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();
  if (forced > 0) return forced;
  const int64_t wide_bytes = (int64_t)kGroupMWide * BM * K * 2;
  return (tiles_m >= kGroupMWide && wide_bytes <= (64ll << 20)) ? kGroupMWide : kGroupM;
}

// Tile hand-out policy: 1 = every CTA draws tiles from a device counter (default), 0 = static stride over the grid.
// With the static stride a CTA that cannot become resident at once - its SM is held by a communication kernel of
// another stream - keeps its whole share of tiles waiting, and the launch takes up to twice as long; drawn tiles go to
// the CTAs that are running. Results do not depend on the policy: every tile is computed whole by one CTA.
static std::atomic<int> g_tile_schedule{[] {
  const char* e = getenv("Q3_GEMM_TILE_SCHEDULE");
  return (e && !strcmp(e, "static")) ? 0 : 1;
}()};
constexpr unsigned kSchedPairs = 4096;

// One zeroed {next tile, CTAs finished} pair for a launch on the current device, or nullptr (static policy). Pairs are
// handed out round-robin; a pair is used again 4096 launches later, long after its launch zeroed it.
inline int sched_pair(int** out) {
  *out = nullptr;
  if (!g_tile_schedule.load(std::memory_order_relaxed)) return Q3_OK;
  static int* base[64] = {};
  static std::mutex lock;
  static std::atomic<unsigned> next{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return Q3_ERR_CUDA;
  int* b = __atomic_load_n(&base[dev], __ATOMIC_ACQUIRE);
  if (!b) {
    std::lock_guard<std::mutex> hold(lock);
    b = base[dev];
    if (!b) {
      if (cudaMalloc(&b, kSchedPairs * 2 * sizeof(int)) != cudaSuccess) return Q3_ERR_CUDA;
      if (cudaMemset(b, 0, kSchedPairs * 2 * sizeof(int)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(b);
        return Q3_ERR_CUDA;
      }
      __atomic_store_n(&base[dev], b, __ATOMIC_RELEASE);
    }
  }
  *out = b + 2 * (next.fetch_add(1, std::memory_order_relaxed) % kSchedPairs);
  return Q3_OK;
}

// CTA pairs (two CTAs per 256-row tile, see Cfg): 1 = used wherever there are at least two 128-row tiles (default),
// 0 = never. Q3_GEMM_CTA_PAIRS=0 sets the initial policy; q3_gemm_cta_pairs() switches at run time.
static std::atomic<int> g_cta_pairs{[] {
  const char* e = getenv("Q3_GEMM_CTA_PAIRS");
  return (e && !strcmp(e, "0")) ? 0 : 1;
}()};

// Persistent launch of the single-CTA kernel (grid = min(tiles, SMs)) or of the pair kernel (clusters of 2, as many
// as can be resident, at most one per 256-row tile).
template <typename K1, typename K2>
int launch_tiles(K1 single, K2 pair, bool use_pair, int smem_single, int smem_pair, DeviceFlags* cfg_single,
                 DeviceFlags* cfg_pair, const GemmMaps& maps, GemmParams& p, cudaStream_t st) {
  if (!use_pair) {
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    if (int rc = ensure_dynamic_smem(single, smem_single, cfg_single); rc != Q3_OK) return rc;
    if (int rc = sched_pair(&p.sched); rc != Q3_OK) return rc;
    single<<<grid, kGemmThreads, smem_single, st>>>(maps, p);
    return launch_status();
  }
  if (int rc = ensure_dynamic_smem(pair, smem_pair, cfg_pair); rc != Q3_OK) return rc;
  if (int rc = sched_pair(&p.sched); rc != Q3_OK) return rc;
  p.prefetch = 0;
  const int64_t tiles = (int64_t)((p.tiles_m + 1) / 2) * p.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)sm_count(), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem_pair;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // as many pairs as can be resident at once (asked once per device), at most one per tile
  static int resident[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return Q3_ERR_CUDA;
  int room = __atomic_load_n(&resident[dev], __ATOMIC_ACQUIRE);
  if (room == 0) {
    if (cudaOccupancyMaxActiveClusters(&room, pair, &cfg) != cudaSuccess || room < 1) {
      cudaGetLastError();
      room = sm_count() / 2;
    }
    __atomic_store_n(&resident[dev], room, __ATOMIC_RELEASE);
  }
  cfg.gridDim = dim3((unsigned)(2 * (tiles < room ? tiles : (int64_t)room)), 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, pair, maps, p);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  return launch_status();
}

template <int BN, typename TO, int EPI>
int launch_gemm(const Operand& A, const Operand& B, const void* b2, GemmParams& p, bool bf16, cudaStream_t st) {
  constexpr bool GATE_UP = (EPI == EPI_GATE_UP);
  using C = Cfg<BN>;
  const bool use_pair = BN == 256 && cdiv(p.M, BM) >= 2 && g_cta_pairs.load(std::memory_order_relaxed) != 0;
  GemmMaps maps;
  int rc;
  if (!A.mn_major) rc = make_tmap_2d(&maps.a[0], A.ptr, bf16, p.M, p.K, A.ld, BK, BM);
  else rc = make_tmap_2d(&maps.a[0], A.ptr, bf16, p.K, p.M, A.ld, 64, BK);
  if (rc != Q3_OK) return rc;
  // K-major B box: all BN rows of the tile, or (pairs, and the two halves of gate/up) 128 of them
  if (!B.mn_major) rc = make_tmap_2d(&maps.b[0], B.ptr, bf16, p.N, p.K, B.ld, BK, (GATE_UP || use_pair) ? BN / 2 : BN);
  else rc = make_tmap_2d(&maps.b[0], B.ptr, bf16, p.K, p.N, B.ld, 64, BK);
  if (rc != Q3_OK) return rc;
  maps.a[1] = maps.a[2] = maps.a[0];
  maps.b[1] = maps.b[2] = maps.b[0];
  if (GATE_UP) {
    rc = make_tmap_2d(&maps.b[1], b2, bf16, p.N, p.K, B.ld, BK, BN / 2);
    if (rc != Q3_OK) return rc;
  }
  p.seg_mode = 0;
  const int n_per_tile = GATE_UP ? BN / 2 : BN;
  p.tiles_m = (int)cdiv(p.M, BM);
  p.tiles_n = (int)cdiv(p.N, n_per_tile);
  p.kblocks = (int)cdiv(p.K, BK);
  p.group_m = pick_group_m(p.tiles_m, p.K);
  p.a_mn = A.mn_major;
  p.b_mn = B.mn_major;
  p.idesc = make_idesc_f16(use_pair ? 2 * BM : BM, BN, bf16, A.mn_major, B.mn_major);
  {
    const char* e = getenv("Q3_GEMM_PREFETCH");
    p.prefetch = e ? atoi(e) : 0;   // measured slower on every shape tried; kept as an experiment switch
  }
  static DeviceFlags configured = {}, configured_pair = {};
  if constexpr (BN == 256) {
    return launch_tiles(gemm_tc_kernel<BN, TO, EPI, false>, gemm_tc_kernel<BN, TO, EPI, true>, use_pair, C::SMEM_BYTES,
                        Cfg<BN, true>::SMEM_BYTES, &configured, &configured_pair, maps, p, st);
  } else {
    return launch_tiles(gemm_tc_kernel<BN, TO, EPI, false>, gemm_tc_kernel<BN, TO, EPI, false>, false, C::SMEM_BYTES,
                        C::SMEM_BYTES, &configured, &configured_pair, maps, p, st);
  }
}

// Up to three products that share an operand in one persistent launch (BN = 256, plain store epilogue):
//   mode 1: C_i[M,N_i] = A[M,K] * B_i[N_i,K]^T          tiles along N walk the segments
//   mode 2: C[M,N]     = sum_i A_i[M,K_i] * B_i[K_i,N]    k-blocks walk the segments (K_i % 64 == 0)
//   mode 3: C_i[M_i,N] = A_i[T,M_i]^T * B[T,N]            tiles along M walk the segments
// All matrices row-major and contiguous. One launch fills the SMs where the small members of a group (the k / v
// projections: 64 tiles on 148 SMs) would leave most of them idle.
template <typename TO>
int launch_grouped(int mode, int count, const void* const* a, const void* const* b, void* const* c, const int64_t* sizes,
                   int64_t M, int64_t N, int64_t K, bool bf16, int* status, cudaStream_t st) {
  constexpr int BN = 256;
  using C = Cfg<BN>;
  GemmMaps maps;
  GemmParams p{};
  p.status = status;
  p.seg_mode = mode;
  int rc = Q3_OK;
  int64_t total = 0;
  // mode 3 counts its 128-row tiles over all segments; the other modes have cdiv(M, 128) of them
  int64_t row_tiles = cdiv(M, BM);
  if (mode == 3) {
    row_tiles = 0;
    for (int i = 0; i < count; ++i) row_tiles += cdiv(sizes[i], BM);
  }
  const bool use_pair = row_tiles >= 2 && g_cta_pairs.load(std::memory_order_relaxed) != 0;
  const int b_box_rows = use_pair ? BN / 2 : BN;     // K-major B (mode 1)
  for (int i = 0; i < 3; ++i) {
    const int j = i < count ? i : count - 1;    // unused slots repeat the last segment
    const int64_t sz = sizes[j];
    if (mode == 1) {
      if (i == 0) rc = make_tmap_2d(&maps.a[0], a[0], bf16, M, K, K, BK, BM);
      if (rc == Q3_OK) rc = make_tmap_2d(&maps.b[i], b[j], bf16, sz, K, K, BK, b_box_rows);
      if (i > 0) maps.a[i] = maps.a[0];
      if (i < count) total += cdiv(sz, BN);
    } else if (mode == 2) {
      rc = make_tmap_2d(&maps.a[i], a[j], bf16, M, sz, sz, BK, BM);
      if (rc == Q3_OK) rc = make_tmap_2d(&maps.b[i], b[j], bf16, sz, N, N, 64, BK);
      if (i < count) total += sz / BK;
    } else {
      rc = make_tmap_2d(&maps.a[i], a[j], bf16, K, sz, sz, 64, BK);
      if (i == 0 && rc == Q3_OK) rc = make_tmap_2d(&maps.b[0], b[0], bf16, K, N, N, 64, BK);
      if (i > 0) maps.b[i] = maps.b[0];
      if (i < count) total += cdiv(sz, BM);
    }
    if (rc != Q3_OK) return rc;
    p.seg_end[i] = (int)total;
    p.seg_c[i] = c[mode == 2 ? 0 : j];
    p.seg_dim[i] = sz;
  }
  p.c0 = c[0];
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = mode == 3 ? (int)total : (int)cdiv(M, BM);
  p.tiles_n = mode == 1 ? (int)total : (int)cdiv(N, BN);
  p.kblocks = mode == 2 ? (int)total : (int)cdiv(K, BK);
  p.group_m = pick_group_m(p.tiles_m, (int64_t)p.kblocks * BK);
  p.a_mn = mode == 3;
  p.b_mn = mode != 1;
  p.idesc = make_idesc_f16(use_pair ? 2 * BM : BM, BN, bf16, p.a_mn != 0, p.b_mn != 0);
  p.prefetch = 0;
  static DeviceFlags configured = {}, configured_pair = {};
  return launch_tiles(gemm_tc_kernel<BN, TO, EPI_STORE, false>, gemm_tc_kernel<BN, TO, EPI_STORE, true>, use_pair,
                      C::SMEM_BYTES, Cfg<BN, true>::SMEM_BYTES, &configured, &configured_pair, maps, p, st);
}

inline int pick_bn(int64_t M, int64_t N) {
  if (N <= 128) return 128;
  const int64_t sms = sm_count();
  const int64_t t256 = cdiv(M, BM) * cdiv(N, 256), t128 = cdiv(M, BM) * cdiv(N, 128);
  // cost ~ waves * time per tile. An N=128 tile does half the work but the tensor core is then limited by
  // shared-memory operand bandwidth (A is re-read per 128 columns), so it costs ~0.62 of an N=256 tile.
  const int64_t c256 = cdiv(t256, sms) * 100, c128 = cdiv(t128, sms) * 62;
  return c128 < c256 ? 128 : 256;
}

}  // namespace tc
}  // namespace q3

using namespace q3;

// Which path q3_gemm takes for these arguments: 1 = tcgen05 tensor cores, 0 = CUDA-core fallback.
extern "C" int q3_gemm_path(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn,
                            const void* c, int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype) {
  if (in_dtype != Q3_BF16 && in_dtype != Q3_F16) return 0;
  if (out_dtype != Q3_F32 && out_dtype != in_dtype) return 0;
  if (M < 1 || N < 1 || K < 1 || M > 2147483647LL / 2 || N > 2147483647LL / 2 || K > 2147483647LL / 2) return 0;
  if (!aligned16(c) || N % (out_dtype == Q3_F32 ? 4 : 8)) return 0;
  tc::Operand A, B;
  if (!tc::classify(a, a_sm, a_sk, M, K, &A)) return 0;
  if (!tc::classify(b, b_sn, b_sk, N, K, &B)) return 0;
  return 1;
}

extern "C" int q3_gemm(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c,
                       int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, int* status,
                       q3_stream_t stream) {
  if (!a || !b || !c) return Q3_ERR_ARG;
  if (M < 1 || N < 1 || K < 1 || a_sm < 1 || a_sk < 1 || b_sk < 1 || b_sn < 1) return Q3_ERR_SHAPE;
  if (in_dtype < Q3_F32 || in_dtype > Q3_F16 || out_dtype < Q3_F32 || out_dtype > Q3_F16) return Q3_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (!q3_gemm_path(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, in_dtype, out_dtype))
    return gemm_simt(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, in_dtype, out_dtype, st);
  tc::Operand A, B;
  tc::classify(a, a_sm, a_sk, M, K, &A);
  tc::classify(b, b_sn, b_sk, N, K, &B);
  tc::GemmParams p{};
  p.c0 = c; p.M = M; p.N = N; p.K = K; p.status = status;
  const bool bf16 = in_dtype == Q3_BF16;
  const int bn = tc::pick_bn(M, N);
  if (out_dtype == Q3_F32)
    return bn == 256 ? tc::launch_gemm<256, float, tc::EPI_STORE>(A, B, nullptr, p, bf16, st)
                     : tc::launch_gemm<128, float, tc::EPI_STORE>(A, B, nullptr, p, bf16, st);
  if (bf16)
    return bn == 256 ? tc::launch_gemm<256, __nv_bfloat16, tc::EPI_STORE>(A, B, nullptr, p, bf16, st)
                     : tc::launch_gemm<128, __nv_bfloat16, tc::EPI_STORE>(A, B, nullptr, p, bf16, st);
  return bn == 256 ? tc::launch_gemm<256, __half, tc::EPI_STORE>(A, B, nullptr, p, bf16, st)
                   : tc::launch_gemm<128, __half, tc::EPI_STORE>(A, B, nullptr, p, bf16, st);
}

// 1 if q3_gate_up_swiglu_fwd runs the fused tensor-core kernel for these arguments.
extern "C" int q3_gate_up_path(const void* x, const void* wg, const void* wu, const void* g, const void* u,
                               const void* y, int64_t M, int64_t N, int64_t K, int dtype) {
  if (dtype != Q3_BF16 && dtype != Q3_F16) return 0;
  if (M < 1 || N < 1 || K < 1 || (K % 8) || (N % 8)) return 0;
  return aligned16(x) && aligned16(wg) && aligned16(wu) && aligned16(g) && aligned16(u) && aligned16(y);
}

extern "C" int q3_gate_up_swiglu_fwd(const void* x, const void* w_gate, const void* w_up, void* gate, void* up,
                                     void* y, int64_t M, int64_t N, int64_t K, int dtype, int* status,
                                     q3_stream_t stream) {
  if (!x || !w_gate || !w_up || !gate || !up || !y) return Q3_ERR_ARG;
  if (M < 1 || N < 1 || K < 1) return Q3_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (!q3_gate_up_path(x, w_gate, w_up, gate, up, y, M, N, K, dtype)) {
    // unfused: two CUDA-core GEMMs and the SwiGLU kernel
    int rc = gemm_simt(x, K, 1, w_gate, 1, K, gate, M, N, K, dtype, dtype, st);
    if (rc != Q3_OK) return rc;
    rc = gemm_simt(x, K, 1, w_up, 1, K, up, M, N, K, dtype, dtype, st);
    if (rc != Q3_OK) return rc;
    return q3_swiglu_fwd(gate, up, y, M * N, dtype, stream);
  }
  tc::Operand A{x, false, K}, B{w_gate, false, K};
  tc::GemmParams p{};
  p.c0 = gate; p.c1 = up; p.c2 = y; p.M = M; p.N = N; p.K = K; p.status = status;
  if (dtype == Q3_BF16) return tc::launch_gemm<256, __nv_bfloat16, tc::EPI_GATE_UP>(A, B, w_up, p, true, st);
  return tc::launch_gemm<256, __half, tc::EPI_GATE_UP>(A, B, w_up, p, false, st);
}

// ---------------------------------------------------------------------------------------------------------
// C (fp32, contiguous [M,N]) += A * B. Same operand rules as q3_gemm; tensor-core path only.
extern "C" int q3_gemm_acc_f32(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn,
                               float* c, int64_t M, int64_t N, int64_t K, int in_dtype, int* status,
                               q3_stream_t stream) {
  if (!a || !b || !c) return Q3_ERR_ARG;
  if (!q3_gemm_path(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, in_dtype, Q3_F32)) return Q3_ERR_ALIGN;
  tc::Operand A, B;
  tc::classify(a, a_sm, a_sk, M, K, &A);
  tc::classify(b, b_sn, b_sk, N, K, &B);
  tc::GemmParams p{};
  p.c0 = c; p.M = M; p.N = N; p.K = K; p.status = status;
  return tc::launch_gemm<256, float, tc::EPI_ACC_F32>(A, B, nullptr, p, in_dtype == Q3_BF16, (cudaStream_t)stream);
}

// C (contiguous [M,N], out_dtype = fp32 or the input type) += A * B: the sum of several products (the input gradient
// of projections that share an input) without separate add kernels. Tensor-core path only.
extern "C" int q3_gemm_acc(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn, void* c,
                           int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, int* status,
                           q3_stream_t stream) {
  if (!a || !b || !c) return Q3_ERR_ARG;
  if (!q3_gemm_path(a, a_sm, a_sk, b, b_sk, b_sn, c, M, N, K, in_dtype, out_dtype)) return Q3_ERR_ALIGN;
  tc::Operand A, B;
  tc::classify(a, a_sm, a_sk, M, K, &A);
  tc::classify(b, b_sn, b_sk, N, K, &B);
  tc::GemmParams p{};
  p.c0 = c; p.M = M; p.N = N; p.K = K; p.status = status;
  const bool bf16 = in_dtype == Q3_BF16;
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == Q3_F32) return tc::launch_gemm<256, float, tc::EPI_ACC_F32>(A, B, nullptr, p, bf16, st);
  if (bf16) return tc::launch_gemm<256, __nv_bfloat16, tc::EPI_ACC_F32>(A, B, nullptr, p, bf16, st);
  return tc::launch_gemm<256, __half, tc::EPI_ACC_F32>(A, B, nullptr, p, bf16, st);
}

// ---------------------------------------------------------------------------------------------------------
// Grouped linear layers that share their input (q/k/v, or gate/up): `count` = 2 or 3 weight matrices W_i [N_i, K].
static int grouped_check(int count, const int64_t* n, int64_t M, int64_t K, int dtype) {
  if (count < 2 || count > 3 || !n) return Q3_ERR_ARG;
  if (dtype != Q3_BF16 && dtype != Q3_F16) return Q3_ERR_DTYPE;
  if (M < 1 || K < 1 || (K % 8)) return Q3_ERR_SHAPE;
  for (int i = 0; i < count; ++i)
    if (n[i] < 1 || (n[i] % 8)) return Q3_ERR_SHAPE;
  return Q3_OK;
}
static bool all_aligned(const void* const* ptrs, int count) {
  for (int i = 0; i < count; ++i)
    if (!ptrs[i] || !aligned16(ptrs[i])) return false;
  return true;
}

// y_i [M, N_i] = x [M, K] * W_i^T, one launch.
extern "C" int q3_linear_fwd_grouped(const void* x, const void* const* weights, void* const* ys, const int64_t* n,
                                     int count, int64_t M, int64_t K, int dtype, int* status, q3_stream_t stream) {
  if (!x || !weights || !ys) return Q3_ERR_ARG;
  int rc = grouped_check(count, n, M, K, dtype);
  if (rc != Q3_OK) return rc;
  if (!aligned16(x) || !all_aligned(weights, count) || !all_aligned((const void* const*)ys, count)) return Q3_ERR_ALIGN;
  const void* a[1] = {x};
  int64_t total = 0;
  for (int i = 0; i < count; ++i) total += n[i];
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q3_BF16) return tc::launch_grouped<__nv_bfloat16>(1, count, a, weights, ys, n, M, total, K, true, status, st);
  return tc::launch_grouped<__half>(1, count, a, weights, ys, n, M, total, K, false, status, st);
}

// dx [M, K] = sum_i dy_i [M, N_i] * W_i [N_i, K], one launch (every N_i a multiple of 64).
extern "C" int q3_linear_dgrad_grouped(const void* const* dys, const void* const* weights, void* dx, const int64_t* n,
                                       int count, int64_t M, int64_t K, int dtype, int* status, q3_stream_t stream) {
  if (!dys || !weights || !dx) return Q3_ERR_ARG;
  int rc = grouped_check(count, n, M, K, dtype);
  if (rc != Q3_OK) return rc;
  for (int i = 0; i < count; ++i)
    if (n[i] % 64) return Q3_ERR_SHAPE;
  if (!aligned16(dx) || !all_aligned(dys, count) || !all_aligned(weights, count)) return Q3_ERR_ALIGN;
  void* c[1] = {dx};
  int64_t total = 0;
  for (int i = 0; i < count; ++i) total += n[i];
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q3_BF16) return tc::launch_grouped<__nv_bfloat16>(2, count, dys, weights, c, n, M, K, total, true, status, st);
  return tc::launch_grouped<__half>(2, count, dys, weights, c, n, M, K, total, false, status, st);
}

// dW_i [N_i, K] = dy_i [M, N_i]^T * x [M, K], one launch.
extern "C" int q3_linear_wgrad_grouped(const void* const* dys, const void* x, void* const* dws, const int64_t* n,
                                       int count, int64_t M, int64_t K, int dtype, int* status, q3_stream_t stream) {
  if (!dys || !x || !dws) return Q3_ERR_ARG;
  int rc = grouped_check(count, n, M, K, dtype);
  if (rc != Q3_OK) return rc;
  if (!aligned16(x) || !all_aligned(dys, count) || !all_aligned((const void* const*)dws, count)) return Q3_ERR_ALIGN;
  const void* b[1] = {x};
  int64_t total = 0;
  for (int i = 0; i < count; ++i) total += n[i];
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q3_BF16) return tc::launch_grouped<__nv_bfloat16>(3, count, dys, b, dws, n, total, K, M, true, status, st);
  return tc::launch_grouped<__half>(3, count, dys, b, dws, n, total, K, M, false, status, st);
}

// dY = dM [M,H] * W_down [H,I] is the gradient of y = silu(G)*U; this forms dG and dU in the GEMM epilogue from the
// saved G and U and never writes dY (one launch instead of q3_gemm + q3_swiglu_bwd, 2 x M x I x 2 bytes less
// traffic). dY is rounded to the storage type before use, so dG / dU equal the two-kernel path bit for bit.
extern "C" int q3_down_dgrad_swiglu_bwd(const void* dm, const void* w_down, const void* gate, const void* up, void* dgate,
                                        void* dup, int64_t M, int64_t I, int64_t H, int dtype, int* status,
                                        q3_stream_t stream) {
  if (!dm || !w_down || !gate || !up || !dgate || !dup) return Q3_ERR_ARG;
  if (M < 1 || I < 1 || H < 1) return Q3_ERR_SHAPE;
  if (dtype != Q3_BF16 && dtype != Q3_F16) return Q3_ERR_DTYPE;
  if ((I % 8) || (H % 8) || !aligned16(dm) || !aligned16(w_down) || !aligned16(gate) || !aligned16(up) ||
      !aligned16(dgate) || !aligned16(dup))
    return Q3_ERR_ALIGN;
  tc::Operand A{dm, false, H}, B{w_down, true, I};
  tc::GemmParams p{};
  p.c0 = dgate; p.c1 = dup; p.aux0 = gate; p.aux1 = up; p.M = M; p.N = I; p.K = H; p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q3_BF16) return tc::launch_gemm<256, __nv_bfloat16, tc::EPI_SWIGLU_BWD>(A, B, nullptr, p, true, st);
  return tc::launch_gemm<256, __half, tc::EPI_SWIGLU_BWD>(A, B, nullptr, p, false, st);
}

extern "C" int64_t q3_linear_ce_tiles(int64_t V_local) { return q3::cdiv(V_local, 256); }

// Logits = hidden [M,K] * weight[V_local,K]^T are produced tile by tile in tensor memory and reduced to
// per-(row, 256-column tile) softmax statistics in the epilogue; they are never written to memory.
extern "C" int q3_linear_ce_stats(const void* hidden, const void* weight, const int64_t* labels_eff, float* part_max,
                                  float* part_sum, float* target, int64_t M, int64_t V_local, int64_t K,
                                  int64_t vocab_start, int64_t ignore_index, int dtype, int* status,
                                  q3_stream_t stream) {
  if (!hidden || !weight || !labels_eff || !part_max || !part_sum || !target) return Q3_ERR_ARG;
  if (M < 1 || V_local < 1 || K < 1) return Q3_ERR_SHAPE;
  if ((dtype != Q3_BF16 && dtype != Q3_F16) || (K % 8) || !aligned16(hidden) || !aligned16(weight)) return Q3_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(target, 0, (size_t)M * 4, st);
  if (e != cudaSuccess) return Q3_ERR_CUDA - (int)e;
  tc::Operand A{hidden, false, K}, B{weight, false, K};
  tc::GemmParams p{};
  p.M = M; p.N = V_local; p.K = K; p.status = status;
  p.labels = labels_eff; p.vocab_start = vocab_start; p.ignore = ignore_index;
  p.part_max = part_max; p.part_sum = part_sum; p.target = target;
  if (dtype == Q3_BF16) return tc::launch_gemm<256, __nv_bfloat16, tc::EPI_CE_STATS>(A, B, nullptr, p, true, st);
  return tc::launch_gemm<256, __half, tc::EPI_CE_STATS>(A, B, nullptr, p, false, st);
}

// dZ [M, Vc] for a slice of Vc vocabulary rows of `weight_chunk` starting at global index vocab_start:
// recomputes that slice of the logits on the tensor cores and applies the softmax gradient in the epilogue.
extern "C" int q3_linear_ce_grad(const void* hidden, const void* weight_chunk, const int64_t* labels_eff,
                                 const float* lse, const float* upstream, const int* counts, void* dz, int64_t M,
                                 int64_t Vc, int64_t K, int64_t vocab_start, int64_t rows_per_rank,
                                 int64_t ignore_index, int dtype, int* status, q3_stream_t stream) {
  if (!hidden || !weight_chunk || !labels_eff || !lse || !upstream || !counts || !dz) return Q3_ERR_ARG;
  if (M < 1 || Vc < 1 || K < 1 || rows_per_rank < 1) return Q3_ERR_SHAPE;
  if ((dtype != Q3_BF16 && dtype != Q3_F16) || (K % 8) || (Vc % 8) || !aligned16(hidden) || !aligned16(weight_chunk) ||
      !aligned16(dz))
    return Q3_ERR_ALIGN;
  tc::Operand A{hidden, false, K}, B{weight_chunk, false, K};
  tc::GemmParams p{};
  p.c0 = dz; p.M = M; p.N = Vc; p.K = K; p.status = status;
  p.labels = labels_eff; p.lse = lse; p.ups = upstream; p.counts = counts; p.rows_per_rank = rows_per_rank;
  p.vocab_start = vocab_start; p.ignore = ignore_index;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == Q3_BF16) return tc::launch_gemm<256, __nv_bfloat16, tc::EPI_CE_GRAD>(A, B, nullptr, p, true, st);
  return tc::launch_gemm<256, __half, tc::EPI_CE_GRAD>(A, B, nullptr, p, false, st);
}

// 1: tiles drawn from a device counter (default), 0: static stride over the grid. Returns the previous policy;
// any other value only queries. Q3_GEMM_TILE_SCHEDULE=static sets the initial policy.
extern "C" int q3_gemm_tile_schedule(int mode) {
  if (mode == 0 || mode == 1) return tc::g_tile_schedule.exchange(mode);
  return tc::g_tile_schedule.load();
}

// 1: two CTAs share every 256-row tile wherever there are at least two 128-row tiles (default), 0: one CTA per
// 128-row tile everywhere. Returns the previous policy; any other value only queries.
extern "C" int q3_gemm_cta_pairs(int mode) {
  if (mode == 0 || mode == 1) return tc::g_cta_pairs.exchange(mode);
  return tc::g_cta_pairs.load();
}
