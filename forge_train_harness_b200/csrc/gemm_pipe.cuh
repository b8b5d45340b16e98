// The tcgen05 GEMM pipeline shared by the plain bf16 GEMM (gemm_sm100.cu) and the GEMMs fused with a tensor-parallel
// collective (comm_gemm_sm100.cu): shared-memory layout, barrier set-up, one ring stage of TMA loads, one ring stage of
// MMAs, the commits that hand stages and accumulators on, and the teardown.  CTAS = 1 is one CTA per 128 x BN tile;
// CTAS = 2 is a CTA pair (tcgen05.mma.cta_group::2) on a 256 x BN tile:
//   * each CTA loads its own 128 rows of A and its own BN/2 rows of B with unicast TMA (no multicast load anywhere),
//   * the ring's "full" barriers live in CTA rank 0 and count the bytes of both CTAs' loads,
//   * CTA rank 0 issues the MMAs for both; one multicast tcgen05.commit signals "stage free" / "accumulator full" in both,
//   * "accumulator empty" collects the eight epilogue warps of the pair in rank 0.
// Every wait is bounded (sm100_ptx.cuh::mbar_wait); a CTA of a pair never exits before its peer (cluster barrier).
#pragma once
#include "sm100_ptx.cuh"

namespace fth {

constexpr int BM = 128;  // rows of A (and accumulator lanes) per CTA
constexpr int BK = 64;   // k extent of one ring stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;  // warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue

template <int BN, int STAGES, int CTAS = 1, int EXTRA_BARS = 0>
struct GemmSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = (BN / CTAS) * BK * 2;  // a CTA of a pair holds half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = STAGES * kStageBytes;  // two 128-row x 128-byte staging buffers
  static constexpr int kEpiBytes = 2 * BM * 128;
  static constexpr int kBarOffset = kEpiOffset + kEpiBytes;
  static constexpr int kNumBars = 2 * STAGES + 4 + EXTRA_BARS;
  static constexpr int kTotal = kBarOffset + ((kNumBars * 8 + 16 + 127) / 128) * 128 + 1024;  // + barriers + alignment slack
};

// Views into the barrier block at the end of the CTA's shared memory.
template <int STAGES, int EXTRA_BARS = 0>
struct PipeBars {
  uint64_t* full;     // [STAGES] a stage's operands have landed
  uint64_t* empty;    // [STAGES] the MMAs that read a stage are done
  uint64_t* tfull;    // [2] an accumulator is complete
  uint64_t* tempty;   // [2] an accumulator has been drained by the epilogue
  uint64_t* extra;    // [EXTRA_BARS] for the kernel's own use
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  __device__ explicit PipeBars(unsigned char* base) {
    full = reinterpret_cast<uint64_t*>(base);
    empty = full + STAGES;
    tfull = empty + STAGES;
    tempty = tfull + 2;
    extra = tempty + 2;
    tmem_slot = reinterpret_cast<uint32_t*>(extra + EXTRA_BARS);
    abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  }
};

__device__ __forceinline__ unsigned char* align_smem_1024(unsigned char* raw) {
  return reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
}

// Barrier initialisation + tensor-memory allocation (2 accumulator stages of BN columns) + the first CTA-wide (pair-wide)
// synchronisation.  `with_tmem` is false for CTAs that run no MMA (copy CTAs of the all-gather kernel).  Returns the
// tensor-memory base column.
template <int BN, int STAGES, int CTAS, int EXTRA_BARS>
__device__ __forceinline__ uint32_t pipe_setup(PipeBars<STAGES, EXTRA_BARS>& b, bool with_tmem) {
  const int warp = threadIdx.x / 32;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&b.full[s], 1);
      mbar_init(&b.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&b.tfull[a], 1);
      mbar_init(&b.tempty[a], 4 * CTAS);  // one arrival per epilogue warp (of both CTAs of a pair)
    }
    for (int s = 0; s < EXTRA_BARS; ++s) mbar_init(&b.extra[s], 1);
    *b.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (with_tmem && warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_pair(b.tmem_slot, 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(b.tmem_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  return with_tmem ? *b.tmem_slot : 0u;
}

// Producer thread: the TMA loads of one ring stage.  `row_a` / `row_b` are THIS CTA's first row of A (128 rows) and of B
// (BN / CTAS rows); `kcol` is the k offset in elements.  Operands are K-major ([rows, K]) or MN-major ([K, rows]).
template <int BN, int CTAS, bool A_MN, bool B_MN>
__device__ __forceinline__ void pipe_load_stage(unsigned char* sa, unsigned char* sb, const CUtensorMap* tmap_a,
                                                const CUtensorMap* tmap_b, int kcol, int row_a, int row_b,
                                                uint64_t* full_bar, uint32_t cta_rank) {
  constexpr int BNH = BN / CTAS;
  constexpr uint32_t kStageBytes = BM * BK * 2 + BNH * BK * 2;
  if constexpr (CTAS == 2) {
    // rank 0's barrier counts the bytes of both CTAs; a peer's bytes may land before the expectation is posted
    const uint32_t fb = map_to_cta(full_bar, 0);
    if (cta_rank == 0) mbar_expect_tx(full_bar, 2 * kStageBytes);
    if constexpr (!A_MN) {
      tma_load_2d_pair(sa, tmap_a, kcol, row_a, fb);
    } else {
#pragma unroll
      for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * 8192, tmap_a, row_a + c * 64, kcol, fb);
    }
    if constexpr (!B_MN) {
      tma_load_2d_pair(sb, tmap_b, kcol, row_b, fb);
    } else {
#pragma unroll
      for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(sb + c * 8192, tmap_b, row_b + c * 64, kcol, fb);
    }
  } else {
    mbar_expect_tx(full_bar, kStageBytes);
    if constexpr (!A_MN) {
      tma_load_2d(sa, tmap_a, kcol, row_a, full_bar);
    } else {
#pragma unroll
      for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, tmap_a, row_a + c * 64, kcol, full_bar);
    }
    if constexpr (!B_MN) {
      tma_load_2d(sb, tmap_b, kcol, row_b, full_bar);
    } else {
#pragma unroll
      for (int c = 0; c < BNH / 64; ++c) tma_load_2d(sb + c * 8192, tmap_b, row_b + c * 64, kcol, full_bar);
    }
  }
}

// MMA thread (CTA rank 0 of a pair): the four k = 16 MMAs of one ring stage into accumulator `d_tmem`.
template <int BN, int CTAS, bool A_MN, bool B_MN>
__device__ __forceinline__ void pipe_mma_stage(uint32_t d_tmem, uint32_t sa, uint32_t sb, bool first_stage) {
  constexpr uint32_t idesc = make_idesc_bf16(BM * CTAS, BN, A_MN, B_MN);
#pragma unroll
  for (int kk = 0; kk < BK / 16; ++kk) {
    const uint64_t adesc = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024) : make_smem_desc(sa + kk * 32, 0, 1024);
    const uint64_t bdesc = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024) : make_smem_desc(sb + kk * 32, 0, 1024);
    const uint32_t acc = (first_stage && kk == 0) ? 0u : 1u;
    if constexpr (CTAS == 2) umma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, acc);
    else umma_bf16_ss(d_tmem, adesc, bdesc, idesc, acc);
  }
}
// "These MMAs are done" on a barrier at the same shared-memory offset of every CTA of the unit.
template <int CTAS>
__device__ __forceinline__ void pipe_commit(uint64_t* bar) {
  if constexpr (CTAS == 2) umma_commit_pair(bar, 3);
  else umma_commit(bar);
}
// One epilogue warp has drained its quarter of an accumulator (lane 0 calls, after tcgen05.fence::before_thread_sync).
template <int CTAS>
__device__ __forceinline__ void pipe_release_acc(uint64_t* tempty_bar) {
  if constexpr (CTAS == 2) mbar_arrive_cluster(map_to_cta(tempty_bar, 0));
  else mbar_arrive(tempty_bar);
}

// End of the kernel: if a wait gave up, let TMA copies that were already issued land before the shared memory is handed
// to another CTA (bounded delay, no barrier that could itself hang); then free the tensor memory.
template <int BN, int CTAS>
__device__ __forceinline__ void pipe_teardown(volatile int* abort_flag, uint32_t tmem_base, bool with_tmem) {
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if constexpr (CTAS == 2) cluster_sync_all();  // no CTA leaves while its peer may still signal its barriers
  if (with_tmem && threadIdx.x / 32 == 1) {
    tc_fence_after();
    if constexpr (CTAS == 2) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
}

// Epilogue helper: 32 lanes x (64 bf16 | 32 fp32) accumulator columns -> one 128-byte row of a 128B-swizzled staging tile.
template <bool OUT_F32>
__device__ __forceinline__ void pipe_stage_row(unsigned char* row_ptr, int r_in_tile, const uint32_t* r, float alpha) {
#pragma unroll
  for (int p8 = 0; p8 < 8; ++p8) {
    uint4 v;
    if constexpr (OUT_F32) {
      v.x = __float_as_uint(__uint_as_float(r[p8 * 4 + 0]) * alpha);
      v.y = __float_as_uint(__uint_as_float(r[p8 * 4 + 1]) * alpha);
      v.z = __float_as_uint(__uint_as_float(r[p8 * 4 + 2]) * alpha);
      v.w = __float_as_uint(__uint_as_float(r[p8 * 4 + 3]) * alpha);
    } else {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[p8 * 8 + e]) * alpha;
      bf16x8 pk = pack8(f);
      v = *reinterpret_cast<uint4*>(&pk);
    }
    *reinterpret_cast<uint4*>(row_ptr + ((p8 ^ (r_in_tile & 7)) * 16)) = v;
  }
}

// Cluster-aware launch: `grid_units` CTAs or CTA pairs.
template <int CTAS, typename Kern, typename... Args>
static inline cudaError_t pipe_launch(Kern kern, int grid_units, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_units * CTAS);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = CTAS;
  at.val.clusterDim.y = 1;
  at.val.clusterDim.z = 1;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// How many CTAs (CTAS = 1) or CTA pairs (CTAS = 2) of `kern` can be resident at once.
template <int CTAS, typename Kern>
static inline int pipe_max_units(Kern kern, size_t smem, int sm_count) {
  if (CTAS == 1) return sm_count;
  cudaLaunchConfig_t q = {};
  q.gridDim = dim3(sm_count / 2 * 2);
  q.blockDim = dim3(kGemmThreads);
  q.dynamicSmemBytes = smem;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = 2;
  at.val.clusterDim.y = 1;
  at.val.clusterDim.z = 1;
  q.attrs = &at;
  q.numAttrs = 1;
  int n_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&n_clusters, kern, &q) != cudaSuccess || n_clusters <= 0) {
    cudaGetLastError();
    n_clusters = sm_count / 2;
  }
  return n_clusters;
}

}  // namespace fth
