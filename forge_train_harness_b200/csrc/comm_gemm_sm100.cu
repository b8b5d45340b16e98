// Tensor-parallel GEMMs fused with their sequence-parallel collective, one kernel each (sm_100a, NVLink peer memory).
//
//   gemm_rs  (row-parallel out-proj / FC2 forward, column-parallel dgrad):  Y_q[M/tp, N] = sum_r A_r[M, K_r] B_r[N, K_r]^T
//       Every rank runs the tcgen05 GEMM on its K slice; the epilogue of each 128-row tile is a TMA REDUCE-ADD (bf16) of
//       the staged tile straight into the OWNER rank's output shard in peer memory.  The reduce-scatter is the epilogue:
//       tile i crosses NVLink while tile i+1 is in the tensor core.  (Megatron semantics; the reference has only the
//       all-reduce form, ref/reference/model_minicpm4_8b_tp.py:209-227, 309-311.)
//   ag_gemm  (column-parallel QKV / FC1 forward, row-parallel dgrad):       Y[M, N_r] = gather_q(X_q)[M, K] B_r[N_r, K]^T
//       A few CTAs of the same launch are COPY CTAs: they pull the peers' row shards into this GPU's own gather buffer with
//       non-multicast bulk copies (peer global -> shared -> local global, each remote byte crosses NVLink once) and publish
//       a flag per 128-row block.  The GEMM CTAs start on the local shard and take remote blocks as their flags arrive
//       (bounded acquire-spin), reading A only from LOCAL memory through TMA.  No TMA load with cluster multicast anywhere.
//
// Cross-rank ordering (who may write or read which buffer when) is the caller's flag barrier; see parallel/fused_tp.py.
#include <cuda.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace fth {

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr int CBM = 128, CBN = 256, CBK = 64, CST = 4;
constexpr int kCgThreads = 192;
constexpr int kCgABytes = CBM * CBK * 2, kCgBBytes = CBN * CBK * 2, kCgStage = kCgABytes + kCgBBytes;
constexpr int kCgEpiOff = CST * kCgStage, kCgBarOff = kCgEpiOff + 2 * CBM * 128, kCgSmem = kCgBarOff + 256 + 1024;
constexpr int kCopyPiece = 32768, kCopySlots = 6;  // copy CTAs reuse the pipeline shared memory as a 6 x 32 KiB ring

struct CMaps {
  CUtensorMap m[8];
};

struct CommArgs {
  int mode;           // 1 = reduce-scatter epilogue, 2 = all-gather prologue
  int tp, rank;
  int rows_per_rank;  // M / tp (multiple of 128)
  int n_copy_ctas;    // mode 2
  int epoch;          // mode 2: flag value that marks "block gathered" for this call
  int* flags;         // mode 2: [M / 128] ints in local memory
  const void* peer_x[8];  // mode 2: every rank's gather buffer (row q*rows_per_rank.. of rank q's buffer is its own shard)
  void* local_x;          // mode 2: this rank's gather buffer
  long long row_bytes;    // mode 2: K * 2
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool B_MN>
__global__ void __launch_bounds__(kCgThreads, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CMaps cmaps, const CommArgs ca, int M, int N, int K, float alpha,
                 int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kCgBarOff);
  uint64_t* empty_bar = full_bar + CST;
  uint64_t* tfull_bar = empty_bar + CST;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* copy_bar = tempty_bar + 2;  // [kCopySlots]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(copy_bar + kCopySlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int m_tiles = M / CBM, n_tiles = (N + CBN - 1) / CBN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + CBK - 1) / CBK;
  const int n_copy = (ca.mode == 2) ? ca.n_copy_ctas : 0;
  const bool is_copy_cta = (int)blockIdx.x < n_copy;
  const int tiles_per_rank = ca.rows_per_rank / CBM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CST; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    for (int s = 0; s < kCopySlots; ++s) mbar_init(&copy_bar[s], 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (!is_copy_cta && warp == 1) { tmem_alloc(tmem_slot, 2 * CBN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (is_copy_cta) {
    // ---------------- all-gather copy CTA: one thread drives bulk copies peer -> shared -> local ----------------
    // The CTA's blocks are one flat stream of 32 KiB pieces through a ring of shared-memory slots: loads run up to
    // kCopySlots - 2 pieces ahead of the stores (also across block boundaries); a block's flag is published when its
    // last store has completed.
    if (threadIdx.x == 0) {
      const long long blk_bytes = (long long)CBM * ca.row_bytes;
      const int ppb = (int)((blk_bytes + kCopyPiece - 1) / kCopyPiece);   // pieces per block
      const int n_remote = (ca.tp - 1) * tiles_per_rank;
      int n_mine = 0;
      for (int i = (int)blockIdx.x; i < n_remote; i += n_copy) ++n_mine;
      const int total = n_mine * ppb;
      // piece j -> (remote block index i, offset)
      auto locate = [&](int j, const char*& src, char*& dst, uint32_t& bytes, int& mb, bool& last) {
        const int i = (int)blockIdx.x + (j / ppb) * n_copy;
        const int q = (ca.rank + 1 + i / tiles_per_rank) % ca.tp;
        mb = q * tiles_per_rank + i % tiles_per_rank;
        const long long o = (long long)(j % ppb) * kCopyPiece;
        bytes = (uint32_t)min((long long)kCopyPiece, blk_bytes - o);
        src = reinterpret_cast<const char*>(ca.peer_x[q]) + (long long)mb * blk_bytes + o;
        dst = reinterpret_cast<char*>(ca.local_x) + (long long)mb * blk_bytes + o;
        last = (j % ppb) == ppb - 1;
      };
      auto issue_load = [&](int j) {
        const char* src; char* dst; uint32_t bytes; int mb; bool last;
        locate(j, src, dst, bytes, mb, last);
        const int sl = j % kCopySlots;
        mbar_expect_tx(&copy_bar[sl], bytes);
        bulk_g2s(smem + sl * kCopyPiece, src, bytes, &copy_bar[sl]);
      };
      int loaded = 0;
      for (; loaded < total && loaded < kCopySlots; ++loaded) issue_load(loaded);
      for (int j = 0; j < total; ++j) {
        const char* src; char* dst; uint32_t bytes; int mb; bool last;
        locate(j, src, dst, bytes, mb, last);
        const int sl = j % kCopySlots;
        if (!mbar_wait(&copy_bar[sl], (uint32_t)((j / kCopySlots) & 1), abort_flag, status, kTimeoutPeerFlag)) break;
        bulk_s2g(dst, smem + sl * kCopyPiece, bytes);
        tma_commit_group();
        if (last) {
          tma_wait_group<0>();          // every store of this block has completed
          fence_proxy_async_all();
          __threadfence();
          st_release_gpu(ca.flags + mb, ca.epoch);
        }
        if (j >= 1 && loaded < total) {
          tma_wait_group_read<1>();     // store j-1 has read its slot: reuse it for the next load
          issue_load(loaded);           // loaded == j - 1 + kCopySlots, same slot as piece j - 1
          ++loaded;
        }
      }
      tma_wait_group<0>();
    }
    __syncthreads();
    return;
  }

  const uint32_t tmem_base = *tmem_slot;
  const int cta = (int)blockIdx.x - n_copy, n_ctas = (int)gridDim.x - n_copy;
  // tile -> (m block, n block).  m fastest in groups of 8; with an all-gather prologue the m order starts at the local shard.
  auto tile_coords = [&](int t, int& mb, int& nb) {
    const int group_m = m_tiles < 8 ? m_tiles : 8;
    const int per_group = group_m * n_tiles;
    const int gidx = t / per_group, r = t % per_group;
    const int m_first = gidx * group_m;
    const int gsz = min(group_m, m_tiles - m_first);
    int ml = m_first + r % gsz;
    nb = r / gsz;
    mb = (ca.mode == 2) ? (ml + ca.rank * tiles_per_rank) % m_tiles : (ml + ((ca.rank + 1) % ca.tp) * tiles_per_rank) % m_tiles;
  };

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += n_ctas) {
        int mb, nb;
        tile_coords(t, mb, nb);
        if (ca.mode == 2 && mb / tiles_per_rank != ca.rank) {
          // wait (bounded) until the copy CTAs have gathered this row block into local memory
          const long long t0 = clock64();
          while (ld_acquire_gpu(ca.flags + mb) != ca.epoch) {
            if (*abort_flag || clock64() - t0 > kSpinLimitCycles) {
              report_status(status, kTimeoutPeerFlag);
              *abort_flag = 1;
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) { ok = false; break; }
          unsigned char* sa = smem + stage * kCgStage;
          unsigned char* sb = sa + kCgABytes;
          mbar_expect_tx(&full_bar[stage], kCgStage);
          tma_load_2d(sa, &tmap_a, kb * CBK, mb * CBM, &full_bar[stage]);
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, kb * CBK, nb * CBN, &full_bar[stage]);
          } else {
#pragma unroll
            for (int c = 0; c < CBN / 64; ++c) tma_load_2d(sb + c * 8192, &tmap_b, nb * CBN + c * 64, kb * CBK, &full_bar[stage]);
          }
          if (++stage == CST) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(CBM, CBN, false, B_MN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += n_ctas) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * CBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kCgStage);
          const uint32_t sb = sa + kCgABytes;
#pragma unroll
          for (int kk = 0; kk < CBK / 16; ++kk) {
            const uint64_t adesc = make_smem_desc(sa + kk * 32, 0, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024) : make_smem_desc(sb + kk * 32, 0, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == CST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int q4 = warp % 4;
    const int r_in_tile = q4 * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    unsigned char* stg = smem + kCgEpiOff;
    int acc = 0, buf = 0;
    uint32_t acc_phase = 0;
    for (int t = cta; t < total_tiles; t += n_ctas) {
      int mb, nb;
      tile_coords(t, mb, nb);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * CBN + ((uint32_t)(q4 * 32) << 16);
      // reduce-scatter epilogue: destination = the output shard of the rank that owns these rows
      const int owner = (ca.mode == 1) ? mb / tiles_per_rank : 0;
      const int dst_row = (ca.mode == 1) ? (mb - owner * tiles_per_rank) * CBM : mb * CBM;
#pragma unroll 1
      for (int c = 0; c < CBN / 64; ++c) {
        const int col0 = nb * CBN + c * 64;
        if (col0 >= N) break;
        uint32_t r[64];
        tmem_ld_32x32(taddr + c * 64, r);
        tmem_ld_32x32(taddr + c * 64 + 32, r + 32);
        tmem_wait_ld();
        if (issuer) tma_wait_group_read<1>();
        named_barrier_sync(1, 128);
        unsigned char* row_ptr = stg + buf * (CBM * 128) + r_in_tile * 128;
#pragma unroll
        for (int p8 = 0; p8 < 8; ++p8) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[p8 * 8 + e]) * alpha;
          bf16x8 pk = pack8(f);
          *reinterpret_cast<uint4*>(row_ptr + ((p8 ^ (r_in_tile & 7)) * 16)) = *reinterpret_cast<uint4*>(&pk);
        }
        fence_proxy_async();
        named_barrier_sync(1, 128);
        if (issuer) {
          if (ca.mode == 1) tma_reduce_add_2d(&cmaps.m[owner], stg + buf * (CBM * 128), col0, dst_row);
          else tma_store_2d(&cmaps.m[0], stg + buf * (CBM * 128), col0, dst_row);
          tma_commit_group();
        }
        buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) {
      tma_wait_group<0>();
      __threadfence_system();  // remote reduce-adds are performed before this kernel is seen to finish
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * CBN); }
}

static int cg_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <bool B_MN>
static int launch_comm_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CMaps& cm, const CommArgs& ca, int M, int N, int K,
                            float alpha, int* status, cudaStream_t stream) {
  auto kern = comm_gemm_kernel<B_MN>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kCgSmem) != cudaSuccess) return -20;
    set = true;
  }
  const int tiles = (M / CBM) * ((N + CBN - 1) / CBN);
  int grid = cg_sm_count();  // mode 2 relies on all CTAs being co-resident: one persistent CTA per SM at most
  const int n_copy = ca.mode == 2 ? ca.n_copy_ctas : 0;
  if (tiles + n_copy < grid) grid = tiles + n_copy;
  kern<<<grid, kCgThreads, kCgSmem, stream>>>(ta, tb, cm, ca, M, N, K, alpha, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace fth

using namespace fth;

extern "C" {

// Row-parallel GEMM + reduce-scatter.  a: [M, K] bf16 (K = this rank's slice); b: [N, K] (b_mn = 0) or [K, N] (b_mn = 1);
// out_shards[q]: rank q's [M/tp, N] bf16 output shard in peer-mapped memory, zeroed by its owner before any rank starts.
int fth_gemm_rs(const void* a, long long lda, const void* b, long long ldb, int b_mn, void* const* out_shards, long long ldo,
                int M, int N, int K, int tp, int rank, float alpha, int* status, cudaStream_t stream) {
  if (tp < 1 || tp > 8 || M % (CBM * tp) || N % 8) return -2;
  CUtensorMap ta, tb;
  CMaps cm;
  int r = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, CBM, CBK);
  if (r) return r;
  r = b_mn ? make_tmap_bf16_2d(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, CBK, 64)
           : make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, CBN, CBK);
  if (r) return r;
  for (int q = 0; q < 8; ++q) {
    r = make_tmap_bf16_2d(&cm.m[q], out_shards[q < tp ? q : 0], (uint64_t)(M / tp), (uint64_t)N, (uint64_t)ldo, CBM, 64);
    if (r) return r;
  }
  CommArgs ca = {};
  ca.mode = 1; ca.tp = tp; ca.rank = rank; ca.rows_per_rank = M / tp;
  return b_mn ? launch_comm_gemm<true>(ta, tb, cm, ca, M, N, K, alpha, status, stream)
              : launch_comm_gemm<false>(ta, tb, cm, ca, M, N, K, alpha, status, stream);
}

// All-gather + column-parallel GEMM.  gather[q]: rank q's [M, K] bf16 gather buffer (peer mapped); each rank has written
// its own row shard [rank*M/tp, (rank+1)*M/tp) into its own buffer.  On return (stream order) this rank's buffer holds all
// M rows and `out` [M, N] = gather x b^T.  flags: [M/128] ints (local), epoch: a value not yet present in them.
int fth_ag_gemm(void* const* gather, long long ldx, const void* b, long long ldb, int b_mn, void* out, long long ldo, int M, int N,
                int K, int tp, int rank, int n_copy_ctas, int* flags, int epoch, float alpha, int* status, cudaStream_t stream) {
  if (tp < 1 || tp > 8 || M % (CBM * tp) || N % 8 || ldx != K) return -2;
  CUtensorMap ta, tb;
  CMaps cm;
  int r = make_tmap_bf16_2d(&ta, gather[rank], (uint64_t)M, (uint64_t)K, (uint64_t)ldx, CBM, CBK);
  if (r) return r;
  r = b_mn ? make_tmap_bf16_2d(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, CBK, 64)
           : make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, CBN, CBK);
  if (r) return r;
  for (int q = 0; q < 8; ++q) {
    r = make_tmap_bf16_2d(&cm.m[q], out, (uint64_t)M, (uint64_t)N, (uint64_t)ldo, CBM, 64);
    if (r) return r;
  }
  CommArgs ca = {};
  ca.mode = 2; ca.tp = tp; ca.rank = rank; ca.rows_per_rank = M / tp;
  {
    const int n_remote = (tp - 1) * (M / tp / CBM);
    int want = n_copy_ctas > 0 ? n_copy_ctas : 16;
    if (want > n_remote) want = n_remote;
    ca.n_copy_ctas = tp > 1 ? want : 0;
  }
  if (tp == 1) ca.mode = 0;
  ca.epoch = epoch; ca.flags = flags;
  for (int q = 0; q < 8; ++q) ca.peer_x[q] = gather[q < tp ? q : 0];
  ca.local_x = gather[rank];
  ca.row_bytes = (long long)K * 2;
  return b_mn ? launch_comm_gemm<true>(ta, tb, cm, ca, M, N, K, alpha, status, stream)
              : launch_comm_gemm<false>(ta, tb, cm, ca, M, N, K, alpha, status, stream);
}

}  // extern "C"
