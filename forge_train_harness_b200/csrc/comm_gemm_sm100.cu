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

#include "gemm_pipe.cuh"

namespace fth {

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr int CBN = 256;
constexpr int kCopyPiece = 32768, kCopySlots = 6;  // copy CTAs reuse the pipeline shared memory as a 6 x 32 KiB ring
template <int CTAS> struct CgCfg { static constexpr int kStages = CTAS == 2 ? 6 : 4; };  // 192 KiB of ring either way

struct CMaps {
  CUtensorMap m[8];
};

struct CommArgs {
  int mode;           // 1 = reduce-scatter epilogue, 2 = all-gather prologue, 0 = plain GEMM (tp = 1)
  int tp, rank;
  int rows_per_rank;  // M / tp (multiple of 128)
  int n_copy_units;   // mode 2: CTAs (or CTA pairs) that only copy
  int epoch;          // mode 2, host-sequenced form: flag value that marks "block gathered" for this call
  int* flags;         // mode 2: [M / 128] ints in local memory
  const void* peer_x[8];  // mode 2: every rank's gather buffer (row q*rows_per_rank.. of rank q's buffer is its own shard)
  void* local_x;          // mode 2: this rank's gather buffer
  long long row_bytes;    // mode 2: K * 2
  // mode 2, self-sequenced form (ctr != nullptr): the call number lives on the device, and "my shard is written" is
  // announced to the peers by the kernel itself instead of by a separate barrier launch before it.
  int* ctr;               // [2] local: {calls completed, CTAs of this call that are done}
  int* ready_local;       // [8] local, written by peers: ready_local[q] = last call for which rank q's shard is in place
  int* ready_peer[8];     // the same array on every rank
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
__device__ __forceinline__ void st_release_sys_s32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool B_MN, int CTAS>
__global__ void __launch_bounds__(kGemmThreads, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CMaps cmaps, const CommArgs ca, int M, int N, int K, float alpha,
                 int* __restrict__ status) {
  constexpr int STAGES = CgCfg<CTAS>::kStages;
  using S = GemmSmem<CBN, STAGES, CTAS, kCopySlots>;
  constexpr int BNH = CBN / CTAS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = align_smem_1024(smem_raw);
  PipeBars<STAGES, kCopySlots> bars(smem + S::kBarOffset);
  volatile int* abort_flag = bars.abort_flag;
  uint64_t* copy_bar = bars.extra;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const int unit_all = (int)blockIdx.x / CTAS, n_units_all = (int)gridDim.x / CTAS;
  const int blocks = M / BM;                          // 128-row blocks (flags, ownership)
  const int m_tiles = blocks / CTAS, n_tiles = (N + CBN - 1) / CBN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  const int n_copy = (ca.mode == 2) ? ca.n_copy_units : 0;
  const bool is_copy_cta = unit_all < n_copy;
  const int blocks_per_rank = ca.rows_per_rank / BM;
  // this call's number: from the device counter (self-sequenced) or from the host
  const int epoch = (ca.mode == 2 && ca.ctr != nullptr) ? ld_volatile_s32(ca.ctr) + 1 : ca.epoch;

  const uint32_t tmem_base = pipe_setup<CBN, STAGES, CTAS, kCopySlots>(bars, !is_copy_cta);

  if (ca.mode == 2 && ca.ctr != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    // This rank's shard was written by an earlier kernel of this stream: tell every peer it may pull it.
    __threadfence_system();
    for (int q = 0; q < ca.tp; ++q)
      if (q != ca.rank) st_release_sys_s32(ca.ready_peer[q] + ca.rank, epoch);
  }

  if (is_copy_cta) {
    // ---------------- all-gather copy CTA: one thread drives bulk copies peer -> shared -> local ----------------
    // The CTA's blocks are one flat stream of 32 KiB pieces through a ring of shared-memory slots: loads run up to
    // kCopySlots - 2 pieces ahead of the stores (also across block boundaries); a block's flag is published when its
    // last store has completed.
    if (threadIdx.x == 0) {
      const int me = (int)blockIdx.x, n_me = n_copy * CTAS;   // every CTA of a copy unit copies
      const long long blk_bytes = (long long)BM * ca.row_bytes;
      const int ppb = (int)((blk_bytes + kCopyPiece - 1) / kCopyPiece);   // pieces per block
      const int n_remote = (ca.tp - 1) * blocks_per_rank;
      int n_mine = 0;
      for (int i = me; i < n_remote; i += n_me) ++n_mine;
      const int total = n_mine * ppb;
      unsigned peers_ready = 0;
      bool ok = true;
      // piece j -> (remote block index i, offset)
      auto locate = [&](int j, const char*& src, char*& dst, uint32_t& bytes, int& mb, int& q, bool& last) {
        const int i = me + (j / ppb) * n_me;
        q = (ca.rank + 1 + i / blocks_per_rank) % ca.tp;
        mb = q * blocks_per_rank + i % blocks_per_rank;
        const long long o = (long long)(j % ppb) * kCopyPiece;
        bytes = (uint32_t)min((long long)kCopyPiece, blk_bytes - o);
        src = reinterpret_cast<const char*>(ca.peer_x[q]) + (long long)mb * blk_bytes + o;
        dst = reinterpret_cast<char*>(ca.local_x) + (long long)mb * blk_bytes + o;
        last = (j % ppb) == ppb - 1;
      };
      auto issue_load = [&](int j) {
        const char* src; char* dst; uint32_t bytes; int mb, q; bool last;
        locate(j, src, dst, bytes, mb, q, last);
        if (ca.ctr != nullptr && !(peers_ready & (1u << q))) {
          // bounded wait until rank q has announced its shard for this call
          const long long t0 = clock64();
          while (ld_acquire_sys_s32(ca.ready_local + q) - epoch < 0) {
            if (*abort_flag || clock64() - t0 > kSpinLimitCycles) {
              report_status(status, kTimeoutPeerFlag);
              *abort_flag = 1;
              ok = false;
              return;
            }
            __nanosleep(64);
          }
          peers_ready |= 1u << q;
        }
        const int sl = j % kCopySlots;
        mbar_expect_tx(&copy_bar[sl], bytes);
        bulk_g2s(smem + sl * kCopyPiece, src, bytes, &copy_bar[sl]);
      };
      int loaded = 0;
      for (; loaded < total && loaded < kCopySlots && ok; ++loaded) issue_load(loaded);
      for (int j = 0; j < total && ok; ++j) {
        const char* src; char* dst; uint32_t bytes; int mb, q; bool last;
        locate(j, src, dst, bytes, mb, q, last);
        const int sl = j % kCopySlots;
        if (!mbar_wait(&copy_bar[sl], (uint32_t)((j / kCopySlots) & 1), abort_flag, status, kTimeoutPeerFlag)) break;
        bulk_s2g(dst, smem + sl * kCopyPiece, bytes);
        tma_commit_group();
        if (last) {
          tma_wait_group<0>();          // every store of this block has completed
          fence_proxy_async_all();
          __threadfence();
          st_release_gpu(ca.flags + mb, epoch);
        }
        if (j >= 1 && loaded < total) {
          tma_wait_group_read<1>();     // store j-1 has read its slot: reuse it for the next load
          issue_load(loaded);           // loaded == j - 1 + kCopySlots, same slot as piece j - 1
          ++loaded;
        }
      }
      tma_wait_group<0>();
    }
  } else {
    const int unit = unit_all - n_copy, n_units = n_units_all - n_copy;
    // tile -> (m tile, n block).  m fastest in groups of 8 row blocks; the m order starts at the local shard (all-gather)
    // or at the next rank's rows (reduce-scatter: the ranks do not all add into the same owner at once).
    const int first_blk = (ca.mode == 2) ? ca.rank * blocks_per_rank : ((ca.rank + 1) % ca.tp) * blocks_per_rank;
    auto tile_coords = [&](int t, int& mt, int& nb) {
      const int group_m = m_tiles < 8 / CTAS ? m_tiles : 8 / CTAS;
      const int per_group = group_m * n_tiles;
      const int gidx = t / per_group, r = t % per_group;
      const int m_first = gidx * group_m;
      const int gsz = min(group_m, m_tiles - m_first);
      const int ml = m_first + r % gsz;
      nb = r / gsz;
      mt = (ml + first_blk / CTAS) % m_tiles;
    };

    if (warp == 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = unit; t < total_tiles && ok; t += n_units) {
          int mt, nb;
          tile_coords(t, mt, nb);
          const int blk = mt * CTAS + (int)cta_rank;  // this CTA's 128-row block
          if (ca.mode == 2 && blk / blocks_per_rank != ca.rank) {
            // wait (bounded) until the copy CTAs have gathered this row block into local memory
            const long long t0 = clock64();
            while (ld_acquire_gpu(ca.flags + blk) != epoch) {
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
            if (!mbar_wait(&bars.empty[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) { ok = false; break; }
            unsigned char* sa = smem + stage * S::kStageBytes;
            pipe_load_stage<CBN, CTAS, false, B_MN>(sa, sa + S::kABytes, &tmap_a, &tmap_b, kb * BK, blk * BM,
                                                    nb * CBN + (int)cta_rank * BNH, &bars.full[stage], cta_rank);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (cta_rank == 0 && elect_one()) {
        int stage = 0, acc = 0;
        uint32_t phase = 0, acc_phase = 0;
        bool ok = true;
        for (int t = unit; t < total_tiles && ok; t += n_units) {
          if (!mbar_wait(&bars.tempty[acc], acc_phase ^ 1, abort_flag, status, kTimeoutTmemEmpty)) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * CBN;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&bars.full[stage], phase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
            pipe_mma_stage<CBN, CTAS, false, B_MN>(d_tmem, sa, sa + S::kABytes, kb == 0);
            pipe_commit<CTAS>(&bars.empty[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          pipe_commit<CTAS>(&bars.tfull[acc]);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
      __syncwarp();
    } else {
      const int q4 = warp % 4;
      const int r_in_tile = q4 * 32 + lane;
      const bool issuer = (threadIdx.x == 64);
      unsigned char* stg = smem + S::kEpiOffset;
      int acc = 0, buf = 0;
      uint32_t acc_phase = 0;
      for (int t = unit; t < total_tiles; t += n_units) {
        int mt, nb;
        tile_coords(t, mt, nb);
        const int blk = mt * CTAS + (int)cta_rank;
        if (!mbar_wait(&bars.tfull[acc], acc_phase, abort_flag, status, kTimeoutTmemFull)) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * CBN + ((uint32_t)(q4 * 32) << 16);
        // reduce-scatter epilogue: destination = the output shard of the rank that owns these rows
        const int owner = (ca.mode == 1) ? blk / blocks_per_rank : 0;
        const int dst_row = (ca.mode == 1) ? (blk - owner * blocks_per_rank) * BM : blk * BM;
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
          pipe_stage_row<false>(stg + buf * (BM * 128) + r_in_tile * 128, r_in_tile, r, alpha);
          fence_proxy_async();
          named_barrier_sync(1, 128);
          if (issuer) {
            if (ca.mode == 1) tma_reduce_add_2d(&cmaps.m[owner], stg + buf * (BM * 128), col0, dst_row);
            else tma_store_2d(&cmaps.m[0], stg + buf * (BM * 128), col0, dst_row);
            tma_commit_group();
          }
          buf ^= 1;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) pipe_release_acc<CTAS>(&bars.tempty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (issuer) {
        tma_wait_group<0>();
        __threadfence_system();  // remote reduce-adds are performed before this kernel is seen to finish
      }
    }
  }

  pipe_teardown<CBN, CTAS>(abort_flag, tmem_base, !is_copy_cta);

  if (ca.mode == 2 && ca.ctr != nullptr && threadIdx.x == 0) {
    // the last CTA to get here closes the call: every CTA read the counter before taking its ticket
    __threadfence();
    const int ticket = atomicAdd(ca.ctr + 1, 1);
    if (ticket == (int)gridDim.x - 1) {
      ca.ctr[1] = 0;
      __threadfence();
      ca.ctr[0] = epoch;
    }
  }
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

template <bool B_MN, int CTAS>
static int launch_comm_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CMaps& cm, CommArgs ca, int n_copy_ctas, int M, int N,
                            int K, float alpha, int* status, cudaStream_t stream) {
  using S = GemmSmem<CBN, CgCfg<CTAS>::kStages, CTAS, kCopySlots>;
  auto kern = comm_gemm_kernel<B_MN, CTAS>;
  static bool set = false;
  static int max_units = 0;
  if (!set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return -20;
    max_units = pipe_max_units<CTAS>(kern, S::kTotal, cg_sm_count());
    set = true;
  }
  const int tiles = (M / (BM * CTAS)) * ((N + CBN - 1) / CBN);
  // mode 2 relies on all CTAs being co-resident (GEMM CTAs wait for copy CTAs): never more units than fit at once
  ca.n_copy_units = ca.mode == 2 ? (n_copy_ctas + CTAS - 1) / CTAS : 0;
  int grid_units = max_units;
  if (tiles + ca.n_copy_units < grid_units) grid_units = tiles + ca.n_copy_units;
  if (grid_units <= ca.n_copy_units) return -4;
  if (pipe_launch<CTAS>(kern, grid_units, S::kTotal, stream, ta, tb, cm, ca, M, N, K, alpha, status) != cudaSuccess) {
    cudaGetLastError();
    return -21;
  }
  return 0;
}

static int dispatch_comm_gemm(const void* a, long long lda, const void* b, long long ldb, int b_mn, const CMaps& cm, const CommArgs& ca,
                              int n_copy_ctas, int M, int N, int K, float alpha, int* status, cudaStream_t stream) {
  const bool pair = (M % (2 * BM)) == 0;  // a CTA pair works on 256 rows
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  if (r) return r;
  r = b_mn ? make_tmap_bf16_2d(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64)
           : make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? CBN / 2 : CBN, BK);
  if (r) return r;
  if (pair) return b_mn ? launch_comm_gemm<true, 2>(ta, tb, cm, ca, n_copy_ctas, M, N, K, alpha, status, stream)
                        : launch_comm_gemm<false, 2>(ta, tb, cm, ca, n_copy_ctas, M, N, K, alpha, status, stream);
  return b_mn ? launch_comm_gemm<true, 1>(ta, tb, cm, ca, n_copy_ctas, M, N, K, alpha, status, stream)
              : launch_comm_gemm<false, 1>(ta, tb, cm, ca, n_copy_ctas, M, N, K, alpha, status, stream);
}

}  // namespace fth

using namespace fth;

extern "C" {

// Row-parallel GEMM + reduce-scatter.  a: [M, K] bf16 (K = this rank's slice); b: [N, K] (b_mn = 0) or [K, N] (b_mn = 1);
// out_shards[q]: rank q's [M/tp, N] bf16 output shard in peer-mapped memory, zeroed by its owner before any rank starts.
int fth_gemm_rs(const void* a, long long lda, const void* b, long long ldb, int b_mn, void* const* out_shards, long long ldo,
                int M, int N, int K, int tp, int rank, float alpha, int* status, cudaStream_t stream) {
  if (tp < 1 || tp > 8 || M % (BM * tp) || N % 8) return -2;
  CMaps cm;
  for (int q = 0; q < 8; ++q) {
    int r = make_tmap_bf16_2d(&cm.m[q], out_shards[q < tp ? q : 0], (uint64_t)(M / tp), (uint64_t)N, (uint64_t)ldo, BM, 64);
    if (r) return r;
  }
  CommArgs ca = {};
  ca.mode = 1; ca.tp = tp; ca.rank = rank; ca.rows_per_rank = M / tp;
  return dispatch_comm_gemm(a, lda, b, ldb, b_mn, cm, ca, 0, M, N, K, alpha, status, stream);
}

// All-gather + column-parallel GEMM.  gather[q]: rank q's [M, K] bf16 gather buffer (peer mapped); each rank has written
// its own row shard [rank*M/tp, (rank+1)*M/tp) into its own buffer.  On return (stream order) this rank's buffer holds all
// M rows and `out` [M, N] = gather x b^T.  flags: [M/128] ints (local).
// Two ways to sequence calls:
//   host-sequenced  (ctr == nullptr): `epoch` is a value not yet present in `flags`, and the caller has made sure (a flag
//                   barrier) that every rank's shard is in place before any rank's kernel starts;
//   self-sequenced  (ctr != nullptr): ctr[2] (local, zero-initialised) counts the calls on the device; ready[q] points at
//                   rank q's 8-int "shard in place" array (peer mapped, zero-initialised).  The kernel announces its own
//                   shard to the peers and its copy CTAs wait (bounded) for each peer's announcement before pulling from
//                   it, so no barrier launch precedes the call and the local tiles start at once.  Every rank must make
//                   the same sequence of self-sequenced calls on one (ctr, ready, flags) set.
int fth_ag_gemm(void* const* gather, long long ldx, const void* b, long long ldb, int b_mn, void* out, long long ldo, int M, int N,
                int K, int tp, int rank, int n_copy_ctas, int* flags, int epoch, int* ctr, void* const* ready, float alpha,
                int* status, cudaStream_t stream) {
  if (tp < 1 || tp > 8 || M % (BM * tp) || N % 8 || ldx != K) return -2;
  CMaps cm;
  for (int q = 0; q < 8; ++q) {
    int r = make_tmap_bf16_2d(&cm.m[q], out, (uint64_t)M, (uint64_t)N, (uint64_t)ldo, BM, 64);
    if (r) return r;
  }
  CommArgs ca = {};
  ca.mode = 2; ca.tp = tp; ca.rank = rank; ca.rows_per_rank = M / tp;
  int n_copy = 0;
  if (tp > 1) {
    const int n_remote = (tp - 1) * (M / tp / BM);
    n_copy = n_copy_ctas > 0 ? n_copy_ctas : 16;
    if (n_copy > n_remote) n_copy = n_remote;
  } else {
    ca.mode = 0;
  }
  ca.epoch = epoch; ca.flags = flags;
  for (int q = 0; q < 8; ++q) ca.peer_x[q] = gather[q < tp ? q : 0];
  ca.local_x = gather[rank];
  ca.row_bytes = (long long)K * 2;
  if (ctr != nullptr && tp > 1) {
    if (ready == nullptr) return -2;
    ca.ctr = ctr;
    for (int q = 0; q < 8; ++q) ca.ready_peer[q] = reinterpret_cast<int*>(ready[q < tp ? q : 0]);
    ca.ready_local = ca.ready_peer[rank];
  }
  return dispatch_comm_gemm(gather[rank], ldx, b, ldb, b_mn, cm, ca, n_copy, M, N, K, alpha, status, stream);
}

}  // extern "C"
