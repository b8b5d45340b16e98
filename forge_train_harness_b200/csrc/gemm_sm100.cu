// Persistent warp-specialised bf16 GEMM for sm_100a: TMA (unicast) -> 128B-swizzled shared memory ->
// tcgen05.mma with fp32 accumulators in tensor memory -> tcgen05.ld epilogue.
//
//   C[M,N] (op)= alpha * sum_k A(m,k) * B(n,k)
//
// Each operand is either K-major (stored [rows = M|N, cols = K], K contiguous) or MN-major (stored
// [rows = K, cols = M|N]), which covers the three GEMMs of a linear layer without any transpose copy:
//   forward  Y  = X W^T      A = X  [M,K]  K-major    B = W  [N,K]  K-major    -> bf16
//   dgrad    dX = dY W       A = dY [M,N'] K-major    B = W  [N',K'] MN-major  -> bf16
//   wgrad    dW += dY^T X    A = dY [T,N'] MN-major   B = X  [T,K'] MN-major   -> fp32, accumulated in place
// These replace every torch.matmul -> cuBLAS call of the reference (forward.py:83,195,198,300;
// backward.py:79,90,389,394); the wgrad epilogue adds straight into the fp32 main_grad buffer, which the
// reference does with a bf16 GEMM followed by .float() and add_ (backward.py:90).
//
// CTA = 6 warps: warp 0 TMA producer, warp 1 MMA issuer (one elected thread) and TMEM owner, warps 2-5
// epilogue (one TMEM lane quarter each).  Tile 128 x BN x 64, 4-6 stage ring, two accumulator stages
// (2 x BN <= 512 TMEM columns) so the epilogue of tile i overlaps the mainloop of tile i+1.  Ragged M / N / K
// are handled by TMA zero fill on loads and predicated stores.  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <tuple>

#include "sm100_ptx.cuh"

namespace fth {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGemmThreads = 192;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = STAGES * kStageBytes;  // two 128-row x 128-byte staging buffers
  static constexpr int kEpiBytes = 2 * BM * 128;
  static constexpr int kBarOffset = kEpiOffset + kEpiBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // + barriers + alignment slack
};

enum EpiMode : int { kEpiBf16 = 0, kEpiF32Accum = 1, kEpiF32Store = 2 };

template <int BN, int STAGES, bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, int M, int N, int K, float alpha, int accumulate,
                 int group_m, int k_splits, int* __restrict__ status) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  // split-K (accumulating fp32 epilogue only): work item = (k split, tile); every split reduce-adds into C
  const int mn_tiles = m_tiles * n_tiles;
  const int total_tiles = mn_tiles * k_splits;
  const int k_blocks_all = (K + BK - 1) / BK;
  const int k_per_split = (k_blocks_all + k_splits - 1) / k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (m_blk, n_blk): groups of `group_m` row blocks, m fastest inside a group, so that
  // concurrently running CTAs share a few B tiles and a few A tiles out of L2.
  auto tile_coords = [&](int t_all, int& mb, int& nb) {
    const int t = t_all % mn_tiles;
    int per_group = group_m * n_tiles;
    int gidx = t / per_group, r = t % per_group;
    int m_first = gidx * group_m;
    int gsz = min(group_m, m_tiles - m_first);
    mb = m_first + r % gsz;
    nb = r / gsz;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, mb, nb);
        const int kb0 = (t / mn_tiles) * k_per_split;
        const int kb1 = min(kb0 + k_per_split, k_blocks_all);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) { ok = false; break; }
          unsigned char* sa = smem + stage * S::kStageBytes;
          unsigned char* sb = sa + S::kABytes;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, kb * BK, mb * BM, &full_bar[stage]);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &tmap_a, mb * BM + c * 64, kb * BK, &full_bar[stage]);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, kb * BK, nb * BN, &full_bar[stage]);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tmap_b, nb * BN + c * 64, kb * BK, &full_bar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb0 = (t / mn_tiles) * k_per_split;
        const int kb1 = min(kb0 + k_per_split, k_blocks_all);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024) : make_smem_desc(sa + kk * 32, 0, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024) : make_smem_desc(sb + kk * 32, 0, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    // TMEM -> registers -> 128B-swizzled shared staging -> TMA store (bf16) or TMA reduce-add (fp32 accumulate).
    // One chunk is 128 rows x 128 bytes (64 bf16 or 32 fp32 columns); two staging buffers alternate.
    const int q = warp % 4;  // TMEM lane quarter this warp may read
    const int r_in_tile = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    constexpr int CW = OUT_F32 ? 32 : 64;  // columns per chunk
    unsigned char* stg = smem + S::kEpiOffset;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, mb, nb);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / CW; ++c) {
        const int col0 = nb * BN + c * CW;
        if (col0 >= N) break;  // uniform across the epilogue warps
        uint32_t r[CW];
        tmem_ld_32x32(taddr + c * CW, r);
        if constexpr (CW == 64) tmem_ld_32x32(taddr + c * CW + 32, r + 32);
        tmem_wait_ld();
        if (issuer) tma_wait_group_read<1>();  // the store that last used this buffer has read it
        named_barrier_sync(1, 128);
        unsigned char* row_ptr = stg + buf * (BM * 128) + r_in_tile * 128;
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
        fence_proxy_async();
        named_barrier_sync(1, 128);
        if (issuer) {
          if (OUT_F32 && accumulate) tma_reduce_add_2d(&tmap_c, stg + buf * (BM * 128), col0, mb * BM);
          else tma_store_2d(&tmap_c, stg + buf * (BM * 128), col0, mb * BM);
          tma_commit_group();
        }
        buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) tma_wait_group<0>();
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up.  Let TMA copies that were already issued land before the CTA's shared memory
    // is handed to another CTA (bounded delay, no barrier that could itself hang).
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---- host side ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D tensor map over a row-major [rows, cols] matrix with `ld` elements between rows, 128-byte swizzle.
static int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -10;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * esize) & 15)) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols) {
  return make_tmap_2d(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, rows, cols, ld, box_rows, box_cols);
}
int make_tmap_f32_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t box_cols) {
  return make_tmap_2d(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ptr, rows, cols, ld, box_rows, box_cols);
}
int make_tmap_u8_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_cols) {
  return make_tmap_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ptr, rows, cols, ld, box_rows, box_cols);
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool OUT_F32>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int M, int N, int K,
                       float alpha, int accumulate, int* status, int max_ctas, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, OUT_F32>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return -20;
    attr_set = true;
  }
  int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  int tiles = m_tiles * n_tiles;
  int grid = tiles < max_ctas ? tiles : max_ctas;
  int group_m = m_tiles < 16 ? m_tiles : 16;
  // split-K when the output has too few tiles to fill the GPU and the epilogue accumulates anyway
  int k_splits = 1;
  if (OUT_F32 && accumulate) {
    const int k_blocks = (K + BK - 1) / BK;
    k_splits = max_ctas / tiles;                 // floor: keep everything in one wave
    if (k_splits > k_blocks / 8) k_splits = k_blocks / 8;
    if (k_splits < 1) k_splits = 1;
    // every split must own at least one k block
    while (k_splits > 1 && ((k_blocks + k_splits - 1) / k_splits) * (k_splits - 1) >= k_blocks) --k_splits;
  }
  grid = tiles * k_splits < max_ctas ? tiles * k_splits : max_ctas;
  kern<<<grid, kGemmThreads, S::kTotal, stream>>>(ta, tb, tc, M, N, K, alpha, accumulate, group_m, k_splits, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace fth

using namespace fth;

extern "C" {

// C[M,N] (op)= alpha * A x B^T in the operand-major sense described at the top of this file.
//   a: K-major -> [M, K] with lda;  MN-major -> [K, M] with lda.   b likewise with N.
//   epi: 0 = store bf16, 1 = fp32 accumulate (C += ...), 2 = fp32 store.
//   bn:  128 or 256 (tile width); 0 = choose.   max_ctas: 0 = one per SM.
int fth_gemm_bf16(const void* a, long long lda, int a_mn_major, const void* b, long long ldb, int b_mn_major, void* c,
                  long long ldc, int M, int N, int K, float alpha, int epi, int bn, int max_ctas, int* status,
                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epi == kEpiBf16 ? (ldc % 8) : (ldc % 4)) return -2;
  if (max_ctas <= 0) max_ctas = sm_count();
  if (bn == 0 && epi == kEpiF32Accum && N > 128) bn = 256;  // split-K fills the GPU; wide tiles reuse A best
  if (bn == 0) {
    // fewer, fatter tiles unless that leaves the last wave mostly empty
    long long t256 = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
    long long t128 = (long long)((M + BM - 1) / BM) * ((N + 127) / 128);
    double w256 = (double)((t256 + max_ctas - 1) / max_ctas) * 2.0;  // cost in units of a 128-wide tile
    double w128 = (double)((t128 + max_ctas - 1) / max_ctas) * 1.15;
    bn = (w256 <= w128) ? 256 : 128;
  }
  CUtensorMap ta, tb;
  int r;
  if (!a_mn_major) r = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  else r = make_tmap_bf16_2d(&ta, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, 64);
  if (r) return r;
  if (!b_mn_major) r = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)bn, BK);
  else r = make_tmap_bf16_2d(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64);
  if (r) return r;
  CUtensorMap tc;
  const bool f32 = epi != kEpiBf16;
  if (f32) r = make_tmap_f32_2d(&tc, c, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, BM, 32);
  else r = make_tmap_bf16_2d(&tc, c, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, BM, 64);
  if (r) return r;
  const int accum = epi == kEpiF32Accum ? 1 : 0;
#define FTH_GEMM_CASE(BN_, ST_, AM_, BM_)                                                                             \
  do {                                                                                                                \
    if (f32) return launch_gemm<BN_, ST_, AM_, BM_, true>(ta, tb, tc, M, N, K, alpha, accum, status, max_ctas, stream); \
    return launch_gemm<BN_, ST_, AM_, BM_, false>(ta, tb, tc, M, N, K, alpha, accum, status, max_ctas, stream);         \
  } while (0)
  if (bn == 256) {
    if (!a_mn_major && !b_mn_major) FTH_GEMM_CASE(256, 4, false, false);
    if (!a_mn_major && b_mn_major) FTH_GEMM_CASE(256, 4, false, true);
    if (a_mn_major && b_mn_major) FTH_GEMM_CASE(256, 4, true, true);
    FTH_GEMM_CASE(256, 4, true, false);
  } else if (bn == 128) {
    if (!a_mn_major && !b_mn_major) FTH_GEMM_CASE(128, 6, false, false);
    if (!a_mn_major && b_mn_major) FTH_GEMM_CASE(128, 6, false, true);
    if (a_mn_major && b_mn_major) FTH_GEMM_CASE(128, 6, true, true);
    FTH_GEMM_CASE(128, 6, true, false);
  }
  return -3;
}

}  // extern "C"
