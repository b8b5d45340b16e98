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
// epilogue (one TMEM lane quarter each).  Tile 128 x BN x 64, 4-8 stage ring, two accumulator stages
// (2 x BN <= 512 TMEM columns) so the epilogue of tile i overlaps the mainloop of tile i+1.  Ragged M / N / K
// are handled by TMA zero fill on loads and predicated stores.  Every mbarrier wait is bounded.
//
// CTAS = 2 is the CTA-pair form (tcgen05.mma.cta_group::2): a cluster of two CTAs on neighbouring SMs computes one
// 256 x BN tile.  Each CTA loads its own 128 rows of A and only HALF of the B tile (its BN/2 rows) with unicast TMA,
// and keeps its own 128 x BN accumulator in its own tensor memory, so per output element the shared-memory fill and
// the L2 -> SM operand traffic drop by a third against the one-CTA 128 x 256 tile.  CTA rank 0 issues the MMAs for
// both; the ring's "full" barriers live in rank 0 and count the bytes of both CTAs' loads, "empty" / "accumulator
// full" are signalled in both CTAs by one multicast tcgen05.commit, "accumulator empty" collects the eight epilogue
// warps of the pair in rank 0.  No TMA load is multicast.
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <tuple>

#include "gemm_pipe.cuh"

namespace fth {

enum EpiMode : int { kEpiBf16 = 0, kEpiF32Accum = 1, kEpiF32Store = 2 };

template <int BN, int STAGES, bool A_MN, bool B_MN, bool OUT_F32, int CTAS>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, int M, int N, int K, float alpha, int accumulate,
                 int group_m, int k_splits, int* __restrict__ status) {
  using S = GemmSmem<BN, STAGES, CTAS>;
  constexpr int BNH = BN / CTAS;       // B rows this CTA loads
  constexpr int TM = BM * CTAS;        // rows of the tile the CTA (pair) computes
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = align_smem_1024(smem_raw);
  PipeBars<STAGES> bars(smem + S::kBarOffset);
  volatile int* abort_flag = bars.abort_flag;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const int unit = (int)blockIdx.x / CTAS, n_units = (int)gridDim.x / CTAS;  // a unit = a CTA or a CTA pair
  const int m_tiles = (M + TM - 1) / TM, n_tiles = (N + BN - 1) / BN;
  // split-K (accumulating fp32 epilogue only): work item = (k split, tile); every split reduce-adds into C
  const int mn_tiles = m_tiles * n_tiles;
  const int total_tiles = mn_tiles * k_splits;
  const int k_blocks_all = (K + BK - 1) / BK;
  const int k_per_split = (k_blocks_all + k_splits - 1) / k_splits;

  const uint32_t tmem_base = pipe_setup<BN, STAGES, CTAS, 0>(bars, true);

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
      for (int t = unit; t < total_tiles && ok; t += n_units) {
        int mb, nb;
        tile_coords(t, mb, nb);
        const int row_a = (mb * CTAS + (int)cta_rank) * BM;   // this CTA's rows of A
        const int row_b = nb * BN + (int)cta_rank * BNH;      // this CTA's rows of B
        const int kb0 = (t / mn_tiles) * k_per_split;
        const int kb1 = min(kb0 + k_per_split, k_blocks_all);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars.empty[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) { ok = false; break; }
          unsigned char* sa = smem + stage * S::kStageBytes;
          pipe_load_stage<BN, CTAS, A_MN, B_MN>(sa, sa + S::kABytes, &tmap_a, &tmap_b, kb * BK, row_a, row_b,
                                                &bars.full[stage], cta_rank);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (cta_rank == 0 && elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += n_units) {
        if (!mbar_wait(&bars.tempty[acc], acc_phase ^ 1, abort_flag, status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb0 = (t / mn_tiles) * k_per_split;
        const int kb1 = min(kb0 + k_per_split, k_blocks_all);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars.full[stage], phase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          pipe_mma_stage<BN, CTAS, A_MN, B_MN>(d_tmem, sa, sa + S::kABytes, kb == kb0);
          pipe_commit<CTAS>(&bars.empty[stage]);  // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        pipe_commit<CTAS>(&bars.tfull[acc]);  // accumulator complete
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
    for (int t = unit; t < total_tiles; t += n_units) {
      int mb, nb;
      tile_coords(t, mb, nb);
      const int row0 = (mb * CTAS + (int)cta_rank) * BM;  // first output row of this CTA
      if (!mbar_wait(&bars.tfull[acc], acc_phase, abort_flag, status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / CW; ++c) {
        const int col0 = nb * BN + c * CW;
        if (col0 >= N || row0 >= M) break;  // uniform across the epilogue warps
        uint32_t r[CW];
        tmem_ld_32x32(taddr + c * CW, r);
        if constexpr (CW == 64) tmem_ld_32x32(taddr + c * CW + 32, r + 32);
        tmem_wait_ld();
        if (issuer) tma_wait_group_read<1>();  // the store that last used this buffer has read it
        named_barrier_sync(1, 128);
        pipe_stage_row<OUT_F32>(stg + buf * (BM * 128) + r_in_tile * 128, r_in_tile, r, alpha);
        fence_proxy_async();
        named_barrier_sync(1, 128);
        if (issuer) {
          if (OUT_F32 && accumulate) tma_reduce_add_2d(&tmap_c, stg + buf * (BM * 128), col0, row0);
          else tma_store_2d(&tmap_c, stg + buf * (BM * 128), col0, row0);
          tma_commit_group();
        }
        buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) pipe_release_acc<CTAS>(&bars.tempty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) tma_wait_group<0>();
  }

  pipe_teardown<BN, CTAS>(abort_flag, tmem_base, true);
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

// Encoded tensor maps are cached: a map depends only on (address, extents, pitch, box, element type), never on the
// contents, and a training step asks for the same few hundred combinations on every micro-batch.  Encoding costs a
// driver call per operand, which an eager (not graph-replayed) step would otherwise pay three times per GEMM.
namespace {
struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  int dt;
  bool operator<(const TmapKey& o) const {
    return std::tie(ptr, rows, cols, ld, box_rows, box_cols, dt) <
           std::tie(o.ptr, o.rows, o.cols, o.ld, o.box_rows, o.box_cols, o.dt);
  }
};
std::mutex g_tmap_mu;
std::map<TmapKey, CUtensorMap> g_tmap_cache;
unsigned long long g_tmap_hits = 0, g_tmap_misses = 0;
constexpr size_t kTmapCacheMax = 8192;
}  // namespace

// 2-D tensor map over a row-major [rows, cols] matrix with `ld` elements between rows, 128-byte swizzle.
static int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int esize, const void* ptr, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * esize) & 15)) return -11;
  const TmapKey key{ptr, rows, cols, ld, box_rows, box_cols, (int)dt};
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      ++g_tmap_hits;
      return 0;
    }
  }
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -10;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -12;
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  if (g_tmap_cache.size() >= kTmapCacheMax) g_tmap_cache.clear();
  g_tmap_cache.emplace(key, *out);
  ++g_tmap_misses;
  return 0;
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

static bool g_deterministic = false;  // one k split per output tile: the fp32 reduce-adds then have a fixed order

// Number of k splits for an accumulating epilogue: fill the last wave without cutting the reduction too thin.
static int choose_k_splits(int tiles, int k_blocks, int units) {
  if (g_deterministic) return 1;
  int max_splits = k_blocks / 8;
  if (max_splits > 16) max_splits = 16;
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= max_splits; ++ks) {
    const int per = (k_blocks + ks - 1) / ks;
    if (per * (ks - 1) >= k_blocks) continue;  // every split must own at least one k block
    const long long items = (long long)tiles * ks;
    const long long waves = (items + units - 1) / units;
    // time ~ waves x (k blocks per item + fixed cost of a tile: pipeline fill + epilogue, about 6 k blocks)
    const double cost = (double)waves * (per + 6.0);
    if (cost < best_cost * 0.97) { best_cost = cost; best = ks; }
  }
  return best;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool OUT_F32, int CTAS>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int M, int N, int K,
                       float alpha, int accumulate, int* status, int max_ctas, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES, CTAS>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, OUT_F32, CTAS>;
  static bool attr_set = false;
  static int max_units = 0;  // CTAs (or CTA pairs) that can be resident at once
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) return -20;
    max_units = pipe_max_units<CTAS>(kern, S::kTotal, sm_count());
    attr_set = true;
  }
  int units = max_ctas / CTAS;
  if (units > max_units) units = max_units;
  if (units < 1) units = 1;
  const int m_tiles = (M + BM * CTAS - 1) / (BM * CTAS), n_tiles = (N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  int group_m = 16 / CTAS;
  if (group_m > m_tiles) group_m = m_tiles;
  // split-K when the output has too few tiles to fill the GPU and the epilogue accumulates anyway
  int k_splits = 1;
  if (OUT_F32 && accumulate) k_splits = choose_k_splits(tiles, (K + BK - 1) / BK, units);
  const long long items = (long long)tiles * k_splits;
  const int grid_units = items < units ? (int)items : units;
  if (pipe_launch<CTAS>(kern, grid_units, S::kTotal, stream, ta, tb, tc, M, N, K, alpha, accumulate, group_m, k_splits, status) !=
      cudaSuccess) {
    cudaGetLastError();
    return -21;
  }
  return 0;
}

// Tile choice.  Candidates: CTA pair 256 x 256, CTA pair 256 x 128, one CTA 128 x 256, one CTA 128 x 128.  The estimate is
// waves x (time one SM spends on its share of a tile); the weights are ratios measured on B200 with the variants timed
// interleaved (FC1 / FC2 / QKV shapes of the 0.5B model, K = 1024 .. 4096), in units of a 128 x 128 block on the pair form.
static void choose_tile(int M, int N, int max_ctas, int* bn, int* ctas) {
  struct Cand { int bn, ctas; double w; };
  const Cand cands[4] = {{256, 2, 2.0}, {128, 2, 1.2}, {256, 1, 2.32}, {128, 1, 1.33}};
  double best = 1e30;
  for (const Cand& c : cands) {
    if (c.ctas == 2 && M <= BM) continue;  // a pair would leave one CTA without rows
    const long long mt = (M + BM * c.ctas - 1) / (BM * c.ctas), nt = (N + c.bn - 1) / c.bn;
    const long long units = max_ctas / c.ctas > 0 ? max_ctas / c.ctas : 1;
    const long long waves = (mt * nt + units - 1) / units;
    const double cost = (double)waves * c.w;
    if (cost < best) { best = cost; *bn = c.bn; *ctas = c.ctas; }
  }
}

}  // namespace fth

using namespace fth;

extern "C" {

void fth_gemm_set_deterministic(int on) { g_deterministic = on != 0; }

void fth_tmap_cache_stats(unsigned long long* hits, unsigned long long* misses) {
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  *hits = g_tmap_hits;
  *misses = g_tmap_misses;
}

// C[M,N] (op)= alpha * A x B^T in the operand-major sense described at the top of this file.
//   a: K-major -> [M, K] with lda;  MN-major -> [K, M] with lda.   b likewise with N.
//   epi: 0 = store bf16, 1 = fp32 accumulate (C += ...), 2 = fp32 store.
//   bn:  tile code.  0 = choose; 128 / 256 = one CTA per 128 x bn tile; -128 / -256 = a CTA pair per 256 x |bn| tile.
//   max_ctas: 0 = one per SM.
int fth_gemm_bf16(const void* a, long long lda, int a_mn_major, const void* b, long long ldb, int b_mn_major, void* c,
                  long long ldc, int M, int N, int K, float alpha, int epi, int bn, int max_ctas, int* status,
                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epi == kEpiBf16 ? (ldc % 8) : (ldc % 4)) return -2;
  if (max_ctas <= 0) max_ctas = sm_count();
  int ctas = 1;
  if (bn < 0) { ctas = 2; bn = -bn; }
  else if (bn == 0) {
    if (epi == kEpiF32Accum) {
      // split-K fills the GPU whatever the tile count: take the widest tile the output has room for
      bn = N > 128 ? 256 : 128;
      ctas = M > 128 ? 2 : 1;
    } else {
      choose_tile(M, N, max_ctas, &bn, &ctas);
    }
  }
  if (bn != 128 && bn != 256) return -3;
  const uint32_t bnh = (uint32_t)(bn / ctas);
  CUtensorMap ta, tb;
  int r;
  if (!a_mn_major) r = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  else r = make_tmap_bf16_2d(&ta, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, 64);
  if (r) return r;
  if (!b_mn_major) r = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, bnh, BK);
  else r = make_tmap_bf16_2d(&tb, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64);
  if (r) return r;
  CUtensorMap tc;
  const bool f32 = epi != kEpiBf16;
  if (f32) r = make_tmap_f32_2d(&tc, c, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, BM, 32);
  else r = make_tmap_bf16_2d(&tc, c, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, BM, 64);
  if (r) return r;
  const int accum = epi == kEpiF32Accum ? 1 : 0;
#define FTH_GEMM_CASE(BN_, ST_, AM_, BM_, CT_)                                                                              \
  do {                                                                                                                      \
    if (f32) return launch_gemm<BN_, ST_, AM_, BM_, true, CT_>(ta, tb, tc, M, N, K, alpha, accum, status, max_ctas, stream); \
    return launch_gemm<BN_, ST_, AM_, BM_, false, CT_>(ta, tb, tc, M, N, K, alpha, accum, status, max_ctas, stream);         \
  } while (0)
#define FTH_GEMM_MAJORS(BN_, ST_, CT_)                                          \
  do {                                                                          \
    if (!a_mn_major && !b_mn_major) FTH_GEMM_CASE(BN_, ST_, false, false, CT_); \
    if (!a_mn_major && b_mn_major) FTH_GEMM_CASE(BN_, ST_, false, true, CT_);   \
    if (a_mn_major && b_mn_major) FTH_GEMM_CASE(BN_, ST_, true, true, CT_);     \
    FTH_GEMM_CASE(BN_, ST_, true, false, CT_);                                  \
  } while (0)
  if (ctas == 2) {
    if (bn == 256) FTH_GEMM_MAJORS(256, 6, 2);
    FTH_GEMM_MAJORS(128, 8, 2);
  }
  if (bn == 256) FTH_GEMM_MAJORS(256, 4, 1);
  FTH_GEMM_MAJORS(128, 6, 1);
  return -3;
}

}  // extern "C"
