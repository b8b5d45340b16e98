// Causal GQA flash attention for sm_100a on the packed kv-group-major QKV activation.
//
// Forward (flash_fwd2_kernel): one CTA owns two 128-row query tiles of one head ("A" and "B", 256 consecutive positions)
// and streams 128-row K/V blocks through a TMA ring shared by both tiles.  S = Q K^T is a tcgen05.mma (operands in
// shared memory) into tensor memory; each tile has two softmax warpgroups (a thread is one query row x 64 of the 128 key
// columns; the halves exchange their row maxima through shared memory and an mbarrier), which read S with tcgen05.ld,
// run the online softmax in the log2 domain and write P as packed bf16 into tensor memory: out of place at head_dim 64
// (so the next S is issued as soon as the current one has been read), over S at head_dim 128.  O += P V is a tcgen05.mma
// with the A operand taken from tensor memory.  O is rescaled in place only when a row's running max moved by more than
// 2^8 (the stale max keeps P bounded by 256), which makes the correction rare.
// Returns the log-sum-exp per row so the backward never replays the forward (the reference's forward drops it
// and its backward re-runs flash-attn under autograd: forward.py:233-235, backward.py:518-527).
//
// Replaces flash_attn_func / _flash_attn_backward (FA2, mma.sync) at forward.py:204-235 and backward.py:473-527.
// Q/K/V are read in place from the QKV GEMM output through one 2-D tensor map (no .contiguous() copies of K and V,
// forward.py:83-93), and the backward writes dQ/dK/dV straight into the packed layout the QKV wgrad/dgrad consume.
#include <type_traits>
#include <cuda.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace fth {

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct FwdSmem {
  static constexpr int kTile = 128 * D * 2;            // one 128 x D bf16 tile
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kQOff = 0;                       // Q_A, Q_B
  static constexpr int kKVOff = 2 * kTile;              // per stage: K tile, V tile
  static constexpr int kBarOff = kKVOff + kStages * 2 * kTile;
  static constexpr int kTotal = kBarOff + 512 + 4096 + 1024;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  // one conversion instruction; doing the rounding with an integer add and a byte permute instead measured slower
  // (forward exp phase 1914 -> 2450 cycles per block): the integer pipe is half rate and the phase is issue bound
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kFwd2Threads = 576;  // warps 0-15 softmax (2 tiles x 2 column halves x 4 lane quarters), 16 TMA, 17 MMA

template <int D>
__global__ void __launch_bounds__(kFwd2Threads, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap, __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out,
                 int S, int n_kv, int g, float scale_log2, int* __restrict__ status, long long* __restrict__ dbg) {
  using L = FwdSmem<D>;
  constexpr int KS = L::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;              // [1]
  uint64_t* kv_full = bars + 1;         // [KS]
  uint64_t* kv_empty = kv_full + KS;    // [KS]
  uint64_t* s_full = kv_empty + KS;     // [2]  S ready (per tile)
  uint64_t* p_full = s_full + 2;        // [2]  P written (and O corrected) by the softmax warpgroup
  uint64_t* o_done = p_full + 2;        // [2]  P V finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(smem + L::kBarOff + 512);  // [2 parities][2 tiles][2 halves][128 rows]
  uint64_t* xbar = reinterpret_cast<uint64_t*>(smem + L::kBarOff + 384);  // [2] per-tile exchange barrier, 8 arrivals (one per warp)
  uint64_t* s_free = xbar + 2;          // [2] per tile: S has been read out of tensor memory (8 arrivals)

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n_pairs = (S + 255) / 256;
  const int pair = n_pairs - 1 - (int)blockIdx.x;  // heaviest (latest) query tiles first
  const int head = blockIdx.y;                      // q head index in kv-group-major order: j * g + i
  const int b = blockIdx.z;
  const int j = head / g, i = head % g;
  const int q0 = pair * 256;
  const bool has_b = q0 + 128 < S;
  const int tA = q0 / 128;
  const int n_blocks = has_b ? tA + 2 : tA + 1;     // kv blocks 0 .. n_blocks-1 (tile A skips the last when has_b)
  const int row_stride = n_kv * (g + 2) * D;
  const int q_col = (j * (g + 2) + i) * D, k_col = (j * (g + 2) + g) * D, v_col = k_col + D;
  const int grow0 = b * S;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 8); mbar_init(&o_done[t], 1); mbar_init(&xbar[t], 8); mbar_init(&s_free[t], 8); }   // one arrival per warp
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 17) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // tensor-memory columns: S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,256+D)  O_B [384,384+D)
  // At head_dim 64 the 512 columns hold S (2 x 128), a separate bf16 P (2 x 64) and O (2 x 64): with P out of place the
  // next S = Q K^T of a tile is issued as soon as its softmax warps have read the current S, and is ready by the time
  // they finish the exp phase.  At head_dim 128 O needs 2 x 128 columns and P overwrites S in place.
  constexpr bool kSepP = (D == 64);
  const uint32_t tm_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tm_p[2] = {kSepP ? tmem_base + 256 : tmem_base, kSepP ? tmem_base + 320 : tmem_base + 128};
  const uint32_t tm_o[2] = {kSepP ? tmem_base + 384 : tmem_base + 256, kSepP ? tmem_base + 448 : tmem_base + 384};

  if (warp == 16) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap);
      const int n_q_tiles = has_b ? 2 : 1;
      mbar_expect_tx(q_full, n_q_tiles * L::kTile);
      for (int t = 0; t < n_q_tiles; ++t)
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(smem + L::kQOff + t * L::kTile + c * 16384, &tmap, q_col + c * 64, grow0 + q0 + t * 128, q_full);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < n_blocks; ++kb) {
        if (!mbar_wait(&kv_empty[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) break;
        unsigned char* sk = smem + L::kKVOff + stage * 2 * L::kTile;
        unsigned char* sv = sk + L::kTile;
        mbar_expect_tx(&kv_full[stage], 2 * L::kTile);
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(sk + c * 16384, &tmap, k_col + c * 64, grow0 + kb * 128, &kv_full[stage]);
          tma_load_2d(sv + c * 16384, &tmap, v_col + c * 64, grow0 + kb * 128, &kv_full[stage]);
        }
        if (++stage == KS) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 17) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, false, true);
      const uint32_t q_addr[2] = {smem_u32(smem + L::kQOff), smem_u32(smem + L::kQOff + L::kTile)};
      auto issue_s = [&](int t, uint32_t k_addr) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_bf16_ss(tm_s[t], make_smem_desc(q_addr[t] + off, 0, 1024), make_smem_desc(k_addr + off, 0, 1024), idesc_s,
                       kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, uint32_t v_addr, bool first) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ts(tm_o[t], kSepP ? tm_p[t] + kk * 8 : tm_s[t] + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8),
                       make_smem_desc(v_addr + kk * 2048, 16384, 1024), idesc_o,
                       (first && kk == 0) ? 0u : 1u);
        umma_commit(&o_done[t]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, status, kTimeoutSmemFull);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t p_phase[2] = {0, 0};
      // number of kv blocks per tile
      const int nb_t[2] = {tA + 1, has_b ? tA + 2 : 0};
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_flag, status, kTimeoutSmemFull);
      if (ok) {
        tc_fence_after();
        const uint32_t k0 = smem_u32(smem + L::kKVOff);
        issue_s(0, k0);
        if (has_b) issue_s(1, k0);
      }
      for (int kb = 0; kb < n_blocks && ok; ++kb) {
        const uint32_t k_cur = smem_u32(smem + L::kKVOff + stage * 2 * L::kTile);
        const uint32_t v_cur = k_cur + L::kTile;
        int nstage = stage + 1;
        uint32_t nphase = phase;
        if (nstage == KS) { nstage = 0; nphase ^= 1; }
        const uint32_t k_next = smem_u32(smem + L::kKVOff + nstage * 2 * L::kTile);
        bool next_ready = false;
        if constexpr (kSepP) {
          // next S of both tiles first (their current S has been read early in the softmax of block kb) ...
          for (int t = 0; t < 2 && ok; ++t) {
            if (kb + 1 >= nb_t[t]) continue;
            if (!mbar_wait(&s_free[t], kb & 1, abort_flag, status, kTimeoutTmemEmpty)) { ok = false; break; }
            if (!next_ready) {
              if (!mbar_wait(&kv_full[nstage], nphase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
              next_ready = true;
            }
            tc_fence_after();
            issue_s(t, k_next);
          }
          // ... then P V of block kb as each tile's P arrives
          for (int t = 0; t < 2 && ok; ++t) {
            if (kb >= nb_t[t]) continue;
            if (!mbar_wait(&p_full[t], p_phase[t], abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
            p_phase[t] ^= 1;
            tc_fence_after();
            issue_pv(t, v_cur, kb == 0);
          }
        } else
        for (int t = 0; t < 2 && ok; ++t) {
          if (kb >= nb_t[t]) continue;
          if (!mbar_wait(&p_full[t], p_phase[t], abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
          p_phase[t] ^= 1;
          tc_fence_after();
          issue_pv(t, v_cur, kb == 0);
          if (kb + 1 < nb_t[t]) {
            if (!next_ready) {
              if (!mbar_wait(&kv_full[nstage], nphase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
              tc_fence_after();
              next_ready = true;
            }
            issue_s(t, k_next);  // runs after P V of this tile: S/P share tensor-memory columns
          }
        }
        umma_commit(&kv_empty[stage]);  // stage free once every MMA issued so far has finished
        stage = nstage;
        phase = nphase;
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax warpgroups: tile t, column half hh, lane quarter qw ----------------
    // Two warpgroups share a query tile: each thread owns one row and 64 of the 128 key columns of a block, so four softmax
    // warps are resident per scheduler.  The two halves exchange their partial row maxima through shared memory (one named
    // barrier per block); the row sums stay partial until the epilogue.
    const int t = warp / 8;
    const int hh = (warp / 4) % 2;
    const int qw = warp % 4;
    const int nb = (t == 0) ? tA + 1 : (has_b ? tA + 2 : 0);
    const int r = qw * 32 + lane;
    const int qrow = q0 + t * 128 + r;
    const uint32_t lane_off = (uint32_t)(qw * 32) << 16;
    const uint32_t s_col = 64 * hh;
    float m_run = -INFINITY, l_run = 0.f;
    uint32_t ph_s = 0, ph_o = 0, ph_x = 0;
    bool ok = true;
    const bool rec = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (warp == 0 || warp == 8) && lane == 0;
    long long* drow = dbg + (warp / 8) * 8 * 64;
#define FTH_TS(i) do { if (rec && kb < 64) drow[(i) * 64 + kb] = clock64(); } while (0)
    for (int kb = 0; kb < nb && ok; ++kb) {
      FTH_TS(0);
      if (!mbar_wait(&s_full[t], ph_s, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
      FTH_TS(1);
      ph_s ^= 1;
      tc_fence_after();
      const bool diag = (kb * 128 + 127 > q0 + t * 128);
      const int kpos0 = kb * 128 + 64 * hh;
      uint32_t sr[64];
      tmem_ld_32x32(tm_s[t] + lane_off + s_col, sr);
      tmem_ld_32x32(tm_s[t] + lane_off + s_col + 32, sr + 32);
      tmem_wait_ld();
      if constexpr (kSepP) { tc_fence_before(); mbar_arrive_warp(&s_free[t]); }
      FTH_TS(2);
      if (diag) {
#pragma unroll
        for (int e = 0; e < 64; ++e)
          if (kpos0 + e > qrow) sr[e] = 0xff800000u;  // -inf
      }
      // three-input max: half the instructions of the pairwise form on the half-rate pipe this phase is bound by
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 64; e += 8) {
        mx0 = fmax3(mx0, __uint_as_float(sr[e]), __uint_as_float(sr[e + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[e + 2]), __uint_as_float(sr[e + 3]));
        mx2 = fmax3(mx2, __uint_as_float(sr[e + 4]), __uint_as_float(sr[e + 5]));
        mx3 = fmax3(mx3, __uint_as_float(sr[e + 6]), __uint_as_float(sr[e + 7]));
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      float* slot = xch + (((kb & 1) * 2 + t) * 2) * 128;
      slot[hh * 128 + r] = mx;
      mbar_arrive_warp(&xbar[t]);
      if (!mbar_wait(&xbar[t], ph_x, abort_flag, status, kTimeoutGeneric)) { ok = false; break; }
      ph_x ^= 1;
      FTH_TS(3);
      mx = fmaxf(mx, slot[(hh ^ 1) * 128 + r]) * scale_log2;
      float m_new = fmaxf(m_run, mx);
      float m_use = (m_new - m_run > kRescaleThreshold) ? m_new : m_run;
      if (m_run == -INFINITY) m_use = m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
      const bool need_fix = (m_use != m_run) && kb > 0;
      if constexpr (kSepP) {
        if (kb > 0) {   // P V of the previous block has read P and finished with O
          if (!mbar_wait(&o_done[t], ph_o, abort_flag, status, kTimeoutTmemEmpty)) { ok = false; break; }
          ph_o ^= 1;
          tc_fence_after();
        }
      }
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float p0 = exp2f(fmaf(__uint_as_float(sr[c * 32 + e]), scale_log2, -m_use));
          const float p1 = exp2f(fmaf(__uint_as_float(sr[c * 32 + e + 1]), scale_log2, -m_use));
          const float p2 = exp2f(fmaf(__uint_as_float(sr[c * 32 + e + 2]), scale_log2, -m_use));
          const float p3 = exp2f(fmaf(__uint_as_float(sr[c * 32 + e + 3]), scale_log2, -m_use));
          rs0 += p0; rs1 += p1; rs2 += p2; rs3 += p3;
          pk[e / 2] = pack_bf16(p0, p1);
          pk[e / 2 + 1] = pack_bf16(p2, p3);
        }
        // P of keys [64hh+32c, +32) -> packed columns [64hh+16c, +16): inside this half's own S columns (already read)
        tmem_st_32x16(kSepP ? tm_p[t] + lane_off + 32 * hh + c * 16 : tm_s[t] + lane_off + s_col + c * 16, pk);
      }
      l_run = l_run * alpha + ((rs0 + rs1) + (rs2 + rs3));
      m_run = m_use;
      FTH_TS(4);
      if (kb > 0) {
        if constexpr (!kSepP) {
          if (!mbar_wait(&o_done[t], ph_o, abort_flag, status, kTimeoutTmemEmpty)) { ok = false; break; }
          ph_o ^= 1;
          tc_fence_after();
        }
        if (__any_sync(0xffffffffu, need_fix)) {   // each half rescales its own D/2 columns of O
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[16];
            tmem_ld_32x16(tm_o[t] + lane_off + hh * (D / 2) + c * 16, rr);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) rr[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
            tmem_st_32x16(tm_o[t] + lane_off + hh * (D / 2) + c * 16, rr);
          }
        }
      }
      FTH_TS(5);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&p_full[t]);
      FTH_TS(6);
    }
#undef FTH_TS
    if (nb > 0 && ok) {
      if (mbar_wait(&o_done[t], ph_o, abort_flag, status, kTimeoutTmemEmpty)) {
        tc_fence_after();
        float* slot = xch + (((nb & 1) * 2 + t) * 2) * 128;   // parity not used by the last block's max exchange
        slot[hh * 128 + r] = l_run;
        mbar_arrive_warp(&xbar[t]);
        if (mbar_wait(&xbar[t], ph_x, abort_flag, status, kTimeoutGeneric)) {
        const float l_tot = l_run + slot[(hh ^ 1) * 128 + r];
        const float inv = 1.f / l_tot;
        __nv_bfloat16* dst = out + (size_t)(grow0 + qrow) * ((size_t)n_kv * g * D) + (size_t)head * D + hh * (D / 2);
#pragma unroll 1
        for (int c = 0; c < D / 64; ++c) {
          uint32_t rr[32];
          tmem_ld_32x32(tm_o[t] + lane_off + hh * (D / 2) + c * 32, rr);
          tmem_wait_ld();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(rr[v * 8 + e]) * inv;
            store8(dst + c * 32 + v * 8, f);
          }
        }
        if (hh == 0) lse_out[((size_t)b * (n_kv * g) + head) * S + qrow] = (m_run + log2f(l_tot)) * 0.6931471805599453f;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if (warp == 17) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}



// =====================================================================================================================
// Backward.
//
// Pre-pass (flash_bwd_prep_kernel): delta[b,h,s] = sum_d dO*O and lse2 = lse*log2(e), one warp per (row, head).
// Main kernel: one CTA per (batch, query head, 128-key block n).  K and V tiles stay resident in shared memory; the CTA
// walks the query blocks m >= n.  Per step, with every product on tcgen05 and every accumulator in tensor memory:
//     S^T  = K Q^T          (128 keys x 128 queries)            SS-MMA
//     dP^T = V dO^T                                              SS-MMA
//     P^T  = exp2(S^T*c - lse2[q]),  dS^T = P^T (dP^T - delta[q]) * scale      (one thread per key row)
//     dV  += P^T dO          A = P^T from tensor memory          TS-MMA   (dO tile reused as an MN-major B operand)
//     dK  += dS^T Q          A = dS^T from tensor memory         TS-MMA   (Q tile reused as an MN-major B operand)
//     dQ   = dS K            A = dS^T from shared memory as an MN-major operand, B = K tile MN-major
// Working on the transposed score tile means no operand ever needs a transposing copy: thread r owns key row r of
// S^T / dP^T, so P^T and dS^T are produced directly in the lane layout tcgen05 wants for an A operand.  dQ tiles are
// summed across the key blocks by TMA reduce-add into an fp32 image of the packed dQKV activation; dK / dV (summed over
// the query heads of a KV group, i.e. over CTAs) use the same path.  A finalize kernel rounds that image to bf16.
// =====================================================================================================================

constexpr int kBwd64Threads = 448;  // head_dim-64 kernel: warps 0-7 compute, 8-11 drain, 12 TMA, 13 MMA
constexpr int kBwdThreads = 320;  // warps 0-7 compute (two warpgroups, 64 query columns each), warp 8 TMA, warp 9 MMA

template <int D>
struct BwdSmem {
  static constexpr int kTile = 128 * D * 2;                       // 128 x D bf16
  static constexpr int kStages = (D == 64) ? 2 : 1;               // Q + dO ring
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kTile;
  static constexpr int kQdOOff = 2 * kTile;                       // per stage: Q tile, dO tile
  static constexpr int kDsOff = kQdOOff + kStages * 2 * kTile;    // dS^T as an MN-major operand: 2 x [128 x 128 B]
  static constexpr int kStgOff = kDsOff + 32768;                  // fp32 staging: one [128 rows x 128 B] per warpgroup
  static constexpr int kVecOff = kStgOff + 32768;                 // per stage: lse2[128], delta[128] fp32
  // augmentation operands (K-major, no swizzle, 8-row groups 256 B apart): a constant [128 x 16] tile of ones and two
  // [128 x 16] tiles with -lse2 / scale_log2 and -delta of the step's queries as bf16 high + low parts in columns 0 and 1
  static constexpr int kOnesOff = kVecOff + kStages * 1024;       // 4 KB
  static constexpr int kAugOff = kOnesOff + 4096;                 // 2 x 4 KB
  static constexpr int kBarOff = kAugOff + 8192;
  static constexpr int kTotal = kBarOff + 512 + 1024;
};

__global__ void flash_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                      const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                                      int B, int S, int nq, int d, float scale) {
  // d / 8 lanes per (row, head): each lane one 16-byte vector of O and of dO, so a warp covers 4 items at head_dim 64.
  // Items run row-fastest inside a head, which makes the delta / lse2 writes and the lse reads contiguous.
  const int lpi = d / 8, ipw = 32 / lpi;
  const int lane = threadIdx.x % 32, sub = lane / lpi, l = lane % lpi;
  const long long rows = (long long)B * S, total = rows * nq;
  const long long warps = (long long)gridDim.x * (blockDim.x / 32);
  for (long long w0 = ((long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32) * ipw; w0 < total; w0 += warps * ipw) {
    const long long w = w0 + sub;
    const bool ok = w < total;
    const int h = ok ? (int)(w / rows) : 0;
    const long long row = ok ? w % rows : 0;  // b*S + s
    float acc = 0.f;
    if (ok) {
      const size_t base = ((size_t)row * nq + h) * d + l * 8;
      float a[8], b8[8];
      load8(o + base, a);
      load8(d_o + base, b8);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += a[e] * b8[e];
    }
    for (int off = lpi / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (ok && l == 0) {
      const int b = (int)(row / S), sq = (int)(row % S);
      const size_t idx = ((size_t)b * nq + h) * S + sq;
      delta[idx] = acc * scale;   // pre-scaled: dS = P * (dP*scale - delta*scale) is one FFMA + one FMUL
      lse2[idx] = lse[idx] * 1.4426950408889634f;
    }
  }
}

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                 const __grid_constant__ CUtensorMap tmap_dqkv, const float* __restrict__ lse2, const float* __restrict__ delta,
                 int S, int n_kv, int g, float scale, float scale_log2, int* __restrict__ status) {
  using L = BwdSmem<D>;
  constexpr int QS = L::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;            // [1]
  uint64_t* q_full = bars + 1;         // [QS]
  uint64_t* q_empty = q_full + QS;     // [QS]
  uint64_t* sdp_full = q_empty + QS;   // S^T and dP^T ready
  uint64_t* pds_full = sdp_full + 1;   // P^T, dS^T written (one arrival per compute warp)
  uint64_t* dq_full = pds_full + 1;    // dV, dK, dQ MMAs of this step finished
  uint64_t* dq_drained = dq_full + 1;  // dQ read out of tensor memory (one arrival per warp)
  uint64_t* aug_full = dq_drained + 1; // augmentation tiles of the step written (one arrival per compute warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aug_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n_blk = S / 128;
  const int n = n_blk - 1 - (int)blockIdx.x;   // key block; cheapest last
  const int head = blockIdx.y;                  // kv-group-major query head index j*g + i
  const int b = blockIdx.z;
  const int j = head / g, i = head % g;
  const int nq = n_kv * g;
  const int q_col = (j * (g + 2) + i) * D, k_col = (j * (g + 2) + g) * D, v_col = k_col + D;
  const int do_col = head * D;
  const int grow0 = b * S;
  const int steps = n_blk - n;                  // query blocks m = n .. n_blk-1
  const float* lse2_h = lse2 + ((size_t)b * nq + head) * S;
  const float* delta_h = delta + ((size_t)b * nq + head) * S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);        // one arrival per compute warp
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 8);
    mbar_init(aug_full, 8);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S^T/P^T [0,128)  dP^T/dS^T [128,256)  D=64: dQ [256,320) dK [320,384) dV [384,448)
  //                                                 D=128: dK [256,384) dV [384,512), dQ reuses [0,128) once P^T is consumed
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128;
  const uint32_t tm_dq = (D == 64) ? tmem_base + 256 : tmem_base;
  const uint32_t tm_dk = (D == 64) ? tmem_base + 320 : tmem_base + 256;
  const uint32_t tm_dv = (D == 64) ? tmem_base + 384 : tmem_base + 384;
  constexpr bool kDqAliasesS = (D != 64);

  if (warp == 8) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_qkv);
      tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(kv_full, 2 * L::kTile);
      for (int c = 0; c < D / 64; ++c) {
        tma_load_2d(smem + L::kKOff + c * 16384, &tmap_qkv, k_col + c * 64, grow0 + n * 128, kv_full);
        tma_load_2d(smem + L::kVOff + c * 16384, &tmap_qkv, v_col + c * 64, grow0 + n * 128, kv_full);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int st = 0; st < steps; ++st) {
        const int m = n + st;
        if (!mbar_wait(&q_empty[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) break;
        unsigned char* sq = smem + L::kQdOOff + stage * 2 * L::kTile;
        unsigned char* sdo = sq + L::kTile;
        float* vec = reinterpret_cast<float*>(smem + L::kVecOff + stage * 1024);
        mbar_expect_tx(&q_full[stage], 2 * L::kTile + 1024);
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(sq + c * 16384, &tmap_qkv, q_col + c * 64, grow0 + m * 128, &q_full[stage]);
          tma_load_2d(sdo + c * 16384, &tmap_do, do_col + c * 64, grow0 + m * 128, &q_full[stage]);
        }
        bulk_load_1d(vec, lse2_h + m * 128, 512, &q_full[stage]);
        bulk_load_1d(vec + 128, delta_h + m * 128, 512, &q_full[stage]);
        if (++stage == QS) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 128, false, false);   // S^T, dP^T: both operands K-major
      constexpr uint32_t idesc_dkv = make_idesc_bf16(128, D, false, true);     // A from TMEM, B MN-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, true, true);       // A = dS^T in smem (MN-major), B = K MN-major
      const uint32_t k_addr = smem_u32(smem + L::kKOff), v_addr = smem_u32(smem + L::kVOff);
      const uint32_t ds_addr = smem_u32(smem + L::kDsOff);
      bool ok = mbar_wait(kv_full, 0, abort_flag, status, kTimeoutSmemFull);
      int stage = 0;
      uint32_t phase = 0, ph_pds = 0, ph_drain = 0, ph_aug = 0;
      auto issue_sdp = [&](uint32_t q_addr, uint32_t do_addr) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_bf16_ss(tm_s, make_smem_desc(k_addr + off, 0, 1024), make_smem_desc(q_addr + off, 0, 1024), idesc_st, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_bf16_ss(tm_dp, make_smem_desc(v_addr + off, 0, 1024), make_smem_desc(do_addr + off, 0, 1024), idesc_st, kk != 0);
        }
        // one more k-step each: ones x (-lse2 / scale_log2) and ones x (-delta), so the accumulators hold the exp2 argument
        // and dP - delta and the compute warps fetch no per-query vectors (their broadcast shared-memory loads were what the
        // math phase waited for)
        const uint64_t ones_desc = make_smem_desc_plain(smem_u32(smem + L::kOnesOff), 128, 256);
        umma_bf16_ss(tm_s, ones_desc, make_smem_desc_plain(smem_u32(smem + L::kAugOff), 128, 256), idesc_st, 1u);
        umma_bf16_ss(tm_dp, ones_desc, make_smem_desc_plain(smem_u32(smem + L::kAugOff + 4096), 128, 256), idesc_st, 1u);
        umma_commit(sdp_full);
      };
      if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag, status, kTimeoutSmemFull);
      if (ok) { ok = mbar_wait(aug_full, ph_aug, abort_flag, status, kTimeoutSmemFull); ph_aug ^= 1; }
      if (ok) {
        tc_fence_after();
        const uint32_t q0a = smem_u32(smem + L::kQdOOff);
        issue_sdp(q0a, q0a + L::kTile);
      }
      for (int st = 0; st < steps && ok; ++st) {
        const uint32_t q_addr = smem_u32(smem + L::kQdOOff + stage * 2 * L::kTile);
        const uint32_t do_addr = q_addr + L::kTile;
        if (!mbar_wait(pds_full, ph_pds, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
        ph_pds ^= 1;
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q   (K dimension = 128 queries, 8 steps of 16)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ts(tm_dv, tm_s + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8), make_smem_desc(do_addr + kk * 2048, 16384, 1024),
                       idesc_dkv, (st | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ts(tm_dk, tm_dp + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8), make_smem_desc(q_addr + kk * 2048, 16384, 1024),
                       idesc_dkv, (st | kk) != 0);
        // dQ = dS K : M = queries, N = D, K dimension = 128 keys
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ss(tm_dq, make_smem_desc(ds_addr + kk * 2048, 16384, 1024), make_smem_desc(k_addr + kk * 2048, 16384, 1024),
                       idesc_dq, kk != 0);
        umma_commit(dq_full);
        umma_commit(&q_empty[stage]);
        int nstage = stage + 1;
        uint32_t nphase = phase;
        if (nstage == QS) { nstage = 0; nphase ^= 1; }
        if (st + 1 < steps) {
          if (!mbar_wait(&q_full[nstage], nphase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          if (kDqAliasesS) {
            if (!mbar_wait(dq_drained, ph_drain, abort_flag, status, kTimeoutTmemEmpty)) { ok = false; break; }
            ph_drain ^= 1;
          }
          if (!mbar_wait(aug_full, ph_aug, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          ph_aug ^= 1;
          tc_fence_after();
          const uint32_t qn = smem_u32(smem + L::kQdOOff + nstage * 2 * L::kTile);
          issue_sdp(qn, qn + L::kTile);
        }
        stage = nstage;
        phase = nphase;
      }
    }
    __syncwarp();
  } else {
    // ---------------- compute warps ----------------
    // Thread (qd, lane) owns key row r = 32*qd + lane; warpgroup h = warp / 4 owns query columns [64h, 64h+64).
    const int qd = warp % 4, h = warp / 4;
    const int r = qd * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const int key = n * 128 + r;
    unsigned char* ds_row = smem + L::kDsOff + h * 16384 + r * 128;   // dS^T operand chunk h (queries 64h..64h+63)
    unsigned char* stg = smem + L::kStgOff + h * 16384;
    const bool issuer = (threadIdx.x == h * 128);
    const int bar_id = 1 + h;
    uint32_t ph_sdp = 0, ph_dq = 0;
    int stage = 0;
    uint32_t qphase = 0;
    bool ok = true;
    // TMA reduce-add of this warpgroup's half of a [128 x D] fp32 tensor-memory tile into the fp32 dQKV image
    auto drain_tile = [&](uint32_t tm_src, int col, int row) {
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        const int cc = h * (D / 64) + c;     // 32-column chunk index handled by this warpgroup
        uint32_t v[32];
        tmem_ld_32x32(tm_src + lane_off + cc * 32, v);
        tmem_wait_ld();
        if (issuer) tma_wait_group_read<0>();  // the previous store has finished reading the staging buffer
        named_barrier_sync(bar_id, 128);
        unsigned char* rowp = stg + r * 128;
#pragma unroll
        for (int p8 = 0; p8 < 8; ++p8)
          *reinterpret_cast<uint4*>(rowp + ((p8 ^ (r & 7)) * 16)) = make_uint4(v[p8 * 4], v[p8 * 4 + 1], v[p8 * 4 + 2], v[p8 * 4 + 3]);
        fence_proxy_async();
        named_barrier_sync(bar_id, 128);
        if (issuer) {
          tma_reduce_add_2d(&tmap_dqkv, stg, col + cc * 32, row);
          tma_commit_group();
        }
      }
    };
    {
      // one-time: zero the augmentation tiles (only columns 0 and 1 are rewritten) and build the ones tile
      const int t = threadIdx.x;   // 0 .. 255
      uint4* z = reinterpret_cast<uint4*>(smem + L::kAugOff);
      for (int i = t; i < 8192 / 16; i += 256) z[i] = make_uint4(0u, 0u, 0u, 0u);
      if (t < 128) {
        unsigned char* one_row = smem + L::kOnesOff + (t >> 3) * 256 + (t & 7) * 16;
        *reinterpret_cast<uint4*>(one_row) = make_uint4(0x3F803F80u, 0u, 0u, 0u);   // bf16 1.0, 1.0, zeros
        *reinterpret_cast<uint4*>(one_row + 128) = make_uint4(0u, 0u, 0u, 0u);
      }
      named_barrier_sync(3, 256);
    }
    const float inv_scale_log2 = 1.f / scale_log2, inv_scale = 1.f / scale;
    for (int st = 0; st < steps && ok; ++st) {
      const int m = n + st;
      // q_full is also what delivers lse2 / delta of this query block
      if (!mbar_wait(&q_full[stage], qphase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
      {
        // thread t < 128 writes the S^T tile's row of query t, thread 128 + t the dP^T tile's: value as bf16 high + low part.
        // The previous step's products have finished reading the tiles (this warp has seen their sdp_full).
        const int t = threadIdx.x, q = t & 127;
        const float* vsrc = reinterpret_cast<const float*>(smem + L::kVecOff + stage * 1024);
        const float val = (t < 128) ? -vsrc[q] * inv_scale_log2 : -vsrc[128 + q] * inv_scale;
        const __nv_bfloat16 hi = __float2bfloat16(val);
        const __nv_bfloat16 lo = __float2bfloat16(val - __bfloat162float(hi));
        unsigned char* dst = smem + L::kAugOff + (t < 128 ? 0 : 4096) + (q >> 3) * 256 + (q & 7) * 16;
        *reinterpret_cast<uint32_t*>(dst) = (uint32_t)__bfloat16_as_ushort(hi) | ((uint32_t)__bfloat16_as_ushort(lo) << 16);
        fence_proxy_async();
        mbar_arrive_warp(aug_full);
      }
      if (!mbar_wait(sdp_full, ph_sdp, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
      ph_sdp ^= 1;
      tc_fence_after();
      const bool diag = (m == n);
      uint32_t sv[64], dv[64];
      tmem_ld_32x32(tm_s + lane_off + 64 * h, sv);
      tmem_ld_32x32(tm_s + lane_off + 64 * h + 32, sv + 32);
      tmem_ld_32x32(tm_dp + lane_off + 64 * h, dv);
      tmem_ld_32x32(tm_dp + lane_off + 64 * h + 32, dv + 32);
      tmem_wait_ld();
      const int q_first = m * 128 + 64 * h;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const int qc = c * 32 + e;
          float p0 = exp2f(__uint_as_float(sv[qc]) * scale_log2);        // the accumulator already holds S - lse
          float p1 = exp2f(__uint_as_float(sv[qc + 1]) * scale_log2);
          if (diag) {
            if (key > q_first + qc) p0 = 0.f;
            if (key > q_first + qc + 1) p1 = 0.f;
          }
          const float d0 = (p0 * scale) * __uint_as_float(dv[qc]);           // ... and dP - delta
          const float d1 = (p1 * scale) * __uint_as_float(dv[qc + 1]);
          pk[e / 2] = pack_bf16(p0, p1);
          dk[e / 2] = pack_bf16(d0, d1);
        }
        // P^T / dS^T of queries [64h+32c, +32) go to packed columns [64h+16c, +16): inside this warpgroup's own
        // S^T / dP^T column range, all of which this thread has already read
        tmem_st_32x16(tm_s + lane_off + 64 * h + c * 16, pk);
        tmem_st_32x16(tm_dp + lane_off + 64 * h + c * 16, dk);
#pragma unroll
        for (int p4 = 0; p4 < 4; ++p4) {
          const int piece = c * 4 + p4;
          *reinterpret_cast<uint4*>(ds_row + ((piece ^ (r & 7)) * 16)) = make_uint4(dk[p4 * 4], dk[p4 * 4 + 1], dk[p4 * 4 + 2], dk[p4 * 4 + 3]);
        }
      }
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_warp(pds_full);
      // drain dQ of this step
      if (!mbar_wait(dq_full, ph_dq, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
      ph_dq ^= 1;
      tc_fence_after();
      drain_tile(tm_dq, q_col, grow0 + m * 128);
      tc_fence_before();
      mbar_arrive_warp(dq_drained);
      if (++stage == QS) { stage = 0; qphase ^= 1; }
    }
    if (ok) {
      // the last dq_full also covers the final dK / dV accumulation
      drain_tile(tm_dk, k_col, grow0 + n * 128);
      drain_tile(tm_dv, v_col, grow0 + n * 128);
    }
    if (issuer) tma_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------------------------------------
// head_dim 64 backward, software-pipelined.  Same math and data flow as flash_bwd_kernel, but the 128-query block of a step
// is handled as two 64-query halves with their own barriers, so the long serial chain of a step (commit -> tensor-memory
// load -> exp / dS math -> tensor-memory store -> fence -> barrier -> next MMA) of one half runs while the tensor core
// works on the other half and on the next step:
//     MMA order:  ... | dV_A dK_A (i) | S_A dP_A (i+1) | dV_B dK_B (i) | dQ (i) | S_B dP_B (i+1) | dV_A dK_A (i+1) | ...
// Warpgroup h computes half h.  dS^T lives in a double-buffered shared-memory operand and dQ in a double-buffered
// tensor-memory tile; tensor memory (512 columns): S^T 128, dP^T 128, dK 64, dV 64, dQ 64, K 32, V 32.
// ---------------------------------------------------------------------------------------------------------------------
struct Bwd64Smem {
  static constexpr int kTile = 128 * 64 * 2;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kTile;
  static constexpr int kQdOOff = 2 * kTile;              // 2 stages x (Q tile, dO tile)
  static constexpr int kDsOff = kQdOOff + 4 * kTile;     // 2 buffers x 2 chunks x [128 x 128 B]
  static constexpr int kStgOff = kDsOff + 65536;         // one [128 x 128 B] fp32 staging buffer per warpgroup
  // "augmentation" operands (see the kernel): a constant [128 x 16] tile of ones and, per stage, four [64 x 16] tiles
  // (S^T half 0 / 1, dP^T half 0 / 1) holding -lse2 / scale_log2 resp. -delta split into two bf16, all K-major, no swizzle
  static constexpr int kOnesOff = kStgOff + 32768;       // 4 KB
  static constexpr int kAugOff = kOnesOff + 4096;        // 2 stages x 4 x 2 KB
  static constexpr int kBarOff = kAugOff + 16384;
  static constexpr int kTotal = kBarOff + 512 + 1024;
};

__global__ void __launch_bounds__(kBwd64Threads, 1)
flash_bwd64_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_q64,
                   const __grid_constant__ CUtensorMap tmap_do64,
                   const __grid_constant__ CUtensorMap tmap_dqkv, const float* __restrict__ lse2, const float* __restrict__ delta,
                   int S, int n_kv, int g, float scale, float scale_log2, int* __restrict__ status, long long* __restrict__ dbg) {
  using L = Bwd64Smem;
  constexpr int D = 64;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;             // [1]
  uint64_t* q_full = bars + 1;          // [2 stages][2 query halves]: rows 64h .. 64h+63 of the Q and dO tiles
  uint64_t* q_empty = q_full + 4;       // [2][2]
  uint64_t* sdp_full = q_empty + 4;     // [2] per half: S^T and dP^T ready
  uint64_t* pds_full = sdp_full + 2;    // [2] per half: P^T, dS^T written (4 arrivals, one per warp)
  uint64_t* dq_full = pds_full + 2;     // [2] per dQ buffer
  uint64_t* dq_drained = dq_full + 2;   // [2] per dQ buffer (4 arrivals)
  uint64_t* kv_tmem = dq_drained + 1;   // K and V copied into tensor memory (4 arrivals); dq_full / dq_drained use slot 0 only
  uint64_t* aug_full = dq_drained + 2;  // [2] per stage: augmentation tiles written (4 arrivals, one per drain warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aug_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n_blk = S / 128;
  const int n = n_blk - 1 - (int)blockIdx.x;
  const int head = blockIdx.y;
  const int b = blockIdx.z;
  const int j = head / g, i = head % g;
  const int nq = n_kv * g;
  const int q_col = (j * (g + 2) + i) * D, k_col = (j * (g + 2) + g) * D, v_col = k_col + D;
  const int do_col = head * D;
  const int grow0 = b * S;
  const int steps = n_blk - n;
  const float* lse2_h = lse2 + ((size_t)b * nq + head) * S;
  const float* delta_h = delta + ((size_t)b * nq + head) * S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(kv_tmem, 4);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[2 * s], 1); mbar_init(&q_full[2 * s + 1], 1);
      mbar_init(&q_empty[2 * s], 1); mbar_init(&q_empty[2 * s + 1], 1);
      mbar_init(&sdp_full[s], 1); mbar_init(&pds_full[s], 4);     // one arrival per warp
      mbar_init(&dq_full[s], 1); mbar_init(&dq_drained[s], 4);
      mbar_init(&aug_full[s], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 13) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dk = tmem_base + 256, tm_dv = tmem_base + 320;
  const uint32_t tm_dq0 = tmem_base + 384;  // one 64-column buffer
  // K and V as bf16 A operands in tensor memory (32 columns each): S^T = K Q^T and dP^T = V dO^T then fetch only their
  // 2 KB B operand from shared memory per MMA instead of 6 KB, and the shared-memory ports are what these MMAs wait for
  const uint32_t tm_k = tmem_base + 448, tm_v = tmem_base + 480;

  if (warp == 12) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_qkv);
      tma_prefetch_desc(&tmap_q64);
      tma_prefetch_desc(&tmap_do64);
      mbar_expect_tx(kv_full, 2 * L::kTile);
      tma_load_2d(smem + L::kKOff, &tmap_qkv, k_col, grow0 + n * 128, kv_full);
      tma_load_2d(smem + L::kVOff, &tmap_qkv, v_col, grow0 + n * 128, kv_full);
      // Q and dO arrive per query half: half h of a stage is free as soon as the dV / dK products of that half have
      // read it, half a step before the whole tile would be, which keeps the loads ahead of the shortened steps
      bool live = true;
      for (int st = 0; st < steps && live; ++st) {
        const int stage = st & 1;
        const uint32_t phase = (st >> 1) & 1;
        const int m = n + st;
        unsigned char* sq = smem + L::kQdOOff + stage * 2 * L::kTile;
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&q_empty[2 * stage + h], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) { live = false; break; }
          mbar_expect_tx(&q_full[2 * stage + h], L::kTile);
          tma_load_2d(sq + h * 8192, &tmap_q64, q_col, grow0 + m * 128 + 64 * h, &q_full[2 * stage + h]);
          tma_load_2d(sq + L::kTile + h * 8192, &tmap_do64, do_col, grow0 + m * 128 + 64 * h, &q_full[2 * stage + h]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 13) {
    if (elect_one()) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);   // S^T / dP^T half: 128 keys x 64 queries
      constexpr uint32_t idesc_dkv = make_idesc_bf16(128, D, false, true);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, true, true);
      const uint32_t k_addr = smem_u32(smem + L::kKOff), v_addr = smem_u32(smem + L::kVOff);
      bool ok = mbar_wait(kv_full, 0, abort_flag, status, kTimeoutSmemFull);
      if (ok) ok = mbar_wait(kv_tmem, 0, abort_flag, status, kTimeoutTmemFull);
      // S^T_h = K Q_h^T and dP^T_h = V dO_h^T for query half h of the tile in `stage`
      auto issue_sdp = [&](int stage, int h) {
        const uint32_t q_addr = smem_u32(smem + L::kQdOOff + stage * 2 * L::kTile) + h * 8192;
        const uint32_t do_addr = q_addr + L::kTile;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(tm_s + 64 * h, tm_k + kk * 8, make_smem_desc(q_addr + kk * 32, 0, 1024), idesc_st, kk != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(tm_dp + 64 * h, tm_v + kk * 8, make_smem_desc(do_addr + kk * 32, 0, 1024), idesc_st, kk != 0);
        // fifth k-step: ones x (-lse2 / scale_log2) resp. ones x (-delta), so the accumulators already hold the exponent
        // argument and dP - delta and no thread has to fetch per-query vectors
        const uint32_t aug = smem_u32(smem + L::kAugOff + stage * 8192);
        const uint64_t ones_desc = make_smem_desc_plain(smem_u32(smem + L::kOnesOff), 128, 256);
        umma_bf16_ss(tm_s + 64 * h, ones_desc, make_smem_desc_plain(aug + h * 2048, 128, 256), idesc_st, 1u);
        umma_bf16_ss(tm_dp + 64 * h, ones_desc, make_smem_desc_plain(aug + 4096 + h * 2048, 128, 256), idesc_st, 1u);
        umma_commit(&sdp_full[h]);
      };
      // dV += P_h^T dO_h ; dK += dS_h^T Q_h  (64 queries = 4 steps of 16)
      auto issue_dkv = [&](int stage, int h, bool first) {
        const uint32_t q_addr = smem_u32(smem + L::kQdOOff + stage * 2 * L::kTile);
        const uint32_t do_addr = q_addr + L::kTile;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(tm_dv, tm_s + 64 * h + kk * 8, make_smem_desc(do_addr + (4 * h + kk) * 2048, 16384, 1024), idesc_dkv,
                       !(first && kk == 0));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(tm_dk, tm_dp + 64 * h + kk * 8, make_smem_desc(q_addr + (4 * h + kk) * 2048, 16384, 1024), idesc_dkv,
                       !(first && kk == 0));
      };
      if (ok) ok = mbar_wait(&aug_full[0], 0, abort_flag, status, kTimeoutSmemFull);
      if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag, status, kTimeoutSmemFull);
      if (ok) { tc_fence_after(); issue_sdp(0, 0); }
      if (ok) ok = mbar_wait(&q_full[1], 0, abort_flag, status, kTimeoutSmemFull);
      if (ok) { tc_fence_after(); issue_sdp(0, 1); }
      const bool mrec = dbg != nullptr && blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && blockIdx.z == 0;
#define FTH_MS(i) do { if (mrec && st < 64) dbg[(16 + (i)) * 64 + st] = clock64(); } while (0)
      for (int st = 0; st < steps && ok; ++st) {
        const int stage = st & 1, nstage = stage ^ 1;
        const uint32_t ph = st & 1;
        const bool more = st + 1 < steps;
        // ---- half A
        FTH_MS(0);
        if (!mbar_wait(&pds_full[0], ph, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        FTH_MS(1);
        issue_dkv(stage, 0, st == 0);
        umma_commit(&q_empty[2 * stage]);
        if (more) {
          if (!mbar_wait(&q_full[2 * nstage], ((st + 1) >> 1) & 1, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          if (!mbar_wait(&aug_full[nstage], ((st + 1) >> 1) & 1, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          tc_fence_after();
          FTH_MS(2);
          issue_sdp(nstage, 0);
        }
        FTH_MS(3);
        // ---- half B
        if (!mbar_wait(&pds_full[1], ph, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        FTH_MS(4);
        issue_dkv(stage, 1, false);
        umma_commit(&q_empty[2 * stage + 1]);
        // the next S^T / dP^T of this half goes first: warpgroup 1 waits for it, nobody waits for dQ
        if (more) {
          if (!mbar_wait(&q_full[2 * nstage + 1], ((st + 1) >> 1) & 1, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          tc_fence_after();
          issue_sdp(nstage, 1);
        }
        // ---- dQ(st) = dS K into buffer st & 1 (free once dQ(st-2) was drained)
        if (st >= 1) {   // the drain warps have read dQ(st - 1) out of the (single) buffer
          if (!mbar_wait(&dq_drained[0], (st - 1) & 1, abort_flag, status, kTimeoutTmemEmpty)) { ok = false; break; }
          tc_fence_after();
        }
        FTH_MS(5);
        const uint32_t ds_addr = smem_u32(smem + L::kDsOff + (st & 1) * 32768);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_ss(tm_dq0, make_smem_desc(ds_addr + kk * 2048, 16384, 1024),
                       make_smem_desc(k_addr + kk * 2048, 16384, 1024), idesc_dq, kk != 0);
        umma_commit(&dq_full[0]);
        FTH_MS(6);
      }
#undef FTH_MS
    }
    __syncwarp();
  } else if (warp >= 8 && warp < 12) {
    // ---------------- drain warps: dQ of every step, then dK and dV, tensor memory -> TMA reduce-add ----------------
    const int qd = warp - 8;
    const int r = qd * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    unsigned char* stg = smem + L::kStgOff;               // two [128 x 128 B] chunks = the 64 fp32 columns of a tile
    const bool issuer = (threadIdx.x == 256);
    auto drain64 = [&](uint32_t tm_src, int col, int row, uint64_t* release_bar) {
      if (issuer) tma_wait_group_read<0>();
      named_barrier_sync(3, 128);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tm_src + lane_off + c * 32, v);
        tmem_wait_ld();
        if (c == 1 && release_bar != nullptr) { tc_fence_before(); mbar_arrive_warp(release_bar); }   // the tile may be overwritten now
        unsigned char* rowp = stg + c * 16384 + r * 128;
#pragma unroll
        for (int p8 = 0; p8 < 8; ++p8)
          *reinterpret_cast<uint4*>(rowp + ((p8 ^ (r & 7)) * 16)) = make_uint4(v[p8 * 4], v[p8 * 4 + 1], v[p8 * 4 + 2], v[p8 * 4 + 3]);
      }
      fence_proxy_async();
      named_barrier_sync(3, 128);
      if (issuer) {
        tma_reduce_add_2d(&tmap_dqkv, stg, col, row);
        tma_reduce_add_2d(&tmap_dqkv, stg + 16384, col + 32, row);
        tma_commit_group();
      }
    };
    // Augmentation tiles.  Thread t of the 128 owns query t of a step: -lse2 / scale_log2 and -delta (the pre-pass stores
    // delta * scale) as bf16 hi + lo pairs in columns 0 and 1 of its row; the constant tile has ones in those two columns.
    const float inv_scale_log2 = 1.f / scale_log2, inv_scale = 1.f / scale;
    auto write_aug = [&](int st_for) {
      const int m = n + st_for, hq = r >> 6, ql = r & 63;
      const float vs = -lse2_h[m * 128 + r] * inv_scale_log2, vd = -delta_h[m * 128 + r] * inv_scale;
      const __nv_bfloat16 s_hi = __float2bfloat16(vs), d_hi = __float2bfloat16(vd);
      const __nv_bfloat16 s_lo = __float2bfloat16(vs - __bfloat162float(s_hi)), d_lo = __float2bfloat16(vd - __bfloat162float(d_hi));
      unsigned char* base = smem + L::kAugOff + (st_for & 1) * 8192 + hq * 2048 + (ql >> 3) * 256 + (ql & 7) * 16;
      *reinterpret_cast<uint32_t*>(base) = (uint32_t)__bfloat16_as_ushort(s_hi) | ((uint32_t)__bfloat16_as_ushort(s_lo) << 16);
      *reinterpret_cast<uint32_t*>(base + 4096) = (uint32_t)__bfloat16_as_ushort(d_hi) | ((uint32_t)__bfloat16_as_ushort(d_lo) << 16);
      fence_proxy_async();
      mbar_arrive_warp(&aug_full[st_for & 1]);
    };
    {
      // one-time: zero both stages' tiles (only columns 0 and 1 are ever rewritten) and build the ones tile
      uint4* z = reinterpret_cast<uint4*>(smem + L::kAugOff);
      for (int i = r; i < 16384 / 16; i += 128) z[i] = make_uint4(0u, 0u, 0u, 0u);
      unsigned char* one_row = smem + L::kOnesOff + (r >> 3) * 256 + (r & 7) * 16;
      *reinterpret_cast<uint4*>(one_row) = make_uint4(0x3F803F80u, 0u, 0u, 0u);          // bf16 1.0, 1.0, then zeros
      *reinterpret_cast<uint4*>(one_row + 128) = make_uint4(0u, 0u, 0u, 0u);
      named_barrier_sync(3, 128);   // the zero fill of other threads' rows is complete before anybody writes values
      write_aug(0);
      if (steps > 1) write_aug(1);
    }
    bool ok = mbar_wait(kv_full, 0, abort_flag, status, kTimeoutSmemFull);
    if (ok) {
      // row r of the 128B-swizzled K / V tile -> lane r, 32 columns of packed bf16 (the layout a tensor-memory A operand has)
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const unsigned char* rowp = smem + (which == 0 ? L::kKOff : L::kVOff) + r * 128;
        uint32_t w[32];
#pragma unroll
        for (int p8 = 0; p8 < 8; ++p8) {
          const uint4 q4 = *reinterpret_cast<const uint4*>(rowp + ((p8 ^ (r & 7)) * 16));
          w[p8 * 4] = q4.x; w[p8 * 4 + 1] = q4.y; w[p8 * 4 + 2] = q4.z; w[p8 * 4 + 3] = q4.w;
        }
        tmem_st_32x16((which == 0 ? tm_k : tm_v) + lane_off, w);
        tmem_st_32x16((which == 0 ? tm_k : tm_v) + lane_off + 16, w + 16);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(kv_tmem);
    }
    for (int st = 0; st < steps && ok; ++st) {
      if (!mbar_wait(&dq_full[0], st & 1, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      // dq_full(st) also covers the S^T / dP^T products of step st + 1, so the tiles of parity st + 1 can take step st + 3
      // (and, the first time round, those of parity 0 step 2): always more than a step ahead of the MMA warp's need
      if (st == 0 && steps > 2) write_aug(2);
      if (st + 3 < steps) write_aug(st + 3);
      drain64(tm_dq0, q_col, grow0 + (n + st) * 128, &dq_drained[0]);
    }
    if (ok) {   // the last dQ commit also covers the final dK / dV accumulation
      drain64(tm_dk, k_col, grow0 + n * 128, nullptr);
      drain64(tm_dv, v_col, grow0 + n * 128, nullptr);
    }
    if (issuer) tma_wait_group<0>();
  } else if (warp < 8) {
    // ---------------- compute warps: warpgroup h owns query half h of every step ----------------
    const int qd = warp % 4, h = warp / 4;
    const int r = qd * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const int key = n * 128 + r;
    bool ok = true;
    const bool rec = dbg != nullptr && blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && blockIdx.z == 0 && qd == 0 && lane == 0;
    long long* drow = dbg + h * 8 * 64;
#define FTH_TS(i) do { if (rec && st < 64) drow[(i) * 64 + st] = clock64(); } while (0)
    for (int st = 0; st < steps && ok; ++st) {
      const int m = n + st, stage = st & 1;
      FTH_TS(0);
      FTH_TS(6);
      if (!mbar_wait(&sdp_full[h], st & 1, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
      FTH_TS(1);
      tc_fence_after();
      const bool diag = (m == n);
      const int q_first = m * 128 + 64 * h;
      unsigned char* ds_row = smem + L::kDsOff + (st & 1) * 32768 + h * 16384 + r * 128;
      // Four 16-column chunks with a rolling prefetch: the tensor-memory load of chunk c+1 is in flight during the math
      // of chunk c.  The bf16 P^T / dS^T of chunk c land on columns [8c, 8c+8) of the warpgroup's own range, all of
      // which chunks <= c have already read.
      auto math = [&](auto diag_tag) {
        constexpr bool kDiag = decltype(diag_tag)::value;
        uint32_t sv[2][16], dv[2][16];
        tmem_ld_32x16(tm_s + lane_off + 64 * h, sv[0]);
        tmem_ld_32x16(tm_dp + lane_off + 64 * h, dv[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_wait_ld();
          if (c == 0) FTH_TS(2);
          if (c < 3) {
            tmem_ld_32x16(tm_s + lane_off + 64 * h + (c + 1) * 16, sv[(c + 1) & 1]);
            tmem_ld_32x16(tm_dp + lane_off + 64 * h + (c + 1) * 16, dv[(c + 1) & 1]);
          }
          uint32_t pk[8], dk[8];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            float p[4], d[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              p[e] = exp2f(__uint_as_float(sv[c & 1][q4 * 4 + e]) * scale_log2);   // the accumulator already holds S - lse
              if (kDiag) { if (key > q_first + c * 16 + q4 * 4 + e) p[e] = 0.f; }
              d[e] = (p[e] * scale) * __uint_as_float(dv[c & 1][q4 * 4 + e]);       // ... and dP - delta
            }
            pk[q4 * 2] = pack_bf16(p[0], p[1]); pk[q4 * 2 + 1] = pack_bf16(p[2], p[3]);
            dk[q4 * 2] = pack_bf16(d[0], d[1]); dk[q4 * 2 + 1] = pack_bf16(d[2], d[3]);
          }
          tmem_st_32x8(tm_s + lane_off + 64 * h + c * 8, pk);
          tmem_st_32x8(tm_dp + lane_off + 64 * h + c * 8, dk);
#pragma unroll
          for (int p2 = 0; p2 < 2; ++p2) {
            const int piece = c * 2 + p2;
            *reinterpret_cast<uint4*>(ds_row + ((piece ^ (r & 7)) * 16)) = make_uint4(dk[p2 * 4], dk[p2 * 4 + 1], dk[p2 * 4 + 2], dk[p2 * 4 + 3]);
          }
        }
      };
      if (diag) math(std::true_type{}); else math(std::false_type{});
      FTH_TS(3);
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive_warp(&pds_full[h]);
      FTH_TS(4);
      FTH_TS(5);
    }
#undef FTH_TS
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if (warp == 13) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// fp32 image -> bf16 packed dQKV.  With a RoPE table the inverse rotation (the RoPE backward) of the q and k head
// slots is applied on the way, so the gradient needs no separate RoPE pass.
__global__ void dqkv_finalize_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, const float* __restrict__ table,
                                     int M, int S, int n_kv, int g, int d) {
  const int half = d / 2, vph = half / 8;
  const int slots = n_kv * (g + 2);
  const size_t total = (size_t)M * slots * vph;
  const size_t row_stride = (size_t)slots * d;
  for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
    const int vec = it % vph;
    const size_t t = it / vph;
    const int sl = t % slots;
    const int row = t / slots;
    const size_t off = (size_t)row * row_stride + (size_t)sl * d + vec * 8;
    float x1[8], x2[8];
    load8(src + off, x1);
    load8(src + off + half, x2);
    if (table != nullptr && (sl % (g + 2)) <= g) {
      const float* tb = table + (size_t)(row % S) * d + vec * 8;
      float c[8], sn[8];
      load8(tb, c);
      load8(tb + half, sn);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a = x1[i], b = x2[i];
        x1[i] = a * c[i] + b * sn[i];
        x2[i] = b * c[i] - a * sn[i];
      }
    }
    store8(dst + off, x1);
    store8(dst + off + half, x2);
  }
}

int make_tmap_f32_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t box_cols);

}  // namespace fth

using namespace fth;

extern "C" {

// qkv: [B*S, n_kv*(g+2)*d] bf16 packed; out: [B*S, n_kv*g*d] bf16; lse: [B, n_kv*g, S] fp32.  S % 128 == 0, d in {64,128}.
static long long* g_fwd_dbg = nullptr;
// Optional timeline buffer (2 x 8 x 64 clock64 stamps of CTA (0,0,0)'s softmax phases); nullptr disables.
void fth_flash_fwd_set_debug(long long* buf) { g_fwd_dbg = buf; }

int fth_flash_fwd(const void* qkv, void* out, float* lse, int B, int S, int n_kv, int g, int d, int* status,
                  cudaStream_t stream) {
  if (S % 128 || (d != 64 && d != 128)) return -2;
  CUtensorMap tm;
  const uint64_t rs = (uint64_t)n_kv * (g + 2) * d;
  int r = make_tmap_bf16_2d(&tm, qkv, (uint64_t)B * S, rs, rs, 128, 64);
  if (r) return r;
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)d);
  dim3 grid((S + 255) / 256, n_kv * g, B);
  if (d == 64) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(flash_fwd2_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<64>::kTotal); set = true; }
    flash_fwd2_kernel<64><<<grid, kFwd2Threads, FwdSmem<64>::kTotal, stream>>>(tm, (__nv_bfloat16*)out, lse, S, n_kv, g, scale_log2, status, g_fwd_dbg);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(flash_fwd2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<128>::kTotal); set = true; }
    flash_fwd2_kernel<128><<<grid, kFwd2Threads, FwdSmem<128>::kTotal, stream>>>(tm, (__nv_bfloat16*)out, lse, S, n_kv, g, scale_log2, status, g_fwd_dbg);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// Scratch: `scratch_f32` holds [B*S, qkv_dim] fp32 (zeroed here) followed by delta and lse2, each [B, nq, S] fp32.
static long long* g_bwd_dbg = nullptr;
void fth_flash_bwd_set_debug(long long* buf) { g_bwd_dbg = buf; }

size_t fth_flash_bwd_scratch_bytes(int B, int S, int n_kv, int g, int d) {
  return ((size_t)B * S * n_kv * (g + 2) * d + 2 * (size_t)B * n_kv * g * S) * sizeof(float);
}

int fth_flash_bwd(const void* d_out, const void* qkv, const void* out, const float* lse, void* dqkv, void* scratch_f32,
                  const float* rope_table, int B, int S, int n_kv, int g, int d, int* status, cudaStream_t stream) {
  if (S % 128 || (d != 64 && d != 128)) return -2;
  const int nq = n_kv * g;
  const uint64_t rs = (uint64_t)n_kv * (g + 2) * d;
  const size_t n_img = (size_t)B * S * rs;
  float* img = reinterpret_cast<float*>(scratch_f32);
  float* delta = img + n_img;
  float* lse2 = delta + (size_t)B * nq * S;
  cudaMemsetAsync(img, 0, n_img * sizeof(float), stream);
  {
    long long warps = ((long long)B * S * nq + (256 / d) - 1) / (256 / d);
    int blocks = (int)((warps + 7) / 8);
    if (blocks > 148 * 16) blocks = 148 * 16;
    flash_bwd_prep_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, lse, delta, lse2,
                                                     B, S, nq, d, 1.f / sqrtf((float)d));
  }
  CUtensorMap tq, tdo, tdq;
  int r = make_tmap_bf16_2d(&tq, qkv, (uint64_t)B * S, rs, rs, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tdo, d_out, (uint64_t)B * S, (uint64_t)nq * d, (uint64_t)nq * d, 128, 64);
  if (r) return r;
  CUtensorMap tq64, tdo64;   // 64-row boxes: the head_dim-64 kernel loads Q and dO per query half
  r = make_tmap_bf16_2d(&tq64, qkv, (uint64_t)B * S, rs, rs, 64, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tdo64, d_out, (uint64_t)B * S, (uint64_t)nq * d, (uint64_t)nq * d, 64, 64);
  if (r) return r;
  r = make_tmap_f32_2d(&tdq, img, (uint64_t)B * S, rs, rs, 128, 32);
  if (r) return r;
  const float scale = 1.f / sqrtf((float)d);
  dim3 grid(S / 128, nq, B);
  if (d == 64) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(flash_bwd64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd64Smem::kTotal); set = true; }
    flash_bwd64_kernel<<<grid, kBwd64Threads, Bwd64Smem::kTotal, stream>>>(tq, tq64, tdo64, tdq, lse2, delta, S, n_kv, g, scale,
                                                                        scale * 1.4426950408889634f, status, g_bwd_dbg);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(flash_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<128>::kTotal); set = true; }
    flash_bwd_kernel<128><<<grid, kBwdThreads, BwdSmem<128>::kTotal, stream>>>(tq, tdo, tdq, lse2, delta, S, n_kv, g, scale,
                                                                              scale * 1.4426950408889634f, status);
  }
  if (cudaGetLastError() != cudaSuccess) return -21;
  size_t items = (size_t)B * S * n_kv * (g + 2) * (d / 16);
  int blocks = (int)((items + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  dqkv_finalize_kernel<<<blocks, 256, 0, stream>>>(img, (__nv_bfloat16*)dqkv, rope_table, B * S, S, n_kv, g, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
