// Causal GQA flash attention for sm_100a on the packed kv-group-major QKV activation.
//
// Forward: one CTA owns two 128-row query tiles of one head ("A" and "B", 256 consecutive positions) and streams
// 128-row K/V blocks through a TMA ring shared by both tiles.  S = Q K^T is a tcgen05.mma (operands in shared
// memory) into tensor memory; two softmax warpgroups (one per tile, one thread per query row) read S with
// tcgen05.ld, run the online softmax in the log2 domain, write P as packed bf16 back into the SAME tensor-memory
// columns, and O += P V is a tcgen05.mma with the A operand taken from tensor memory.  While one tile's softmax
// runs, the tensor core works on the other tile (ping-pong).  O is rescaled in place only when a row's running
// max moved by more than 2^8 (the stale max keeps P bounded by 256), which makes the correction rare.
// Returns the log-sum-exp per row so the backward never replays the forward (the reference's forward drops it
// and its backward re-runs flash-attn under autograd: forward.py:233-235, backward.py:518-527).
//
// Replaces flash_attn_func / _flash_attn_backward (FA2, mma.sync) at forward.py:204-235 and backward.py:473-527.
// Q/K/V are read in place from the QKV GEMM output through one 2-D tensor map (no .contiguous() copies of K and V,
// forward.py:83-93), and the backward writes dQ/dK/dV straight into the packed layout the QKV wgrad/dgrad consume.
#include <cuda.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace fth {

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr int kFwdThreads = 320;  // warps 0-3 softmax A, 4-7 softmax B, 8 TMA, 9 MMA
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct FwdSmem {
  static constexpr int kTile = 128 * D * 2;            // one 128 x D bf16 tile
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kQOff = 0;                       // Q_A, Q_B
  static constexpr int kKVOff = 2 * kTile;              // per stage: K tile, V tile
  static constexpr int kBarOff = kKVOff + kStages * 2 * kTile;
  static constexpr int kTotal = kBarOff + 512 + 1024;
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap, __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out,
                 int S, int n_kv, int g, float scale_log2, int* __restrict__ status) {
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
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 128); mbar_init(&o_done[t], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // tensor-memory columns: S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,256+D)  O_B [384,384+D)
  const uint32_t tm_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tm_o[2] = {tmem_base + 256, tmem_base + 384};

  if (warp == 8) {
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
  } else if (warp == 9) {
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
          umma_bf16_ts(tm_o[t], tm_s[t] + kk * 8, make_smem_desc(v_addr + kk * 2048, 16384, 1024), idesc_o,
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
    // ---------------- softmax warpgroups ----------------
    const int t = warp / 4;                 // tile 0 = A, 1 = B
    const int qw = warp % 4;
    const int nb = (t == 0) ? tA + 1 : (has_b ? tA + 2 : 0);
    const int qrow = q0 + t * 128 + qw * 32 + lane;   // query position of this thread's row
    const uint32_t lane_off = (uint32_t)(qw * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    uint32_t ph_s = 0, ph_o = 0;
    bool ok = true;
    for (int kb = 0; kb < nb && ok; ++kb) {
      if (!mbar_wait(&s_full[t], ph_s, abort_flag, status, kTimeoutTmemFull)) { ok = false; break; }
      ph_s ^= 1;
      tc_fence_after();
      const bool diag = (kb * 128 + 127 > q0 + t * 128);  // block touches the causal boundary
      const int kpos0 = kb * 128;
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tm_s[t] + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float v = __uint_as_float(r[e]);
          if (diag && kpos0 + c * 32 + e > qrow) v = -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      mx *= scale_log2;
      float m_new = fmaxf(m_run, mx);
      // keep the stale max unless it moved a lot (P stays <= 2^8); always take it on the first block
      float m_use = (m_new - m_run > kRescaleThreshold) ? m_new : m_run;
      if (m_run == -INFINITY) m_use = m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
      const bool need_fix = (m_use != m_run) && kb > 0;
      // pass 2: P = exp2(s*scale - m), row sum, packed bf16 into the S columns
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32], pk[16];
        tmem_ld_32x32(tm_s[t] + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float v0 = __uint_as_float(r[e]) * scale_log2 - m_use, v1 = __uint_as_float(r[e + 1]) * scale_log2 - m_use;
          float p0 = exp2f(v0), p1 = exp2f(v1);
          if (diag) {
            if (kpos0 + c * 32 + e > qrow) p0 = 0.f;
            if (kpos0 + c * 32 + e + 1 > qrow) p1 = 0.f;
          }
          rs += p0 + p1;
          pk[e / 2] = pack_bf16(p0, p1);
        }
        // all four chunks of S have been read by this thread before any P column it aliases is needed?  P chunk c
        // occupies columns [16c, 16c+16) which alias S columns of chunk c/2 <= c, already consumed.
        tmem_st_32x16(tm_s[t] + lane_off + c * 16, pk);
      }
      l_run = l_run * alpha + rs;
      m_run = m_use;
      // O correction (needs the previous P V of this tile to be complete)
      if (kb > 0) {
        if (!mbar_wait(&o_done[t], ph_o, abort_flag, status, kTimeoutTmemEmpty)) { ok = false; break; }
        ph_o ^= 1;
        tc_fence_after();
        if (__any_sync(0xffffffffu, need_fix)) {
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t r[16];
            tmem_ld_32x16(tm_o[t] + lane_off + c * 16, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_32x16(tm_o[t] + lane_off + c * 16, r);
          }
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }
    // epilogue: O / l -> bf16, lse
    if (nb > 0 && ok) {
      if (mbar_wait(&o_done[t], ph_o, abort_flag, status, kTimeoutTmemEmpty)) {
        tc_fence_after();
        const float inv = 1.f / l_run;
        __nv_bfloat16* dst = out + (size_t)(grow0 + qrow) * ((size_t)n_kv * g * D) + (size_t)head * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tm_o[t] + lane_off + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * inv;
            store8(dst + c * 32 + v * 8, f);
          }
        }
        lse_out[((size_t)b * (n_kv * g) + head) * S + qrow] = (m_run + log2f(l_run)) * 0.6931471805599453f;
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
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace fth

using namespace fth;

extern "C" {

// qkv: [B*S, n_kv*(g+2)*d] bf16 packed; out: [B*S, n_kv*g*d] bf16; lse: [B, n_kv*g, S] fp32.  S % 128 == 0, d in {64,128}.
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
    if (!set) { cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<64>::kTotal); set = true; }
    flash_fwd_kernel<64><<<grid, kFwdThreads, FwdSmem<64>::kTotal, stream>>>(tm, (__nv_bfloat16*)out, lse, S, n_kv, g, scale_log2, status);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<128>::kTotal); set = true; }
    flash_fwd_kernel<128><<<grid, kFwdThreads, FwdSmem<128>::kTotal, stream>>>(tm, (__nv_bfloat16*)out, lse, S, n_kv, g, scale_log2, status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
