// MXFP8 (OCP microscaling: e4m3 payload, one e8m0 scale per 32 elements along the contraction dimension) for sm_100a:
// quantisation kernels for both orientations and a persistent warp-specialised block-scaled GEMM on
// tcgen05.mma.kind::mxf8f6f4.block_scale with the scale factors staged in tensor memory by tcgen05.cp.
//
// The reference trains in bf16 only (every matmul is torch.matmul -> cuBLAS, forward.py:83,195,198,300); this file is
// the block-scaled fp8 option of the 8B tensor-parallel target.  A linear layer needs three products, and the scale
// blocks must always run along the contraction dimension, so every operand exists in up to two quantised copies:
//   forward  Y  = X  W^T   contraction K : X  row-quantised [M,K],  W  row-quantised [N,K]
//   dgrad    dX = dY W     contraction N : dY row-quantised [M,N],  W  col-quantised, stored transposed [K,N]
//   wgrad    dW = dY^T X   contraction M : dY col-quantised, stored transposed [N,M]; X col-quantised, stored [K,M]
// "col-quantised" writes the transpose, so the GEMM below only ever sees K-major operands: C[M,N] = A[M,K] B[N,K]^T.
//
// Scale-factor storage (chosen so that no shuffle is needed between global memory and tensor memory): for every 128
// rows x 4 scale blocks (= 128 elements of K) one 512-byte chunk, byte (r % 32) * 16 + (r / 32) * 4 + (kb % 4); chunks
// are laid out [ceil(rows / 128)][ceil(K / 128)].  One chunk is exactly what one tcgen05.cp.32x128b.warpx4 moves: 32
// lanes x 16 bytes, replicated to the four 32-lane quarters of tensor memory, which is where the block-scaled MMA
// looks up the scale of accumulator row r: lane r % 32, 32-bit column r / 32, byte = scale-block id from the
// instruction descriptor.
//
// GEMM CTA = 6 warps: warp 0 TMA producer (payload tiles by tensor map, scale chunks by 1-D bulk copy), warp 1 MMA
// issuer and TMEM owner, warps 2-5 epilogue.  Tile 128 x 128 x 128, 5-stage ring, two accumulator stages.  Every
// mbarrier wait is bounded.
#include <cstdlib>

#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace fth {

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);
int make_tmap_f32_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t box_cols);
int make_tmap_u8_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_cols);

// ---- quantisation ---------------------------------------------------------------------------------------------

// e8m0 exponent byte of ceil_pow2(amax / 448): the smallest power of two s with amax / s <= 448 (e4m3 max).
__device__ __forceinline__ uint32_t e8m0_of_amax(float amax) {
  const float v = amax * (1.0f / 448.0f);
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = (bits >> 23) & 0xFF;
  if (bits & 0x7FFFFF) e += 1;            // not an exact power of two: round the exponent up
  if (e > 254) e = 254;
  return e;                               // 0 for amax == 0 (and for denormal quotients): scale 2^-127
}
__device__ __forceinline__ float inv_scale_of_e8m0(uint32_t e) {
  // 2^(127 - e) as a float; e = 0 would need 2^127 (representable), e = 254 gives 2^-127 (denormal, fine as a factor)
  return e == 254 ? __uint_as_float(0x00400000u) : __uint_as_float((254u - e) << 23);
}
__device__ __forceinline__ size_t sf_offset(int r, int kb, int k_chunks) {
  return ((size_t)(r >> 7) * k_chunks + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Row orientation: x [R, C] bf16 (row pitch ld) -> q [R, C] e4m3, scale blocks of 32 along C.  One thread per block.
__global__ void mxfp8_quant_row_kernel(const __nv_bfloat16* __restrict__ x, long long ld, uint8_t* __restrict__ q,
                                       uint8_t* __restrict__ sf, int R, int C) {
  const int blocks_per_row = C / 32, k_chunks = (blocks_per_row + 3) / 4;
  const long long total = (long long)R * blocks_per_row;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(it / blocks_per_row), kb = (int)(it % blocks_per_row);
    const __nv_bfloat16* src = x + (size_t)r * ld + kb * 32;
    float v[32];
#pragma unroll
    for (int i = 0; i < 4; ++i) load8(src + i * 8, v + i * 8);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const uint32_t e = e8m0_of_amax(amax);
    const float inv = inv_scale_of_e8m0(e);
    uint4 o[2];
    uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
    for (int i = 0; i < 8; ++i) ow[i] = pack4_e4m3(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
    uint4* dst = reinterpret_cast<uint4*>(q + (size_t)r * C + kb * 32);
    dst[0] = o[0];
    dst[1] = o[1];
    sf[sf_offset(r, kb, k_chunks)] = (uint8_t)e;
  }
}

// Column orientation: x [R, C] bf16 -> q^T [C, R] e4m3 with scale blocks of 32 along R (the contraction dimension of a
// product that reduces over rows).  A CTA takes a 32-row x 64-column patch; a thread owns one column of it.
__global__ void mxfp8_quant_col_kernel(const __nv_bfloat16* __restrict__ x, long long ld, uint8_t* __restrict__ qt,
                                       uint8_t* __restrict__ sf, int R, int C) {
  const int row_blocks = R / 32, col_tiles = (C + 63) / 64, k_chunks = (row_blocks + 3) / 4;
  const long long total = (long long)row_blocks * col_tiles;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const int rb = (int)(t / col_tiles), c = (int)(t % col_tiles) * 64 + threadIdx.x;
    if (c >= C) continue;
    const __nv_bfloat16* src = x + (size_t)rb * 32 * ld + c;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(src[(size_t)i * ld]);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const uint32_t e = e8m0_of_amax(amax);
    const float inv = inv_scale_of_e8m0(e);
    uint4 o[2];
    uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
    for (int i = 0; i < 8; ++i) ow[i] = pack4_e4m3(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
    uint4* dst = reinterpret_cast<uint4*>(qt + (size_t)c * R + rb * 32);
    dst[0] = o[0];
    dst[1] = o[1];
    sf[sf_offset(c, rb, k_chunks)] = (uint8_t)e;
  }
}

// Row orientation, coalesced form: four neighbouring lanes own one 32-element block, each one 16-byte vector of it, so a warp
// reads 512 contiguous bytes per instruction and writes 256; the block's amax is combined with two xor shuffles.
__global__ void mxfp8_quant_row4_kernel(const __nv_bfloat16* __restrict__ x, long long ld, uint8_t* __restrict__ q,
                                        uint8_t* __restrict__ sf, int R, int C) {
  const int vec_per_row = C / 8, k_chunks = (C / 32 + 3) / 4;
  const long long total = (long long)R * vec_per_row, stride = (long long)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // (row, vector-in-row) of this thread's first vector, then advanced by the grid stride without a division per vector
  long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int r = (int)(it / vec_per_row), vr = (int)(it % vec_per_row);
  const int dr = (int)(stride / vec_per_row), dv = (int)(stride % vec_per_row);
  for (; it - lane < total; it += stride) {
    const bool live = it < total;
    float v[8];
    if (live) load8(x + (size_t)r * ld + vr * 8, v);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (live) {
      const uint32_t e = e8m0_of_amax(amax);
      const float inv = inv_scale_of_e8m0(e);
      uint2 o;
      o.x = pack4_e4m3(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
      o.y = pack4_e4m3(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
      *reinterpret_cast<uint2*>(q + (size_t)r * C + vr * 8) = o;
      if ((vr & 3) == 0) sf[sf_offset(r, vr >> 2, k_chunks)] = (uint8_t)e;
    }
    r += dr;
    vr += dv;
    if (vr >= vec_per_row) { vr -= vec_per_row; ++r; }
  }
}

// Column orientation, coalesced form: a CTA stages a 32-row x 256-column patch in shared memory with 16-byte row loads
// (512 contiguous bytes per row), then thread c reads column c of the patch, quantises its 32 values and writes one
// 32-byte sector of q^T.
constexpr int kColTile = 256;
__global__ void mxfp8_quant_col_tile_kernel(const __nv_bfloat16* __restrict__ x, long long ld, uint8_t* __restrict__ qt,
                                            uint8_t* __restrict__ sf, int R, int C) {
  __shared__ __align__(16) __nv_bfloat16 patch[32][kColTile + 8];
  const int row_blocks = R / 32, col_tiles = (C + kColTile - 1) / kColTile, k_chunks = (row_blocks + 3) / 4;
  const long long total = (long long)row_blocks * col_tiles;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const int rb = (int)(t / col_tiles), c0 = (int)(t % col_tiles) * kColTile;
    __syncthreads();   // the previous patch has been consumed
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int v = threadIdx.x + k * 256, row = v / (kColTile / 8), cv = v % (kColTile / 8);
      const int col = c0 + cv * 8;
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      if (col < C) w = *reinterpret_cast<const uint4*>(x + (size_t)(rb * 32 + row) * ld + col);
      *reinterpret_cast<uint4*>(&patch[row][cv * 8]) = w;
    }
    __syncthreads();
    const int c = c0 + threadIdx.x;
    if (c < C) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(patch[i][threadIdx.x]);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
      const uint32_t e = e8m0_of_amax(amax);
      const float inv = inv_scale_of_e8m0(e);
      uint4 o[2];
      uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) ow[i] = pack4_e4m3(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
      uint4* dst = reinterpret_cast<uint4*>(qt + (size_t)c * R + rb * 32);
      dst[0] = o[0];
      dst[1] = o[1];
      sf[sf_offset(c, rb, k_chunks)] = (uint8_t)e;
    }
  }
}

// ---- block-scaled GEMM --------------------------------------------------------------------------------------------

constexpr int XBM = 128, XBN = 128, XBK = 128, XSTAGES = 5;
constexpr int kMxThreads = 192;

struct MxSmem {
  static constexpr int kABytes = XBM * XBK;          // e4m3: one byte per element, rows of 128 B = one swizzle atom
  static constexpr int kBBytes = XBN * XBK;
  static constexpr int kSfBytes = 512;               // one chunk each for A and B per stage
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSfOffset = XSTAGES * kStageBytes;
  static constexpr int kEpiOffset = kSfOffset + XSTAGES * 2 * kSfBytes;
  static constexpr int kEpiBytes = 2 * XBM * 128;
  static constexpr int kBarOffset = kEpiOffset + kEpiBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
};

// Instruction descriptor of kind::mxf8f6f4.block_scale: e4m3 x e4m3, e8m0 scales, both operands K-major.
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int M, int N, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4)                 // scale-block (byte) id of B inside its 32-bit tensor-memory column
         | (0u << 7) | (0u << 10)       // A, B format: e4m3
         | ((uint32_t)(N >> 3) << 17)
         | (1u << 23)                   // scale format: e8m0
         | ((uint32_t)(M >> 4) << 24)
         | (a_sf_id << 29);
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mxf8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem,
                                             uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void bulk_load_1d_mx(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <bool OUT_F32>
__global__ void __launch_bounds__(kMxThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb,
                  int M, int N, int K, float alpha, int accumulate, int* __restrict__ status) {
  using S = MxSmem;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + XSTAGES;
  uint64_t* tfull_bar = empty_bar + XSTAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int m_tiles = (M + XBM - 1) / XBM, n_tiles = (N + XBN - 1) / XBN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + XBK - 1) / XBK;   // also the number of scale chunks per 128 rows
  constexpr uint32_t kTmemCols = 512;         // 2 x 128 accumulator columns + 2 x (4 + 4) scale columns, power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < XSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf = tmem_base + 2 * XBN;   // two sets of 4 columns SFA + 4 columns SFB

  // m fastest inside groups of 16 row blocks: concurrently running CTAs share B tiles out of L2
  const int group_m = m_tiles < 16 ? m_tiles : 16;
  auto tile_coords = [&](int t, int& mb, int& nb) {
    int per_group = group_m * n_tiles;
    int gidx = t / per_group, r = t % per_group;
    int m_first = gidx * group_m;
    int gsz = min(group_m, m_tiles - m_first);
    mb = m_first + r % gsz;
    nb = r / gsz;
  };

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, mb, nb);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, kTimeoutSmemEmpty)) { ok = false; break; }
          unsigned char* sa = smem + stage * S::kStageBytes;
          unsigned char* sb = sa + S::kABytes;
          unsigned char* ssf = smem + S::kSfOffset + stage * 2 * S::kSfBytes;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes + 2 * S::kSfBytes);
          tma_load_2d(sa, &tmap_a, kb * XBK, mb * XBM, &full_bar[stage]);
          tma_load_2d(sb, &tmap_b, kb * XBK, nb * XBN, &full_bar[stage]);
          bulk_load_1d_mx(ssf, sfa + ((size_t)mb * k_blocks + kb) * 512, 512, &full_bar[stage]);
          bulk_load_1d_mx(ssf + 512, sfb + ((size_t)nb * k_blocks + kb) * 512, 512, &full_bar[stage]);
          if (++stage == XSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t sfbuf = 0;   // the scale columns alternate between two sets from one k block to the next
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * XBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, kTimeoutSmemFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          const uint32_t ssf = smem_u32(smem + S::kSfOffset + stage * 2 * S::kSfBytes);
          const uint32_t t_sfa = tmem_sf + sfbuf * 8, t_sfb = t_sfa + 4;
          sfbuf ^= 1;
          // scale chunks: shared memory -> tensor memory (same pipe and issue order as the MMAs that read them)
          tmem_cp_32x128b_warpx4(t_sfa, make_smem_desc_plain(ssf, 16, 128));
          tmem_cp_32x128b_warpx4(t_sfb, make_smem_desc_plain(ssf + 512, 16, 128));
#pragma unroll
          for (int kk = 0; kk < XBK / 32; ++kk) {
            const uint64_t adesc = make_smem_desc(sa + kk * 32, 0, 1024);
            const uint64_t bdesc = make_smem_desc(sb + kk * 32, 0, 1024);
            umma_mxf8_ss(d_tmem, adesc, bdesc, make_idesc_mxf8(XBM, XBN, kk, kk), t_sfa, t_sfb, (kb != 0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == XSTAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // epilogue: TMEM -> registers -> 128B-swizzled staging -> TMA store (bf16 / fp32) or TMA reduce-add (fp32 accumulate)
    const int q = warp % 4;
    const int r_in_tile = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    constexpr int CW = OUT_F32 ? 32 : 64;
    unsigned char* stg = smem + S::kEpiOffset;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, mb, nb);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * XBN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < XBN / CW; ++c) {
        const int col0 = nb * XBN + c * CW;
        if (col0 >= N) break;
        uint32_t r[CW];
        tmem_ld_32x32(taddr + c * CW, r);
        if constexpr (CW == 64) tmem_ld_32x32(taddr + c * CW + 32, r + 32);
        tmem_wait_ld();
        if (issuer) tma_wait_group_read<1>();
        named_barrier_sync(1, 128);
        unsigned char* row_ptr = stg + buf * (XBM * 128) + r_in_tile * 128;
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
          if (OUT_F32 && accumulate) tma_reduce_add_2d(&tmap_c, stg + buf * (XBM * 128), col0, mb * XBM);
          else tma_store_2d(&tmap_c, stg + buf * (XBM * 128), col0, mb * XBM);
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

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { __nanosleep(200); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int mx_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace fth

using namespace fth;

extern "C" {

// Bytes of the scale-factor array for a [rows, K] operand (K % 32 == 0): whole 512-byte chunks.
size_t fth_mxfp8_sf_bytes(int rows, int K) { return (size_t)((rows + 127) / 128) * ((K / 32 + 3) / 4) * 512; }

// colwise = 0: q [R, C] with blocks along C (needs C % 32 == 0).  colwise = 1: q^T [C, R] with blocks along R (R % 32 == 0).
// `sf` must hold fth_mxfp8_sf_bytes(R, C) resp. (C, R) bytes and be zero-initialised by the caller when rows or K / 32
// do not fill whole chunks (unused scale bytes then read as 2^-127 and multiply zero-filled payload).
int fth_mxfp8_quant(const void* x, long long ld, void* q, void* sf, int R, int C, int colwise, cudaStream_t stream) {
  if (R <= 0 || C <= 0) return 0;
  if (ld % 8) return -1;
  if (!colwise) {
    if (C % 32) return -2;
    long long total = (long long)R * (C / 32);
    int grid = (int)((total + 255) / 256);
    if (grid > mx_sm_count() * 16) grid = mx_sm_count() * 16;
    // coalesced form (4 lanes per block); FTH_MXFP8_QUANT_V1=1 (both orientations) or =row selects the one-thread-per-block
    // kernel (same bits)
    static const bool v1 = getenv("FTH_MXFP8_QUANT_V1") != nullptr &&
                           (getenv("FTH_MXFP8_QUANT_V1")[0] == '1' || getenv("FTH_MXFP8_QUANT_V1")[0] == 'r');
    if (v1) {
      mxfp8_quant_row_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, R, C);
    } else {
      long long vecs = (long long)R * (C / 8);
      int g4 = (int)((vecs + 255) / 256);
      if (g4 > mx_sm_count() * 16) g4 = mx_sm_count() * 16;
      mxfp8_quant_row4_kernel<<<g4, 256, 0, stream>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, R, C);
    }
  } else {
    if (R % 32 || R % 16) return -2;
    long long total = (long long)(R / 32) * ((C + 63) / 64);
    int grid = (int)(total < (long long)mx_sm_count() * 32 ? total : (long long)mx_sm_count() * 32);
    static const bool v1c = getenv("FTH_MXFP8_QUANT_V1") != nullptr &&
                            (getenv("FTH_MXFP8_QUANT_V1")[0] == '1' || getenv("FTH_MXFP8_QUANT_V1")[0] == 'c');
    if (v1c || C % 8) {   // the tiled kernel loads 16-byte vectors along the columns
      mxfp8_quant_col_kernel<<<grid, 64, 0, stream>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, R, C);
    } else {
      long long tiles = (long long)(R / 32) * ((C + kColTile - 1) / kColTile);
      int gt = (int)(tiles < (long long)mx_sm_count() * 8 ? tiles : (long long)mx_sm_count() * 8);
      mxfp8_quant_col_tile_kernel<<<gt, 256, 0, stream>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, R, C);
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// C[M,N] (op)= alpha * A[M,K] B[N,K]^T with e4m3 payloads (row pitch K bytes, K % 16 == 0) and e8m0 scale chunks.
//   epi: 0 = store bf16, 1 = fp32 accumulate (C += ...), 2 = fp32 store.
int fth_gemm_mxfp8(const void* a, const void* sfa, const void* b, const void* sfb, void* c, long long ldc, int M, int N, int K,
                   float alpha, int epi, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 32) return -1;
  if (epi == 0 ? (ldc % 8) : (ldc % 4)) return -2;
  CUtensorMap ta, tb, tc;
  int r = make_tmap_u8_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)K, XBM, XBK);
  if (r) return r;
  r = make_tmap_u8_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)K, XBN, XBK);
  if (r) return r;
  const bool f32 = epi != 0;
  r = f32 ? make_tmap_f32_2d(&tc, c, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, XBM, 32)
          : make_tmap_bf16_2d(&tc, c, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, XBM, 64);
  if (r) return r;
  const int tiles = ((M + XBM - 1) / XBM) * ((N + XBN - 1) / XBN);
  const int grid = tiles < mx_sm_count() ? tiles : mx_sm_count();
  static bool set0 = false, set1 = false;
  if (f32) {
    if (!set1) { if (cudaFuncSetAttribute(gemm_mxfp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem::kTotal) != cudaSuccess) return -20; set1 = true; }
    gemm_mxfp8_kernel<true><<<grid, kMxThreads, MxSmem::kTotal, stream>>>(ta, tb, tc, (const uint8_t*)sfa, (const uint8_t*)sfb, M, N, K,
                                                                       alpha, epi == 1 ? 1 : 0, status);
  } else {
    if (!set0) { if (cudaFuncSetAttribute(gemm_mxfp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem::kTotal) != cudaSuccess) return -20; set0 = true; }
    gemm_mxfp8_kernel<false><<<grid, kMxThreads, MxSmem::kTotal, stream>>>(ta, tb, tc, (const uint8_t*)sfa, (const uint8_t*)sfb, M, N, K,
                                                                        alpha, 0, status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
