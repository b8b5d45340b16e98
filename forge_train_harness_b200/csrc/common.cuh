// Shared device helpers for the sm_100a kernels: vector types, reductions, status words, bounded waits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fth {

// ---- status words -------------------------------------------------------------------------
// A kernel that gives up on a wait writes one of these into a device status word and returns;
// the host reads the word after the step's event sync and raises.  No kernel traps or spins forever.
enum StatusCode : int {
  kOk = 0,
  kTimeoutSmemFull = 1,    // consumer waited for a TMA stage that never arrived
  kTimeoutSmemEmpty = 2,   // producer waited for a stage that was never released
  kTimeoutTmemFull = 3,    // epilogue waited for an accumulator that was never committed
  kTimeoutTmemEmpty = 4,   // MMA issuer waited for an accumulator that was never drained
  kTimeoutPeerFlag = 5,    // a flag another GPU should have written never changed
  kTimeoutGeneric = 6,
  kBadIndex = 7,           // an input check found an index outside its valid range (debug checks; no wait involved)
};

constexpr long long kSpinLimitCycles = 4000000000LL;  // ~2 s at B200 clocks

__device__ __forceinline__ void report_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// ---- small utilities ------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// 8-element vector load/store for bf16 (16 B) and float (2 x 16 B) rows, converting to fp32 registers.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  bf16x8 v = *reinterpret_cast<const bf16x8*>(p);
  unpack8(v, f);
}
__device__ __forceinline__ void load8(const float* p, float* f) {
  float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  *reinterpret_cast<bf16x8*>(p) = pack8(f);
}
__device__ __forceinline__ void store8(float* p, const float* f) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}

}  // namespace fth
