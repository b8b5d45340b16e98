// Collectives fused with their neighbouring compute, over NVLink / NVSwitch peer memory (sm_100a).
//
// Every rank maps every peer's symmetric buffers (same offset = same logical element).  The kernels below address peers
// with plain global loads / stores on those mappings (and, as an option, with multimem.* on the NVSwitch multicast
// mapping); none of them issues a TMA load from another GPU's memory.
//
//   peer_barrier_kernel          flag barrier over the DP (or TP) group: release-store an epoch into every peer's pad, then
//                                a BOUNDED acquire-spin on the own pad.  Monotonic epochs, nothing is ever reset.
//   dp_reduce_scatter_kernel     this rank's slice of a gradient bucket = sum over ranks (fixed rank order, fp32) of the
//                                peers' buckets, written in place, fused with the sum of squares the clip needs.
//                                Replaces NCCL reduce-scatter + a separate norm pass (zero_optimizer.py:152-254).
//   adamw_push_kernel            AdamW on the owned fp32 master / moments, and the rounded bf16 parameter is stored straight
//                                into EVERY rank's parameter buffer: the parameter all-gather costs no extra pass over memory
//                                (replaces _fused_adamw_ + bf16 sync + all_gather_bf16, train_loop.py:1227-1328,
//                                zero_optimizer.py:346-385).
//   *_mm variants                the same with multimem.ld_reduce / multimem.st through the switch (opt-in).
#include "common.cuh"

namespace fth {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// pads.p[r] points at rank r's pad: `world` uint32 slots per barrier lane.  One thread per peer (one warp).
// `epoch_dev` (optional): the barrier numbers itself from a device counter (epoch = *epoch_dev + 1, written back when the
// barrier has completed), so the same launch can be replayed from a CUDA graph; every rank makes the same sequence of calls.
__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, int lane_slot, int* status,
                                    long long limit_cycles, uint32_t* epoch_dev) {
  const int t = threadIdx.x;
  if (epoch_dev != nullptr) {
    epoch = *reinterpret_cast<volatile uint32_t*>(epoch_dev) + 1;
    __syncwarp();                      // every lane has read the counter before lane 0 may advance it
    if (t == 0) *epoch_dev = epoch;    // advanced even if the wait below runs out: the ranks stay in step
  }
  if (t >= world) return;
  __threadfence_system();
  uint32_t* remote = reinterpret_cast<uint32_t*>(pads.p[t]) + lane_slot * kMaxPeers + rank;
  st_release_sys(remote, epoch);
  const uint32_t* local = reinterpret_cast<const uint32_t*>(pads.p[rank]) + lane_slot * kMaxPeers + t;
  const long long t0 = clock64();
  while ((int)(ld_acquire_sys(local) - epoch) < 0) {
    if (clock64() - t0 > limit_cycles) {
      report_status(status, kTimeoutPeerFlag);
      return;
    }
    __nanosleep(64);
  }
}

// out slice [start, start+count) of this rank's buffer = sum_r peer[r][start + i]; partial sums of squares per block.
__global__ void dp_reduce_scatter_kernel(PeerPtrs grads, long long start, long long count, int world, int rank,
                                         double* __restrict__ sumsq_partial) {
  __shared__ float red[32];
  const long long n4 = count / 4;
  float* own = reinterpret_cast<float*>(grads.p[rank]) + start;
  float acc = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + start)[i];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    reinterpret_cast<float4*>(own)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += (reinterpret_cast<const float*>(grads.p[r]) + start)[i];
    own[i] = s;
    acc += s * s;
  }
  acc = warp_sum(acc);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < blockDim.x / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = (double)t;
  }
}

// The same through the NVSwitch: one multimem.ld_reduce per 16 bytes does the cross-rank sum in the fabric.
__global__ void dp_reduce_scatter_mm_kernel(const float* __restrict__ mc_grads, float* __restrict__ own_grads, long long start,
                                            long long count, double* __restrict__ sumsq_partial) {
  __shared__ float red[32];
  const long long n4 = count / 4;
  float acc = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 s;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w)
                 : "l"(mc_grads + start + i * 4)
                 : "memory");
    reinterpret_cast<float4*>(own_grads + start)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < blockDim.x / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = (double)t;
  }
}

__global__ void sum_partials_kernel(const double* __restrict__ partial, int nb, float* __restrict__ out_accum) {
  __shared__ double red[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) acc += partial[i];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < (int)blockDim.x / 32; ++i) t += red[i];
    *out_accum += (float)t;
  }
}

struct AdamSegC {
  long long shard_off;
  long long flat_off;
  int n;
  float lr_mult;
  float wd;
  int pad;
};

// AdamW on the owned shard; the bf16 result goes to every rank's parameter buffer (mc_param != nullptr: one multimem.st).
__global__ void adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                  const float* __restrict__ grad, PeerPtrs params, __nv_bfloat16* mc_param, int world,
                                  const AdamSegC* __restrict__ segs, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, float bc1, float rsqrt_bc2, const float* __restrict__ grad_scale) {
  const AdamSegC sg = segs[blockIdx.x];
  const float gs = *grad_scale;
  const float l = lr * sg.lr_mult;
  const float decay = 1.f - l * weight_decay * sg.wd;
  const float step = __fdiv_rn(l, bc1);
  float* w = master + sg.shard_off;
  float* mm = m + sg.shard_off;
  float* vv = v + sg.shard_off;
  const float* g = grad + sg.flat_off;
  const int n8 = sg.n / 8;
  for (int i = threadIdx.x; i < n8; i += blockDim.x) {
    float ww[8], ma[8], va[8], ga[8];
    load8(w + i * 8, ww);
    load8(mm + i * 8, ma);
    load8(vv + i * 8, va);
    load8(g + i * 8, ga);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gg = ga[k] * gs;
      ww[k] *= decay;
      ma[k] += (gg - ma[k]) * (1.f - beta1);
      va[k] = va[k] * beta2 + gg * gg * (1.f - beta2);
      ww[k] -= __fdiv_rn(step * ma[k], __fsqrt_rn(va[k]) * rsqrt_bc2 + eps);  // IEEE sqrt / divide whatever the build's fast-math flag says
    }
    store8(w + i * 8, ww);
    store8(mm + i * 8, ma);
    store8(vv + i * 8, va);
    const bf16x8 pk = pack8(ww);
    const long long off = sg.flat_off + (long long)i * 8;
    if (mc_param != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(&pk);
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_param + off), "f"(__uint_as_float(u.x)),
                   "f"(__uint_as_float(u.y)), "f"(__uint_as_float(u.z)), "f"(__uint_as_float(u.w))
                   : "memory");
    } else {
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) *reinterpret_cast<bf16x8*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + off) = pk;
    }
  }
  for (int i = n8 * 8 + threadIdx.x; i < sg.n; i += blockDim.x) {
    float gg = g[i] * gs, ww = w[i] * decay;
    float ma = mm[i] + (gg - mm[i]) * (1.f - beta1);
    float va = vv[i] * beta2 + gg * gg * (1.f - beta2);
    ww -= __fdiv_rn(step * ma, __fsqrt_rn(va) * rsqrt_bc2 + eps);
    w[i] = ww; mm[i] = ma; vv[i] = va;
    const __nv_bfloat16 b = __float2bfloat16(ww);
    for (int r = 0; r < world; ++r) reinterpret_cast<__nv_bfloat16*>(params.p[r])[sg.flat_off + i] = b;
  }
}

}  // namespace fth

using namespace fth;

extern "C" {

int fth_peer_barrier(void* const* pads, int rank, int world, unsigned epoch, int lane_slot, int* status, double limit_s,
                     unsigned* epoch_dev, cudaStream_t stream) {
  if (world > kMaxPeers) return -2;
  PeerPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < world ? pads[i] : nullptr;
  long long limit = (long long)(limit_s * 1.9e9);
  peer_barrier_kernel<<<1, 32, 0, stream>>>(pp, rank, world, epoch, lane_slot, status, limit, epoch_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

int fth_dp_reduce_scatter_blocks(void) { return 148 * 4; }

// grads[r]: base of rank r's flat fp32 gradient buffer.  sumsq_accum (device float) is incremented by the slice's sum of
// squares.  mc_grads (multicast mapping of the same buffer) may be NULL: then peers are read one by one in rank order.
int fth_dp_reduce_scatter(void* const* grads, const void* mc_grads, long long start, long long count, int world, int rank,
                          double* partial, float* sumsq_accum, cudaStream_t stream) {
  if (world > kMaxPeers || (start % 4) != 0) return -2;
  const int nb = fth_dp_reduce_scatter_blocks();
  if (mc_grads != nullptr) {
    if (count % 4) return -2;
    dp_reduce_scatter_mm_kernel<<<nb, 512, 0, stream>>>((const float*)mc_grads, (float*)grads[rank], start, count, partial);
  } else {
    PeerPtrs pp;
    for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < world ? grads[i] : nullptr;
    dp_reduce_scatter_kernel<<<nb, 512, 0, stream>>>(pp, start, count, world, rank, partial);
  }
  sum_partials_kernel<<<1, 256, 0, stream>>>(partial, nb, sumsq_accum);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

int fth_adamw_push(float* master, float* m, float* v, const float* grad, void* const* params, void* mc_param, int world,
                   const void* seg_table, int n_segs, float lr, float beta1, float beta2, float eps, float weight_decay,
                   float bc1, float rsqrt_bc2, const float* grad_scale, cudaStream_t stream) {
  if (world > kMaxPeers) return -2;
  if (n_segs <= 0) return 0;
  PeerPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < world ? params[i] : nullptr;
  adamw_push_kernel<<<n_segs, 512, 0, stream>>>(master, m, v, grad, pp, (__nv_bfloat16*)mc_param, world, (const AdamSegC*)seg_table,
                                                lr, beta1, beta2, eps, weight_decay, bc1, rsqrt_bc2, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
