// Memory-bound fused kernels (sm_100a): RMSNorm fwd / residual+RMSNorm fwd / RMSNorm bwd (dx + dW),
// RoPE, SwiGLU fwd/bwd, embedding fwd/bwd with the muP scale, residual add, fused cross-entropy
// (loss + in-place logits gradient), segment AdamW with low-precision write-back, sum of squares.
//
// They replace the reference's Triton kernels (workload/src/training_engine_tensor/triton_kernels.py:
// _rms_norm_fwd_kernel 172-204, _rms_norm_residual_fwd_kernel 248-289, _rms_norm_bwd_kernel 349-390,
// _swiglu_fwd_kernel 453-491, _swiglu_bwd_kernel 539-597, _ce_bwd_kernel 652-706, _rope_kernel 785-867)
// and the ATen kernels around them (F.cross_entropy forward, embedding_dense_backward, _fused_adamw_).
// All math is fp32 in registers; activations are bf16 in memory; every access is a 16-byte vector.
// Nothing here is a port: e.g. the norm backward also produces the weight gradient (the reference
// re-reads x in PyTorch for it, triton_kernels.py:430-433), the cross-entropy keeps a whole vocabulary
// row in shared memory so logits are read from HBM once, and RMSNorm has no H <= 2048 limit.
#include "common.cuh"

namespace fth {

constexpr int kRowThreads = 256;

template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* smem, int row_slot, int lane_in_row) {
  if constexpr (TPR <= 32) {
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  } else {
    v = warp_sum(v);
    constexpr int WPR = TPR / 32;
    int w = lane_in_row / 32;
    __syncthreads();
    if ((lane_in_row & 31) == 0) smem[row_slot * WPR + w] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < WPR; ++i) t += smem[row_slot * WPR + i];
    return t;
  }
}

// y = rmsnorm(r) * w * out_scale, r = x (+ res * res_scale, rounded to bf16 and written to r_out).
template <int TPR, int VPT>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res, float res_scale,
    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ r_out, __nv_bfloat16* __restrict__ y,
    float* __restrict__ rstd_out, int M, int H, float eps, float out_scale) {
  __shared__ float smem[kRowThreads / 32];
  constexpr int RPB = kRowThreads / TPR;
  const int slot = threadIdx.x / TPR, lane = threadIdx.x % TPR;
  float wv[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    int c = (v * TPR + lane) * 8;
    if (c < H) load8(w + c, wv[v]);
  }
  const int groups = (M + RPB - 1) / RPB;
  for (int g = blockIdx.x; g < groups; g += gridDim.x) {
    const int row = g * RPB + slot;
    const bool ok = row < M;
    float xv[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      int c = (v * TPR + lane) * 8;
      if (ok && c < H) {
        load8(x + (size_t)row * H + c, xv[v]);
        if (res != nullptr) {
          float rv[8];
          load8(res + (size_t)row * H + c, rv);
#pragma unroll
          for (int i = 0; i < 8; ++i) xv[v][i] = __bfloat162float(__float2bfloat16(xv[v][i] + rv[i] * res_scale));
          store8(r_out + (size_t)row * H + c, xv[v]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += xv[v][i] * xv[v][i];
      }
    }
    ss = row_sum<TPR>(ss, smem, slot, lane);
    const float rstd = __frsqrt_rn(__fdiv_rn(ss, (float)H) + eps);  // IEEE-rounded, one per row: independent of the fast-math flag
    if (ok && lane == 0) rstd_out[row] = rstd;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      int c = (v * TPR + lane) * 8;
      if (ok && c < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = xv[v][i] * rstd * wv[v][i] * out_scale;
        store8(y + (size_t)row * H + c, o);
      }
    }
  }
}

// dx = rstd*(g*w - xhat*mean(g*w*xhat)) (+ dres); per-block partial dW = sum_rows g*xhat.
template <int TPR, int VPT>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_bwd_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
    float* __restrict__ dw_partial, int M, int H, float out_scale) {
  __shared__ float smem[kRowThreads / 32];
  __shared__ float dw_s[kRowThreads * 8];
  constexpr int RPB = kRowThreads / TPR;
  const int slot = threadIdx.x / TPR, lane = threadIdx.x % TPR;
  float wv[VPT][8], dwv[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    int c = (v * TPR + lane) * 8;
    if (c < H) load8(w + c, wv[v]);
#pragma unroll
    for (int i = 0; i < 8; ++i) dwv[v][i] = 0.f;
  }
  const int groups = (M + RPB - 1) / RPB;
  for (int g = blockIdx.x; g < groups; g += gridDim.x) {
    const int row = g * RPB + slot;
    const bool ok = row < M;
    const float rstd = ok ? rstd_in[row] : 0.f;
    float gv[VPT][8], xh[VPT][8];
    bf16x8 dr[VPT];   // the residual-stream gradient is fetched with dy and x, not after the row reduction
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      int c = (v * TPR + lane) * 8;
      if (ok && c < H) {
        if (dres != nullptr) dr[v] = *reinterpret_cast<const bf16x8*>(dres + (size_t)row * H + c);
        load8(dy + (size_t)row * H + c, gv[v]);
        load8(x + (size_t)row * H + c, xh[v]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          gv[v][i] *= out_scale;
          xh[v][i] *= rstd;
          dwv[v][i] += gv[v][i] * xh[v][i];
          gv[v][i] *= wv[v][i];
          dot += gv[v][i] * xh[v][i];
        }
      }
    }
    dot = row_sum<TPR>(dot, smem, slot, lane) / (float)H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      int c = (v * TPR + lane) * 8;
      if (ok && c < H) {
        float o[8];
        if (dres != nullptr) unpack8(dr[v], o);
        else {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += rstd * (gv[v][i] - xh[v][i] * dot);
        store8(dx + (size_t)row * H + c, o);
      }
    }
  }
  // combine the RPB row slots of this block, write one partial row per block
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) dw_s[threadIdx.x * 8 + i] = dwv[v][i];
    __syncthreads();
    if (slot == 0) {
      int c = (v * TPR + lane) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float t = 0.f;
          for (int s = 0; s < RPB; ++s) t += dw_s[(s * TPR + lane) * 8 + i];
          o[i] = t;
        }
        store8(dw_partial + (size_t)blockIdx.x * H + c, o);
      }
    }
  }
}

// main_grad[c] += sum_b partial[b][c].  Block = 32 columns x 32 row-slices; the slices are combined in shared memory.
__global__ void colsum_add_kernel(const float* __restrict__ partial, float* __restrict__ out, int nb, int H) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float t = 0.f;
  if (c < H)
    for (int b = threadIdx.y; b < nb; b += 32) t += partial[(size_t)b * H + c];
  red[threadIdx.y][threadIdx.x] = t;
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) a += red[i][threadIdx.x];
    out[c] += a;
  }
}

// ---- per-head q/k RMSNorm (Qwen3 variant), on the packed kv-group-major QKV layout ------------------------------------------
// A head vector of d = 64 / 128 bf16 is owned by d / 8 neighbouring lanes (8 or 16), each holding one 16-byte vector; the sum
// of squares is combined with xor shuffles inside that lane group.  v heads pass through.  Every lane of a warp runs the
// shuffles (lanes past the end, and lanes on a v head, feed zeros / ignore the result), so no shuffle sits in divergent code.
__global__ void qk_norm_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                                   const __nv_bfloat16* __restrict__ wk, __nv_bfloat16* __restrict__ out,
                                   float* __restrict__ rstd_out, int M, int n_kv, int g, int d, float eps) {
  const int tph = d / 8, hpr = n_kv * (g + 2);
  const size_t total = (size_t)M * hpr * tph, stride = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // (row, head slot) of this thread's first vector; advanced by the grid stride (a multiple of the lane-group size, so the
  // vector position inside the head never changes) without a division per vector
  size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const int vec = (int)(it % tph);
  size_t row = (it / tph) / hpr;
  int hs = (int)((it / tph) % hpr);
  const size_t dslot = stride / tph, drow = dslot / hpr;
  const int dhs = (int)(dslot % hpr);
  for (; it - lane < total; it += stride, row += drow, hs += dhs) {
    if (hs >= hpr) { hs -= hpr; ++row; }
    const bool live = it < total;
    const int hh = hs % (g + 2);
    const size_t off = (row * hpr + hs) * (size_t)d + vec * 8;
    float f[8];
    if (live) load8(qkv + off, f);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    for (int o = tph / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!live) continue;
    if (hh <= g) {
      const float r = __frsqrt_rn(__fdiv_rn(ss, (float)d) + eps);
      float w[8];
      load8((hh < g ? wq : wk) + vec * 8, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * r * w[i];
      if (vec == 0) rstd_out[(row * n_kv + hs / (g + 2)) * (size_t)(g + 1) + hh] = r;
    }
    store8(out + off, f);
  }
}

// Backward, in place on dqkv: dx = rstd * (g*w - xhat * mean(g*w*xhat)) for q and k heads; v heads untouched.  Weight gradients:
// every thread keeps its 8 columns' sums for q heads and for the k head in registers over all rows it visits (its column
// position never changes: the grid stride is a multiple of the lane-group size), the block combines them in a fixed order
// in shared memory and writes one partial row per block; colsum_add_kernel adds the partial rows into main_grad.
__global__ void qk_norm_bwd_kernel(__nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ qkv_pre,
                                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ wq,
                                   const __nv_bfloat16* __restrict__ wk, float* __restrict__ partial_q,
                                   float* __restrict__ partial_k, int M, int n_kv, int g, int d) {
  __shared__ float red[256][17];
  const int tph = d / 8, hpr = n_kv * (g + 2);
  const size_t total = (size_t)M * hpr * tph, stride = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int vec = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) % tph);
  float wqv[8], wkv[8], accq[8], acck[8];
  load8(wq + vec * 8, wqv);
  load8(wk + vec * 8, wkv);
#pragma unroll
  for (int i = 0; i < 8; ++i) accq[i] = acck[i] = 0.f;
  size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  size_t row = (it / tph) / hpr;
  int hs = (int)((it / tph) % hpr);
  const size_t dslot = stride / tph, drow = dslot / hpr;
  const int dhs = (int)(dslot % hpr);
  for (; it - lane < total; it += stride, row += drow, hs += dhs) {
    if (hs >= hpr) { hs -= hpr; ++row; }
    const bool live = it < total;
    const int hh = hs % (g + 2);
    const bool normed = live && hh <= g;
    const size_t off = (row * hpr + hs) * (size_t)d + vec * 8;
    float gq[8], x[8];
    float r = 0.f, dot = 0.f;
    if (normed) {
      load8(dqkv + off, gq);
      load8(qkv_pre + off, x);
      r = rstd[(row * n_kv + hs / (g + 2)) * (size_t)(g + 1) + hh];
      const bool is_q = hh < g;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] *= r;                       // xhat
        const float dwc = gq[i] * x[i];  // weight-gradient contribution
        accq[i] += is_q ? dwc : 0.f;
        acck[i] += is_q ? 0.f : dwc;
        gq[i] *= is_q ? wqv[i] : wkv[i];  // g * w
        dot += gq[i] * x[i];
      }
    }
    for (int o = tph / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (normed) {
      const float mean = __fdiv_rn(dot, (float)d);
#pragma unroll
      for (int i = 0; i < 8; ++i) gq[i] = r * (gq[i] - x[i] * mean);
      store8(dqkv + off, gq);
    }
  }
  // block combine: thread t holds columns vec(t)*8 .. +8; threads t, t + tph, t + 2 tph, ... share a column group
#pragma unroll
  for (int i = 0; i < 8; ++i) { red[threadIdx.x][i] = accq[i]; red[threadIdx.x][8 + i] = acck[i]; }
  __syncthreads();
  if ((int)threadIdx.x < 2 * d) {
    const int which = threadIdx.x / d, col = threadIdx.x % d;   // 0: q columns, 1: k columns
    const int v0 = col / 8, e = col % 8;
    float a = 0.f;
    for (int t = v0; t < (int)blockDim.x; t += tph) a += red[t][which * 8 + e];
    (which ? partial_k : partial_q)[(size_t)blockIdx.x * d + col] = a;
  }
}

// In-place rotate-half RoPE on the q and k heads of the packed kv-group-major QKV activation.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ table, int M, int S,
                            int n_kv, int g, int d, float sign) {
  // A thread owns one 16-byte vector position of the row (head slot, vector) and walks down the rows, so the index
  // arithmetic (divisions by g + 1 and d / 16) happens once per thread, not once per element.
  const int half = d / 2, vph = half / 8;  // vectors per half head
  const int ipr = n_kv * (g + 1) * vph;    // vector pairs per row
  const int row_stride = n_kv * (g + 2) * d;
  const int tpr = ipr < (int)blockDim.x ? ipr : (int)blockDim.x;
  const int rpb = blockDim.x / tpr;
  const int my_row = threadIdx.x / tpr;
  if (my_row >= rpb) return;
  for (int rem = threadIdx.x % tpr; rem < ipr; rem += tpr) {
    const int vec = rem % vph, sl = rem / vph;
    const int j = sl / (g + 1), hh = sl % (g + 1);
    const int col = (j * (g + 2) + hh) * d + vec * 8;
    for (int row = blockIdx.x * rpb + my_row; row < M; row += gridDim.x * rpb) {
      __nv_bfloat16* p = qkv + (size_t)row * row_stride + col;
      const float* tb = table + (size_t)(row % S) * d + vec * 8;
      float x1[8], x2[8], c[8], sn[8], o1[8], o2[8];
      load8(p, x1);
      load8(p + half, x2);
      load8(tb, c);
      load8(tb + half, sn);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float si = sn[i] * sign;
        o1[i] = x1[i] * c[i] - x2[i] * si;
        o2[i] = x2[i] * c[i] + x1[i] * si;
      }
      store8(p, o1);
      store8(p + half, o2);
    }
  }
}

__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int M, int F) {
  const int vpr = F / 8;
  const size_t total = (size_t)M * vpr;
  for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
    int row = it / vpr, c = (it % vpr) * 8;
    float a[8], b[8], o[8];
    load8(gu + (size_t)row * 2 * F + c, a);
    load8(gu + (size_t)row * 2 * F + F + c, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = a[i] / (1.f + __expf(-a[i])) * b[i];
    store8(out + (size_t)row * F + c, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dinter, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, int M, int F) {
  const int vpr = F / 8;
  const size_t total = (size_t)M * vpr;
  for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
    int row = it / vpr, c = (it % vpr) * 8;
    float a[8], b[8], d[8], dg[8], du[8];
    load8(gu + (size_t)row * 2 * F + c, a);
    load8(gu + (size_t)row * 2 * F + F + c, b);
    load8(dinter + (size_t)row * F + c, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float sig = 1.f / (1.f + __expf(-a[i]));
      dg[i] = d[i] * b[i] * sig * (1.f + a[i] * (1.f - sig));
      du[i] = d[i] * a[i] * sig;
    }
    store8(dgu + (size_t)row * 2 * F + c, dg);
    store8(dgu + (size_t)row * 2 * F + F + c, du);
  }
}

__global__ void residual_add_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ a,
                                    float scale, __nv_bfloat16* __restrict__ out, size_t n8) {
  for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < n8; it += (size_t)gridDim.x * blockDim.x) {
    float x[8], y[8];
    load8(h + it * 8, x);
    load8(a + it * 8, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] += y[i] * scale;
    store8(out + it * 8, x);
  }
}

// out[row] = weight[ids[row] - vocab_start] * scale (zero outside the local vocabulary shard)
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, int M, int H, int vocab_start, int vocab_local,
                                     float scale) {
  const int vpr = H / 8;
  const size_t total = (size_t)M * vpr;
  for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
    int row = it / vpr, c = (it % vpr) * 8;
    int id = ids[row] - vocab_start;
    float f[8];
    if (id >= 0 && id < vocab_local) {
      load8(w + (size_t)id * H + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] *= scale;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    store8(out + (size_t)row * H + c, f);
  }
}

// Debug input check: the embedding and cross-entropy kernels treat an id outside the local vocabulary range as "another
// rank's token" and skip it, which is right under vocabulary parallelism and hides a corrupt batch without it.  This kernel
// looks at the GLOBAL range: an id outside [lo, hi) sets status kBadIndex and records the first offending position
// (atomicMin) in where[0]; it touches nothing else.
__global__ void check_ids_kernel(const int* __restrict__ ids, size_t n, int lo, int hi, int* status, int* where) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    int v = ids[i];
    if (v < lo || v >= hi) {
      report_status(status, kBadIndex);
      if (where != nullptr) atomicMin(where, (int)(i < 0x7fffffff ? i : 0x7fffffff));
    }
  }
}

__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ ids,
                                     float* __restrict__ main_grad, int M, int H, int vocab_start, int vocab_local,
                                     float scale) {
  const int vpr = H / 8;
  const size_t total = (size_t)M * vpr;
  for (size_t it = blockIdx.x * (size_t)blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
    int row = it / vpr, c = (it % vpr) * 8;
    int id = ids[row] - vocab_start;
    if (id < 0 || id >= vocab_local) continue;
    float f[8];
    load8(dout + (size_t)row * H + c, f);
    float4* dst = reinterpret_cast<float4*>(main_grad + (size_t)id * H + c);
    atomicAdd(dst, make_float4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale));
    atomicAdd(dst + 1, make_float4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale));
  }
}

// Deterministic form: the rows are visited token by token in a fixed order.  `order` lists the row indices sorted by
// token id (stable, so equal ids keep their row order), `seg_start[s] .. seg_start[s+1]` is the run of rows of one token
// and `seg_id[s]` that token (already relative to the shard and inside it).  One block per run sums its rows in that
// order in fp32 and adds the total to main_grad once: no atomics, the result does not depend on the schedule.
__global__ void embedding_bwd_det_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ order,
                                         const int* __restrict__ seg_start, const int* __restrict__ seg_id,
                                         float* __restrict__ main_grad, int n_seg, int H, float scale) {
  const int vpr = H / 8;
  for (int s = blockIdx.x; s < n_seg; s += gridDim.x) {
    const int r0 = seg_start[s], r1 = seg_start[s + 1];
    float* dst = main_grad + (size_t)seg_id[s] * H;
    for (int v = threadIdx.x; v < vpr; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = r0; j < r1; ++j) {
        float f[8];
        load8(dout + (size_t)order[j] * H + v * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
      float cur[8];
      load8(dst + v * 8, cur);
#pragma unroll
      for (int e = 0; e < 8; ++e) cur[e] += acc[e] * scale;
      store8(dst + v * 8, cur);
    }
  }
}

// ---- fused cross-entropy ------------------------------------------------------------------------
constexpr int kCeThreads = 1024;

__device__ __forceinline__ void block_max_sum(float& mx, float& sm, float* red) {
  // combine per-thread (max, sum-of-exp relative to max) pairs over the block
  float m2 = warp_max(mx);
  sm = (mx == -INFINITY) ? 0.f : sm * __expf(mx - m2);
  sm = warp_sum(sm);
  int w = threadIdx.x / 32, l = threadIdx.x % 32;
  if (l == 0) { red[w] = m2; red[32 + w] = sm; }
  __syncthreads();
  int nw = blockDim.x / 32;
  float a = l < nw ? red[l] : -INFINITY, b = l < nw ? red[32 + l] : 0.f;
  float m3 = warp_max(a);
  b *= (a == -INFINITY) ? 0.f : __expf(a - m3);
  b = warp_sum(b);
  mx = m3;
  sm = b;
  __syncthreads();
}

// mode 0: fused single-shard: nll + in-place gradient.  mode 1: statistics only (max, sumexp, target logit).
// mode 2: gradient only from a given lse.  Rows live in shared memory when they fit (kSmemRow).
template <bool kSmemRow>
__global__ void __launch_bounds__(kCeThreads) cross_entropy_kernel(
    __nv_bfloat16* __restrict__ logits, const int* __restrict__ labels, const float* __restrict__ mask,
    float* __restrict__ nll, float* __restrict__ st_max, float* __restrict__ st_sum, float* __restrict__ st_tgt,
    const float* __restrict__ lse_in, int M, int V, long long ld, int vocab_start, float grad_scale, int mode) {
  // rows are `ld` elements apart (ld % 8 == 0); a row's last 16-byte vector may reach past V: those elements count as
  // -inf in the statistics and get a zero gradient
  extern __shared__ __align__(16) unsigned char ce_smem[];
  __shared__ float red[64];
  bf16x8* rowbuf = reinterpret_cast<bf16x8*>(ce_smem);
  const int nvec = (V + 7) / 8;
  const int tail = V & 7;   // valid elements of the last vector, 0 = all eight
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    bf16x8* grow = reinterpret_cast<bf16x8*>(logits + (size_t)row * ld);
    const int lab = labels[row] - vocab_start;
    const bool has = lab >= 0 && lab < V;
    float lse;
    if (mode != 2) {
      float mx = -INFINITY, sm = 0.f;
      // four independent 16-byte loads in flight per thread
      for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * blockDim.x) {
        bf16x8 p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * blockDim.x;
          if (v < nvec) p[u] = grow[v];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * blockDim.x;
          if (v < nvec) {
            if (kSmemRow) rowbuf[v] = p[u];
            float f[8];
            unpack8(p[u], f);
            if (tail && v == nvec - 1) {
#pragma unroll
              for (int i = 1; i < 8; ++i)
                if (i >= tail) f[i] = -INFINITY;
            }
            float m8 = f[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) m8 = fmaxf(m8, f[i]);
            if (m8 > mx) { sm *= __expf(mx - m8); mx = m8; }
#pragma unroll
            for (int i = 0; i < 8; ++i) sm += __expf(f[i] - mx);
          }
        }
      }
      block_max_sum(mx, sm, red);
      float tgt = has ? __bfloat162float(logits[(size_t)row * ld + lab]) : 0.f;
      if (mode == 1) {
        if (threadIdx.x == 0) { st_max[row] = mx; st_sum[row] = sm; st_tgt[row] = tgt; }
        continue;
      }
      lse = mx + __logf(sm);
      if (threadIdx.x == 0) nll[row] = (lse - tgt) * mask[row];
    } else {
      lse = lse_in[row];
    }
    const float gs = mask[row] * grad_scale;
    __syncthreads();
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      bf16x8 p = (kSmemRow && mode != 2) ? rowbuf[v] : grow[v];
      float f[8];
      unpack8(p, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float g = __expf(f[i] - lse);
        if (has && v * 8 + i == lab) g -= 1.f;
        f[i] = (tail && v * 8 + i >= V) ? 0.f : g * gs;
      }
      grow[v] = pack8(f);
    }
    __syncthreads();
  }
}

// ---- AdamW over a table of segments ---------------------------------------------------------------
struct AdamSeg {
  long long shard_off;  // into master / m / v
  long long flat_off;   // into the flat gradient / parameter buffers
  int n;
  float lr_mult;
  float wd;  // 0 or 1: whether weight decay applies
  int pad;
};

template <typename PT>
__global__ void adamw_segments_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                      const float* __restrict__ grad, PT* __restrict__ param,
                                      const AdamSeg* __restrict__ segs, float lr, float beta1, float beta2, float eps,
                                      float weight_decay, float bc1, float rsqrt_bc2, const float* __restrict__ grad_scale) {
  const AdamSeg sg = segs[blockIdx.x];
  const float gs = *grad_scale;
  const float l = lr * sg.lr_mult;
  const float decay = 1.f - l * weight_decay * sg.wd;
  const float step = __fdiv_rn(l, bc1);
  float* w = master + sg.shard_off;
  float* mm = m + sg.shard_off;
  float* vv = v + sg.shard_off;
  const float* g = grad + sg.flat_off;
  PT* p = param + sg.flat_off;
  const int n4 = sg.n / 4;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    float4 w4 = reinterpret_cast<float4*>(w)[i], m4 = reinterpret_cast<float4*>(mm)[i], v4 = reinterpret_cast<float4*>(vv)[i];
    float4 g4 = reinterpret_cast<const float4*>(g)[i];
    float ww[4] = {w4.x, w4.y, w4.z, w4.w}, ma[4] = {m4.x, m4.y, m4.z, m4.w}, va[4] = {v4.x, v4.y, v4.z, v4.w};
    float ga[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      ww[k] *= decay;
      ma[k] += (ga[k] - ma[k]) * (1.f - beta1);
      va[k] = va[k] * beta2 + ga[k] * ga[k] * (1.f - beta2);
      ww[k] -= __fdiv_rn(step * ma[k], __fsqrt_rn(va[k]) * rsqrt_bc2 + eps);  // IEEE sqrt / divide whatever the build's fast-math flag says
    }
    reinterpret_cast<float4*>(w)[i] = make_float4(ww[0], ww[1], ww[2], ww[3]);
    reinterpret_cast<float4*>(mm)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(vv)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if constexpr (sizeof(PT) == 2) {
      reinterpret_cast<__nv_bfloat162*>(p)[2 * i] = __floats2bfloat162_rn(ww[0], ww[1]);
      reinterpret_cast<__nv_bfloat162*>(p)[2 * i + 1] = __floats2bfloat162_rn(ww[2], ww[3]);
    } else {
      reinterpret_cast<float4*>(p)[i] = make_float4(ww[0], ww[1], ww[2], ww[3]);
    }
  }
  for (int i = n4 * 4 + threadIdx.x; i < sg.n; i += blockDim.x) {
    float gg = g[i] * gs, ww = w[i] * decay;
    float ma = mm[i] + (gg - mm[i]) * (1.f - beta1);
    float va = vv[i] * beta2 + gg * gg * (1.f - beta2);
    ww -= __fdiv_rn(step * ma, __fsqrt_rn(va) * rsqrt_bc2 + eps);
    w[i] = ww; mm[i] = ma; vv[i] = va;
    if constexpr (sizeof(PT) == 2) p[i] = __float2bfloat16(ww); else p[i] = ww;
  }
}

__global__ void sumsq_partial_kernel(const float* __restrict__ x, size_t n, double* __restrict__ partial) {
  __shared__ float red[32];
  float acc = 0.f;
  const size_t n4 = n / 4;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    float4 a = reinterpret_cast<const float4*>(x)[i];
    acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  for (size_t i = n4 * 4 + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    acc += x[i] * x[i];
  acc = warp_sum(acc);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < blockDim.x / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partial[blockIdx.x] = (double)t;
  }
}

__global__ void sumsq_final_kernel(const double* __restrict__ partial, int nb, float* __restrict__ out) {
  __shared__ double red[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) acc += partial[i];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < (int)blockDim.x / 32; ++i) t += red[i];
    *out = (float)t;
  }
}

// ---- host launchers (plain C ABI; the torch binding layer passes raw pointers and the stream) ----------
static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

// Wide layout for the bandwidth-bound training shapes: as many threads per row as there are 16-byte vectors (up to 256),
// so a thread holds one vector per array, registers stay low and every SM keeps its full 2048 threads of loads in flight.
static int row_cfg_wide(int H, int& tpr, int& vpt) {
  int vecs = H / 8;
  tpr = 32;
  while (tpr < 256 && vecs > tpr) tpr *= 2;
  vpt = (vecs + tpr - 1) / tpr;
  return (H % 8 == 0 && vpt <= 4) ? 0 : -1;
}

#define FTH_ROW_DISPATCH_WIDE(KERNEL, ...)                                                 \
  do {                                                                                     \
    switch (tpr * 8 + vpt) {                                                               \
      case 32 * 8 + 1: KERNEL<32, 1><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break;   \
      case 64 * 8 + 1: KERNEL<64, 1><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break;   \
      case 128 * 8 + 1: KERNEL<128, 1><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break; \
      case 256 * 8 + 1: KERNEL<256, 1><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break; \
      case 256 * 8 + 2: KERNEL<256, 2><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break; \
      case 256 * 8 + 3: KERNEL<256, 3><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break; \
      case 256 * 8 + 4: KERNEL<256, 4><<<grid, kRowThreads, 0, stream>>>(__VA_ARGS__); break; \
      default: return -1;                                                                  \
    }                                                                                      \
  } while (0)

}  // namespace fth

using namespace fth;

extern "C" {

int fth_rmsnorm_fwd(const void* x, const void* res, float res_scale, const void* w, void* r_out, void* y,
                    float* rstd, int M, int H, float eps, float out_scale, cudaStream_t stream) {
  int tpr, vpt;
  if (row_cfg_wide(H, tpr, vpt)) return -1;
  int rpb = kRowThreads / tpr;
  int grid = min((M + rpb - 1) / rpb, num_sms() * 8);
  FTH_ROW_DISPATCH_WIDE(rmsnorm_fwd_kernel, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, res_scale,
                   (const __nv_bfloat16*)w, (__nv_bfloat16*)r_out, (__nv_bfloat16*)y, rstd, M, H, eps, out_scale);
  return 0;
}

// Number of partial rows (= blocks) the backward kernel writes for M rows of width H.
int fth_rmsnorm_bwd_blocks(int M, int H) {
  int tpr, vpt;
  if (row_cfg_wide(H, tpr, vpt)) return -1;
  int rpb = kRowThreads / tpr;
  return min((M + rpb - 1) / rpb, num_sms() * 8);
}

int fth_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                    float* dw_partial, float* dw_main_grad, int M, int H, float out_scale, cudaStream_t stream) {
  int tpr, vpt;
  if (row_cfg_wide(H, tpr, vpt)) return -1;
  int grid = fth_rmsnorm_bwd_blocks(M, H);
  FTH_ROW_DISPATCH_WIDE(rmsnorm_bwd_kernel, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,
                   (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw_partial, M, H, out_scale);
  colsum_add_kernel<<<(H + 31) / 32, dim3(32, 32), 0, stream>>>(dw_partial, dw_main_grad, grid, H);
  return 0;
}

int fth_qk_norm_blocks(int M, int n_kv, int g, int d) {
  if (d != 64 && d != 128) return -1;
  size_t total = (size_t)M * n_kv * (g + 2) * (d / 8);
  return (int)min((total + 255) / 256, (size_t)num_sms() * 8);
}

int fth_qk_norm_fwd(const void* qkv, const void* wq, const void* wk, void* out, float* rstd, int M, int n_kv, int g, int d,
                    float eps, cudaStream_t stream) {
  const int grid = fth_qk_norm_blocks(M, n_kv, g, d);
  if (grid < 0) return -1;
  if (grid == 0) return 0;
  qk_norm_fwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk,
                                               (__nv_bfloat16*)out, rstd, M, n_kv, g, d, eps);
  return 0;
}

// partial: fth_qk_norm_blocks(...) x 2 x d floats of scratch (q rows first, then k rows)
int fth_qk_norm_bwd(void* dqkv, const void* qkv_pre, const float* rstd, const void* wq, const void* wk, float* partial,
                    float* dwq_main, float* dwk_main, int M, int n_kv, int g, int d, cudaStream_t stream) {
  const int grid = fth_qk_norm_blocks(M, n_kv, g, d);
  if (grid < 0) return -1;
  if (grid == 0) return 0;
  float* pq = partial;
  float* pk = partial + (size_t)grid * d;
  qk_norm_bwd_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)dqkv, (const __nv_bfloat16*)qkv_pre, rstd,
                                               (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, pq, pk, M, n_kv, g, d);
  colsum_add_kernel<<<(d + 31) / 32, dim3(32, 32), 0, stream>>>(pq, dwq_main, grid, d);
  colsum_add_kernel<<<(d + 31) / 32, dim3(32, 32), 0, stream>>>(pk, dwk_main, grid, d);
  return 0;
}

int fth_rope(void* qkv, const float* table, int M, int S, int n_kv, int g, int d, float sign, cudaStream_t stream) {
  if (d % 16) return -1;
  const int ipr = n_kv * (g + 1) * (d / 16);
  const int rpb = 256 / (ipr < 256 ? ipr : 256);
  int grid = min((M + rpb - 1) / rpb, num_sms() * 8);
  rope_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)qkv, table, M, S, n_kv, g, d, sign);
  return 0;
}

int fth_swiglu_fwd(const void* gu, void* out, int M, int F, cudaStream_t stream) {
  if (F % 8) return -1;
  size_t total = (size_t)M * (F / 8);
  int grid = (int)min((total + 255) / 256, (size_t)num_sms() * 16);
  swiglu_fwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, M, F);
  return 0;
}

int fth_swiglu_bwd(const void* dinter, const void* gu, void* dgu, int M, int F, cudaStream_t stream) {
  if (F % 8) return -1;
  size_t total = (size_t)M * (F / 8);
  int grid = (int)min((total + 255) / 256, (size_t)num_sms() * 16);
  swiglu_bwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dinter, (const __nv_bfloat16*)gu,
                                              (__nv_bfloat16*)dgu, M, F);
  return 0;
}

int fth_residual_add(const void* h, const void* a, float scale, void* out, size_t n, cudaStream_t stream) {
  if (n % 8) return -1;
  size_t n8 = n / 8;
  int grid = (int)min((n8 + 255) / 256, (size_t)num_sms() * 16);
  residual_add_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)a, scale,
                                                (__nv_bfloat16*)out, n8);
  return 0;
}

int fth_embedding_fwd(const int* ids, const void* w, void* out, int M, int H, int vocab_start, int vocab_local,
                      float scale, cudaStream_t stream) {
  if (H % 8) return -1;
  size_t total = (size_t)M * (H / 8);
  int grid = (int)min((total + 255) / 256, (size_t)num_sms() * 16);
  embedding_fwd_kernel<<<grid, 256, 0, stream>>>(ids, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, H, vocab_start,
                                                 vocab_local, scale);
  return 0;
}

int fth_check_ids(const int* ids, size_t n, int lo, int hi, int* status, int* where, cudaStream_t stream) {
  if (n == 0) return 0;
  int grid = (int)min((n + 255) / 256, (size_t)num_sms() * 4);
  check_ids_kernel<<<grid, 256, 0, stream>>>(ids, n, lo, hi, status, where);
  return 0;
}

int fth_embedding_bwd(const void* dout, const int* ids, float* main_grad, int M, int H, int vocab_start,
                      int vocab_local, float scale, cudaStream_t stream) {
  if (H % 8) return -1;
  size_t total = (size_t)M * (H / 8);
  int grid = (int)min((total + 255) / 256, (size_t)num_sms() * 16);
  embedding_bwd_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dout, ids, main_grad, M, H, vocab_start,
                                                 vocab_local, scale);
  return 0;
}

int fth_embedding_bwd_det(const void* dout, const int* order, const int* seg_start, const int* seg_id, float* main_grad,
                          int n_seg, int H, float scale, cudaStream_t stream) {
  if (H % 8) return -1;
  if (n_seg <= 0) return 0;
  const int threads = H / 8 < 128 ? 64 : 128;
  const int grid = n_seg < num_sms() * 16 ? n_seg : num_sms() * 16;
  embedding_bwd_det_kernel<<<grid, threads, 0, stream>>>((const __nv_bfloat16*)dout, order, seg_start, seg_id, main_grad,
                                                        n_seg, H, scale);
  return 0;
}

int fth_cross_entropy(void* logits, const int* labels, const float* mask, float* nll, float* st_max, float* st_sum,
                      float* st_tgt, const float* lse_in, int M, int V, long long ld, int vocab_start, float grad_scale,
                      int mode, cudaStream_t stream) {
  if (ld % 8 || ld < V) return -1;
  size_t row_bytes = (size_t)((V + 7) / 8) * 16;
  static int max_smem = 0;
  if (max_smem == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  }
  bool fits = mode != 2 && row_bytes + 1024 <= (size_t)max_smem;
  if (fits) {
    cudaFuncSetAttribute(cross_entropy_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes);
    int per_sm = max(1, (int)(((size_t)max_smem) / (row_bytes + 1024)));
    int grid = min(M, num_sms() * min(per_sm, 4));
    cross_entropy_kernel<true><<<grid, kCeThreads, row_bytes, stream>>>(
        (__nv_bfloat16*)logits, labels, mask, nll, st_max, st_sum, st_tgt, lse_in, M, V, ld, vocab_start, grad_scale, mode);
  } else {
    int grid = min(M, num_sms() * 4);
    cross_entropy_kernel<false><<<grid, kCeThreads, 0, stream>>>(
        (__nv_bfloat16*)logits, labels, mask, nll, st_max, st_sum, st_tgt, lse_in, M, V, ld, vocab_start, grad_scale, mode);
  }
  return 0;
}

int fth_adamw_segments(float* master, float* m, float* v, const float* grad, void* param, int param_is_bf16,
                       const void* seg_table, int n_segs, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float bc1, float rsqrt_bc2, const float* grad_scale, cudaStream_t stream) {
  if (n_segs <= 0) return 0;
  if (param_is_bf16)
    adamw_segments_kernel<__nv_bfloat16><<<n_segs, 512, 0, stream>>>(master, m, v, grad, (__nv_bfloat16*)param,
                                                                    (const AdamSeg*)seg_table, lr, beta1, beta2, eps,
                                                                    weight_decay, bc1, rsqrt_bc2, grad_scale);
  else
    adamw_segments_kernel<float><<<n_segs, 512, 0, stream>>>(master, m, v, grad, (float*)param, (const AdamSeg*)seg_table,
                                                            lr, beta1, beta2, eps, weight_decay, bc1, rsqrt_bc2, grad_scale);
  return 0;
}

int fth_sumsq_blocks() { return num_sms() * 4; }

int fth_sumsq(const float* x, size_t n, double* partial, float* out, cudaStream_t stream) {
  int nb = fth_sumsq_blocks();
  sumsq_partial_kernel<<<nb, 512, 0, stream>>>(x, n, partial);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial, nb, out);
  return 0;
}

}  // extern "C"

// =====================================================================================================================
// RMSNorm backward without any allocation (declared in noalloc.h).
//
// Same kernels as fth_rmsnorm_bwd above, but the per-block partial sums of the weight gradient live in a file-scope
// device array instead of a caller-provided buffer, so a caller that cannot allocate device memory can still run it.
// =====================================================================================================================
namespace fth {
constexpr int kNoAllocMaxH = 4096;       // widest row supported by this entry point
constexpr int kNoAllocMaxBlocks = 296;   // partial rows (= thread blocks) it will launch at most
constexpr int kNoAllocMaxDevices = 64;
// 296 x 4096 fp32 = 4.625 MiB, resident on every GPU that loads this library until the process exits.
static __device__ __align__(256) float g_rmsnorm_bwd_partials[kNoAllocMaxBlocks * kNoAllocMaxH];
// Device address of the array above, per device.  The array's NAME is only a host-side handle in host code; the
// address a kernel can use comes from cudaGetSymbolAddress, queried once per device with that device current.
static float* g_rmsnorm_bwd_partials_addr[kNoAllocMaxDevices] = {nullptr};

static int noalloc_fail(char* err, size_t err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) {
    size_t i = 0;
    for (; msg[i] != '\0' && i + 1 < err_len; ++i) err[i] = msg[i];
    err[i] = '\0';
  }
  return code;
}
}  // namespace fth

extern "C" int fth_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                       void* dx, float* dw_main_grad, int M, int H, float out_scale, cudaStream_t stream,
                                       char* err, size_t err_len) {
  using namespace fth;
  if (M <= 0 || H <= 0) return noalloc_fail(err, err_len, -1, "fth_rmsnorm_bwd_noalloc: M and H must be positive");
  if (H > kNoAllocMaxH)
    return noalloc_fail(err, err_len, -2, "fth_rmsnorm_bwd_noalloc: H exceeds the built-in scratch (max 4096 columns); use fth_rmsnorm_bwd with your own buffer");
  int tpr, vpt;
  if (row_cfg_wide(H, tpr, vpt)) return noalloc_fail(err, err_len, -3, "fth_rmsnorm_bwd_noalloc: H must be a multiple of 8");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices)
    return noalloc_fail(err, err_len, -4, "fth_rmsnorm_bwd_noalloc: no current CUDA device (or device ordinal >= 64)");
  if (g_rmsnorm_bwd_partials_addr[dev] == nullptr) {
    // one-time set-up for this device (this is why the first call should not happen inside a stream capture)
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_rmsnorm_bwd_partials) != cudaSuccess || p == nullptr)
      return noalloc_fail(err, err_len, -5, "fth_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed for the scratch array");
    g_rmsnorm_bwd_partials_addr[dev] = p;
  }
  float* partial = g_rmsnorm_bwd_partials_addr[dev];
  const int rpb = kRowThreads / tpr;
  int grid = (M + rpb - 1) / rpb;
  if (grid > kNoAllocMaxBlocks) grid = kNoAllocMaxBlocks;
  // Every launched block writes its whole partial row (zeros if it had no rows), and the column sum reads exactly
  // `grid` rows, so nothing left in the array by an earlier call is ever read: no clearing is needed.
  FTH_ROW_DISPATCH_WIDE(rmsnorm_bwd_kernel, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,
                   (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, partial, M, H, out_scale);
  colsum_add_kernel<<<(H + 31) / 32, dim3(32, 32), 0, stream>>>(partial, dw_main_grad, grid, H);
  if (cudaGetLastError() != cudaSuccess) return noalloc_fail(err, err_len, -6, "fth_rmsnorm_bwd_noalloc: kernel launch failed");
  return 0;
}
