// C ABI of the sm_100a kernel library (every launcher takes raw device pointers and a stream, returns 0 on
// success or a negative code for an unsupported shape / failed launch).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int fth_rmsnorm_fwd(const void* x, const void* res, float res_scale, const void* w, void* r_out, void* y, float* rstd,
                    int M, int H, float eps, float out_scale, cudaStream_t stream);
int fth_rmsnorm_bwd_blocks(int M, int H);
int fth_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                    float* dw_partial, float* dw_main_grad, int M, int H, float out_scale, cudaStream_t stream);
// per-head q/k RMSNorm on the packed QKV layout (d = 64 or 128).  fwd writes a new tensor (v heads copied) + rstd [M, n_kv, g+1];
// bwd is in place on dqkv and accumulates the two weight gradients; `partial` = fth_qk_norm_blocks() x 2 x d floats.
int fth_qk_norm_blocks(int M, int n_kv, int g, int d);
int fth_qk_norm_fwd(const void* qkv, const void* wq, const void* wk, void* out, float* rstd, int M, int n_kv, int g, int d,
                    float eps, cudaStream_t stream);
int fth_qk_norm_bwd(void* dqkv, const void* qkv_pre, const float* rstd, const void* wq, const void* wk, float* partial,
                    float* dwq_main, float* dwk_main, int M, int n_kv, int g, int d, cudaStream_t stream);
int fth_rope(void* qkv, const float* table, int M, int S, int n_kv, int g, int d, float sign, cudaStream_t stream);
int fth_swiglu_fwd(const void* gu, void* out, int M, int F, cudaStream_t stream);
int fth_swiglu_bwd(const void* dinter, const void* gu, void* dgu, int M, int F, cudaStream_t stream);
int fth_residual_add(const void* h, const void* a, float scale, void* out, size_t n, cudaStream_t stream);
// debug input check: ids outside [lo, hi) set status 7 and record the first bad position in where[0] (atomicMin)
int fth_check_ids(const int* ids, size_t n, int lo, int hi, int* status, int* where, cudaStream_t stream);
int fth_embedding_fwd(const int* ids, const void* w, void* out, int M, int H, int vocab_start, int vocab_local, float scale,
                      cudaStream_t stream);
int fth_embedding_bwd(const void* dout, const int* ids, float* main_grad, int M, int H, int vocab_start, int vocab_local,
                      float scale, cudaStream_t stream);
int fth_embedding_bwd_det(const void* dout, const int* order, const int* seg_start, const int* seg_id, float* main_grad,
                          int n_seg, int H, float scale, cudaStream_t stream);
int fth_cross_entropy(void* logits, const int* labels, const float* mask, float* nll, float* st_max, float* st_sum,
                      float* st_tgt, const float* lse_in, int M, int V, long long ld, int vocab_start, float grad_scale,
                      int mode, cudaStream_t stream);
int fth_adamw_segments(float* master, float* m, float* v, const float* grad, void* param, int param_is_bf16,
                       const void* seg_table, int n_segs, float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bc1, float rsqrt_bc2, const float* grad_scale, cudaStream_t stream);
int fth_sumsq_blocks(void);
int fth_sumsq(const float* x, size_t n, double* partial, float* out, cudaStream_t stream);
int fth_gemm_bf16(const void* a, long long lda, int a_mn_major, const void* b, long long ldb, int b_mn_major, void* c,
                  long long ldc, int M, int N, int K, float alpha, int epi, int bn, int max_ctas, int* status,
                  cudaStream_t stream);

// Deterministic mode: one k split per output tile, so the fp32 reduce-adds of an accumulating epilogue have a fixed order.
void fth_gemm_set_deterministic(int on);
void fth_tmap_cache_stats(unsigned long long* hits, unsigned long long* misses);

int fth_flash_fwd(const void* qkv, void* out, float* lse, int B, int S, int n_kv, int g, int d, int* status,
                  cudaStream_t stream);

void fth_flash_fwd_set_debug(long long* buf);
void fth_flash_bwd_set_debug(long long* buf);
size_t fth_flash_bwd_scratch_bytes(int B, int S, int n_kv, int g, int d);
int fth_flash_bwd(const void* d_out, const void* qkv, const void* out, const float* lse, void* dqkv, void* scratch_f32,
                  const float* rope_table, int B, int S, int n_kv, int g, int d, int* status, cudaStream_t stream);

int fth_peer_barrier(void* const* pads, int rank, int world, unsigned epoch, int lane_slot, int* status, double limit_s,
                     unsigned* epoch_dev, cudaStream_t stream);
int fth_dp_reduce_scatter_blocks(void);
int fth_dp_reduce_scatter(void* const* grads, const void* mc_grads, long long start, long long count, int world, int rank,
                          double* partial, float* sumsq_accum, cudaStream_t stream);
int fth_adamw_push(float* master, float* m, float* v, const float* grad, void* const* params, void* mc_param, int world,
                   const void* seg_table, int n_segs, float lr, float beta1, float beta2, float eps, float weight_decay,
                   float bc1, float rsqrt_bc2, const float* grad_scale, cudaStream_t stream);

int fth_gemm_rs(const void* a, long long lda, const void* b, long long ldb, int b_mn, void* const* out_shards, long long ldo,
                int M, int N, int K, int tp, int rank, float alpha, int* status, cudaStream_t stream);
int fth_ag_gemm(void* const* gather, long long ldx, const void* b, long long ldb, int b_mn, void* out, long long ldo, int M, int N,
                int K, int tp, int rank, int n_copy_ctas, int* flags, int epoch, int* ctr, void* const* ready, float alpha,
                int* status, cudaStream_t stream);

// MXFP8 (e4m3 payload + e8m0 scale per 32 elements of the contraction dimension); see mxfp8_sm100.cu.
size_t fth_mxfp8_sf_bytes(int rows, int K);
int fth_mxfp8_quant(const void* x, long long ld, void* q, void* sf, int R, int C, int colwise, cudaStream_t stream);
int fth_gemm_mxfp8(const void* a, const void* sfa, const void* b, const void* sfb, void* c, long long ldc, int M, int N, int K,
                   float alpha, int epi, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
