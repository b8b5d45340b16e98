// Torch bindings: tensors in, raw pointers + the current CUDA stream out to the extern "C" launchers.
// Output tensors and scratch buffers come from torch's caching allocator (graph-capture safe).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// Number of kernels of this library launched (or captured into a CUDA graph) by this process.
int64_t g_launches = 0;
int64_t launch_count() { return g_launches; }

void check(int rc, const char* what, int kernels = 1) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc);
  g_launches += kernels;
}

void need_bf16(const at::Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), n, " must be a contiguous CUDA bf16 tensor");
}
// 2-D bf16 whose rows may be padded: unit inner stride, row stride a multiple of 8 elements (16 bytes)
void need_bf16_rows(const at::Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1 && t.stride(0) % 8 == 0 &&
                  t.stride(0) >= t.size(1) && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0,
              n, " must be a CUDA bf16 matrix with unit inner stride and 16-byte aligned rows");
}
void need_f32(const at::Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), n, " must be a contiguous CUDA fp32 tensor");
}
void need_i32(const at::Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), n, " must be a contiguous CUDA int32 tensor");
}

at::Tensor g_status;  // one int per process: first non-zero code a kernel reported

int* status_ptr() {
  if (!g_status.defined()) g_status = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA));
  return g_status.data_ptr<int>();
}

int read_status(bool reset) {
  if (!g_status.defined()) return 0;
  int v = g_status.cpu().item<int>();
  if (reset && v) g_status.zero_();
  return v;
}

// `y_out` (optional): where the normalised rows go, e.g. this rank's rows of an all-gather buffer, instead of a new tensor.
std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& res, double res_scale,
                                    const at::Tensor& w, double eps, double out_scale, const c10::optional<at::Tensor>& y_out) {
  need_bf16(x, "x");
  need_bf16(w, "w");
  const int M = x.size(0), H = x.size(1);
  at::Tensor y;
  if (y_out.has_value()) {
    need_bf16(*y_out, "y_out");
    TORCH_CHECK(y_out->dim() == 2 && y_out->size(0) == M && y_out->size(1) == H, "rmsnorm_fwd: y_out shape");
    y = *y_out;
  } else {
    y = at::empty_like(x);
  }
  at::Tensor rstd = at::empty({M}, x.options().dtype(at::kFloat));
  at::Tensor r;
  const void* resp = nullptr;
  void* rp = nullptr;
  if (res.has_value()) {
    need_bf16(*res, "res");
    r = at::empty_like(x);
    resp = res->data_ptr();
    rp = r.data_ptr();
  }
  check(fth_rmsnorm_fwd(x.data_ptr(), resp, (float)res_scale, w.data_ptr(), rp, y.data_ptr(), rstd.data_ptr<float>(), M, H,
                        (float)eps, (float)out_scale, cur_stream()), "rmsnorm_fwd");
  if (res.has_value()) return {r, y, rstd};
  return {y, rstd};
}

at::Tensor rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd,
                       const c10::optional<at::Tensor>& dres, at::Tensor& dw_main_grad, double out_scale) {
  need_bf16(dy, "dy");
  need_bf16(x, "x");
  need_bf16(w, "w");
  need_f32(rstd, "rstd");
  need_f32(dw_main_grad, "dw_main_grad");
  const int M = x.size(0), H = x.size(1);
  const int nb = fth_rmsnorm_bwd_blocks(M, H);
  TORCH_CHECK(nb > 0, "unsupported hidden size for rmsnorm_bwd");
  at::Tensor dx = at::empty_like(x);
  at::Tensor partial = at::empty({nb, H}, x.options().dtype(at::kFloat));
  const void* dr = nullptr;
  if (dres.has_value()) {
    need_bf16(*dres, "dres");
    dr = dres->data_ptr();
  }
  check(fth_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dr, dx.data_ptr(),
                        partial.data_ptr<float>(), dw_main_grad.data_ptr<float>(), M, H, (float)out_scale, cur_stream()),
        "rmsnorm_bwd", 2);
  return dx;
}

void rope_(at::Tensor& qkv, const at::Tensor& table, int64_t S, int64_t n_kv, int64_t g, int64_t d, double sign) {
  need_bf16(qkv, "qkv");
  need_f32(table, "table");
  TORCH_CHECK(qkv.size(1) == n_kv * (g + 2) * d && table.size(1) == d && table.size(0) >= S, "rope shape mismatch");
  check(fth_rope(qkv.data_ptr(), table.data_ptr<float>(), (int)qkv.size(0), (int)S, (int)n_kv, (int)g, (int)d, (float)sign,
                 cur_stream()), "rope");
}

// Per-head q/k RMSNorm (Qwen3 variant) on the packed QKV activation.  Returns (normalised copy, rstd [M, n_kv, g + 1]).
std::vector<at::Tensor> qk_norm_fwd(const at::Tensor& qkv, const at::Tensor& wq, const at::Tensor& wk, double eps, int64_t n_kv,
                                    int64_t g, int64_t d) {
  need_bf16(qkv, "qkv");
  need_bf16(wq, "q_norm weight");
  need_bf16(wk, "k_norm weight");
  TORCH_CHECK(qkv.dim() == 2 && qkv.is_contiguous() && qkv.size(1) == n_kv * (g + 2) * d && wq.numel() == d && wk.numel() == d,
              "qk_norm_fwd shape mismatch");
  const int M = qkv.size(0);
  at::Tensor out = at::empty_like(qkv);
  at::Tensor rstd = at::empty({M, n_kv, g + 1}, qkv.options().dtype(at::kFloat));
  check(fth_qk_norm_fwd(qkv.data_ptr(), wq.data_ptr(), wk.data_ptr(), out.data_ptr(), rstd.data_ptr<float>(), M, (int)n_kv, (int)g,
                        (int)d, (float)eps, cur_stream()), "qk_norm_fwd");
  return {out, rstd};
}

// In place on dqkv; accumulates into the two fp32 main-grad vectors.
void qk_norm_bwd_(at::Tensor& dqkv, const at::Tensor& qkv_pre, const at::Tensor& rstd, const at::Tensor& wq, const at::Tensor& wk,
                  at::Tensor& dwq_main, at::Tensor& dwk_main, int64_t n_kv, int64_t g, int64_t d) {
  need_bf16(dqkv, "dqkv");
  need_bf16(qkv_pre, "qkv_pre");
  need_f32(rstd, "rstd");
  need_f32(dwq_main, "q_norm main_grad");
  need_f32(dwk_main, "k_norm main_grad");
  const int M = dqkv.size(0);
  TORCH_CHECK(dqkv.is_contiguous() && qkv_pre.is_contiguous() && dqkv.sizes() == qkv_pre.sizes() && dqkv.size(1) == n_kv * (g + 2) * d &&
              rstd.numel() == (int64_t)M * n_kv * (g + 1) && dwq_main.numel() == d && dwk_main.numel() == d, "qk_norm_bwd shape mismatch");
  const int nb = fth_qk_norm_blocks(M, (int)n_kv, (int)g, (int)d);
  TORCH_CHECK(nb >= 0, "qk_norm: head_dim must be 64 or 128");
  at::Tensor partial = at::empty({2 * (int64_t)std::max(nb, 1) * d}, rstd.options());
  check(fth_qk_norm_bwd(dqkv.data_ptr(), qkv_pre.data_ptr(), rstd.data_ptr<float>(), wq.data_ptr(), wk.data_ptr(),
                        partial.data_ptr<float>(), dwq_main.data_ptr<float>(), dwk_main.data_ptr<float>(), M, (int)n_kv, (int)g, (int)d,
                        cur_stream()), "qk_norm_bwd");
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
  need_bf16(gu, "gate_up");
  const int M = gu.size(0), F = gu.size(1) / 2;
  at::Tensor out = at::empty({M, F}, gu.options());
  check(fth_swiglu_fwd(gu.data_ptr(), out.data_ptr(), M, F, cur_stream()), "swiglu_fwd");
  return out;
}

at::Tensor swiglu_bwd(const at::Tensor& dinter, const at::Tensor& gu) {
  need_bf16(gu, "gate_up");
  need_bf16(dinter, "dinter");
  const int M = gu.size(0), F = gu.size(1) / 2;
  at::Tensor out = at::empty_like(gu);
  check(fth_swiglu_bwd(dinter.data_ptr(), gu.data_ptr(), out.data_ptr(), M, F, cur_stream()), "swiglu_bwd");
  return out;
}

at::Tensor residual_add(const at::Tensor& h, const at::Tensor& a, double scale) {
  need_bf16(h, "h");
  need_bf16(a, "a");
  at::Tensor out = at::empty_like(h);
  check(fth_residual_add(h.data_ptr(), a.data_ptr(), (float)scale, out.data_ptr(), (size_t)h.numel(), cur_stream()),
        "residual_add");
  return out;
}

at::Tensor g_bad_pos;  // first position a debug input check found out of range (INT_MAX = none)

// Debug input check (off the hot path unless asked for): every id must lie in [lo, hi).  Nothing is read back here; a bad id
// shows up as status 7 at the step's status check, and bad_index_position() says where.
void check_ids(const at::Tensor& ids, int64_t lo, int64_t hi) {
  need_i32(ids, "ids");
  if (!g_bad_pos.defined()) g_bad_pos = at::full({1}, 0x7fffffff, at::TensorOptions().dtype(at::kInt).device(at::kCUDA));
  check(fth_check_ids(ids.data_ptr<int>(), (size_t)ids.numel(), (int)lo, (int)hi, status_ptr(), g_bad_pos.data_ptr<int>(),
                      cur_stream()), "check_ids");
}

int64_t bad_index_position(bool reset) {
  if (!g_bad_pos.defined()) return -1;
  int v = g_bad_pos.cpu().item<int>();
  if (reset && v != 0x7fffffff) g_bad_pos.fill_(0x7fffffff);
  return v == 0x7fffffff ? -1 : v;
}

at::Tensor embedding_fwd(const at::Tensor& ids, const at::Tensor& w, double scale, int64_t vocab_start) {
  need_i32(ids, "ids");
  need_bf16(w, "weight");
  const int M = ids.numel(), H = w.size(1);
  at::Tensor out = at::empty({M, H}, w.options());
  check(fth_embedding_fwd(ids.data_ptr<int>(), w.data_ptr(), out.data_ptr(), M, H, (int)vocab_start, (int)w.size(0),
                          (float)scale, cur_stream()), "embedding_fwd");
  return out;
}

void embedding_bwd(const at::Tensor& dout, const at::Tensor& ids, at::Tensor& main_grad, double scale, int64_t vocab_start) {
  need_bf16(dout, "dout");
  need_i32(ids, "ids");
  need_f32(main_grad, "main_grad");
  check(fth_embedding_bwd(dout.data_ptr(), ids.data_ptr<int>(), main_grad.data_ptr<float>(), (int)ids.numel(),
                          (int)main_grad.size(1), (int)vocab_start, (int)main_grad.size(0), (float)scale, cur_stream()),
        "embedding_bwd");
}

// Deterministic embedding backward: `order` = row indices sorted (stably) by token id, `seg_start` [n_seg + 1] the runs of
// equal ids in that order, `seg_id` [n_seg] each run's row of main_grad (ids outside this vocabulary shard already removed).
void embedding_bwd_det(const at::Tensor& dout, const at::Tensor& order, const at::Tensor& seg_start, const at::Tensor& seg_id,
                       at::Tensor& main_grad, double scale) {
  need_bf16(dout, "dout");
  need_i32(order, "order");
  need_i32(seg_start, "seg_start");
  need_i32(seg_id, "seg_id");
  need_f32(main_grad, "main_grad");
  TORCH_CHECK(seg_start.numel() == seg_id.numel() + 1, "embedding_bwd_det: seg_start needs n_seg + 1 entries");
  check(fth_embedding_bwd_det(dout.data_ptr(), order.data_ptr<int>(), seg_start.data_ptr<int>(), seg_id.data_ptr<int>(),
                              main_grad.data_ptr<float>(), (int)seg_id.numel(), (int)main_grad.size(1), (float)scale, cur_stream()),
        "embedding_bwd_det");
}

// mode 0: returns nll; logits overwritten with the gradient.
at::Tensor cross_entropy(at::Tensor& logits, const at::Tensor& labels, const at::Tensor& mask, double grad_scale,
                         int64_t vocab_start) {
  need_bf16_rows(logits, "logits");
  need_i32(labels, "labels");
  need_f32(mask, "mask");
  const int M = logits.size(0), V = logits.size(1);
  at::Tensor nll = at::empty({M}, mask.options());
  check(fth_cross_entropy(logits.data_ptr(), labels.data_ptr<int>(), mask.data_ptr<float>(), nll.data_ptr<float>(), nullptr,
                          nullptr, nullptr, nullptr, M, V, logits.stride(0), (int)vocab_start, (float)grad_scale, 0, cur_stream()),
        "cross_entropy");
  return nll;
}

std::vector<at::Tensor> ce_stats(at::Tensor& logits, const at::Tensor& labels, const at::Tensor& mask, int64_t vocab_start) {
  need_bf16_rows(logits, "logits");
  need_i32(labels, "labels");
  need_f32(mask, "mask");
  const int M = logits.size(0), V = logits.size(1);
  at::Tensor mx = at::empty({M}, mask.options()), sm = at::empty({M}, mask.options()), tg = at::empty({M}, mask.options());
  check(fth_cross_entropy(logits.data_ptr(), labels.data_ptr<int>(), mask.data_ptr<float>(), nullptr, mx.data_ptr<float>(),
                          sm.data_ptr<float>(), tg.data_ptr<float>(), nullptr, M, V, logits.stride(0), (int)vocab_start, 1.f, 1, cur_stream()),
        "ce_stats");
  return {mx, sm, tg};
}

void ce_grad(at::Tensor& logits, const at::Tensor& labels, const at::Tensor& mask, const at::Tensor& lse, double grad_scale,
             int64_t vocab_start) {
  need_bf16_rows(logits, "logits");
  need_i32(labels, "labels");
  need_f32(mask, "mask");
  need_f32(lse, "lse");
  check(fth_cross_entropy(logits.data_ptr(), labels.data_ptr<int>(), mask.data_ptr<float>(), nullptr, nullptr, nullptr, nullptr,
                          lse.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), logits.stride(0), (int)vocab_start,
                          (float)grad_scale, 2, cur_stream()), "ce_grad");
}

void adamw_segments(at::Tensor& master, at::Tensor& m, at::Tensor& v, const at::Tensor& grad, at::Tensor& param,
                    const at::Tensor& table, int64_t n_segs, double lr, double beta1, double beta2, double eps, double wd,
                    int64_t step, const at::Tensor& grad_scale) {
  need_f32(master, "master");
  need_f32(m, "m");
  need_f32(v, "v");
  need_f32(grad, "grad");
  need_f32(grad_scale, "grad_scale");
  TORCH_CHECK(param.is_cuda() && param.is_contiguous(), "param must be a contiguous CUDA tensor");
  const bool bf = param.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf || param.scalar_type() == at::kFloat, "param must be bf16 or fp32");
  const double bc1 = 1.0 - std::pow(beta1, (double)step), bc2 = 1.0 - std::pow(beta2, (double)step);
  check(fth_adamw_segments(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr<float>(),
                           param.data_ptr(), bf ? 1 : 0, table.data_ptr(), (int)n_segs, (float)lr, (float)beta1, (float)beta2,
                           (float)eps, (float)wd, (float)bc1, (float)(1.0 / std::sqrt(bc2)), grad_scale.data_ptr<float>(),
                           cur_stream()), "adamw_segments");
}

at::Tensor sumsq(const at::Tensor& x) {
  need_f32(x, "x");
  at::Tensor partial = at::empty({fth_sumsq_blocks()}, x.options().dtype(at::kDouble));
  at::Tensor out = at::empty({}, x.options());
  check(fth_sumsq(x.data_ptr<float>(), (size_t)x.numel(), partial.data_ptr<double>(), out.data_ptr<float>(), cur_stream()),
        "sumsq", 2);
  return out;
}

// C = alpha * A B^T (see gemm_sm100.cu).  `a`/`b` are 2-D bf16 with unit inner stride; `*_mn` says the stored
// matrix is [K, M|N] instead of [M|N, K].  epi: 0 bf16 store, 1 fp32 accumulate into `c`, 2 fp32 store.
at::Tensor gemm(const at::Tensor& a, bool a_mn, const at::Tensor& b, bool b_mn, c10::optional<at::Tensor> c, double alpha,
                int64_t epi, int64_t bn, int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "bf16 CUDA inputs");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "2-D operands with unit inner stride");
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "reduction dims differ: ", K, " vs ", Kb);
  at::Tensor out;
  if (c.has_value()) {
    out = *c;
    TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "bad output");
    TORCH_CHECK(out.scalar_type() == (epi == 0 ? at::kBFloat16 : at::kFloat), "output dtype does not match epilogue");
  } else {
    TORCH_CHECK(epi != 1, "accumulating epilogue needs an output tensor");
    out = at::empty({M, N}, a.options().dtype(epi == 0 ? at::kBFloat16 : at::kFloat));
  }
  check(fth_gemm_bf16(a.data_ptr(), a.stride(0), a_mn ? 1 : 0, b.data_ptr(), b.stride(0), b_mn ? 1 : 0, out.data_ptr(),
                      out.stride(0), (int)M, (int)N, (int)K, (float)alpha, (int)epi, (int)bn, (int)max_ctas, status_ptr(),
                      cur_stream()), "gemm_bf16");
  return out;
}

// MXFP8 quantisation of a 2-D bf16 matrix.  colwise = false: payload [R, C], scale blocks along C.  colwise = true: payload
// of the TRANSPOSE [C, R], scale blocks along R.  Returns {payload uint8, scale chunks uint8}.
std::vector<at::Tensor> mxfp8_quant(const at::Tensor& x, bool colwise) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 8 == 0 &&
                  (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "mxfp8_quant: bf16 CUDA matrix with 16-byte aligned rows");
  const int64_t R = x.size(0), C = x.size(1);
  const int64_t rows = colwise ? C : R, K = colwise ? R : C;
  TORCH_CHECK(K % 32 == 0, "mxfp8_quant: the quantised dimension must be a multiple of 32, got ", K);
  at::Tensor q = at::empty({rows, K}, x.options().dtype(at::kByte));
  const int64_t sfb = (int64_t)fth_mxfp8_sf_bytes((int)rows, (int)K);
  // whole chunks are read by the GEMM: bytes no block writes must not be the e8m0 NaN pattern
  at::Tensor sf = ((K / 32) % 4 == 0 && rows % 128 == 0) ? at::empty({sfb}, q.options()) : at::zeros({sfb}, q.options());
  check(fth_mxfp8_quant(x.data_ptr(), x.stride(0), q.data_ptr(), sf.data_ptr(), (int)R, (int)C, colwise ? 1 : 0, cur_stream()),
        "mxfp8_quant");
  return {q, sf};
}

// C = alpha * A B^T on MXFP8 operands (payload [M|N, K] uint8 + scale chunks).  epi as in gemm().
at::Tensor gemm_mxfp8(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb,
                      c10::optional<at::Tensor> c, double alpha, int64_t epi) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kByte && b.scalar_type() == at::kByte && a.is_contiguous() &&
                  b.is_contiguous() && a.dim() == 2 && b.dim() == 2, "gemm_mxfp8: contiguous uint8 payloads");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(b.size(1) == K, "gemm_mxfp8: reduction dims differ");
  TORCH_CHECK(sfa.numel() >= (int64_t)fth_mxfp8_sf_bytes((int)M, (int)K) && sfb.numel() >= (int64_t)fth_mxfp8_sf_bytes((int)N, (int)K),
              "gemm_mxfp8: scale arrays too small");
  at::Tensor out;
  if (c.has_value()) {
    out = *c;
    TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "bad output");
    TORCH_CHECK(out.scalar_type() == (epi == 0 ? at::kBFloat16 : at::kFloat), "output dtype does not match epilogue");
  } else {
    TORCH_CHECK(epi != 1, "accumulating epilogue needs an output tensor");
    out = at::empty({M, N}, a.options().dtype(epi == 0 ? at::kBFloat16 : at::kFloat));
  }
  check(fth_gemm_mxfp8(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), out.data_ptr(), out.stride(0), (int)M, (int)N,
                       (int)K, (float)alpha, (int)epi, status_ptr(), cur_stream()), "gemm_mxfp8");
  return out;
}

// Causal GQA attention on the packed QKV activation.  Returns {out [M, n_kv*g*d] bf16, lse [B, n_kv*g, S] fp32}.
std::vector<at::Tensor> flash_fwd(const at::Tensor& qkv, int64_t S, int64_t n_kv, int64_t g, int64_t d) {
  need_bf16(qkv, "qkv");
  const int64_t M = qkv.size(0), B = M / S;
  TORCH_CHECK(M % S == 0 && qkv.size(1) == n_kv * (g + 2) * d, "qkv shape mismatch");
  at::Tensor out = at::empty({M, n_kv * g * d}, qkv.options());
  at::Tensor lse = at::empty({B, n_kv * g, S}, qkv.options().dtype(at::kFloat));
  check(fth_flash_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), (int)B, (int)S, (int)n_kv, (int)g, (int)d,
                      status_ptr(), cur_stream()), "flash_fwd");
  return {out, lse};
}

at::Tensor flash_bwd(const at::Tensor& dout, const at::Tensor& qkv, const at::Tensor& out, const at::Tensor& lse,
                     const c10::optional<at::Tensor>& rope_table, int64_t S, int64_t n_kv, int64_t g, int64_t d) {
  need_bf16(dout, "dout");
  need_bf16(qkv, "qkv");
  need_bf16(out, "out");
  need_f32(lse, "lse");
  const int64_t M = qkv.size(0), B = M / S;
  at::Tensor dqkv = at::empty_like(qkv);
  const size_t bytes = fth_flash_bwd_scratch_bytes((int)B, (int)S, (int)n_kv, (int)g, (int)d);
  at::Tensor scratch = at::empty({(int64_t)(bytes / 4)}, qkv.options().dtype(at::kFloat));
  const float* tab = nullptr;
  if (rope_table.has_value()) {
    need_f32(*rope_table, "rope_table");
    TORCH_CHECK(rope_table->size(0) >= S && rope_table->size(1) == d, "rope table shape mismatch");
    tab = rope_table->data_ptr<float>();
  }
  check(fth_flash_bwd(dout.data_ptr(), qkv.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), dqkv.data_ptr(),
                      scratch.data_ptr(), tab, (int)B, (int)S, (int)n_kv, (int)g, (int)d, status_ptr(), cur_stream()), "flash_bwd", 3);
  return dqkv;
}

// ---- peer-memory collectives (pointers come from torch symmetric memory: handle.buffer_ptrs / multicast_ptr) ----------
// `epoch_dev` (int32[lanes], optional): number the barrier from a device counter instead of `epoch` (graph-replayable).
void peer_barrier(const std::vector<int64_t>& pads, int64_t rank, int64_t epoch, int64_t lane_slot, double limit_s,
                  c10::optional<at::Tensor> epoch_dev) {
  std::vector<void*> p(pads.size());
  for (size_t i = 0; i < pads.size(); ++i) p[i] = reinterpret_cast<void*>(pads[i]);
  unsigned* ed = nullptr;
  if (epoch_dev.has_value()) {
    need_i32(*epoch_dev, "epoch_dev");
    TORCH_CHECK(epoch_dev->numel() > lane_slot, "peer_barrier: epoch_dev needs one counter per lane");
    ed = reinterpret_cast<unsigned*>(epoch_dev->data_ptr<int>()) + lane_slot;
  }
  check(fth_peer_barrier(p.data(), (int)rank, (int)pads.size(), (unsigned)epoch, (int)lane_slot, status_ptr(), limit_s, ed,
                         cur_stream()), "peer_barrier");
}

void dp_reduce_scatter(const std::vector<int64_t>& grads, int64_t mc_grads, int64_t start, int64_t count, int64_t rank,
                       at::Tensor& sumsq_accum) {
  need_f32(sumsq_accum, "sumsq_accum");
  std::vector<void*> p(grads.size());
  for (size_t i = 0; i < grads.size(); ++i) p[i] = reinterpret_cast<void*>(grads[i]);
  at::Tensor partial = at::empty({fth_dp_reduce_scatter_blocks()}, sumsq_accum.options().dtype(at::kDouble));
  check(fth_dp_reduce_scatter(p.data(), reinterpret_cast<const void*>(mc_grads), start, count, (int)grads.size(), (int)rank,
                              partial.data_ptr<double>(), sumsq_accum.data_ptr<float>(), cur_stream()), "dp_reduce_scatter", 2);
}

void adamw_push(at::Tensor& master, at::Tensor& m, at::Tensor& v, const at::Tensor& grad, const std::vector<int64_t>& params,
                int64_t mc_param, const at::Tensor& table, int64_t n_segs, double lr, double beta1, double beta2, double eps,
                double wd, int64_t step, const at::Tensor& grad_scale) {
  need_f32(master, "master");
  need_f32(m, "m");
  need_f32(v, "v");
  need_f32(grad, "grad");
  need_f32(grad_scale, "grad_scale");
  std::vector<void*> p(params.size());
  for (size_t i = 0; i < params.size(); ++i) p[i] = reinterpret_cast<void*>(params[i]);
  const double bc1 = 1.0 - std::pow(beta1, (double)step), bc2 = 1.0 - std::pow(beta2, (double)step);
  check(fth_adamw_push(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr<float>(), p.data(),
                       reinterpret_cast<void*>(mc_param), (int)params.size(), table.data_ptr(), (int)n_segs, (float)lr, (float)beta1,
                       (float)beta2, (float)eps, (float)wd, (float)bc1, (float)(1.0 / std::sqrt(bc2)), grad_scale.data_ptr<float>(),
                       cur_stream()), "adamw_push");
}

// a [M, K_local] x b -> reduce-scatter into the owners' [M/tp, N] shards (pointers into symmetric memory, zeroed by the owners).
void gemm_rs(const at::Tensor& a, const at::Tensor& b, bool b_mn, const std::vector<int64_t>& out_shards, int64_t N, int64_t rank,
             double alpha) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && a.dim() == 2 && a.stride(1) == 1, "a: 2-D bf16");
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 2 && b.stride(1) == 1, "b: 2-D bf16");
  std::vector<void*> p(out_shards.size());
  for (size_t i = 0; i < p.size(); ++i) p[i] = reinterpret_cast<void*>(out_shards[i]);
  check(fth_gemm_rs(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), b_mn ? 1 : 0, p.data(), N, (int)a.size(0), (int)N,
                    (int)a.size(1), (int)p.size(), (int)rank, (float)alpha, status_ptr(), cur_stream()), "gemm_rs");
}

// gather buffers [M, K] (symmetric; own shard already written) x b -> out [M, N]; this rank's buffer ends up fully gathered.
// `ctr` / `ready` select the self-sequenced form (see fth_ag_gemm); pass None / [] for the host-sequenced one.
at::Tensor ag_gemm(const std::vector<int64_t>& gather, int64_t M, int64_t K, const at::Tensor& b, bool b_mn, int64_t rank,
                   int64_t n_copy_ctas, at::Tensor& flags, int64_t epoch, double alpha, c10::optional<at::Tensor> ctr,
                   const std::vector<int64_t>& ready) {
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 2 && b.stride(1) == 1, "b: 2-D bf16");
  need_i32(flags, "flags");
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  std::vector<void*> p(gather.size());
  for (size_t i = 0; i < p.size(); ++i) p[i] = reinterpret_cast<void*>(gather[i]);
  std::vector<void*> rp(ready.size());
  for (size_t i = 0; i < rp.size(); ++i) rp[i] = reinterpret_cast<void*>(ready[i]);
  int* ctr_ptr = nullptr;
  if (ctr.has_value()) {
    need_i32(*ctr, "ctr");
    TORCH_CHECK(ctr->numel() >= 2 && rp.size() == p.size(), "ag_gemm: ctr needs 2 ints and one ready array per rank");
    ctr_ptr = ctr->data_ptr<int>();
  }
  at::Tensor out = at::empty({M, N}, b.options());
  check(fth_ag_gemm(p.data(), K, b.data_ptr(), b.stride(0), b_mn ? 1 : 0, out.data_ptr(), N, (int)M, (int)N, (int)K, (int)p.size(),
                    (int)rank, (int)n_copy_ctas, flags.data_ptr<int>(), (int)epoch, ctr_ptr, ctr_ptr ? rp.data() : nullptr,
                    (float)alpha, status_ptr(), cur_stream()),
        "ag_gemm");
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_", &rope_);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("residual_add", &residual_add);
  m.def("qk_norm_fwd", &qk_norm_fwd);
  m.def("qk_norm_bwd_", &qk_norm_bwd_);
  m.def("check_ids", &check_ids);
  m.def("bad_index_position", &bad_index_position);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("embedding_bwd_det", &embedding_bwd_det);
  m.def("cross_entropy", &cross_entropy);
  m.def("ce_stats", &ce_stats);
  m.def("ce_grad", &ce_grad);
  m.def("adamw_segments", &adamw_segments);
  m.def("sumsq", &sumsq);
  m.def("gemm", &gemm);
  m.def("gemm_set_deterministic", [](bool on) { fth_gemm_set_deterministic(on ? 1 : 0); });
  m.def("tmap_cache_stats", []() {
    unsigned long long h = 0, mi = 0;
    fth_tmap_cache_stats(&h, &mi);
    return std::vector<int64_t>{(int64_t)h, (int64_t)mi};
  });
  m.def("mxfp8_quant", &mxfp8_quant);
  m.def("gemm_mxfp8", &gemm_mxfp8);
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_fwd_set_debug", [](int64_t p) { fth_flash_fwd_set_debug(reinterpret_cast<long long*>(p)); });
  m.def("flash_bwd", &flash_bwd);
  m.def("flash_bwd_set_debug", [](int64_t p) { fth_flash_bwd_set_debug(reinterpret_cast<long long*>(p)); });
  m.def("gemm_rs", &gemm_rs);
  m.def("ag_gemm", &ag_gemm);
  m.def("peer_barrier", &peer_barrier);
  m.def("dp_reduce_scatter", &dp_reduce_scatter);
  m.def("adamw_push", &adamw_push);
  m.def("read_status", &read_status);
  m.def("launch_count", &launch_count);
}
