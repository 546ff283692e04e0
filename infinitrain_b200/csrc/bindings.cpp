// Python bindings of the native layer: tensor-checked wrappers around the C launch interface of
// the sm_100a kernels (csrc/kernels/kernels.h), the multi-GPU kernels (csrc/comm/comm.h) and the
// host runtime (csrc/runtime/runtime.h).  Nothing here allocates on the hot path except the
// per-device status word, created once.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <string>
#include <vector>

#include "comm/comm.h"
#include "kernels/kernels.h"
#include "runtime/runtime.h"

namespace {

int dt(const at::Tensor& t) {
  if (t.scalar_type() == at::kFloat) return kItbF32;
  if (t.scalar_type() == at::kBFloat16) return kItbBF16;
  TORCH_CHECK(false, "infinitrain_b200: unsupported dtype ", t.scalar_type());
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "infinitrain_b200 kernel '", what, "' failed with code ", rc,
              rc > 0 ? std::string(" (") + cudaGetErrorString(static_cast<cudaError_t>(rc)) + ")"
                     : std::string(" (bad argument: alignment / shape / dtype)"));
}
const void* optr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr() : nullptr;
}

// Per-device status word that kernels with bounded waits write on time-out.
at::Tensor& status_word(int device) {
  static std::vector<at::Tensor> words(64);
  if (!words[device].defined())
    words[device] = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device];
}

int64_t kernel_status() {
  int dev = at::cuda::current_device();
  return status_word(dev).cpu()[0].item<int64_t>();
}
void kernel_status_reset() {
  int dev = at::cuda::current_device();
  status_word(dev).zero_();
}

// ------------------------------------------------------------------ GEMM
// Kernel choice: 0 = one CTA per 128 x 256 tile, 1 = CTA pairs on 256 x 256 tiles.
int g_gemm_mode = 1;
void set_gemm_mode(int64_t mode) { g_gemm_mode = static_cast<int>(mode); }
int64_t get_gemm_mode() { return g_gemm_mode; }
// bit 0: attention backward on tcgen05, bit 1: attention forward on tcgen05 (flash_attn_tc.cu);
// a cleared bit selects the mma.sync kernel of flash_attn.cu for that pass.
int g_attn_mode = 3;
void set_attn_mode(int64_t mode) { g_attn_mode = static_cast<int>(mode); }
int64_t get_attn_mode() { return g_attn_mode; }

// C[M,N] = A . B^T-like product; see kernels.h for the layout flags.
void gemm(const at::Tensor& a, bool a_mn, const at::Tensor& b, bool b_mn, int64_t M, int64_t N,
          int64_t K, at::Tensor& c, const c10::optional<at::Tensor>& c2,
          const c10::optional<at::Tensor>& bias, const c10::optional<at::Tensor>& residual,
          const c10::optional<at::Tensor>& aux, int64_t flags, int64_t split_k) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16,
              "gemm: bf16 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2, "gemm: 2-D tensors required");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1,
              "gemm: innermost dimension must be contiguous");
  c10::cuda::CUDAGuard guard(a.device());
  ItbGemmArgs g{};
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.A = a.data_ptr();
  g.lda = a.stride(0);
  g.a_mn_major = a_mn;
  g.B = b.data_ptr();
  g.ldb = b.stride(0);
  g.b_mn_major = b_mn;
  TORCH_CHECK(a_mn ? (a.size(0) == K && a.size(1) == M) : (a.size(0) == M && a.size(1) == K),
              "gemm: A shape mismatch");
  TORCH_CHECK(b_mn ? (b.size(0) == K && b.size(1) == N) : (b.size(0) == N && b.size(1) == K),
              "gemm: B shape mismatch");
  TORCH_CHECK(c.size(0) == M && c.size(1) >= N, "gemm: C shape mismatch");
  const bool f32 = flags & kGemmOutF32;
  TORCH_CHECK(c.scalar_type() == (f32 ? at::kFloat : at::kBFloat16), "gemm: C dtype mismatch");
  g.C = c.data_ptr();
  g.ldc = c.stride(0);
  if (flags & kGemmGeluDual) {
    TORCH_CHECK(c2.has_value() && c2->scalar_type() == at::kBFloat16 &&
                    c2->stride(0) == c.stride(0) && !f32,
                "gemm: gelu dual output needs a bf16 C2 with C's layout");
    g.C2 = c2->data_ptr();
  }
  if (flags & kGemmBias) {
    TORCH_CHECK(bias.has_value() && bias->scalar_type() == at::kFloat && bias->numel() >= N,
                "gemm: fp32 bias of length N required");
    g.bias = static_cast<const float*>(bias->data_ptr());
  }
  if (flags & kGemmResidual) {
    TORCH_CHECK(residual.has_value() && residual->scalar_type() == c.scalar_type() &&
                    residual->stride(1) == 1,
                "gemm: residual must have C's dtype");
    g.residual = residual->data_ptr();
    g.ldr = residual->stride(0);
  }
  if (flags & kGemmDGelu) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && aux->stride(1) == 1,
                "gemm: bf16 aux required");
    g.aux = aux->data_ptr();
    g.ld_aux = aux->stride(0);
  }
  g.flags = static_cast<int>(flags);
  g.split_k = static_cast<int>(split_k);
  g.err = status_word(a.get_device()).data_ptr<int>();
  if (g_gemm_mode == 1 && M > 128)
    check_rc(itb_gemm_bf16_pair(&g, cur_stream()), "gemm_bf16_tcgen05_pair");
  else
    check_rc(itb_gemm_bf16(&g, cur_stream()), "gemm_bf16_tcgen05");
}

// ------------------------------------------------------------------ norms
std::vector<at::Tensor> layernorm_fwd(const at::Tensor& x, const at::Tensor& gamma,
                                      const c10::optional<at::Tensor>& beta, double eps,
                                      at::ScalarType out_dtype) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "layernorm: contiguous input required");
  const int C = x.size(-1);
  const int rows = x.numel() / C;
  auto y = torch::empty_like(x, x.options().dtype(out_dtype));
  auto mean = torch::empty({rows}, x.options().dtype(at::kFloat));
  auto rstd = torch::empty({rows}, x.options().dtype(at::kFloat));
  check_rc(itb_layernorm_fwd(x.data_ptr(), dt(x), gamma.data_ptr<float>(),
                             static_cast<const float*>(optr(beta)), y.data_ptr(), dt(y),
                             mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, C,
                             static_cast<float>(eps), cur_stream()),
           "layernorm_fwd");
  return {y, mean, rstd};
}
// dres (optional): gradient of the residual stream past the norm, added to dx in the same pass;
// dgamma_out / dbeta_out / dres_sum_out (optional fp32 [C]): gradients are ACCUMULATED into these
// tensors (views of a flat gradient buffer) instead of being returned; want_dres_sum without an
// output tensor returns the column sums of dres as a fresh tensor.
std::vector<at::Tensor> layernorm_bwd(const at::Tensor& dy, const at::Tensor& x,
                                      const at::Tensor& gamma, const at::Tensor& mean,
                                      const at::Tensor& rstd, bool has_beta,
                                      const c10::optional<at::Tensor>& dres,
                                      const c10::optional<at::Tensor>& dgamma_out,
                                      const c10::optional<at::Tensor>& dbeta_out,
                                      const c10::optional<at::Tensor>& dres_sum_out, bool want_dres_sum) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous(), "layernorm_bwd: contiguous tensors required");
  const int C = x.size(-1);
  const int rows = x.numel() / C;
  auto dx = torch::empty_like(x);
  if (dres) TORCH_CHECK(dres->is_contiguous() && dres->scalar_type() == dx.scalar_type() && dres->numel() == x.numel(),
                        "layernorm_bwd: dres must match dx");
  int acc = 0;
  auto f32 = x.options().dtype(at::kFloat);
  at::Tensor dgamma = dgamma_out ? *dgamma_out : torch::empty({C}, f32);
  at::Tensor dbeta = dbeta_out ? *dbeta_out : torch::empty({C}, f32);
  at::Tensor dsum;
  if (dres && (dres_sum_out || want_dres_sum)) dsum = dres_sum_out ? *dres_sum_out : torch::empty({C}, f32);
  if (dgamma_out) acc |= 1;
  if (dbeta_out) acc |= 2;
  if (dres_sum_out) acc |= 4;
  for (const at::Tensor* t : {&dgamma, &dbeta})
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == C, "layernorm_bwd: fp32 [C] outputs");
  auto partial = torch::empty({itb_norm_partial_rows(rows), 3 * C}, f32);
  check_rc(itb_layernorm_bwd_res(dy.data_ptr(), dt(dy), x.data_ptr(), dt(x), gamma.data_ptr<float>(),
                                 mean.data_ptr<float>(), rstd.data_ptr<float>(), dres ? dres->data_ptr() : nullptr,
                                 dx.data_ptr(), dt(dx), dgamma.data_ptr<float>(), dbeta.data_ptr<float>(),
                                 dsum.defined() ? dsum.data_ptr<float>() : nullptr, partial.data_ptr<float>(), rows, C,
                                 acc, cur_stream()),
           "layernorm_bwd");
  return {dx, dgamma, dbeta, dsum};
}
std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& gamma, double eps,
                                    at::ScalarType out_dtype) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "rmsnorm: contiguous input required");
  const int C = x.size(-1);
  const int rows = x.numel() / C;
  auto y = torch::empty_like(x, x.options().dtype(out_dtype));
  auto rstd = torch::empty({rows}, x.options().dtype(at::kFloat));
  check_rc(itb_rmsnorm_fwd(x.data_ptr(), dt(x), gamma.data_ptr<float>(), y.data_ptr(), dt(y),
                           rstd.data_ptr<float>(), rows, C, static_cast<float>(eps), cur_stream()),
           "rmsnorm_fwd");
  return {y, rstd};
}
std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x,
                                    const at::Tensor& gamma, const at::Tensor& rstd,
                                    const c10::optional<at::Tensor>& dres,
                                    const c10::optional<at::Tensor>& dgamma_out,
                                    const c10::optional<at::Tensor>& dres_sum_out, bool want_dres_sum) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous(), "rmsnorm_bwd: contiguous tensors required");
  const int C = x.size(-1);
  const int rows = x.numel() / C;
  auto dx = torch::empty_like(x);
  if (dres) TORCH_CHECK(dres->is_contiguous() && dres->scalar_type() == dx.scalar_type() && dres->numel() == x.numel(),
                        "rmsnorm_bwd: dres must match dx");
  auto f32 = x.options().dtype(at::kFloat);
  at::Tensor dgamma = dgamma_out ? *dgamma_out : torch::empty({C}, f32);
  TORCH_CHECK(dgamma.scalar_type() == at::kFloat && dgamma.is_contiguous() && dgamma.numel() == C, "rmsnorm_bwd: fp32 [C] output");
  at::Tensor dsum;
  if (dres && (dres_sum_out || want_dres_sum)) dsum = dres_sum_out ? *dres_sum_out : torch::empty({C}, f32);
  const int acc = (dgamma_out ? 1 : 0) | (dres_sum_out ? 4 : 0);
  auto partial = torch::empty({itb_norm_partial_rows(rows), 3 * C}, f32);
  check_rc(itb_rmsnorm_bwd_res(dy.data_ptr(), dt(dy), x.data_ptr(), dt(x), gamma.data_ptr<float>(),
                               rstd.data_ptr<float>(), dres ? dres->data_ptr() : nullptr, dx.data_ptr(), dt(dx),
                               dgamma.data_ptr<float>(), dsum.defined() ? dsum.data_ptr<float>() : nullptr,
                               partial.data_ptr<float>(), rows, C, acc, cur_stream()),
           "rmsnorm_bwd");
  return {dx, dgamma, dsum};
}

// ------------------------------------------------------------------ activations
at::Tensor gelu_fwd(const at::Tensor& x) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "gelu: contiguous input required");
  auto y = torch::empty_like(x);
  check_rc(itb_gelu_fwd(x.data_ptr(), y.data_ptr(), dt(x), x.numel(), cur_stream()), "gelu_fwd");
  return y;
}
at::Tensor gelu_bwd(const at::Tensor& dy, const at::Tensor& x) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dy.scalar_type() == x.scalar_type(),
              "gelu_bwd: contiguous tensors of one dtype required");
  auto dx = torch::empty_like(x);
  check_rc(itb_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), dt(x), x.numel(), cur_stream()),
           "gelu_bwd");
  return dx;
}
// a, b: [rows, F] views (row stride ld, unit column stride) -> out [rows, F] contiguous
at::Tensor swiglu_fwd(const at::Tensor& a, const at::Tensor& b) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 &&
                  a.stride(0) == b.stride(0) && a.scalar_type() == b.scalar_type(),
              "swiglu: 2-D views with equal row strides required");
  auto out = torch::empty({a.size(0), a.size(1)}, a.options());
  check_rc(itb_swiglu_fwd(a.data_ptr(), b.data_ptr(), a.stride(0), out.data_ptr(), out.stride(0),
                          dt(a), a.size(0), a.size(1), cur_stream()),
           "swiglu_fwd");
  return out;
}
// Returns dab [rows, 2F]: columns [0,F) = da, [F,2F) = db.
at::Tensor swiglu_bwd(const at::Tensor& dout, const at::Tensor& a, const at::Tensor& b) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(dout.dim() == 2 && dout.stride(1) == 1 && a.stride(1) == 1 && b.stride(1) == 1 &&
                  a.stride(0) == b.stride(0),
              "swiglu_bwd: bad layout");
  const int64_t F = a.size(1);
  auto dab = torch::empty({a.size(0), 2 * F}, a.options());
  check_rc(itb_swiglu_bwd(dout.data_ptr(), dout.stride(0), a.data_ptr(), b.data_ptr(), a.stride(0),
                          dab.data_ptr(), static_cast<char*>(dab.data_ptr()) + F * dab.element_size(),
                          dab.stride(0), dt(a), a.size(0), F, cur_stream()),
           "swiglu_bwd");
  return dab;
}

// ------------------------------------------------------------------ rope
void rope_inplace(at::Tensor& qkv, const at::Tensor& freqs, int64_t B, int64_t T, int64_t n_heads,
                  int64_t D, int64_t row_stride, int64_t pos0, bool inverse) {
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(freqs.scalar_type() == at::kFloat && freqs.is_contiguous(), "rope: fp32 table");
  TORCH_CHECK(freqs.size(0) >= pos0 + T, "rope: table too short");
  check_rc(itb_rope_inplace(qkv.data_ptr(), dt(qkv), freqs.data_ptr<float>(), B, T, n_heads, D,
                            row_stride, pos0, inverse, cur_stream()),
           "rope");
}

// ------------------------------------------------------------------ embedding
at::Tensor embedding_fwd(const at::Tensor& idx, const at::Tensor& wte,
                         const c10::optional<at::Tensor>& wpe, int64_t pos0, int64_t vocab_start,
                         at::ScalarType out_dtype) {
  c10::cuda::CUDAGuard guard(wte.device());
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous() && idx.dim() == 2,
              "embedding: int64 [B,T] indices");
  const int B = idx.size(0), T = idx.size(1), C = wte.size(1);
  auto out = torch::empty({B, T, C}, wte.options().dtype(out_dtype));
  check_rc(itb_embedding_fwd(idx.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()) : nullptr,
                             wte.data_ptr(), optr(wpe), dt(wte), out.data_ptr(), dt(out), B, T, C,
                             pos0, vocab_start, vocab_start + wte.size(0), cur_stream()),
           "embedding_fwd");
  return out;
}
void embedding_bwd(const at::Tensor& idx, const at::Tensor& dout,
                   const c10::optional<at::Tensor>& dwte, const c10::optional<at::Tensor>& dwpe,
                   int64_t pos0, int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(dout.device());
  TORCH_CHECK(dout.is_contiguous() && dout.dim() == 3, "embedding_bwd: contiguous [B,T,C]");
  const int B = dout.size(0), T = dout.size(1), C = dout.size(2);
  int64_t vend = vocab_start + (dwte.has_value() ? dwte->size(0) : 0);
  check_rc(itb_embedding_bwd(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()),
                             dout.data_ptr(), dt(dout),
                             dwte.has_value() ? dwte->data_ptr<float>() : nullptr,
                             dwpe.has_value() ? dwpe->data_ptr<float>() : nullptr, B, T, C, pos0,
                             vocab_start, vend, cur_stream()),
           "embedding_bwd");
}

// ------------------------------------------------------------------ cross entropy
// logits [rows, ld] (first V columns valid).  Returns {loss_mean[1], lse[rows], row_loss[rows]}.
std::vector<at::Tensor> ce_fwd(const at::Tensor& logits, const at::Tensor& target, int64_t V) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "ce: 2-D logits");
  TORCH_CHECK(target.scalar_type() == at::kLong && target.is_contiguous(), "ce: int64 targets");
  const int rows = logits.size(0);
  auto f32 = logits.options().dtype(at::kFloat);
  auto loss = torch::zeros({1}, f32);
  auto lse = torch::empty({rows}, f32);
  auto row_loss = torch::empty({rows}, f32);
  check_rc(itb_ce_fwd(logits.data_ptr(), dt(logits), logits.stride(0),
                      reinterpret_cast<const long long*>(target.data_ptr<int64_t>()),
                      row_loss.data_ptr<float>(), lse.data_ptr<float>(), loss.data_ptr<float>(),
                      rows, V, cur_stream()),
           "ce_fwd");
  return {loss, lse, row_loss};
}
void ce_bwd(at::Tensor& logits, const at::Tensor& target, const at::Tensor& lse,
            const at::Tensor& grad_out, int64_t V, bool ignore_oob) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(grad_out.scalar_type() == at::kFloat && grad_out.numel() == 1, "ce_bwd: fp32 scalar");
  check_rc(itb_ce_bwd(logits.data_ptr(), dt(logits), logits.stride(0),
                      reinterpret_cast<const long long*>(target.data_ptr<int64_t>()),
                      lse.data_ptr<float>(), grad_out.data_ptr<float>(), logits.size(0), V,
                      ignore_oob, cur_stream()),
           "ce_bwd");
}

// ------------------------------------------------------------------ optimizer
void adamw(at::Tensor& p, const at::Tensor& g, at::Tensor& m, at::Tensor& v,
           const c10::optional<at::Tensor>& shadow, double lr, double b1, double b2, double eps,
           double wd, double bc1, double bc2, double grad_scale,
           const c10::optional<at::Tensor>& dev_hyper) {
  c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(!dev_hyper.has_value() || (dev_hyper->scalar_type() == at::kFloat && dev_hyper->numel() >= 3 &&
                                         dev_hyper->is_cuda()),
              "adamw: dev_hyper must be a CUDA fp32 tensor [lr, 1/bc1, 1/bc2]");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(),
              "adamw: contiguous flat buffers required");
  TORCH_CHECK(p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
                  v.scalar_type() == at::kFloat,
              "adamw: fp32 master weights and state required");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(),
              "adamw: size mismatch");
  check_rc(itb_adamw(p.data_ptr<float>(), g.data_ptr(), dt(g), m.data_ptr<float>(),
                     v.data_ptr<float>(), const_cast<void*>(optr(shadow)), p.numel(), lr, b1, b2,
                     eps, wd, bc1, bc2, grad_scale, static_cast<const float*>(optr(dev_hyper)),
                     cur_stream()),
           "adamw");
}
void adam_advance(at::Tensor& hyper, double b1, double b2) {
  c10::cuda::CUDAGuard guard(hyper.device());
  TORCH_CHECK(hyper.is_cuda() && hyper.scalar_type() == at::kFloat && hyper.numel() >= 4, "adam_advance: fp32[4]");
  check_rc(itb_adam_advance(hyper.data_ptr<float>(), b1, b2, cur_stream()), "adam_advance");
}
void sgd(at::Tensor& p, const at::Tensor& g, const c10::optional<at::Tensor>& shadow, double lr,
         double grad_scale) {
  c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && p.scalar_type() == at::kFloat,
              "sgd: contiguous fp32 weights required");
  check_rc(itb_sgd(p.data_ptr<float>(), g.data_ptr(), dt(g), const_cast<void*>(optr(shadow)),
                   p.numel(), lr, grad_scale, cur_stream()),
           "sgd");
}

// ------------------------------------------------------------------ utilities
void cast_into(const at::Tensor& src, at::Tensor& dst) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel(),
              "cast: contiguous tensors of equal size required");
  check_rc(itb_cast(src.data_ptr(), dt(src), dst.data_ptr(), dt(dst), src.numel(), cur_stream()),
           "cast");
}
// Column sums of a [rows, N] matrix; with `into` (fp32 [N]) the sums are ADDED to that tensor (a view
// of a flat gradient buffer) and it is returned.
at::Tensor colsum(const at::Tensor& x, const c10::optional<at::Tensor>& into) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "colsum: 2-D row-major input");
  const int rows = x.size(0), N = x.size(1);
  at::Tensor out = into ? *into : torch::empty({N}, x.options().dtype(at::kFloat));
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == N, "colsum: fp32 [N] output");
  auto partial = torch::empty({itb_colsum_partial_rows(rows), N}, x.options().dtype(at::kFloat));
  check_rc(itb_colsum(x.data_ptr(), dt(x), x.stride(0), out.data_ptr<float>(),
                      partial.data_ptr<float>(), rows, N, into ? 1 : 0, cur_stream()),
           "colsum");
  return out;
}

// ------------------------------------------------------------------ attention
// q [B,T,H,D], k/v [B,T,KV,D] (views with unit stride on D, head stride D) -> {o [B,T,H,D], lse}
ItbAttnArgs attn_args(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                      bool causal) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "attention: [B,T,H,D] tensors");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16,
              "attention: bf16 required");
  const int64_t D = q.size(3);
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && q.stride(2) == D &&
                  k.stride(2) == D && v.stride(2) == D,
              "attention: heads must be packed along the last two dimensions");
  ItbAttnArgs a{};
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.q_row_stride = q.stride(1);
  a.k_row_stride = k.stride(1);
  a.v_row_stride = v.stride(1);
  a.q_batch_stride = q.stride(0);
  a.k_batch_stride = k.stride(0);
  a.v_batch_stride = v.stride(0);
  a.B = q.size(0);
  a.T = q.size(1);
  a.H = q.size(2);
  a.KV = k.size(2);
  a.D = D;
  a.scale = static_cast<float>(scale);
  a.causal = causal;
  return a;
}
std::vector<at::Tensor> flash_attn_fwd(const at::Tensor& q, const at::Tensor& k,
                                       const at::Tensor& v, double scale, bool causal) {
  c10::cuda::CUDAGuard guard(q.device());
  ItbAttnArgs a = attn_args(q, k, v, scale, causal);
  auto o = torch::empty({a.B, a.T, a.H, a.D}, q.options());
  auto lse = torch::empty({a.B, a.H, a.T}, q.options().dtype(at::kFloat));
  a.o = o.data_ptr();
  a.o_row_stride = o.stride(1);
  a.o_batch_stride = o.stride(0);
  a.lse = lse.data_ptr<float>();
  if (g_attn_mode & 2)
    check_rc(itb_flash_attn_fwd_tc(&a, status_word(q.get_device()).data_ptr<int>(), cur_stream()),
             "flash_attn_fwd_tc");
  else
    check_rc(itb_flash_attn_fwd(&a, cur_stream()), "flash_attn_fwd");
  return {o, lse};
}
// dq/dk/dv are written into caller-provided views (e.g. column blocks of one packed dqkv buffer).
void flash_attn_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                    const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse, at::Tensor& dq,
                    at::Tensor& dk, at::Tensor& dv, double scale, bool causal) {
  c10::cuda::CUDAGuard guard(q.device());
  ItbAttnArgs a = attn_args(q, k, v, scale, causal);
  TORCH_CHECK(o.is_contiguous() && dout.is_contiguous(), "attention bwd: contiguous o and dout");
  TORCH_CHECK(dq.strides() == q.strides() && dk.strides() == k.strides() &&
                  dv.strides() == v.strides(),
              "attention bwd: gradient views must share the strides of q/k/v");
  a.o = o.data_ptr();
  a.o_row_stride = o.stride(1);
  a.o_batch_stride = o.stride(0);
  a.lse = lse.data_ptr<float>();
  a.dout = dout.data_ptr();
  a.dq = dq.data_ptr();
  a.dk = dk.data_ptr();
  a.dv = dv.data_ptr();
  auto f32 = q.options().dtype(at::kFloat);
  auto delta = torch::empty({a.B, a.H, a.T}, f32);
  auto dq_accum = torch::empty({a.B, a.T, a.H, a.D}, f32);
  a.delta = delta.data_ptr<float>();
  a.dq_accum = dq_accum.data_ptr<float>();
  at::Tensor dkv_accum;
  if ((g_attn_mode & 1) && itb_flash_attn_bwd_parts(a.B, a.T, a.H, a.KV, a.causal) > 1) {
    dkv_accum = torch::empty({2, a.B, a.T, a.KV, a.D}, f32);
    a.dkv_accum = dkv_accum.data_ptr<float>();
  }
  if (g_attn_mode & 1)
    check_rc(itb_flash_attn_bwd_tc(&a, status_word(q.get_device()).data_ptr<int>(), cur_stream()),
             "flash_attn_bwd_tc");
  else
    check_rc(itb_flash_attn_bwd(&a, cur_stream()), "flash_attn_bwd");
}

}  // namespace

void bind_comm(pybind11::module_& m);
void bind_runtime(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "infinitrain_b200 native layer (sm_100a kernels, NVLink kernels, host runtime)";
  m.attr("GEMM_OUT_F32") = static_cast<int>(kGemmOutF32);
  m.attr("GEMM_ATOMIC") = static_cast<int>(kGemmAtomic);
  m.attr("GEMM_ACCUM") = static_cast<int>(kGemmAccum);
  m.attr("GEMM_BIAS") = static_cast<int>(kGemmBias);
  m.attr("GEMM_RESIDUAL") = static_cast<int>(kGemmResidual);
  m.attr("GEMM_GELU_DUAL") = static_cast<int>(kGemmGeluDual);
  m.attr("GEMM_DGELU") = static_cast<int>(kGemmDGelu);
  m.attr("GEMM_PROBE_NO_LOAD") = static_cast<int>(kGemmProbeNoLoad);
  m.attr("GEMM_PROBE_NO_MMA") = static_cast<int>(kGemmProbeNoMma);
  m.def("kernel_status", &kernel_status);
  m.def("kernel_status_reset", &kernel_status_reset);
  m.def("gemm", &gemm);
  m.def("set_gemm_mode", &set_gemm_mode);
  m.def("set_attn_mode", &set_attn_mode);
  m.def("get_attn_mode", &get_attn_mode);
  m.def("get_gemm_mode", &get_gemm_mode);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("gamma"),
        pybind11::arg("mean"), pybind11::arg("rstd"), pybind11::arg("has_beta"), pybind11::arg("dres") = pybind11::none(),
        pybind11::arg("dgamma_out") = pybind11::none(), pybind11::arg("dbeta_out") = pybind11::none(),
        pybind11::arg("dres_sum_out") = pybind11::none(), pybind11::arg("want_dres_sum") = false);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("gamma"), pybind11::arg("rstd"),
        pybind11::arg("dres") = pybind11::none(), pybind11::arg("dgamma_out") = pybind11::none(),
        pybind11::arg("dres_sum_out") = pybind11::none(), pybind11::arg("want_dres_sum") = false);
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("rope_inplace", &rope_inplace);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd", &ce_bwd);
  m.def("adamw", &adamw, pybind11::arg("p"), pybind11::arg("g"), pybind11::arg("m"), pybind11::arg("v"),
        pybind11::arg("shadow"), pybind11::arg("lr"), pybind11::arg("b1"), pybind11::arg("b2"),
        pybind11::arg("eps"), pybind11::arg("wd"), pybind11::arg("bc1"), pybind11::arg("bc2"),
        pybind11::arg("grad_scale"), pybind11::arg("dev_hyper") = pybind11::none());
  m.def("adam_advance", &adam_advance);
  m.def("sgd", &sgd);
  m.def("cast_into", &cast_into);
  m.def("colsum", &colsum, pybind11::arg("x"), pybind11::arg("into") = pybind11::none());
  m.def("flash_attn_fwd", &flash_attn_fwd);
  m.def("flash_attn_bwd", &flash_attn_bwd);
  bind_comm(m);
  bind_runtime(m);
}
