// Fused ops of the C++ frontend on a B200: torch::autograd::Function wrappers around the C launch
// interface of the sm_100a kernels (csrc/kernels/kernels.h).  Included by ops.h under ITB_WITH_CUDA;
// the program links against infinitrain_b200/_C.so, which exports the itb_* launchers.
//
// Mixed precision as in the Python layer: bf16 activations and bf16 weight shadows into the tcgen05
// GEMM, fp32 accumulation, fp32 weight / bias / norm gradients, fp32 statistics.
#pragma once
#include "profiler.h"
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cmath>
#include <unordered_map>

#include "../../kernels/kernels.h"
#include "module.h"

namespace itb {
namespace ops {
namespace fused {

using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline int code(const Tensor& t) {
  if (t.scalar_type() == torch::kFloat32) return kItbF32;
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, "itb: fp32 or bf16 tensor expected");
  return kItbBF16;
}
inline void check(int rc, const char* what) { TORCH_CHECK(rc == 0, "itb kernel '", what, "' failed with code ", rc); }
inline int64_t pad64(int64_t n) { return (n + 63) / 64 * 64; }
inline Tensor contig(const Tensor& t) { return t.is_contiguous() ? t : t.contiguous(); }

// Status word of the bounded waits, one per device; 0 = no wait gave up.
inline Tensor& status_word(int device) {
  static std::vector<Tensor> words(64);
  if (!words[device].defined())
    words[device] = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device];
}
inline int64_t kernel_status() { return status_word(at::cuda::current_device()).cpu()[0].item<int64_t>(); }

// bf16 copy of an fp32 weight, cached per tensor and refreshed when the weight's version moved.  An
// entry holds a weak reference to its tensor: the tensor's address cannot be handed to another tensor
// while the entry exists (a new weight can never pick up a dead weight's copy), and entries of dead
// tensors are dropped the next time the table grows.
struct Shadow {
  Tensor bf16;
  int64_t version = -1;
  c10::weak_intrusive_ptr<c10::TensorImpl> owner{c10::intrusive_ptr<c10::TensorImpl>()};
};
inline std::unordered_map<const void*, Shadow>& shadows() {
  static std::unordered_map<const void*, Shadow> m;
  return m;
}
inline Shadow& shadow_entry(const Tensor& w) {
  auto& table = shadows();
  auto it = table.find(w.unsafeGetTensorImpl());
  if (it != table.end() && !it->second.owner.expired()) return it->second;
  if (it == table.end() && table.size() % 64 == 63)
    for (auto dead = table.begin(); dead != table.end();) dead = dead->second.owner.expired() ? table.erase(dead) : std::next(dead);
  Shadow& s = table[w.unsafeGetTensorImpl()];
  s = Shadow{};
  s.owner = c10::weak_intrusive_ptr<c10::TensorImpl>(w.getIntrusivePtr());
  return s;
}
inline Tensor weight_lp(const Tensor& w) {
  if (w.scalar_type() == torch::kBFloat16) return w.detach();
  auto& s = shadow_entry(w);
  int64_t ver = static_cast<int64_t>(w._version());
  if (s.bf16.defined() && s.version == ver && s.bf16.device() == w.device()) return s.bf16;
  if (!s.bf16.defined() || s.bf16.sizes() != w.sizes() || s.bf16.device() != w.device())
    s.bf16 = torch::empty(w.sizes(), w.options().dtype(torch::kBFloat16).requires_grad(false));
  Tensor wc = contig(w.detach());
  check(itb_cast(wc.data_ptr(), kItbF32, s.bf16.data_ptr(), kItbBF16, wc.numel(), stream()), "cast");
  s.version = ver;
  return s.bf16;
}
// An optimizer that wrote the shadow itself stamps it with the weight's new version.
inline void mark_shadow_fresh(const Tensor& w) {
  auto it = shadows().find(w.unsafeGetTensorImpl());
  if (it != shadows().end() && !it->second.owner.expired()) it->second.version = static_cast<int64_t>(w._version());
}
inline Tensor shadow_of(const Tensor& w) {
  weight_lp(w);
  return shadow_entry(w).bf16;
}

inline Tensor as_bf16_2d(const Tensor& x) {
  Tensor x2 = x.reshape({-1, x.size(-1)});
  if (x2.scalar_type() != torch::kBFloat16) x2 = x2.to(torch::kBFloat16);
  if (x2.stride(-1) != 1 || x2.stride(0) % 8 || reinterpret_cast<uintptr_t>(x2.data_ptr()) % 16) x2 = x2.contiguous();
  return x2;
}

// C[M, N] (+)= A . B with the layout flags of kernels.h, on CTA pairs.
inline void gemm(const Tensor& a, bool a_mn, const Tensor& b, bool b_mn, int64_t M, int64_t N, int64_t K, Tensor& c,
                 const Tensor& c2, const Tensor& bias, const Tensor& residual, const Tensor& aux, int flags) {
  c10::cuda::CUDAGuard guard(a.device());
  ItbGemmArgs g{};
  g.M = static_cast<int>(M), g.N = static_cast<int>(N), g.K = static_cast<int>(K);
  g.A = a.data_ptr(), g.lda = a.stride(0), g.a_mn_major = a_mn;
  g.B = b.data_ptr(), g.ldb = b.stride(0), g.b_mn_major = b_mn;
  g.C = c.data_ptr(), g.ldc = c.stride(0);
  g.C2 = c2.defined() ? c2.data_ptr() : nullptr;
  g.bias = bias.defined() ? bias.data_ptr<float>() : nullptr;
  g.residual = residual.defined() ? residual.data_ptr() : nullptr;
  g.ldr = residual.defined() ? residual.stride(0) : 0;
  g.aux = aux.defined() ? aux.data_ptr() : nullptr;
  g.ld_aux = aux.defined() ? aux.stride(0) : 0;
  g.flags = flags;
  g.split_k = 0;
  g.err = status_word(a.device().index()).data_ptr<int>();
  check(itb_gemm_bf16_pair(&g, stream()), "gemm_bf16_pair");
}

// ------------------------------------------------------------------ linear
struct LinearFn : public torch::autograd::Function<LinearFn> {
  // Optional tensor inputs are std::optional arguments: an undefined Tensor passed to apply() would be
  // recorded as a variable input, and the engine rejects a variable without a device.
  static Tensor forward(AutogradContext* ctx, const Tensor& x, const Tensor& weight, const c10::optional<Tensor>& bias_o,
                        const c10::optional<Tensor>& residual_o, bool gelu) {
    const Tensor bias = bias_o.value_or(Tensor()), residual = residual_o.value_or(Tensor());
    int64_t K = x.size(-1), N = weight.size(0);
    Tensor x2 = as_bf16_2d(x);
    int64_t M = x2.size(0), ld = pad64(N);
    Tensor w = weight_lp(weight);
    bool out_f32 = residual.defined() && residual.scalar_type() == torch::kFloat32;
    Tensor out = torch::empty({M, ld}, x.options().dtype(out_f32 ? torch::kFloat32 : torch::kBFloat16).requires_grad(false));
    int flags = (out_f32 ? kGemmOutF32 : 0) | (bias.defined() ? kGemmBias : 0);
    Tensor pre, res2;
    if (residual.defined()) {
      res2 = residual.reshape({M, N});
      if (res2.stride(-1) != 1) res2 = res2.contiguous();
      flags |= kGemmResidual;
    }
    if (gelu) {
      TORCH_CHECK(!residual.defined(), "gelu and residual epilogues are not combined");
      pre = torch::empty({M, ld}, x.options().dtype(torch::kBFloat16).requires_grad(false));
      gemm(x2, false, w, false, M, N, K, pre, out, bias, Tensor(), Tensor(), flags | kGemmGeluDual);
    } else {
      gemm(x2, false, w, false, M, N, K, out, Tensor(), bias, res2, Tensor(), flags);
    }
    ctx->save_for_backward({x2, weight, pre});
    ctx->saved_data["has_bias"] = bias.defined();
    ctx->saved_data["has_res"] = residual.defined();
    ctx->saved_data["gelu"] = gelu;
    ctx->saved_data["x_shape"] = x.sizes().vec();
    ctx->saved_data["x_bf16"] = x.scalar_type() == torch::kBFloat16;
    ctx->saved_data["res_f32"] = out_f32;
    Tensor y = ld != N ? out.slice(1, 0, N) : out;
    auto shape = x.sizes().vec();
    shape.back() = N;
    return y.view(shape);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("linear[bwd]", grads[0]);
    auto saved = ctx->get_saved_variables();
    Tensor x2 = saved[0], weight = saved[1], pre = saved[2];
    Tensor dy = grads[0];
    int64_t M = x2.size(0), K = x2.size(1), N = weight.size(0);
    bool has_res = ctx->saved_data["has_res"].toBool(), gelu = ctx->saved_data["gelu"].toBool();
    Tensor d_res;
    if (has_res) d_res = dy.to(ctx->saved_data["res_f32"].toBool() ? torch::kFloat32 : torch::kBFloat16);
    Tensor dy2 = dy.reshape({M, N});
    if (dy2.scalar_type() != torch::kBFloat16) dy2 = dy2.to(torch::kBFloat16);
    if (dy2.stride(-1) != 1 || dy2.stride(0) % 8 || reinterpret_cast<uintptr_t>(dy2.data_ptr()) % 16) dy2 = dy2.contiguous();
    if (gelu) {   // fold gelu'(h) into the incoming gradient with one pointwise pass
      Tensor dyc = contig(dy2), prec = contig(pre.size(1) != N ? pre.slice(1, 0, N) : pre);
      Tensor folded = torch::empty_like(dyc);
      check(itb_gelu_bwd(dyc.data_ptr(), prec.data_ptr(), folded.data_ptr(), kItbBF16, dyc.numel(), stream()), "gelu_bwd");
      dy2 = folded;
    }
    Tensor dx, dw, db;
    if (ctx->needs_input_grad(0)) {
      Tensor w = weight_lp(weight);
      Tensor dx2 = torch::empty({M, K}, dy2.options());
      gemm(dy2, false, w, true, M, K, N, dx2, Tensor(), Tensor(), Tensor(), Tensor(), 0);
      dx = dx2.view(ctx->saved_data["x_shape"].toIntVector());
      if (!ctx->saved_data["x_bf16"].toBool()) dx = dx.to(torch::kFloat32);
    }
    if (ctx->needs_input_grad(1)) {
      dw = torch::zeros({N, K}, dy2.options().dtype(torch::kFloat32));
      gemm(dy2, true, x2, true, N, K, M, dw, Tensor(), Tensor(), Tensor(), Tensor(), kGemmOutF32 | kGemmAtomic);
      if (weight.scalar_type() != torch::kFloat32) dw = dw.to(weight.scalar_type());
    }
    if (ctx->saved_data["has_bias"].toBool() && ctx->needs_input_grad(2)) {
      if (N % 8 == 0) {
        db = torch::empty({N}, dy2.options().dtype(torch::kFloat32));
        Tensor partial = torch::empty({itb_colsum_partial_rows(static_cast<int>(M)), N}, db.options());
        check(itb_colsum(dy2.data_ptr(), kItbBF16, dy2.stride(0), db.data_ptr<float>(), partial.data_ptr<float>(),
                         static_cast<int>(M), static_cast<int>(N), 0, stream()), "colsum");
      } else {
        db = dy2.to(torch::kFloat32).sum(0);
      }
    }
    return {dx, dw, db, d_res, Tensor()};
  }
};
inline Tensor linear(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& b, const c10::optional<Tensor>& r,
                     bool gelu) {
  return LinearFn::apply(x, w, b, r, gelu);
}

// ------------------------------------------------------------------ normalisation
inline torch::Dtype norm_out_dtype(const Tensor& x) {
  return (x.scalar_type() == torch::kBFloat16 || (autocast_state().enabled && autocast_state().dtype == torch::kBFloat16))
             ? torch::kBFloat16 : torch::kFloat32;
}
struct LayerNormFn : public torch::autograd::Function<LayerNormFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x, const Tensor& gamma, const c10::optional<Tensor>& beta_o,
                        double eps) {
    const Tensor beta = beta_o.value_or(Tensor());
    Tensor xc = contig(x);
    int64_t C = xc.size(-1), rows = xc.numel() / C;
    Tensor y = torch::empty(xc.sizes(), xc.options().dtype(norm_out_dtype(x)).requires_grad(false));
    Tensor mean = torch::empty({rows}, xc.options().dtype(torch::kFloat32).requires_grad(false)), rstd = torch::empty_like(mean);
    check(itb_layernorm_fwd(xc.data_ptr(), code(xc), gamma.data_ptr<float>(), beta.defined() ? beta.data_ptr<float>() : nullptr,
                            y.data_ptr(), code(y), mean.data_ptr<float>(), rstd.data_ptr<float>(), static_cast<int>(rows),
                            static_cast<int>(C), static_cast<float>(eps), stream()), "layernorm_fwd");
    ctx->save_for_backward({xc, gamma, mean, rstd});
    ctx->saved_data["has_beta"] = beta.defined();
    return y;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("layernorm[bwd]", grads[0]);
    auto s = ctx->get_saved_variables();
    Tensor x = s[0], gamma = s[1], mean = s[2], rstd = s[3];
    Tensor dy = contig(grads[0]);
    if (dy.scalar_type() == torch::kFloat32 && x.scalar_type() == torch::kBFloat16) dy = dy.to(torch::kBFloat16);
    int64_t C = x.size(-1), rows = x.numel() / C;
    Tensor dx = torch::empty_like(x);
    Tensor dg = torch::empty({C}, gamma.options().requires_grad(false)), db = torch::empty_like(dg);
    Tensor partial = torch::empty({itb_norm_partial_rows(static_cast<int>(rows)), 3 * C}, dg.options());
    check(itb_layernorm_bwd(dy.data_ptr(), code(dy), x.data_ptr(), code(x), gamma.data_ptr<float>(), mean.data_ptr<float>(),
                            rstd.data_ptr<float>(), dx.data_ptr(), code(dx), dg.data_ptr<float>(), db.data_ptr<float>(),
                            partial.data_ptr<float>(), static_cast<int>(rows), static_cast<int>(C), 0, stream()),
          "layernorm_bwd");
    return {dx, dg, ctx->saved_data["has_beta"].toBool() ? db : Tensor(), Tensor()};
  }
};
inline Tensor layernorm(const Tensor& x, const Tensor& g, const c10::optional<Tensor>& b, double eps) {
  return LayerNormFn::apply(x, g, b, eps);
}
struct RMSNormFn : public torch::autograd::Function<RMSNormFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x, const Tensor& gamma, double eps) {
    Tensor xc = contig(x);
    int64_t C = xc.size(-1), rows = xc.numel() / C;
    Tensor y = torch::empty(xc.sizes(), xc.options().dtype(norm_out_dtype(x)).requires_grad(false));
    Tensor rstd = torch::empty({rows}, xc.options().dtype(torch::kFloat32).requires_grad(false));
    check(itb_rmsnorm_fwd(xc.data_ptr(), code(xc), gamma.data_ptr<float>(), y.data_ptr(), code(y), rstd.data_ptr<float>(),
                          static_cast<int>(rows), static_cast<int>(C), static_cast<float>(eps), stream()), "rmsnorm_fwd");
    ctx->save_for_backward({xc, gamma, rstd});
    return y;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("rmsnorm[bwd]", grads[0]);
    auto s = ctx->get_saved_variables();
    Tensor x = s[0], gamma = s[1], rstd = s[2];
    Tensor dy = contig(grads[0]);
    if (dy.scalar_type() == torch::kFloat32 && x.scalar_type() == torch::kBFloat16) dy = dy.to(torch::kBFloat16);
    int64_t C = x.size(-1), rows = x.numel() / C;
    Tensor dx = torch::empty_like(x), dg = torch::empty({C}, gamma.options().requires_grad(false));
    Tensor partial = torch::empty({itb_norm_partial_rows(static_cast<int>(rows)), 3 * C}, dg.options());
    check(itb_rmsnorm_bwd(dy.data_ptr(), code(dy), x.data_ptr(), code(x), gamma.data_ptr<float>(), rstd.data_ptr<float>(),
                          dx.data_ptr(), code(dx), dg.data_ptr<float>(), partial.data_ptr<float>(), static_cast<int>(rows),
                          static_cast<int>(C), 0, stream()), "rmsnorm_bwd");
    return {dx, dg, Tensor()};
  }
};
inline Tensor rmsnorm(const Tensor& x, const Tensor& g, double eps) { return RMSNormFn::apply(x, g, eps); }

// ------------------------------------------------------------------ activations
struct GeluFn : public torch::autograd::Function<GeluFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x) {
    Tensor xc = contig(x), y = torch::empty_like(xc);
    check(itb_gelu_fwd(xc.data_ptr(), y.data_ptr(), code(xc), xc.numel(), stream()), "gelu_fwd");
    ctx->save_for_backward({xc});
    return y;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("gelu[bwd]", grads[0]);
    Tensor x = ctx->get_saved_variables()[0];
    Tensor dy = contig(grads[0].to(x.scalar_type())), dx = torch::empty_like(x);
    check(itb_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), code(x), x.numel(), stream()), "gelu_bwd");
    return {dx};
  }
};
inline Tensor gelu(const Tensor& x) { return GeluFn::apply(x); }

// out = a * silu(b) for the two column halves (a, b) of one [rows, 2F] matrix.
struct SwiGLUFn : public torch::autograd::Function<SwiGLUFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& ab) {
    int64_t F = ab.size(-1) / 2;
    Tensor ab2 = ab.reshape({-1, 2 * F});
    if (ab2.stride(-1) != 1) ab2 = ab2.contiguous();
    int64_t rows = ab2.size(0), eb = ab2.element_size();
    Tensor out = torch::empty({rows, F}, ab2.options().requires_grad(false));
    const char* base = static_cast<const char*>(ab2.data_ptr());
    check(itb_swiglu_fwd(base, base + F * eb, ab2.stride(0), out.data_ptr(), F, code(ab2), static_cast<int>(rows),
                         static_cast<int>(F), stream()), "swiglu_fwd");
    ctx->save_for_backward({ab2});
    ctx->saved_data["shape"] = ab.sizes().vec();
    auto shape = ab.sizes().vec();
    shape.back() = F;
    return out.view(shape);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("swiglu[bwd]", grads[0]);
    Tensor ab2 = ctx->get_saved_variables()[0];
    int64_t F = ab2.size(1) / 2, rows = ab2.size(0), eb = ab2.element_size();
    Tensor d2 = grads[0].reshape({-1, F}).to(ab2.scalar_type());
    if (d2.stride(-1) != 1) d2 = d2.contiguous();
    Tensor dab = torch::empty_like(ab2);
    const char* base = static_cast<const char*>(ab2.data_ptr());
    char* dbase = static_cast<char*>(dab.data_ptr());
    check(itb_swiglu_bwd(d2.data_ptr(), d2.stride(0), base, base + F * eb, ab2.stride(0), dbase, dbase + F * eb,
                         dab.stride(0), code(ab2), static_cast<int>(rows), static_cast<int>(F), stream()), "swiglu_bwd");
    return {dab.view(ctx->saved_data["shape"].toIntVector())};
  }
};
inline Tensor swiglu_packed(const Tensor& ab) { return SwiGLUFn::apply(ab); }

// ------------------------------------------------------------------ attention
// Causal flash attention on a packed [B, T, (H + 2 KV) D] bf16 projection, RoPE applied in place to
// the q and k heads first and un-applied on their gradients.
struct AttentionFn : public torch::autograd::Function<AttentionFn> {
  static void fill(ItbAttnArgs* a, const Tensor& qkv, const Tensor& o, const Tensor& lse, int64_t H, int64_t KV, int64_t D,
                   bool causal) {
    const char* base = static_cast<const char*>(qkv.data_ptr());
    a->q = base, a->k = base + 2 * H * D, a->v = base + 2 * (H + KV) * D;
    a->o = o.data_ptr(), a->lse = lse.data_ptr<float>();
    a->q_row_stride = a->k_row_stride = a->v_row_stride = qkv.stride(1);
    a->q_batch_stride = a->k_batch_stride = a->v_batch_stride = qkv.stride(0);
    a->o_row_stride = H * D, a->o_batch_stride = qkv.size(1) * H * D;
    a->B = static_cast<int>(qkv.size(0)), a->T = static_cast<int>(qkv.size(1));
    a->H = static_cast<int>(H), a->KV = static_cast<int>(KV), a->D = static_cast<int>(D);
    a->scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(D)));
    a->causal = causal;
  }
  static Tensor forward(AutogradContext* ctx, const Tensor& qkv_in, int64_t H, int64_t KV, int64_t D,
                        const c10::optional<Tensor>& freqs_o, int64_t pos0, bool causal) {
    const Tensor freqs = freqs_o.value_or(Tensor());
    Tensor qkv = qkv_in.scalar_type() == torch::kBFloat16 ? qkv_in : qkv_in.to(torch::kBFloat16);
    int64_t B = qkv.size(0), T = qkv.size(1);
    if (!qkv.is_contiguous()) qkv = qkv.contiguous();
    if (freqs.defined())
      check(itb_rope_inplace(qkv.data_ptr(), kItbBF16, freqs.data_ptr<float>(), static_cast<int>(B), static_cast<int>(T),
                             static_cast<int>(H + KV), static_cast<int>(D), qkv.stride(1), static_cast<int>(pos0), 0, stream()),
            "rope");
    Tensor o = torch::empty({B, T, H, D}, qkv.options().requires_grad(false));
    Tensor lse = torch::empty({B, H, T}, qkv.options().dtype(torch::kFloat32).requires_grad(false));
    ItbAttnArgs a{};
    fill(&a, qkv, o, lse, H, KV, D, causal);
    check(itb_flash_attn_fwd_tc(&a, status_word(qkv.device().index()).data_ptr<int>(), stream()), "flash_attn_fwd_tc");
    ctx->save_for_backward({qkv, o, lse, freqs});
    ctx->saved_data["meta"] = std::vector<int64_t>{H, KV, D, pos0, causal};
    return o.view({B, T, H * D});
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("attention_packed[bwd]", grads[0]);
    auto s = ctx->get_saved_variables();
    Tensor qkv = s[0], o = s[1], lse = s[2], freqs = s[3];
    auto meta = ctx->saved_data["meta"].toIntVector();
    int64_t H = meta[0], KV = meta[1], D = meta[2], pos0 = meta[3];
    int64_t B = qkv.size(0), T = qkv.size(1);
    Tensor dqkv = torch::empty_like(qkv);
    Tensor dout = grads[0].reshape({B, T, H, D});
    if (dout.scalar_type() != torch::kBFloat16) dout = dout.to(torch::kBFloat16);
    dout = contig(dout);
    Tensor delta = torch::empty({B, H, T}, lse.options());
    Tensor dq_accum = torch::empty({B, T, H, D}, lse.options());
    ItbAttnArgs a{};
    fill(&a, qkv, o, lse, H, KV, D, meta[4] != 0);
    char* dbase = static_cast<char*>(dqkv.data_ptr());
    a.dout = dout.data_ptr();
    a.dq = dbase, a.dk = dbase + 2 * H * D, a.dv = dbase + 2 * (H + KV) * D;
    a.delta = delta.data_ptr<float>(), a.dq_accum = dq_accum.data_ptr<float>();
    Tensor dkv_accum;   // few key tiles and KV heads: several CTAs share a key tile and sum dK / dV here
    if (itb_flash_attn_bwd_parts(a.B, a.T, a.H, a.KV, a.causal) > 1) {
      dkv_accum = torch::empty({2, B, T, KV, D}, lse.options());
      a.dkv_accum = dkv_accum.data_ptr<float>();
    }
    check(itb_flash_attn_bwd_tc(&a, status_word(qkv.device().index()).data_ptr<int>(), stream()), "flash_attn_bwd_tc");
    if (freqs.defined())
      check(itb_rope_inplace(dqkv.data_ptr(), kItbBF16, freqs.data_ptr<float>(), static_cast<int>(B), static_cast<int>(T),
                             static_cast<int>(H + KV), static_cast<int>(D), dqkv.stride(1), static_cast<int>(pos0), 1, stream()),
            "rope_inverse");
    return {dqkv, Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};
inline Tensor attention_packed(const Tensor& qkv, int64_t H, int64_t KV, int64_t D, const c10::optional<Tensor>& freqs,
                               int64_t pos0, bool causal) {
  return AttentionFn::apply(qkv, H, KV, D, freqs, pos0, causal);
}

// ------------------------------------------------------------------ embedding
struct EmbeddingFn : public torch::autograd::Function<EmbeddingFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& idx_in, const Tensor& wte, const c10::optional<Tensor>& wpe_o,
                        int64_t pos0) {
    const Tensor wpe = wpe_o.value_or(Tensor());
    Tensor idx = contig(idx_in);
    int64_t B = idx.size(0), T = idx.size(1), C = wte.size(1);
    bool lp = autocast_state().enabled && autocast_state().dtype == torch::kBFloat16;
    Tensor out = torch::empty({B, T, C}, wte.options().dtype(lp ? torch::kBFloat16 : torch::kFloat32).requires_grad(false));
    check(itb_embedding_fwd(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), wte.data_ptr(),
                            wpe.defined() ? wpe.data_ptr() : nullptr, kItbF32, out.data_ptr(), code(out), static_cast<int>(B),
                            static_cast<int>(T), static_cast<int>(C), static_cast<int>(pos0), 0, static_cast<int>(wte.size(0)),
                            stream()), "embedding_fwd");
    ctx->save_for_backward({idx, wte, wpe});
    ctx->saved_data["pos0"] = pos0;
    return out;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("embedding[bwd]", grads[0]);
    auto s = ctx->get_saved_variables();
    Tensor idx = s[0], wte = s[1], wpe = s[2];
    Tensor dout = contig(grads[0]);
    int64_t B = idx.size(0), T = idx.size(1), C = wte.size(1);
    Tensor dwte = torch::zeros_like(wte), dwpe = wpe.defined() ? torch::zeros_like(wpe) : Tensor();
    check(itb_embedding_bwd(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), dout.data_ptr(), code(dout),
                            dwte.data_ptr<float>(), dwpe.defined() ? dwpe.data_ptr<float>() : nullptr, static_cast<int>(B),
                            static_cast<int>(T), static_cast<int>(C), static_cast<int>(ctx->saved_data["pos0"].toInt()), 0,
                            static_cast<int>(wte.size(0)), stream()), "embedding_bwd");
    return {Tensor(), dwte, dwpe, Tensor()};
  }
};
inline Tensor embedding(const Tensor& idx, const Tensor& wte, const c10::optional<Tensor>& wpe, int64_t pos0) {
  return EmbeddingFn::apply(idx, wte, wpe, pos0);
}

// ------------------------------------------------------------------ cross entropy
// Mean softmax cross-entropy; the backward pass overwrites the logits buffer with the gradient.
struct CrossEntropyFn : public torch::autograd::Function<CrossEntropyFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& logits, const Tensor& target) {
    int64_t V = logits.size(-1);
    Tensor l2 = logits.reshape({-1, V});
    if (l2.stride(-1) != 1) l2 = l2.contiguous();
    Tensor t = contig(target.reshape({-1}));
    int64_t rows = l2.size(0);
    auto f32 = l2.options().dtype(torch::kFloat32).requires_grad(false);
    Tensor row_loss = torch::empty({rows}, f32), lse = torch::empty({rows}, f32), loss = torch::zeros({1}, f32);
    check(itb_ce_fwd(l2.data_ptr(), code(l2), l2.stride(0), reinterpret_cast<const long long*>(t.data_ptr<int64_t>()),
                     row_loss.data_ptr<float>(), lse.data_ptr<float>(), loss.data_ptr<float>(), static_cast<int>(rows),
                     static_cast<int>(V), stream()), "ce_fwd");
    ctx->save_for_backward({l2, t, lse});
    ctx->saved_data["shape"] = logits.sizes().vec();
    return loss.reshape({});
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    ITB_PROFILE("cross_entropy[bwd]", grads[0]);
    auto s = ctx->get_saved_variables();
    Tensor l2 = s[0], t = s[1], lse = s[2];
    Tensor g = grads[0].reshape({1}).to(torch::kFloat32);
    check(itb_ce_bwd(l2.data_ptr(), code(l2), l2.stride(0), reinterpret_cast<const long long*>(t.data_ptr<int64_t>()),
                     lse.data_ptr<float>(), g.data_ptr<float>(), static_cast<int>(l2.size(0)), static_cast<int>(l2.size(1)), 1,
                     stream()), "ce_bwd");
    return {l2.view(ctx->saved_data["shape"].toIntVector()), Tensor()};
  }
};
inline Tensor cross_entropy(const Tensor& logits, const Tensor& target) { return CrossEntropyFn::apply(logits, target); }

}  // namespace fused
}  // namespace ops
}  // namespace itb
