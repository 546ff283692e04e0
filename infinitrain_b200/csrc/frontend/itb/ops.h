// Functional ops of the C++ frontend.
//
// Every op has one entry point.  On a CUDA tensor under bf16 autocast (or on bf16 activations) it runs
// this library's sm_100a kernels through the fused autograd functions of ops_fused.h (compiled in with
// -DITB_WITH_CUDA and linked against _C.so); anywhere else it is the plain libtorch formulation, which
// is also the fp32 oracle.  Math follows the reference's kernels: tanh GELU
// (src/nn/modules/activations.cc:15-19), gate order c_fc(x) * silu(c_fc2(x))
// (src/nn/modules/transformer/mlp.cc:84-90), interleaved-pair RoPE
// (src/nn/modules/transformer/utils.cc:9-29), mean cross-entropy (src/kernels/cpu/cross_entropy.cc:17-98).
#pragma once
#include <functional>
#include <cmath>

#include "module.h"
#include "profiler.h"

namespace itb {

// Thread-local autocast state (reference: include/autocast.h: Linear / Matmul run in the low-precision
// type, normalisation and the loss in fp32).
struct AutocastState {
  bool enabled = false;
  torch::Dtype dtype = torch::kBFloat16;
};
inline AutocastState& autocast_state() {
  static thread_local AutocastState s;
  return s;
}
class AutocastGuard {
 public:
  AutocastGuard(torch::Dtype dtype, bool enabled = true) : prev_(autocast_state()) {
    autocast_state().enabled = enabled && dtype != torch::kFloat32;
    autocast_state().dtype = dtype;
  }
  ~AutocastGuard() { autocast_state() = prev_; }

 private:
  AutocastState prev_;
};

namespace ops {

// Function-level observation (the precision checker's level 2): when a hook is installed, every op below
// reports its tensor arguments and its result once per call; an op that calls another op reports for itself only.
using FunctionHook = std::function<void(const char* name, const TensorList& inputs, const Tensor& output)>;
inline FunctionHook& function_hook() {
  static FunctionHook h;
  return h;
}
inline bool& inside_function_hook() {
  static thread_local bool inside = false;
  return inside;
}
inline bool function_hook_wanted() { return static_cast<bool>(function_hook()) && !inside_function_hook(); }
struct FunctionHookScope {
  FunctionHookScope() { inside_function_hook() = true; }
  ~FunctionHookScope() { inside_function_hook() = false; }
};
inline Tensor report_function(const char* name, const TensorList& inputs, const Tensor& output) {
  function_hook()(name, inputs, output);
  return output;
}
inline Tensor or_undefined(const c10::optional<Tensor>& t) { return t.has_value() ? *t : Tensor(); }
// Runs `call` with the hook off and reports (name, inputs, result).
#define ITB_FUNCTION_HOOK(name, inputs, call)                                  \
  if (::itb::ops::function_hook_wanted()) {                                     \
    ::itb::Tensor itb_hook_out;                                                 \
    {                                                                           \
      ::itb::ops::FunctionHookScope itb_hook_scope;                             \
      itb_hook_out = (call);                                                    \
    }                                                                           \
    return ::itb::ops::report_function(name, inputs, itb_hook_out);            \
  }

inline bool use_fused(const Tensor& x) {
#ifdef ITB_WITH_CUDA
  return x.is_cuda() && (x.scalar_type() == torch::kBFloat16 ||
                         (autocast_state().enabled && autocast_state().dtype == torch::kBFloat16));
#else
  (void)x;
  return false;
#endif
}

}  // namespace ops
}  // namespace itb

#ifdef ITB_WITH_CUDA
#include "ops_fused.h"
#endif

namespace itb {
namespace ops {

inline Tensor new_gelu(const Tensor& x) {
  const double k = std::sqrt(2.0 / M_PI);
  return 0.5 * x * (1.0 + torch::tanh(k * (x + 0.044715 * x.pow(3))));
}

// y = x W^T (+ bias) (+ gelu) (+ residual)
inline Tensor linear(const Tensor& x, const Tensor& weight, const c10::optional<Tensor>& bias = c10::nullopt,
                     const c10::optional<Tensor>& residual = c10::nullopt, bool gelu = false) {
  ITB_FUNCTION_HOOK("Linear", (TensorList{x, weight, or_undefined(bias), or_undefined(residual)}), ::itb::ops::linear(x, weight, bias, residual, gelu));
  ITB_PROFILE("linear", x);
#ifdef ITB_WITH_CUDA
  if (use_fused(x) && x.size(-1) % 8 == 0 && weight.is_cuda()) return fused::linear(x, weight, bias, residual, gelu);
#endif
  Tensor y;
  if (autocast_state().enabled && x.scalar_type() == torch::kFloat32 && !x.is_cuda()) {
    // CPU emulation of the autocast of Linear: operands rounded to the low-precision type, fp32 accumulate
    auto lp = autocast_state().dtype;
    y = torch::linear(x.to(lp).to(torch::kFloat32), weight.to(lp).to(torch::kFloat32),
                      bias.has_value() ? *bias : Tensor());
  } else {
    y = torch::linear(x, weight.to(x.scalar_type()), bias.has_value() ? bias->to(x.scalar_type()) : Tensor());
  }
  if (gelu) y = new_gelu(y);
  if (residual.has_value()) y = y + *residual;
  return y;
}

inline Tensor layernorm(const Tensor& x, const Tensor& gamma, const c10::optional<Tensor>& beta, double eps = 1e-5) {
  ITB_FUNCTION_HOOK("LayerNorm", (TensorList{x, gamma, or_undefined(beta)}), ::itb::ops::layernorm(x, gamma, beta, eps));
  ITB_PROFILE("layernorm", x);
#ifdef ITB_WITH_CUDA
  if (x.is_cuda() && gamma.scalar_type() == torch::kFloat32 && x.size(-1) % 8 == 0 && x.size(-1) <= 6144)
    return fused::layernorm(x, gamma, beta, eps);
#endif
  auto xf = x.to(torch::kFloat32);
  auto mean = xf.mean(-1, true);
  auto var = (xf - mean).pow(2).mean(-1, true);          // two-pass variance in fp32
  auto y = (xf - mean) * torch::rsqrt(var + eps) * gamma;
  if (beta.has_value()) y = y + *beta;
  return y.to(x.scalar_type());
}

inline Tensor rmsnorm(const Tensor& x, const Tensor& gamma, double eps = 1e-6) {
  ITB_FUNCTION_HOOK("RMSNorm", (TensorList{x, gamma}), ::itb::ops::rmsnorm(x, gamma, eps));
  ITB_PROFILE("rmsnorm", x);
#ifdef ITB_WITH_CUDA
  if (x.is_cuda() && gamma.scalar_type() == torch::kFloat32 && x.size(-1) % 8 == 0 && x.size(-1) <= 6144)
    return fused::rmsnorm(x, gamma, eps);
#endif
  auto xf = x.to(torch::kFloat32);
  return (xf * torch::rsqrt(xf.pow(2).mean(-1, true) + eps) * gamma).to(x.scalar_type());
}

inline Tensor gelu(const Tensor& x) {
  ITB_FUNCTION_HOOK("Gelu", (TensorList{x}), ::itb::ops::gelu(x));
  ITB_PROFILE("gelu", x);
#ifdef ITB_WITH_CUDA
  if (x.is_cuda() && (x.scalar_type() == torch::kFloat32 || x.scalar_type() == torch::kBFloat16))
    return fused::gelu(x);
#endif
  return new_gelu(x);
}

inline Tensor swiglu(const Tensor& a, const Tensor& b) {
  ITB_FUNCTION_HOOK("SwiGLU", (TensorList{a, b}), ::itb::ops::swiglu(a, b));
  ITB_PROFILE("swiglu", a);
#ifdef ITB_WITH_CUDA
  if (a.is_cuda() && a.size(-1) % 8 == 0 && (a.scalar_type() == torch::kFloat32 || a.scalar_type() == torch::kBFloat16))
    return fused::swiglu_packed(torch::cat({a, b}, -1));
#endif
  return a * (b * torch::sigmoid(b));
}

// [end, head_dim / 2, 2] table of (cos, sin).
inline Tensor precompute_freqs_cis(int64_t head_dim, int64_t end, double theta = 10000.0,
                                   torch::Device device = torch::kCPU) {
  auto opt = torch::TensorOptions().dtype(torch::kFloat32).device(device);
  auto inv = 1.0 / torch::pow(theta, torch::arange(0, head_dim, 2, opt) / static_cast<double>(head_dim));
  auto ang = torch::outer(torch::arange(end, opt), inv);
  return torch::stack({ang.cos(), ang.sin()}, -1).contiguous();
}

// x [B, T, H, D] with interleaved (even, odd) pairs.
inline Tensor apply_rope(const Tensor& x, const Tensor& freqs, int64_t pos0 = 0) {
  ITB_PROFILE("apply_rope", x);
  auto B = x.size(0), T = x.size(1), H = x.size(2), D = x.size(3);
  auto xf = x.to(torch::kFloat32).reshape({B, T, H, D / 2, 2});
  auto f = freqs.slice(0, pos0, pos0 + T);
  auto c = f.select(-1, 0).view({1, T, 1, D / 2}), s = f.select(-1, 1).view({1, T, 1, D / 2});
  auto x0 = xf.select(-1, 0), x1 = xf.select(-1, 1);
  return torch::stack({x0 * c - x1 * s, x0 * s + x1 * c}, -1).reshape({B, T, H, D}).to(x.scalar_type());
}

// Causal self-attention on a packed projection [B, T, (H + 2 KV) D] -> [B, T, H D]; softmax in fp32,
// grouped-query attention by repeating the KV heads.
inline Tensor attention_packed(const Tensor& qkv, int64_t H, int64_t KV, int64_t D,
                               const c10::optional<Tensor>& freqs = c10::nullopt, int64_t pos0 = 0,
                               bool causal = true) {
  ITB_FUNCTION_HOOK("Attention", (TensorList{qkv}), ::itb::ops::attention_packed(qkv, H, KV, D, freqs, pos0, causal));
  ITB_PROFILE("attention_packed", qkv);
#ifdef ITB_WITH_CUDA
  if (qkv.is_cuda() && (D == 64 || D == 128) && use_fused(qkv))
    return fused::attention_packed(qkv, H, KV, D, freqs, pos0, causal);
#endif
  auto B = qkv.size(0), T = qkv.size(1);
  auto q = qkv.slice(-1, 0, H * D).reshape({B, T, H, D});
  auto k = qkv.slice(-1, H * D, (H + KV) * D).reshape({B, T, KV, D});
  auto v = qkv.slice(-1, (H + KV) * D, (H + 2 * KV) * D).reshape({B, T, KV, D});
  if (freqs.has_value()) {
    q = apply_rope(q, *freqs, pos0);
    k = apply_rope(k, *freqs, pos0);
  }
  auto qf = q.to(torch::kFloat32), kf = k.to(torch::kFloat32), vf = v.to(torch::kFloat32);
  if (KV != H) {
    kf = kf.repeat_interleave(H / KV, 2);
    vf = vf.repeat_interleave(H / KV, 2);
  }
  auto s = torch::einsum("bthd,bshd->bhts", {qf, kf}) * (1.0 / std::sqrt(static_cast<double>(D)));
  if (causal) {
    auto mask = torch::ones({T, T}, torch::TensorOptions().dtype(torch::kBool).device(qkv.device())).tril();
    s = s.masked_fill(mask.logical_not(), -std::numeric_limits<float>::infinity());
  }
  auto p = s.softmax(-1);
  return torch::einsum("bhts,bshd->bthd", {p, vf}).to(qkv.scalar_type()).reshape({B, T, H * D});
}

// Token (+ position) embedding.
inline Tensor embedding(const Tensor& idx, const Tensor& wte, const c10::optional<Tensor>& wpe = c10::nullopt,
                        int64_t pos0 = 0) {
  ITB_FUNCTION_HOOK("Embedding", (TensorList{wte, or_undefined(wpe)}), ::itb::ops::embedding(idx, wte, wpe, pos0));
  ITB_PROFILE("embedding", idx);
#ifdef ITB_WITH_CUDA
  if (wte.is_cuda() && wte.scalar_type() == torch::kFloat32 && wte.size(1) % 8 == 0 && idx.dim() == 2)
    return fused::embedding(idx, wte, wpe, pos0);
#endif
  auto out = torch::embedding(wte, idx);
  if (wpe.has_value()) out = out + wpe->slice(0, pos0, pos0 + idx.size(1));
  return out;
}

// Mean cross-entropy over all rows, statistics in fp32.
// Mean over rows of -log softmax(logits)[target]; targets are class indices as int64 or as uint8 (the
// reference's loss takes both, src/kernels/cpu/cross_entropy.cc).
inline Tensor cross_entropy(const Tensor& logits, const Tensor& target_in) {
  ITB_FUNCTION_HOOK("CrossEntropy", (TensorList{logits}), ::itb::ops::cross_entropy(logits, target_in));
  ITB_PROFILE("cross_entropy", logits);
  const Tensor target = target_in.scalar_type() == torch::kLong ? target_in : target_in.to(torch::kLong);
#ifdef ITB_WITH_CUDA
  if (logits.is_cuda() && (logits.scalar_type() == torch::kFloat32 || logits.scalar_type() == torch::kBFloat16))
    return fused::cross_entropy(logits, target);
#endif
  auto l2 = logits.to(torch::kFloat32).reshape({-1, logits.size(-1)});
  return torch::nll_loss(torch::log_softmax(l2, -1), target.reshape({-1}));
}

}  // namespace ops
}  // namespace itb
