// The generic Transformer of the C++ frontend, instantiated as GPT-2 or LLaMA-3 by its config
// (reference: infini_train/include/nn/modules/transformer/transformer_config.h:23-61 and
// src/nn/modules/transformer/{causal_self_attention,mlp,transformer}.cc).  State-dict names follow the
// reference's layout (transformer.wte.weight, transformer.h.<i>.attn.c_attn.weight, ..., lm_head.weight),
// so weight files, checkpoints and LoRA targets carry over.
#pragma once
#include "layers.h"
#include "precision.h"

namespace itb {
namespace nn {

enum class AttentionType { kStandard, kRoPE };
enum class MLPType { kGELU, kSwiGLU };
enum class NormType { kLayerNorm, kRMSNorm };

struct TransformerConfig {
  int64_t block_size = 1024, vocab_size = 50304, original_vocab_size = 50257;
  int64_t n_layer = 12, n_head = 12, n_kv_head = 12, n_embd = 768;
  AttentionType attention_type = AttentionType::kStandard;
  MLPType activation_type = MLPType::kGELU;
  NormType norm_type = NormType::kLayerNorm;
  bool add_bias_linear = true, add_bias_lm_head = false, tie_weights = true;
  double ffn_expansion_ratio = 4.0;
  c10::optional<double> ffn_dim_multiplier = c10::nullopt;
  int64_t multiple_of = 1;
  double rope_theta = 500000.0, norm_eps = 1e-5;
  bool use_scaled_rope = false;
  int64_t max_gen_batch_size = 4;

  bool UseGQA() const { return n_kv_head < n_head; }
  int64_t head_dim() const { return n_embd / n_head; }
  // MLP width (reference: src/nn/modules/transformer/mlp.cc:24-38)
  int64_t ffn_hidden() const {
    int64_t h = static_cast<int64_t>(n_embd * ffn_expansion_ratio);
    if (activation_type == MLPType::kSwiGLU) h = 2 * h / 3;
    if (ffn_dim_multiplier.has_value()) h = static_cast<int64_t>(std::llround(h * *ffn_dim_multiplier));
    return (h + multiple_of - 1) / multiple_of * multiple_of;
  }
  static TransformerConfig GPT2() {
    TransformerConfig c;
    c.vocab_size = 50257;
    return c;
  }
  static TransformerConfig LLaMA3() {   // the 1B shape
    TransformerConfig c;
    c.block_size = 8192, c.vocab_size = c.original_vocab_size = 128256;
    c.n_layer = 16, c.n_head = 32, c.n_kv_head = 8, c.n_embd = 2048;
    c.attention_type = AttentionType::kRoPE, c.activation_type = MLPType::kSwiGLU, c.norm_type = NormType::kRMSNorm;
    c.add_bias_linear = false, c.tie_weights = false;
    c.ffn_dim_multiplier = 1.5, c.multiple_of = 256;
    return c;
  }
};

inline std::shared_ptr<Module> MakeNorm(const TransformerConfig& c) {
  if (c.norm_type == NormType::kLayerNorm) return std::make_shared<LayerNorm>(c.n_embd);
  return std::make_shared<RMSNorm>(c.n_embd, c.norm_eps);
}

class CausalSelfAttention : public Module {
 public:
  explicit CausalSelfAttention(const TransformerConfig& c) : Module("CausalSelfAttention"), config(c) {
    TORCH_CHECK(c.n_embd % c.n_head == 0, "n_embd must be divisible by n_head");
    TORCH_CHECK(c.n_head % c.n_kv_head == 0, "n_head must be divisible by n_kv_head");
    int64_t D = c.head_dim();
    register_module("c_attn", std::make_shared<Linear>(c.n_embd, (c.n_head + 2 * c.n_kv_head) * D, c.add_bias_linear));
    register_module("c_proj", std::make_shared<Linear>(c.n_embd, c.n_embd, c.add_bias_linear));
  }
  // children are looked up by name on every call, so a wrapper put in their place (LoRA) takes over
  std::shared_ptr<Linear> linear(const char* name) const { return std::static_pointer_cast<Linear>(mutable_module(name)); }
  // in: x, [freqs_cis]; residual is added in the projection's epilogue
  Tensor forward(const Tensor& x, const c10::optional<Tensor>& freqs, const c10::optional<Tensor>& residual) {
    if (utils::aligned_mode()) {   // through the children's call operators, so that their hooks see the tensors
      Tensor qkv = (*mutable_module("c_attn"))(x);
      auto rope = config.attention_type == AttentionType::kRoPE ? freqs : c10::nullopt;
      Tensor y = (*mutable_module("c_proj"))(ops::attention_packed(qkv, config.n_head, config.n_kv_head, config.head_dim(), rope, 0, true));
      return residual.has_value() ? y + *residual : y;
    }
    Tensor qkv = linear("c_attn")->forward(x);
    auto rope = config.attention_type == AttentionType::kRoPE ? freqs : c10::nullopt;
    Tensor y = ops::attention_packed(qkv, config.n_head, config.n_kv_head, config.head_dim(), rope, 0, true);
    return linear("c_proj")->forward(y, residual);
  }
  TensorList Forward(const TensorList& in) override {
    return {forward(in[0], in.size() > 1 ? c10::optional<Tensor>(in[1]) : c10::nullopt, c10::nullopt)};
  }
  TransformerConfig config;
};

class MLP : public Module {
 public:
  explicit MLP(const TransformerConfig& c) : Module("MLP"), config(c) {
    int64_t hidden = c.ffn_hidden();
    register_module("c_fc", std::make_shared<Linear>(c.n_embd, hidden, c.add_bias_linear));
    if (c.activation_type == MLPType::kSwiGLU)
      register_module("c_fc2", std::make_shared<Linear>(c.n_embd, hidden, c.add_bias_linear));
    register_module("c_proj", std::make_shared<Linear>(hidden, c.n_embd, c.add_bias_linear));
    // activation modules under the reference's names; the fused path does not go through them
    if (c.activation_type == MLPType::kSwiGLU) register_module("silu", std::make_shared<SwiGLU>());
    else register_module("gelu", std::make_shared<NewGELU>());
  }
  std::shared_ptr<Linear> linear(const char* name) const { return std::static_pointer_cast<Linear>(mutable_module(name)); }
  Tensor forward(const Tensor& x, const c10::optional<Tensor>& residual) {
    if (utils::aligned_mode()) {
      Tensor h;
      if (config.activation_type == MLPType::kSwiGLU)
        h = (*mutable_module("c_fc"))(x) * (*mutable_module("silu"))((*mutable_module("c_fc2"))(x));
      else
        h = (*mutable_module("gelu"))((*mutable_module("c_fc"))(x));
      Tensor y = (*mutable_module("c_proj"))(h);
      return residual.has_value() ? y + *residual : y;
    }
    if (config.activation_type == MLPType::kSwiGLU)
      return linear("c_proj")->forward(ops::swiglu(linear("c_fc")->forward(x), linear("c_fc2")->forward(x)), residual);
    return linear("c_proj")->forward(linear("c_fc")->forward(x, c10::nullopt, /*gelu=*/true), residual);
  }
  TensorList Forward(const TensorList& in) override { return {forward(in[0], c10::nullopt)}; }
  TransformerConfig config;
};

// Pre-norm residual block: x + attn(ln_1(x)), then x + mlp(ln_2(x)).
class TransformerLayer : public Module {
 public:
  explicit TransformerLayer(const TransformerConfig& c) : Module("Layer") {   // the reference's type name
    ln_1 = register_module("ln_1", MakeNorm(c));
    attn = register_module("attn", std::make_shared<CausalSelfAttention>(c));
    ln_2 = register_module("ln_2", MakeNorm(c));
    mlp = register_module("mlp", std::make_shared<MLP>(c));
  }
  Tensor forward(const Tensor& x, const c10::optional<Tensor>& freqs) {
    if (utils::aligned_mode()) {
      TensorList a_in = {(*ln_1)(x)};
      if (freqs.has_value()) a_in.push_back(*freqs);
      Tensor h = x + (*attn)(a_in)[0];
      return h + (*mlp)(TensorList{(*ln_2)(h)})[0];
    }
    Tensor h = attn->forward((*ln_1)(x), freqs, x);
    return mlp->forward((*ln_2)(h), h);
  }
  TensorList Forward(const TensorList& in) override {
    return {forward(in[0], in.size() > 1 ? c10::optional<Tensor>(in[1]) : c10::nullopt)};
  }
  std::shared_ptr<Module> ln_1, ln_2;
  std::shared_ptr<CausalSelfAttention> attn;
  std::shared_ptr<MLP> mlp;
};

class TransformerModel : public Module {
 public:
  explicit TransformerModel(const TransformerConfig& c) : Module("Transformer"), config(c) {   // the reference's type name
    auto body = std::make_shared<ModuleDict>();
    wte = std::make_shared<Embedding>(c.vocab_size, c.n_embd);
    body->insert("wte", wte);
    if (c.attention_type == AttentionType::kStandard) {
      wpe = std::make_shared<Embedding>(c.block_size, c.n_embd);
      body->insert("wpe", wpe);
    }
    h = std::make_shared<ModuleList>();
    for (int64_t i = 0; i < c.n_layer; ++i) h->push_back(std::make_shared<TransformerLayer>(c));
    body->insert("h", h);
    ln_f = MakeNorm(c);
    body->insert("ln_f", ln_f);
    register_module("transformer", body);
    register_module("lm_head", std::make_shared<Linear>(c.n_embd, c.vocab_size, c.add_bias_lm_head));
    if (c.tie_weights) wte->tie(lm_head()->weight);   // one tensor serves the lookup and the projection
  }
  // idx [B, T] int64 -> logits [B, T, vocab]
  Tensor forward(const Tensor& idx) {
    int64_t T = idx.size(1);
    TORCH_CHECK(T <= config.block_size, "sequence longer than block_size");
    const bool aligned = utils::aligned_mode();
    Tensor x;
    if (aligned) {
      x = (*wte)(idx);
      if (wpe) x = x + (*wpe)(torch::arange(T, torch::TensorOptions().dtype(torch::kInt64).device(idx.device())));
    } else {
      x = ops::embedding(idx, wte->weight, wpe ? c10::optional<Tensor>(wpe->weight) : c10::nullopt, 0);
    }
    c10::optional<Tensor> freqs;
    if (config.attention_type == AttentionType::kRoPE) {
      if (!freqs_cis_.defined() || freqs_cis_.device() != x.device())
        freqs_cis_ = ops::precompute_freqs_cis(config.head_dim(), 2 * config.block_size, config.rope_theta, x.device());
      freqs = freqs_cis_.slice(0, 0, T);
    }
    if (aligned) {
      for (auto& layer : *h) {
        TensorList in = {x};
        if (freqs.has_value()) in.push_back(*freqs);
        x = (*layer)(in)[0];
      }
      return (*mutable_module("lm_head"))((*ln_f)(x));
    }
    for (auto& layer : *h) x = std::static_pointer_cast<TransformerLayer>(layer)->forward(x, freqs);
    return lm_head()->forward((*ln_f)(x));
  }
  TensorList Forward(const TensorList& in) override { return {forward(in[0])}; }

  TransformerConfig config;
  std::shared_ptr<Embedding> wte, wpe;
  std::shared_ptr<ModuleList> h;
  std::shared_ptr<Module> ln_f;
  std::shared_ptr<Linear> lm_head() const { return std::static_pointer_cast<Linear>(mutable_module("lm_head")); }

 private:
  Tensor freqs_cis_;
};

}  // namespace nn
}  // namespace itb
