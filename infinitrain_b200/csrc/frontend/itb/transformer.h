// The generic Transformer of the C++ frontend, instantiated as GPT-2 or LLaMA-3 by its config
// (reference: infini_train/include/nn/modules/transformer/transformer_config.h:23-61 and
// src/nn/modules/transformer/{causal_self_attention,mlp,transformer}.cc).  State-dict names follow the
// reference's layout (transformer.wte.weight, transformer.h.<i>.attn.c_attn.weight, ..., lm_head.weight),
// so weight files, checkpoints and LoRA targets carry over.
#pragma once
#include "layers.h"
#include "precision.h"
#include "tensor_parallel.h"

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

// Every linear of the Transformer is a tensor-parallel layer that degrades to a plain Linear with one
// tensor-parallel rank (reference: tensor_parallel.cc:31-34, causal_self_attention.cc:21-75).
inline std::shared_ptr<Linear> MakeColumnLinear(int64_t in, int64_t out, bool bias) {
  if (parallel::env().tp() == 1) return std::make_shared<Linear>(in, out, bias);
  return std::make_shared<parallel::ColumnParallelLinear>(in, out, bias, /*gather_output=*/false, /*input_is_parallel=*/false,
                                                          /*skip_bias_add=*/false, parallel::env().sequence_parallel);
}
inline std::shared_ptr<Linear> MakeRowLinear(int64_t in, int64_t out, bool bias) {
  if (parallel::env().tp() == 1) return std::make_shared<Linear>(in, out, bias);
  return std::make_shared<parallel::RowParallelLinear>(in, out, bias, /*reduce_output=*/true, /*input_is_parallel=*/true,
                                                       /*skip_bias_add=*/false, parallel::env().sequence_parallel);
}

class CausalSelfAttention : public Module {
 public:
  explicit CausalSelfAttention(const TransformerConfig& c) : Module("CausalSelfAttention"), config(c) {
    TORCH_CHECK(c.n_embd % c.n_head == 0, "n_embd must be divisible by n_head");
    TORCH_CHECK(c.n_head % c.n_kv_head == 0, "n_head must be divisible by n_kv_head");
    const int64_t D = c.head_dim(), tp = parallel::env().tp();
    TORCH_CHECK(c.n_head % tp == 0 && c.n_kv_head % tp == 0, "head counts must be divisible by the tensor-parallel size");
    local_heads = c.n_head / tp, local_kv_heads = c.n_kv_head / tp;
    register_module("c_attn", MakeColumnLinear(c.n_embd, (c.n_head + 2 * c.n_kv_head) * D, c.add_bias_linear));
    register_module("c_proj", MakeRowLinear(c.n_embd, c.n_embd, c.add_bias_linear));
  }
  int64_t local_heads = 0, local_kv_heads = 0;   // heads of this tensor-parallel rank (the fused QKV rows are [q_r | k_r | v_r])
  // children are looked up by name on every call, so a wrapper put in their place (LoRA) takes over
  std::shared_ptr<Linear> linear(const char* name) const { return std::static_pointer_cast<Linear>(mutable_module(name)); }
  // in: x, [freqs_cis]; residual is added in the projection's epilogue
  Tensor forward(const Tensor& x, const c10::optional<Tensor>& freqs, const c10::optional<Tensor>& residual) {
    if (utils::aligned_mode()) {   // through the children's call operators, so that their hooks see the tensors
      Tensor qkv = (*mutable_module("c_attn"))(x);
      auto rope = config.attention_type == AttentionType::kRoPE ? freqs : c10::nullopt;
      Tensor y = (*mutable_module("c_proj"))(ops::attention_packed(qkv, local_heads, local_kv_heads, config.head_dim(), rope, 0, true));
      return residual.has_value() ? y + *residual : y;
    }
    Tensor qkv = linear("c_attn")->forward(x);
    auto rope = config.attention_type == AttentionType::kRoPE ? freqs : c10::nullopt;
    Tensor y = ops::attention_packed(qkv, local_heads, local_kv_heads, config.head_dim(), rope, 0, true);
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
    register_module("c_fc", MakeColumnLinear(c.n_embd, hidden, c.add_bias_linear));
    if (c.activation_type == MLPType::kSwiGLU) register_module("c_fc2", MakeColumnLinear(c.n_embd, hidden, c.add_bias_linear));
    register_module("c_proj", MakeRowLinear(hidden, c.n_embd, c.add_bias_linear));
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

// GPT-2 or LLaMA-3 depending on the config; with pipeline parallelism a rank holds only its stage:
// the embeddings on the first stage, its chunks of consecutive layers (round robin over the stages,
// reference pipeline_parallel.cc:42-77), the final norm and the head on the last stage.  State-dict
// names are the reference's, with stage-local layer indices (transformer.h.<i>...).
class TransformerModel : public Module {
 public:
  explicit TransformerModel(const TransformerConfig& c) : Module("Transformer"), config(c) {   // the reference's type name
    const auto& pe = parallel::env();
    TORCH_CHECK(c.vocab_size % pe.tp() == 0, "Vocab size should be divisible by TP world size");
    stage = parallel::GetStageInfo(static_cast<int>(c.n_layer), pe.pp(), pe.pp_rank, pe.vpp);
    auto body = std::make_shared<ModuleDict>();
    if (stage.is_first_stage) {
      if (pe.tp() > 1) wte = std::make_shared<parallel::VocabParallelEmbedding>(c.vocab_size, c.n_embd, pe.sequence_parallel);
      else wte = std::make_shared<Embedding>(c.vocab_size, c.n_embd);
      body->insert("wte", wte);
      if (c.attention_type == AttentionType::kStandard) {
        wpe = std::make_shared<Embedding>(c.block_size, c.n_embd);
        body->insert("wpe", wpe);
      }
    }
    h = std::make_shared<ModuleList>();
    auto ranges = stage.layer_ranges_per_chunk;
    std::sort(ranges.begin(), ranges.end());
    for (const auto& r : ranges) {
      chunk_begin.push_back(static_cast<int64_t>(h->size()));
      for (int i = r.first; i < r.second; ++i) h->push_back(std::make_shared<TransformerLayer>(c));
    }
    chunk_begin.push_back(static_cast<int64_t>(h->size()));
    body->insert("h", h);
    if (stage.is_last_stage) {
      ln_f = MakeNorm(c);
      body->insert("ln_f", ln_f);
    }
    register_module("transformer", body);
    if (stage.is_last_stage) register_module("lm_head", MakeColumnLinear(c.n_embd, c.vocab_size, c.add_bias_lm_head));
    // one tensor serves the lookup and the projection (only possible when one stage holds both)
    if (c.tie_weights && pe.pp() == 1) wte->tie(lm_head()->weight);
  }
  int64_t num_chunks() const { return static_cast<int64_t>(chunk_begin.size()) - 1; }
  // index into h of the layer numbered `global` in the whole model, -1 when another stage holds it
  int64_t local_layer(int64_t global) const {
    int64_t at = 0;
    for (const auto& r : stage.layer_ranges_per_chunk) {
      if (global >= r.first && global < r.second) return at + (global - r.first);
      at += r.second - r.first;
    }
    return -1;
  }

  // ---- the three pieces a pipeline schedule strings together
  // idx [B, T] int64 -> the residual stream [B, T (/ sp), C]
  Tensor embed(const Tensor& idx) {
    const int64_t T = idx.size(1);
    TORCH_CHECK(T <= config.block_size, "sequence longer than block_size");
    const auto& pe = parallel::env();
    if (pe.tp() == 1) {
      if (utils::aligned_mode()) {
        Tensor x = (*wte)(idx);
        if (wpe) x = x + (*wpe)(torch::arange(T, torch::TensorOptions().dtype(torch::kInt64).device(idx.device())));
        return x;
      }
      return ops::embedding(idx, wte->weight, wpe ? c10::optional<Tensor>(wpe->weight) : c10::nullopt, 0);
    }
    Tensor x = std::static_pointer_cast<parallel::VocabParallelEmbedding>(wte)->lookup(idx);
    if (wpe) {   // positions are added after the reduction; under sequence parallelism this rank holds a slice of T
      const int64_t t_local = x.size(1), start = pe.sequence_parallel ? pe.tp_rank * t_local : 0;
      x = x + wpe->weight.slice(0, start, start + t_local).to(x.scalar_type());
    }
    return x;
  }
  // the layers of local chunk `ci` (all layers when ci < 0); T_full is the sequence length before any sharding
  Tensor run_layers(Tensor x, int64_t ci, int64_t T_full) {
    c10::optional<Tensor> freqs;
    if (config.attention_type == AttentionType::kRoPE) {
      if (!freqs_cis_.defined() || freqs_cis_.device() != x.device())
        freqs_cis_ = ops::precompute_freqs_cis(config.head_dim(), 2 * config.block_size, config.rope_theta, x.device());
      freqs = freqs_cis_.slice(0, 0, T_full);
    }
    const int64_t b = ci < 0 ? 0 : chunk_begin[ci], e = ci < 0 ? static_cast<int64_t>(h->size()) : chunk_begin[ci + 1];
    const bool aligned = utils::aligned_mode();
    for (int64_t i = b; i < e; ++i) {
      auto layer = h->at(static_cast<size_t>(i));
      if (aligned) {
        TensorList in = {x};
        if (freqs.has_value()) in.push_back(*freqs);
        x = (*layer)(in)[0];
      } else {
        x = std::static_pointer_cast<TransformerLayer>(layer)->forward(x, freqs);
      }
    }
    return x;
  }
  // final norm + output projection: logits [B, T, vocab / tp]
  Tensor head(const Tensor& x) {
    if (utils::aligned_mode()) return (*mutable_module("lm_head"))((*ln_f)(x));
    return lm_head()->forward((*ln_f)(x));
  }
  // One local chunk of a pipeline stage: `in` is the token ids for the first chunk of the first stage,
  // the previous chunk's activation otherwise; the last chunk of the last stage returns logits.
  Tensor forward_chunk(int64_t ci, const Tensor& in, int64_t T_full) {
    Tensor x = (stage.is_first_stage && ci == 0) ? embed(in) : in;
    x = run_layers(x, ci, T_full);
    return (stage.is_last_stage && ci == num_chunks() - 1) ? head(x) : x;
  }
  // idx [B, T] int64 -> logits [B, T, vocab / tp] (whole model on this rank: pp == 1)
  Tensor forward(const Tensor& idx) {
    TORCH_CHECK(stage.is_first_stage && stage.is_last_stage, "forward() needs the whole model; use forward_chunk under pipeline parallelism");
    return head(run_layers(embed(idx), -1, idx.size(1)));
  }
  TensorList Forward(const TensorList& in) override { return {forward(in[0])}; }

  // Parameters that are replicated over the tensor-parallel group but see a slice of the sequence
  // under sequence parallelism: their gradients are partial sums (norm weights, position table,
  // row-parallel biases).
  TensorList SequenceParallelReplicated() const {
    TensorList out;
    for (const auto& [name, p] : NamedParameters()) {
      const bool norm = name.find("ln_") != std::string::npos;
      const bool row_bias = name.size() > 11 && name.compare(name.size() - 11, 11, "c_proj.bias") == 0;
      if (norm || row_bias || name.find("wpe.weight") != std::string::npos) out.push_back(p);
    }
    return out;
  }

  TransformerConfig config;
  parallel::StageInfo stage;
  std::vector<int64_t> chunk_begin;     // first layer (index into h) of every local chunk, plus the end
  std::shared_ptr<Embedding> wte, wpe;
  std::shared_ptr<ModuleList> h;
  std::shared_ptr<Module> ln_f;
  std::shared_ptr<Linear> lm_head() const { return std::static_pointer_cast<Linear>(mutable_module("lm_head")); }

 private:
  Tensor freqs_cis_;
};

}  // namespace nn
}  // namespace itb
