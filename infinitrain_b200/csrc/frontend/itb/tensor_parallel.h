// Tensor and sequence parallelism (Megatron style) for the C++ frontend.
//
// Reference: infini_train/src/nn/parallel/tensor_parallel.cc -- region functions :133-232,
// ColumnParallelLinear :270-315, RowParallelLinear :324-370, VocabParallelEmbedding :379-434,
// VocabParallelCrossEntropy :436-572.
//
// Activations are [B, T, C].  Under sequence parallelism the tensors between blocks are sharded along
// T over the tensor-parallel group: an all-gather precedes every column-parallel linear and a
// reduce-scatter follows every row-parallel linear (and the embedding).  The collectives work along
// dim 1 directly (the reference transposes T to the front around each of them).
#pragma once
#include "layers.h"
#include "process_group.h"

namespace itb {
namespace parallel {

inline std::shared_ptr<ProcessGroup> TP() {
  auto g = tp_group();
  return g && g->size() > 1 ? g : nullptr;
}

// ------------------------------------------------------------------ raw collectives on activations
inline Tensor AllReduceSum(const Tensor& x, ProcessGroup& g) {
  Tensor t = x.contiguous().clone();
  g.AllReduce(t, ReduceOp::kSum);
  return t;
}
// [.., s, ..] on every rank -> [.., n s, ..] along `dim`
inline Tensor GatherAlong(const Tensor& x, ProcessGroup& g, int64_t dim) {
  const int64_t n = g.size();
  Tensor in = x.contiguous();
  std::vector<int64_t> shape = {n};
  for (int64_t d : in.sizes()) shape.push_back(d);
  Tensor out = torch::empty(shape, in.options());
  g.AllGather(out, in);
  if (dim == 0) {
    std::vector<int64_t> s(in.sizes().begin(), in.sizes().end());
    s[0] *= n;
    return out.view(s);
  }
  std::vector<int64_t> s(in.sizes().begin(), in.sizes().end());
  s[dim] *= n;
  return out.movedim(0, dim).reshape(s);
}
// [.., n s, ..] on every rank -> this rank's [.., s, ..] of the sum along `dim`
inline Tensor ReduceScatterAlong(const Tensor& x, ProcessGroup& g, int64_t dim) {
  const int64_t n = g.size();
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
  TORCH_CHECK(shape[dim] % n == 0, "reduce-scatter dimension must divide by the group size");
  Tensor in = x;
  if (dim != 0) {
    std::vector<int64_t> split(shape.begin(), shape.begin() + dim);
    split.push_back(n);
    split.push_back(shape[dim] / n);
    split.insert(split.end(), shape.begin() + dim + 1, shape.end());
    in = x.reshape(split).movedim(dim, 0);     // rank r's shard becomes contiguous block r
  }
  in = in.contiguous();
  shape[dim] /= n;
  Tensor out = torch::empty(shape, x.options());
  g.ReduceScatter(out, in, ReduceOp::kSum);
  return out;
}
inline Tensor SplitAlong(const Tensor& x, ProcessGroup& g, int64_t dim) { return x.chunk(g.size(), dim)[g.rank()].contiguous(); }
inline int64_t SeqDim(const Tensor& x) { return x.dim() >= 3 ? 1 : 0; }

// ------------------------------------------------------------------ region functions (autograd nodes)
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

// identity forward, all-reduce of the gradient backward
struct CopyToTPRegion : torch::autograd::Function<CopyToTPRegion> {
  static Tensor forward(AutogradContext*, const Tensor& x) { return x.view_as(x); }
  static variable_list backward(AutogradContext*, variable_list g) {
    auto grp = TP();
    return {grp ? AllReduceSum(g[0], *grp) : g[0]};
  }
};
// all-reduce forward, identity backward
struct ReduceFromTPRegion : torch::autograd::Function<ReduceFromTPRegion> {
  static Tensor forward(AutogradContext*, const Tensor& x) {
    auto grp = TP();
    return grp ? AllReduceSum(x, *grp) : x.view_as(x);
  }
  static variable_list backward(AutogradContext*, variable_list g) { return {g[0]}; }
};
// keep this rank's slice of the last dimension forward, all-gather backward
struct ScatterToTPRegion : torch::autograd::Function<ScatterToTPRegion> {
  static Tensor forward(AutogradContext*, const Tensor& x) {
    auto grp = TP();
    return grp ? SplitAlong(x, *grp, x.dim() - 1) : x.view_as(x);
  }
  static variable_list backward(AutogradContext*, variable_list g) {
    auto grp = TP();
    return {grp ? GatherAlong(g[0], *grp, g[0].dim() - 1) : g[0]};
  }
};
// all-gather along the last dimension forward, slice backward
struct GatherFromTPRegion : torch::autograd::Function<GatherFromTPRegion> {
  static Tensor forward(AutogradContext*, const Tensor& x) {
    auto grp = TP();
    return grp ? GatherAlong(x, *grp, x.dim() - 1) : x.view_as(x);
  }
  static variable_list backward(AutogradContext*, variable_list g) {
    auto grp = TP();
    return {grp ? SplitAlong(g[0], *grp, g[0].dim() - 1) : g[0]};
  }
};
// reduce-scatter along the sequence forward, all-gather backward
struct ReduceScatterToSPRegion : torch::autograd::Function<ReduceScatterToSPRegion> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x) {
    auto grp = TP();
    ctx->saved_data["dim"] = SeqDim(x);
    return grp ? ReduceScatterAlong(x, *grp, SeqDim(x)) : x.view_as(x);
  }
  static variable_list backward(AutogradContext* ctx, variable_list g) {
    auto grp = TP();
    return {grp ? GatherAlong(g[0], *grp, ctx->saved_data["dim"].toInt()) : g[0]};
  }
};
// all-gather along the sequence forward, reduce-scatter backward
struct GatherFromSPRegion : torch::autograd::Function<GatherFromSPRegion> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x) {
    auto grp = TP();
    ctx->saved_data["dim"] = SeqDim(x);
    return grp ? GatherAlong(x, *grp, SeqDim(x)) : x.view_as(x);
  }
  static variable_list backward(AutogradContext* ctx, variable_list g) {
    auto grp = TP();
    return {grp ? ReduceScatterAlong(g[0], *grp, ctx->saved_data["dim"].toInt()) : g[0]};
  }
};

// ------------------------------------------------------------------ layers
// y = x W^T + b with W split along the OUTPUT dimension: weight [out / tp, in].  A Linear by
// inheritance, so that code written against Linear (the Transformer blocks, LoRA) takes it as is.
class ColumnParallelLinear : public nn::Linear {
 public:
  ColumnParallelLinear(int64_t in_features, int64_t out_features, bool bias = true, bool gather_output = false,
                       bool input_is_parallel = false, bool skip_bias_add = false, bool sequence_parallel = false)
      : nn::Linear(in_features, Shard(out_features), bias), gather_output_(gather_output), input_is_parallel_(input_is_parallel),
        skip_bias_add_(skip_bias_add), sequence_parallel_(sequence_parallel && env().tp() > 1), out_features_global_(out_features) {
    set_type("ColumnParallelLinear");
  }
  Tensor forward(const Tensor& x_in, const c10::optional<Tensor>& residual = c10::nullopt, bool gelu = false) override {
    Tensor x = x_in;
    if (sequence_parallel_) x = GatherFromSPRegion::apply(x);
    else if (!input_is_parallel_ && TP()) x = CopyToTPRegion::apply(x);
    Tensor y = ops::linear(x, weight, skip_bias_add_ ? c10::nullopt : opt(bias), c10::nullopt, gelu);
    if (gather_output_) y = GatherFromTPRegion::apply(y);
    return residual.has_value() ? y + *residual : y;
  }
  int64_t out_features_global() const { return out_features_global_; }
  bool gather_output() const { return gather_output_; }
  bool input_is_parallel() const { return input_is_parallel_; }
  bool skip_bias_add() const { return skip_bias_add_; }
  bool sequence_parallel() const { return sequence_parallel_; }

 private:
  static int64_t Shard(int64_t n) {
    TORCH_CHECK(n % env().tp() == 0, "out_features must be divisible by the tensor-parallel size");
    return n / env().tp();
  }
  bool gather_output_, input_is_parallel_, skip_bias_add_, sequence_parallel_;
  int64_t out_features_global_;
};

// y = x W^T + b with W split along the INPUT dimension: weight [out, in / tp]; the partial products
// are summed over the group (all-reduce, or reduce-scatter along the sequence under sequence
// parallelism), then bias and residual are added once.
class RowParallelLinear : public nn::Linear {
 public:
  RowParallelLinear(int64_t in_features, int64_t out_features, bool bias = true, bool reduce_output = true,
                    bool input_is_parallel = true, bool skip_bias_add = false, bool sequence_parallel = false)
      : nn::Linear(Shard(in_features), out_features, bias), reduce_output_(reduce_output), input_is_parallel_(input_is_parallel),
        skip_bias_add_(skip_bias_add), sequence_parallel_(sequence_parallel && env().tp() > 1) {
    TORCH_CHECK(!(sequence_parallel_ && !input_is_parallel), "sequence parallelism needs a parallel input");
    set_type("RowParallelLinear");
  }
  Tensor forward(const Tensor& x_in, const c10::optional<Tensor>& residual = c10::nullopt, bool gelu = false) override {
    TORCH_CHECK(!gelu, "a row-parallel linear has no activation epilogue");
    Tensor x = input_is_parallel_ ? x_in : ScatterToTPRegion::apply(x_in);
    auto add_bias = skip_bias_add_ ? c10::nullopt : opt(bias);
    if (!TP() || !reduce_output_) return ops::linear(x, weight, add_bias, residual);
    Tensor y = ops::linear(x, weight);
    y = sequence_parallel_ ? ReduceScatterToSPRegion::apply(y) : ReduceFromTPRegion::apply(y);
    if (add_bias.has_value()) y = y + add_bias->to(y.scalar_type());
    return residual.has_value() ? y + *residual : y;
  }
  bool reduce_output() const { return reduce_output_; }
  bool input_is_parallel() const { return input_is_parallel_; }
  bool skip_bias_add() const { return skip_bias_add_; }
  bool sequence_parallel() const { return sequence_parallel_; }

 private:
  static int64_t Shard(int64_t n) {
    TORCH_CHECK(n % env().tp() == 0, "in_features must be divisible by the tensor-parallel size");
    return n / env().tp();
  }
  bool reduce_output_, input_is_parallel_, skip_bias_add_, sequence_parallel_;
};

// Embedding table split along the vocabulary: weight [V / tp, C]; ids owned by other ranks contribute
// zero rows and the partial results are summed (all-reduce, or reduce-scatter along the sequence).
class VocabParallelEmbedding : public nn::Embedding {
 public:
  VocabParallelEmbedding(int64_t num_embeddings, int64_t embedding_dim, bool reduce_scatter_embeddings = false)
      : nn::Embedding(Shard(num_embeddings), embedding_dim), vocab_global_(num_embeddings),
        reduce_scatter_(reduce_scatter_embeddings && env().tp() > 1) {
    set_type("VocabParallelEmbedding");
    vocab_start_ = env().tp_rank * weight.size(0);
    vocab_end_ = vocab_start_ + weight.size(0);
  }
  Tensor lookup(const Tensor& tokens) {
    auto grp = TP();
    if (!grp) return torch::embedding(weight, tokens);
    Tensor mine = (tokens >= vocab_start_) & (tokens < vocab_end_);
    Tensor local = (tokens - vocab_start_).masked_fill(~mine, 0);
    Tensor out = torch::embedding(weight, local) * mine.unsqueeze(-1).to(weight.scalar_type());
    return reduce_scatter_ ? ReduceScatterToSPRegion::apply(out) : ReduceFromTPRegion::apply(out);
  }
  TensorList Forward(const TensorList& in) override { return {lookup(in[0])}; }
  int64_t vocab_start() const { return vocab_start_; }
  int64_t vocab_end() const { return vocab_end_; }

 private:
  static int64_t Shard(int64_t n) {
    TORCH_CHECK(n % env().tp() == 0, "num_embeddings must be divisible by the tensor-parallel size");
    return n / env().tp();
  }
  int64_t vocab_global_, vocab_start_ = 0, vocab_end_ = 0;
  bool reduce_scatter_;
};

// Cross-entropy over logits sharded along the vocabulary, with ONE collective: every rank reduces its
// shard to (log-sum-exp, target logit where it owns the target column), the per-row pairs are
// all-gathered and merged; backward writes softmax_global - onehot for the local columns.  (The
// reference composes ~20 ops and three all-reduces: tensor_parallel.cc:436-541.)
struct VocabParallelCEFn : torch::autograd::Function<VocabParallelCEFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& logits, const Tensor& target, int64_t valid_local, int64_t vocab_start) {
    auto grp = TP();
    const int64_t V = logits.size(-1);
    Tensor l2 = logits.reshape({-1, V}).to(torch::kFloat32);
    const int64_t rows = l2.size(0);
    Tensor t_local = target.reshape({-1}) - vocab_start;
    Tensor own = (t_local >= 0) & (t_local < valid_local);
    Tensor lse_local, tgt;
    if (valid_local > 0) {
      Tensor lv = l2.slice(1, 0, valid_local);
      lse_local = torch::logsumexp(lv, {-1});
      Tensor picked = lv.gather(1, t_local.clamp(0, valid_local - 1).unsqueeze(1)).squeeze(1);
      tgt = torch::where(own, picked, torch::zeros_like(picked));
    } else {
      lse_local = torch::full({rows}, -1e30, l2.options());
      tgt = torch::zeros({rows}, l2.options());
    }
    Tensor lse = lse_local, tgt_all = tgt;
    if (grp) {
      Tensor stats = torch::stack({lse_local, tgt}, 0).contiguous();            // [2, rows]
      Tensor all = torch::empty({grp->size(), 2, rows}, stats.options());
      grp->AllGather(all, stats);
      lse = torch::logsumexp(all.select(1, 0), {0});
      tgt_all = all.select(1, 1).sum(0);
    }
    ctx->save_for_backward({l2, t_local, lse, own});
    ctx->saved_data["valid"] = valid_local;
    ctx->saved_data["shape"] = logits.sizes().vec();
    ctx->saved_data["dtype"] = static_cast<int64_t>(logits.scalar_type());
    return (lse - tgt_all).view(target.sizes());
  }
  static variable_list backward(AutogradContext* ctx, variable_list g) {
    auto s = ctx->get_saved_variables();
    Tensor l2 = s[0], t_local = s[1], lse = s[2], own = s[3];
    const int64_t valid = ctx->saved_data["valid"].toInt();
    Tensor p = torch::exp(l2 - lse.unsqueeze(1));
    if (valid < p.size(1)) p.slice(1, valid).zero_();
    Tensor onehot = torch::zeros_like(p);
    if (valid > 0) onehot.scatter_(1, t_local.clamp(0, valid - 1).unsqueeze(1), own.to(p.scalar_type()).unsqueeze(1));
    Tensor grad = (p - onehot) * g[0].reshape({-1, 1}).to(torch::kFloat32);
    return {grad.view(ctx->saved_data["shape"].toIntVector()).to(static_cast<torch::ScalarType>(ctx->saved_data["dtype"].toInt())),
            Tensor(), Tensor(), Tensor()};
  }
};

// Mean over all tokens of the vocabulary-parallel cross-entropy (columns past vocab_size_original are
// padding and carry no probability).
class VocabParallelCrossEntropyLoss : public Module {
 public:
  explicit VocabParallelCrossEntropyLoss(int64_t vocab_size_original = 0)
      : Module("VocabParallelCrossEntropyLoss"), vocab_original_(vocab_size_original) {}
  Tensor forward(const Tensor& logits, const Tensor& target) {
    const int64_t V_local = logits.size(-1), tp = env().tp();
    const int64_t V_orig = vocab_original_ > 0 ? vocab_original_ : V_local * tp;
    TORCH_CHECK(V_orig <= V_local * tp, "original vocab size must be <= padded vocab size");
    const int64_t start = (TP() ? env().tp_rank : 0) * V_local;
    const int64_t valid = std::max<int64_t>(0, std::min<int64_t>(V_local, V_orig - start));
    return VocabParallelCEFn::apply(logits, target, valid, start).reshape({-1}).mean();
  }
  TensorList Forward(const TensorList& in) override { return {forward(in[0], in[1])}; }

 private:
  int64_t vocab_original_;
};

// Sums, over the tensor-parallel group, the gradients of parameters that are replicated on its ranks
// but see only a slice of the sequence under sequence parallelism (norm weights, position table,
// row-parallel biases).  Call it after backward and before the optimizer step.
// `always`: the listed gradients are partial with or without sequence parallelism (replicated adapter
// factors next to a split one).
inline int AllReduceSequenceParallelGrads(const TensorList& replicated, bool always = false) {
  auto grp = TP();
  if (!grp || !(env().sequence_parallel || always)) return 0;
  TensorList grads;
  for (const Tensor& p : replicated)
    if (p.grad().defined()) grads.push_back(p.grad());
  if (grads.empty()) return 0;
  TensorList flat_parts;
  for (auto& g : grads) flat_parts.push_back(g.reshape({-1}).to(torch::kFloat32));
  Tensor flat = torch::cat(flat_parts).contiguous();
  grp->AllReduce(flat, ReduceOp::kSum);
  torch::NoGradGuard ng;
  int64_t off = 0;
  for (auto& g : grads) {
    g.copy_(flat.narrow(0, off, g.numel()).view_as(g));
    off += g.numel();
  }
  return static_cast<int>(grads.size());
}

}  // namespace parallel
}  // namespace itb
