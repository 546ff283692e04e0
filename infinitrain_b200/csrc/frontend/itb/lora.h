// LoRA for the C++ frontend (reference: infini_train/src/nn/lora/{lora_config,lora_linear,lora_utils}.cc):
// y = base(x) + (alpha / r) (x A^T) B^T with A [r, in] Kaiming-uniform and B [out, r] zeros, base frozen;
// injection by dotted-suffix targets, merge / unmerge, merge-and-unload, adapter files (magic
// 0x4C4F5241, version 1, fp32) that the reference and the Python layer read and write too.
#pragma once
#include <algorithm>
#include <fstream>
#include <set>
#include <sstream>

#include "transformer.h"

namespace itb {
namespace nn {
namespace lora {

struct LoRAConfig {
  int64_t rank = 8;
  double alpha = 16.0;
  double dropout = 0.0;   // accepted, unused (as in the reference)
  // 0: A factors are drawn from the global stream in injection order (the reference's behaviour).  Otherwise every
  // adapter draws from a generator of its own, seeded with this value and its module's whole-model path: the
  // initial adapters are then the same whatever layout (tensor / pipeline split, stage order) builds the model.
  uint32_t seed = 0;
  std::set<std::string> target_modules = {"c_attn", "c_proj"};
  double Scaling() const { return alpha / static_cast<double>(rank); }
  // A module matches when its dotted path equals a target or ends with ".target"
  // ("attn.c_proj" does not match "mlp.c_proj").
  bool ShouldApplyLoRA(const std::string& path) const {
    for (const auto& t : target_modules) {
      if (path == t) return true;
      if (path.size() > t.size() && path.compare(path.size() - t.size() - 1, t.size() + 1, "." + t) == 0) return true;
    }
    return false;
  }
};
// "c_attn, attn.c_proj ,," -> {"c_attn", "attn.c_proj"}
inline std::set<std::string> ParseLoRATargetModules(const std::string& spec) {
  std::set<std::string> out;
  std::stringstream ss(spec);
  std::string item;
  while (std::getline(ss, item, ',')) {
    size_t a = item.find_first_not_of(" \t"), b = item.find_last_not_of(" \t");
    if (a != std::string::npos) out.insert(item.substr(a, b - a + 1));
  }
  return out;
}

// One wrapper for the three kinds of base layer.  Around a tensor-parallel base the low-rank factors
// follow the base's split (reference: infini_train/src/nn/lora/lora_parallel_linear.cc):
//   column-parallel base, W [out / tp, in]:  A [r, in] replicated, B [out / tp, r] split like W's rows;
//   row-parallel base,    W [out, in / tp]:  A [r, in / tp] split like W's columns, B [out, r] replicated;
//     the rank-r partial products x_local A^T are summed over the group (all-reduce, or reduce-scatter
//     along the sequence) beside the base's partial outputs, B is applied after the sum.
// A is drawn at its FULL shape on every rank from the shared initialisation stream and then cut, so a
// tensor-parallel run starts from the adapters a one-rank run starts from.  The replicated factor sees
// only this rank's part of the product in backward (A of a column base always, B of a row base under
// sequence parallelism): PartialGradParameters() lists them for the sum over the group that has to
// precede the optimizer step.
class LoRALinear : public Linear {
 public:
  enum class Kind { kPlain, kColumn, kRow };
  // `generator`: where A is drawn from (null: the global stream)
  LoRALinear(const std::shared_ptr<Linear>& base, const LoRAConfig& config, std::mt19937* generator = nullptr)
      : Linear(*base, "LoRALinear"), config(config) {
    Init(in_features(), /*a_cols_begin=*/0, generator);
  }
  LoRALinear(const std::shared_ptr<parallel::ColumnParallelLinear>& base, const LoRAConfig& config, std::mt19937* generator = nullptr)
      : Linear(*base, "LoRAColumnParallelLinear"), config(config), kind_(Kind::kColumn), column_(base) {
    Init(in_features(), 0, generator);
  }
  LoRALinear(const std::shared_ptr<parallel::RowParallelLinear>& base, const LoRAConfig& config, std::mt19937* generator = nullptr)
      : Linear(*base, "LoRARowParallelLinear"), config(config), kind_(Kind::kRow), row_(base) {
    const auto& pe = parallel::env();
    Init(in_features() * pe.tp(), in_features() * pe.tp_rank, generator);
  }
  Kind kind() const { return kind_; }
  static bool IsLoRAType(const std::string& type) {
    return type == "LoRALinear" || type == "LoRAColumnParallelLinear" || type == "LoRARowParallelLinear";
  }
  Tensor forward(const Tensor& x, const c10::optional<Tensor>& residual = c10::nullopt, bool gelu = false) override {
    TORCH_CHECK(!(merged_ && (lora_A.requires_grad() || lora_B.requires_grad())),
                "Forward() on merged LoRA with requires_grad=true. Call UnmergeWeights() before training.");
    if (kind_ == Kind::kColumn) return ForwardColumn(x, residual, gelu);
    if (kind_ == Kind::kRow) return ForwardRow(x, residual, gelu);
    if (merged_) return ops::linear(x, weight, opt(bias), residual, gelu);
    // the low-rank branch joins before the activation, so a fused GELU epilogue cannot be used here
    Tensor y = ops::linear(x, weight, opt(bias));
    Tensor low = ops::linear(ops::linear(x, lora_A), lora_B);
    y = y + low.to(y.scalar_type()) * config.Scaling();
    if (gelu) y = ops::gelu(y);
    if (residual.has_value()) y = y + *residual;
    return y;
  }
  // this rank's part of (alpha / r) B A, in the shape of this rank's base weight
  Tensor Delta() const {
    return torch::matmul(lora_B.detach().to(torch::kFloat32), lora_A.detach().to(torch::kFloat32)) * config.Scaling();
  }
  void MergeWeights() {
    if (merged_) return;
    torch::NoGradGuard g;
    weight.add_(Delta().to(weight.scalar_type()));
    merged_ = true;
    lora_A.set_requires_grad(false);
    lora_B.set_requires_grad(false);
  }
  void UnmergeWeights() {
    if (!merged_) return;
    torch::NoGradGuard g;
    weight.sub_(Delta().to(weight.scalar_type()));
    merged_ = false;
    lora_A.set_requires_grad(true);
    lora_B.set_requires_grad(true);
  }
  bool IsMerged() const { return merged_; }
  // the factor whose gradient is a partial sum on every tensor-parallel rank (undefined when there is none)
  Tensor PartialGradFactor() const {
    if (kind_ == Kind::kColumn && parallel::env().tp() > 1) return lora_A;
    if (kind_ == Kind::kRow && row_->sequence_parallel()) return lora_B;
    return Tensor();
  }
  LoRAConfig config;
  Tensor lora_A, lora_B;

 private:
  void Init(int64_t in_global, int64_t a_cols_begin, std::mt19937* generator) {
    auto o = weight.options().requires_grad(false);
    Tensor full = torch::empty({config.rank, in_global}, o.device(torch::kCPU));
    init::KaimingUniform(full, std::sqrt(5.0f), init::KaimingMode::kFanIn, init::NonLinearityType::kLeakyReLU, generator);
    lora_A = register_parameter("lora_A", full.slice(1, a_cols_begin, a_cols_begin + in_features()).contiguous().to(weight.device()));
    lora_B = register_parameter("lora_B", torch::zeros({out_features(), config.rank}, o));
    weight.set_requires_grad(false);
    if (bias.defined()) bias.set_requires_grad(false);
  }
  Tensor ForwardColumn(const Tensor& x_in, const c10::optional<Tensor>& residual, bool gelu) {
    Tensor x = x_in;
    if (column_->sequence_parallel()) x = parallel::GatherFromSPRegion::apply(x);
    else if (!column_->input_is_parallel() && parallel::TP()) x = parallel::CopyToTPRegion::apply(x);
    auto b = column_->skip_bias_add() ? c10::nullopt : opt(bias);
    Tensor y;
    if (merged_) {
      y = ops::linear(x, weight, b, c10::nullopt, gelu);
    } else {
      y = ops::linear(x, weight, b);
      y = y + ops::linear(ops::linear(x, lora_A), lora_B).to(y.scalar_type()) * config.Scaling();
      if (gelu) y = ops::gelu(y);
    }
    if (column_->gather_output()) y = parallel::GatherFromTPRegion::apply(y);
    return residual.has_value() ? y + *residual : y;
  }
  Tensor ForwardRow(const Tensor& x_in, const c10::optional<Tensor>& residual, bool gelu) {
    TORCH_CHECK(!gelu, "a row-parallel linear has no activation epilogue");
    Tensor x = row_->input_is_parallel() ? x_in : parallel::ScatterToTPRegion::apply(x_in);
    auto b = row_->skip_bias_add() ? c10::nullopt : opt(bias);
    const bool reduce = parallel::TP() && row_->reduce_output();
    auto sum = [&](const Tensor& t) {
      if (!reduce) return t;
      return row_->sequence_parallel() ? parallel::ReduceScatterToSPRegion::apply(t) : parallel::ReduceFromTPRegion::apply(t);
    };
    Tensor y = sum(ops::linear(x, weight));
    if (!merged_) y = y + ops::linear(sum(ops::linear(x, lora_A)), lora_B).to(y.scalar_type()) * config.Scaling();
    if (b.has_value()) y = y + b->to(y.scalar_type());
    return residual.has_value() ? y + *residual : y;
  }
  bool merged_ = false;
  Kind kind_ = Kind::kPlain;
  std::shared_ptr<parallel::ColumnParallelLinear> column_;
  std::shared_ptr<parallel::RowParallelLinear> row_;
};

// A plain Linear that owns copies of the wrapper's tensors' storage (used by MergeAndUnload).
class UnwrappedLinear : public Linear {
 public:
  explicit UnwrappedLinear(const Linear& merged) : Linear(merged, Linear::kType) {}
};

inline void visit(const std::shared_ptr<Module>& m, const std::string& path,
                  const std::function<void(const std::shared_ptr<Module>& parent, const std::string& name,
                                           const std::string& child_path, const std::shared_ptr<Module>& child)>& fn) {
  for (const auto& name : m->child_names()) {
    auto child = m->mutable_module(name);
    std::string child_path = path.empty() ? name : path + "." + name;
    fn(m, name, child_path, child);
    visit(m->mutable_module(name), child_path, fn);
  }
}

// Puts `replacement` where the module at the dotted `path` sits (reference: lora_utils.cc ReplaceModuleByPath).
inline void ReplaceModuleByPath(const std::shared_ptr<Module>& model, const std::string& path, std::shared_ptr<Module> replacement) {
  TORCH_CHECK(!path.empty(), "ReplaceModuleByPath: the path names a child, the root cannot be replaced");
  std::shared_ptr<Module> parent = model;
  size_t begin = 0;
  while (true) {
    size_t dot = path.find('.', begin);
    std::string name = path.substr(begin, dot == std::string::npos ? std::string::npos : dot - begin);
    TORCH_CHECK(parent->has_module(name), "ReplaceModuleByPath: no module '", name, "' on the way to '", path, "'");
    if (dot == std::string::npos) {
      parent->replace_module(name, std::move(replacement));
      return;
    }
    parent = parent->mutable_module(name);
    begin = dot + 1;
  }
}

inline bool IsLoRAParameterName(const std::string& name) {
  return name.size() >= 6 && (name.compare(name.size() - 6, 6, "lora_A") == 0 || name.compare(name.size() - 6, 6, "lora_B") == 0);
}

inline void FreezeBaseModel(const std::shared_ptr<Module>& model) {
  for (auto& [name, p] : model->NamedParameters()) {
    bool is_lora = name.size() >= 6 && (name.compare(name.size() - 6, 6, "lora_A") == 0 || name.compare(name.size() - 6, 6, "lora_B") == 0);
    Tensor t = p;
    t.set_requires_grad(is_lora);
  }
}
inline void UnfreezeModel(const std::shared_ptr<Module>& model) { model->set_requires_grad(true); }

inline std::string GlobalLayerName(const TransformerModel& model, const std::string& name);

// Wraps every Linear whose path matches a target; everything else is frozen.
inline std::shared_ptr<Module> InjectLoRALayers(const std::shared_ptr<Module>& model, const LoRAConfig& config) {
  auto transformer = std::dynamic_pointer_cast<TransformerModel>(model);
  visit(model, "", [&](const std::shared_ptr<Module>& parent, const std::string& name, const std::string& path,
                       const std::shared_ptr<Module>& child) {
    if (!config.ShouldApplyLoRA(path)) return;
    // config.seed: a generator per adapter, keyed by the module's path in the whole model (FNV-1a of the name)
    std::mt19937 own;
    std::mt19937* gen = nullptr;
    if (config.seed != 0) {
      uint32_t h = 2166136261u;
      for (unsigned char c : transformer ? GlobalLayerName(*transformer, path) : path) h = (h ^ c) * 16777619u;
      own.seed(config.seed ^ h);
      gen = &own;
    }
    if (child->type() == Linear::kType)
      parent->replace_module(name, std::make_shared<LoRALinear>(std::static_pointer_cast<Linear>(child), config, gen));
    else if (child->type() == "ColumnParallelLinear")
      parent->replace_module(name, std::make_shared<LoRALinear>(std::static_pointer_cast<parallel::ColumnParallelLinear>(child), config, gen));
    else if (child->type() == "RowParallelLinear")
      parent->replace_module(name, std::make_shared<LoRALinear>(std::static_pointer_cast<parallel::RowParallelLinear>(child), config, gen));
  });
  return model;
}
inline std::shared_ptr<Module> GetLoRAModel(const std::shared_ptr<Module>& model, const LoRAConfig& config) {
  InjectLoRALayers(model, config);
  FreezeBaseModel(model);
  return model;
}
inline std::vector<std::shared_ptr<LoRALinear>> LoRAModules(const std::shared_ptr<Module>& model) {
  std::vector<std::shared_ptr<LoRALinear>> out;
  for (auto& [path, m] : model->NamedModules())
    if (LoRALinear::IsLoRAType(m->type())) out.push_back(std::static_pointer_cast<LoRALinear>(m));
  return out;
}
inline TensorList GetLoRAParameters(const std::shared_ptr<Module>& model) {
  TensorList out;
  for (auto& m : LoRAModules(model)) {
    out.push_back(m->lora_A);
    out.push_back(m->lora_B);
  }
  return out;
}
// Every parameter that is not an adapter factor, each tensor once.
inline TensorList GetBaseParameters(const std::shared_ptr<Module>& model) {
  TensorList out;
  std::unordered_set<const void*> seen;
  for (auto& [name, p] : model->NamedParameters())
    if (!IsLoRAParameterName(name) && seen.insert(p.unsafeGetTensorImpl()).second) out.push_back(p);
  return out;
}
// Adapter factors whose gradients are partial sums on every tensor-parallel rank (see LoRALinear).
inline TensorList PartialGradParameters(const std::shared_ptr<Module>& model) {
  TensorList out;
  for (auto& m : LoRAModules(model)) {
    Tensor t = m->PartialGradFactor();
    if (t.defined()) out.push_back(t);
  }
  return out;
}
inline TensorList TrainableParameters(const std::shared_ptr<Module>& model) {
  TensorList out;
  for (auto& p : model->Parameters())
    if (p.requires_grad()) out.push_back(p);
  return out;
}
inline void MergeLoRAWeights(const std::shared_ptr<Module>& model) {
  for (auto& m : LoRAModules(model)) m->MergeWeights();
}
inline void UnmergeLoRAWeights(const std::shared_ptr<Module>& model) {
  for (auto& m : LoRAModules(model)) m->UnmergeWeights();
}
// Folds every adapter into its base weight, puts plain Linears back and makes all parameters trainable.
inline std::shared_ptr<Module> MergeAndUnload(const std::shared_ptr<Module>& model) {
  visit(model, "", [&](const std::shared_ptr<Module>& parent, const std::string& name, const std::string&,
                       const std::shared_ptr<Module>& child) {
    if (!LoRALinear::IsLoRAType(child->type())) return;
    auto l = std::static_pointer_cast<LoRALinear>(child);
    TORCH_CHECK(l->kind() == LoRALinear::Kind::kPlain, "MergeAndUnload of a tensor-parallel adapter: merge with MergeLoRAWeights "
                                                      "and keep the wrapper (it carries the base layer's collectives)");
    l->MergeWeights();
    parent->replace_module(name, std::make_shared<UnwrappedLinear>(*l));
  });
  UnfreezeModel(model);
  return model;
}
inline int64_t CountTrainableParameters(const std::shared_ptr<Module>& model) {
  int64_t n = 0;
  for (auto& p : model->Parameters())
    if (p.requires_grad()) n += p.numel();
  return n;
}
inline int64_t CountTotalParameters(const std::shared_ptr<Module>& model) {
  int64_t n = 0;
  for (auto& p : model->Parameters()) n += p.numel();
  return n;
}
inline std::map<std::string, Tensor> LoRAStateDict(const std::shared_ptr<Module>& model) {
  std::map<std::string, Tensor> out;
  for (auto& [k, v] : model->StateDict()) {
    if (k.size() >= 6 && (k.compare(k.size() - 6, 6, "lora_A") == 0 || k.compare(k.size() - 6, 6, "lora_B") == 0)) out[k] = v;
  }
  return out;
}

// Copies the adapter tensors of `state_dict` into the model; names the model lacks are reported and skipped,
// a shape mismatch is an error (reference: lora_utils.cc LoadLoRAStateDict).
inline void LoadLoRAStateDict(const std::shared_ptr<Module>& model, const std::map<std::string, Tensor>& state_dict) {
  auto own = LoRAStateDict(model);
  torch::NoGradGuard g;
  for (auto& [name, t] : state_dict) {
    auto it = own.find(name);
    if (it == own.end()) {
      std::fprintf(stderr, "[W] LoRA parameter not found in model: %s\n", name.c_str());
      continue;
    }
    TORCH_CHECK(it->second.sizes() == t.sizes(), "LoRA parameter ", name, ": the model holds ", it->second.sizes(), ", the state dict ",
                t.sizes());
    it->second.copy_(t);
  }
}

constexpr uint32_t kLoRAMagic = 0x4C4F5241;
// The adapter file format (magic 0x4C4F5241, version 1, count, then per tensor: name, dims, fp32 values; reference:
// lora_utils.cc:309-406) on any stream, so that the same bytes also travel between ranks.
inline void WriteLoRAStream(std::ostream& f, const std::map<std::string, Tensor>& sd) {
  uint32_t head[3] = {kLoRAMagic, 1, static_cast<uint32_t>(sd.size())};
  f.write(reinterpret_cast<const char*>(head), sizeof(head));
  for (auto& [name, t] : sd) {
    uint32_t len = static_cast<uint32_t>(name.size()), ndim = static_cast<uint32_t>(t.dim());
    f.write(reinterpret_cast<const char*>(&len), 4);
    f.write(name.data(), len);
    f.write(reinterpret_cast<const char*>(&ndim), 4);
    for (int64_t d : t.sizes()) f.write(reinterpret_cast<const char*>(&d), 8);
    Tensor host = t.detach().to(torch::kCPU, torch::kFloat32).contiguous();
    f.write(static_cast<const char*>(host.data_ptr()), host.numel() * 4);
  }
}
inline std::map<std::string, Tensor> ReadLoRAStream(std::istream& f, const std::string& what) {
  uint32_t head[3];
  f.read(reinterpret_cast<char*>(head), sizeof(head));
  TORCH_CHECK(f.good() && head[0] == kLoRAMagic, "Invalid LoRA file format: ", what);
  TORCH_CHECK(head[1] == 1, "Unsupported LoRA file version: ", head[1]);
  std::map<std::string, Tensor> out;
  for (uint32_t i = 0; i < head[2]; ++i) {
    uint32_t len = 0, ndim = 0;
    f.read(reinterpret_cast<char*>(&len), 4);
    TORCH_CHECK(f.good() && len < 4096, "LoRA file is damaged: ", what);
    std::string name(len, '\0');
    f.read(name.data(), len);
    f.read(reinterpret_cast<char*>(&ndim), 4);
    TORCH_CHECK(f.good() && ndim <= 8, "LoRA file is damaged: ", what);
    std::vector<int64_t> dims(ndim);
    for (auto& d : dims) f.read(reinterpret_cast<char*>(&d), 8);
    Tensor t = torch::empty(dims, torch::kFloat32);
    f.read(static_cast<char*>(t.data_ptr()), t.numel() * 4);
    TORCH_CHECK(f.good(), "LoRA file is truncated: ", what);
    out[name] = t;
  }
  return out;
}
inline void SaveLoRAWeights(const std::shared_ptr<Module>& model, const std::string& path) {
  std::ofstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "Failed to open ", path);
  WriteLoRAStream(f, LoRAStateDict(model));
}
inline void LoadLoRAWeights(const std::shared_ptr<Module>& model, const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "Failed to open ", path);
  auto own = model->StateDict();
  torch::NoGradGuard g;
  for (auto& [name, t] : ReadLoRAStream(f, path)) {
    auto it = own.find(name);
    if (it == own.end()) {
      std::fprintf(stderr, "[W] LoRA parameter not found in model: %s\n", name.c_str());
      continue;
    }
    it->second.copy_(t);
  }
}

// ---- one adapter file for the whole model, whatever the layout that trained it
// How this rank's piece of an adapter factor relates to the whole factor.
enum class LoRAShard { kReplicated, kRows, kCols };
inline LoRAShard ShardOf(const LoRALinear& m, const std::string& key) {
  if (parallel::env().tp() <= 1) return LoRAShard::kReplicated;
  const bool is_a = key.size() >= 6 && key.compare(key.size() - 6, 6, "lora_A") == 0;
  if (m.kind() == LoRALinear::Kind::kColumn && !is_a) return LoRAShard::kRows;   // B split like the base's output rows
  if (m.kind() == LoRALinear::Kind::kRow && is_a) return LoRAShard::kCols;       // A split like the base's input columns
  return LoRAShard::kReplicated;
}
// "transformer.h.<local>..." -> "transformer.h.<global>..." for the layers this pipeline stage holds.
inline std::string GlobalLayerName(const TransformerModel& model, const std::string& name) {
  const std::string prefix = "transformer.h.";
  if (name.compare(0, prefix.size(), prefix) != 0) return name;
  const size_t dot = name.find('.', prefix.size());
  const int64_t local = std::stoll(name.substr(prefix.size(), dot - prefix.size()));
  auto ranges = model.stage.layer_ranges_per_chunk;
  std::sort(ranges.begin(), ranges.end());
  int64_t at = 0;
  for (const auto& r : ranges) {
    if (local < at + (r.second - r.first)) return prefix + std::to_string(r.first + (local - at)) + name.substr(dot);
    at += r.second - r.first;
  }
  TORCH_CHECK(false, "layer ", local, " is not one of this stage's");
}
// Rows of a fused QKV projection: every tensor-parallel rank holds [its Q heads | its K heads | its V heads].
inline bool IsFusedQKV(const std::string& key) {
  const std::string tail = "attn.c_attn.lora_B";
  return key.size() >= tail.size() && key.compare(key.size() - tail.size(), tail.size(), tail) == 0;
}

// The adapters of the WHOLE model under global names: column-parallel B factors joined along the output rows (a
// fused QKV projection back into Q | K | V order), row-parallel A factors along the input columns, replicated
// factors from this rank, a stage's local layer numbers turned into global ones.  Collective over this rank's
// tensor-parallel group and its pipeline group; the first pipeline stage gets the whole dict, the others their own.
inline std::map<std::string, Tensor> GatherFullLoRAStateDict(const std::shared_ptr<TransformerModel>& model) {
  const auto& pe = parallel::env();
  auto tp_group = parallel::tp_group();
  auto pp_group = parallel::pp_group();
  const auto& cfg = model->config;
  std::map<std::string, Tensor> mine;
  std::map<std::string, std::shared_ptr<LoRALinear>> owners;
  for (auto& [path, m] : model->NamedModules())
    if (LoRALinear::IsLoRAType(m->type())) owners[path] = std::static_pointer_cast<LoRALinear>(m);
  for (auto& [key, t] : LoRAStateDict(model)) {   // sorted by name: the same order on every rank of the group
    const auto& owner = owners.at(key.substr(0, key.rfind('.')));
    const LoRAShard shard = ShardOf(*owner, key);
    Tensor full = t.detach().to(torch::kFloat32).contiguous();
    if (shard != LoRAShard::kReplicated) {
      Tensor all = torch::empty({pe.tp() * full.numel()}, full.options());
      tp_group->AllGather(all, full.view({-1}));
      std::vector<int64_t> shape = full.sizes().vec();
      shape.insert(shape.begin(), pe.tp());
      all = all.view(shape).cpu();
      TensorList parts;
      if (shard == LoRAShard::kCols) {
        for (int r = 0; r < pe.tp(); ++r) parts.push_back(all[r]);
        full = torch::cat(parts, 1);
      } else if (IsFusedQKV(key)) {
        const int64_t q = cfg.n_head * cfg.head_dim() / pe.tp(), kv = cfg.n_kv_head * cfg.head_dim() / pe.tp();
        for (int64_t begin : {int64_t(0), q, q + kv})
          for (int r = 0; r < pe.tp(); ++r) parts.push_back(all[r].slice(0, begin, begin + (begin == 0 ? q : kv)));
        full = torch::cat(parts, 0);
      } else {
        for (int r = 0; r < pe.tp(); ++r) parts.push_back(all[r]);
        full = torch::cat(parts, 0);
      }
    }
    mine[GlobalLayerName(*model, key)] = full.cpu();
  }
  if (!pp_group || pp_group->size() == 1) return mine;
  // every stage's part, in the file format, to the first stage
  std::ostringstream os;
  WriteLoRAStream(os, mine);
  const std::string bytes = os.str();
  const torch::Device dev = model->Parameters()[0].device();
  Tensor sizes = torch::zeros({pp_group->size()}, torch::dtype(torch::kInt64).device(dev));
  Tensor my_size = torch::full({1}, static_cast<int64_t>(bytes.size()), sizes.options());
  pp_group->AllGather(sizes, my_size);
  sizes = sizes.cpu();
  if (pp_group->rank() != 0) {
    Tensor payload = torch::from_blob(const_cast<char*>(bytes.data()), {static_cast<int64_t>(bytes.size())}, torch::kUInt8).to(dev);
    pp_group->Send({payload}, 0);
    return mine;
  }
  for (int r = 1; r < pp_group->size(); ++r) {
    TensorList in = {torch::empty({sizes[r].item<int64_t>()}, torch::dtype(torch::kUInt8).device(dev))};
    pp_group->Recv(in, r);
    Tensor host = in[0].cpu();
    std::istringstream is(std::string(reinterpret_cast<const char*>(host.data_ptr<uint8_t>()), static_cast<size_t>(host.numel())));
    for (auto& [name, t] : ReadLoRAStream(is, "stage " + std::to_string(r)))
      if (!mine.count(name)) mine[name] = t;
  }
  return mine;
}

// Collective (see GatherFullLoRAStateDict); the rank that holds tensor-parallel rank 0 of the first pipeline stage
// of data-parallel replica 0 writes ONE ordinary adapter file, loadable on any layout, by the Python layer and by
// the reference.
inline void SaveFullLoRAWeights(const std::shared_ptr<TransformerModel>& model, const std::string& path) {
  const auto& pe = parallel::env();
  if (pe.dp_rank != 0) return;   // the other replicas hold the same adapters; their groups are their own
  auto full = GatherFullLoRAStateDict(model);
  if (pe.tp_rank != 0 || pe.pp_rank != 0) return;
  std::ofstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "Failed to open ", path);
  WriteLoRAStream(f, full);
}
// Every rank reads the whole-model file and keeps its own rows / columns / layers.  Returns the number of tensors loaded.
inline int64_t LoadFullLoRAWeights(const std::shared_ptr<TransformerModel>& model, const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "Failed to open ", path);
  auto full = ReadLoRAStream(f, path);
  const auto& pe = parallel::env();
  const auto& cfg = model->config;
  std::map<std::string, std::shared_ptr<LoRALinear>> owners;
  for (auto& [p, m] : model->NamedModules())
    if (LoRALinear::IsLoRAType(m->type())) owners[p] = std::static_pointer_cast<LoRALinear>(m);
  torch::NoGradGuard g;
  int64_t n = 0;
  for (auto& [key, dst] : LoRAStateDict(model)) {
    const std::string gname = GlobalLayerName(*model, key);
    auto it = full.find(gname);
    TORCH_CHECK(it != full.end(), "adapter file ", path, " has no tensor '", gname, "'");
    Tensor src = it->second;
    const LoRAShard shard = ShardOf(*owners.at(key.substr(0, key.rfind('.'))), key);
    const int64_t r = pe.tp_rank, tp = pe.tp();
    if (shard == LoRAShard::kCols) {
      src = src.chunk(tp, 1)[r];
    } else if (shard == LoRAShard::kRows && IsFusedQKV(key)) {
      const int64_t Q = cfg.n_head * cfg.head_dim(), KV = cfg.n_kv_head * cfg.head_dim();
      src = torch::cat({src.slice(0, 0, Q).chunk(tp, 0)[r], src.slice(0, Q, Q + KV).chunk(tp, 0)[r], src.slice(0, Q + KV, Q + 2 * KV).chunk(tp, 0)[r]}, 0);
    } else if (shard == LoRAShard::kRows) {
      src = src.chunk(tp, 0)[r];
    }
    TORCH_CHECK(src.sizes() == dst.sizes(), "adapter tensor ", gname, ": the file gives ", src.sizes(), " for this rank, the model holds ", dst.sizes());
    Tensor d = dst;
    d.copy_(src);
    ++n;
  }
  return n;
}
inline std::string PrintLoRASummary(const std::shared_ptr<Module>& model) {
  int64_t trainable = CountTrainableParameters(model), total = CountTotalParameters(model);
  std::ostringstream os;
  os << "LoRA: " << LoRAModules(model).size() << " adapted layers, trainable " << trainable << " / " << total << " ("
     << 100.0 * static_cast<double>(trainable) / static_cast<double>(total) << " %)";
  return os.str();
}

}  // namespace lora
}  // namespace nn
}  // namespace itb
