// Basic layers of the C++ frontend (reference: infini_train/src/nn/modules/{linear,sparse,
// normalization,activations,loss,container}.cc): same constructor shapes, parameter names
// ("weight", "bias") and initialisation rules.
#pragma once
#include <cmath>
#include <random>

#include "ops.h"

namespace itb {
namespace nn {

// Host-side random initialisation from one global generator, seed 42 (reference:
// src/nn/init.cc:22,35): values are drawn on the CPU and land on the parameter's device later.
inline std::mt19937& global_rng() {
  static std::mt19937 g(42);
  return g;
}
inline void ManualSeed(uint32_t seed) { global_rng().seed(seed); }
namespace init {
// Every draw comes from the global generator unless one is passed (reference: include/nn/init.h:17-54).
inline void Uniform(Tensor t, float lo = 0.0f, float hi = 1.0f, std::mt19937* generator = nullptr) {
  torch::NoGradGuard g;
  std::mt19937& rng = generator ? *generator : global_rng();
  auto host = torch::empty(t.sizes(), torch::kFloat32);
  std::uniform_real_distribution<float> d(lo, hi);
  float* p = host.data_ptr<float>();
  for (int64_t i = 0; i < host.numel(); ++i) p[i] = d(rng);
  t.copy_(host);
}
inline void Normal(Tensor t, float mean = 0.0f, float std = 1.0f, std::mt19937* generator = nullptr) {
  torch::NoGradGuard g;
  std::mt19937& rng = generator ? *generator : global_rng();
  auto host = torch::empty(t.sizes(), torch::kFloat32);
  std::normal_distribution<float> d(mean, std);
  float* p = host.data_ptr<float>();
  for (int64_t i = 0; i < host.numel(); ++i) p[i] = d(rng);
  t.copy_(host);
}
// (fan_in, fan_out) of a weight [out, in, receptive field...].
inline std::pair<int64_t, int64_t> CalculateFanInAndFanOut(const Tensor& t) {
  TORCH_CHECK(t.dim() >= 2, "fan in and fan out need a tensor of at least two dimensions");
  int64_t receptive = 1;
  for (int64_t d = 2; d < t.dim(); ++d) receptive *= t.size(d);
  return {t.size(1) * receptive, t.size(0) * receptive};
}
enum class KaimingMode { kFanIn, kFanOut };
enum class NonLinearityType { kLinear, kConv1D, kConv2D, kConv3D, kConvTransposed1d, kConvTransposed2d, kConvTransposed3d,
                              kSigmoid, kTanh, kReLU, kLeakyReLU, kSELU };
// The gain PyTorch and the reference recommend per non-linearity (`param` = the negative slope of a leaky ReLU).
inline float CalculateGain(NonLinearityType nl, float param = 0.0f) {
  switch (nl) {
    case NonLinearityType::kTanh: return 5.0f / 3.0f;
    case NonLinearityType::kReLU: return std::sqrt(2.0f);
    case NonLinearityType::kLeakyReLU: return std::sqrt(2.0f / (1.0f + param * param));
    case NonLinearityType::kSELU: return 0.75f;
    default: return 1.0f;   // linear, convolutions, sigmoid
  }
}
// U(-bound, bound) with bound = sqrt(3) * gain / sqrt(fan).  The defaults of Linear (a = sqrt(5), fan in, leaky ReLU)
// give bound = 1 / sqrt(fan_in).
inline void KaimingUniform(Tensor t, float a = std::sqrt(5.0f), KaimingMode mode = KaimingMode::kFanIn,
                           NonLinearityType nl = NonLinearityType::kLeakyReLU, std::mt19937* generator = nullptr) {
  auto fans = CalculateFanInAndFanOut(t);
  const float fan = static_cast<float>(mode == KaimingMode::kFanIn ? fans.first : fans.second);
  const float bound = std::sqrt(3.0f) * CalculateGain(nl, a) / std::sqrt(fan);
  Uniform(t, -bound, bound, generator);
}
inline void Ones(Tensor t) {
  torch::NoGradGuard g;
  t.fill_(1);
}
inline void Zeros(Tensor t) {
  torch::NoGradGuard g;
  t.zero_();
}
inline Tensor Arange(int64_t start, int64_t end, torch::Dtype dtype = torch::kInt64, torch::Device device = torch::kCPU) {
  return torch::arange(start, end, torch::TensorOptions().dtype(dtype).device(device));
}
}  // namespace init

class Linear : public Module {
 public:
  static constexpr const char* kType = "Linear";
  Linear(int64_t in_features, int64_t out_features, bool bias = true) : Module(kType) {
    weight = register_parameter("weight", torch::empty({out_features, in_features}));
    init::KaimingUniform(weight);
    if (bias) {
      this->bias = register_parameter("bias", torch::empty({out_features}));
      float bound = 1.0f / std::sqrt(static_cast<float>(in_features));
      init::Uniform(this->bias, -bound, bound);
    }
  }
  TensorList Forward(const TensorList& in) override { return {forward(in[0])}; }
  // y = x W^T + b, optionally through tanh-GELU or plus a residual (fused into the GEMM epilogue on a B200)
  virtual Tensor forward(const Tensor& x, const c10::optional<Tensor>& residual = c10::nullopt, bool gelu = false) {
    return ops::linear(x, weight, opt(bias), residual, gelu);
  }
  static c10::optional<Tensor> opt(const Tensor& t) { return t.defined() ? c10::optional<Tensor>(t) : c10::nullopt; }
  int64_t in_features() const { return weight.size(1); }
  int64_t out_features() const { return weight.size(0); }
  Tensor weight, bias;

 protected:
  // Adopts another Linear's tensors (a wrapper around an existing layer shares its storage).
  Linear(const Linear& base, const char* type) : Module(type) {
    alias_parameter("weight", base.weight);
    weight = base.weight;
    if (base.bias.defined()) {
      alias_parameter("bias", base.bias);
      bias = base.bias;
    }
  }
};

class Embedding : public Module {
 public:
  static constexpr const char* kType = "Embedding";
  Embedding(int64_t num_embeddings, int64_t embedding_dim) : Module(kType) {
    weight = register_parameter("weight", torch::empty({num_embeddings, embedding_dim}));
    init::Normal(weight, 0.0f, 1.0f);
  }
  TensorList Forward(const TensorList& in) override { return {ops::embedding(in[0], weight)}; }
  // Lets a model share this table with its output projection.
  void tie(const Tensor& shared) {
    alias_parameter("weight", shared);
    weight = shared;
  }
  Tensor weight;
};

class LayerNorm : public Module {
 public:
  static constexpr const char* kType = "LayerNorm";
  explicit LayerNorm(int64_t dim, double eps = 1e-5) : Module(kType), eps(eps) {
    weight = register_parameter("weight", torch::ones({dim}));
    bias = register_parameter("bias", torch::zeros({dim}));
  }
  TensorList Forward(const TensorList& in) override { return {ops::layernorm(in[0], weight, bias, eps)}; }
  Tensor weight, bias;
  double eps;
};

class RMSNorm : public Module {
 public:
  static constexpr const char* kType = "RMSNorm";
  explicit RMSNorm(int64_t dim, double eps = 1e-6) : Module(kType), eps(eps) {
    weight = register_parameter("weight", torch::ones({dim}));
  }
  TensorList Forward(const TensorList& in) override { return {ops::rmsnorm(in[0], weight, eps)}; }
  Tensor weight;
  double eps;
};

class Sigmoid : public Module {
 public:
  Sigmoid() : Module("Sigmoid") {}
  TensorList Forward(const TensorList& in) override { return {torch::sigmoid(in[0])}; }
};
class NewGELU : public Module {
 public:
  NewGELU() : Module("NewGELU") {}
  TensorList Forward(const TensorList& in) override { return {ops::gelu(in[0])}; }
};
// One input: x * sigmoid(x), the reference's module of this name (src/nn/modules/activations.cc:21-23);
// two inputs: the gated product in[0] * silu(in[1]) in one fused op.
class SwiGLU : public Module {
 public:
  SwiGLU() : Module("SwiGLU") {}
  TensorList Forward(const TensorList& in) override {
    if (in.size() == 1) return {in[0] * torch::sigmoid(in[0])};
    return {ops::swiglu(in[0], in[1])};
  }
};
class CrossEntropyLoss : public Module {
 public:
  CrossEntropyLoss() : Module("CrossEntropyLoss") {}
  TensorList Forward(const TensorList& in) override { return {ops::cross_entropy(in[0], in[1])}; }
};

// Children named "0", "1", ...; Forward chains them.
class Sequential : public Module {
 public:
  explicit Sequential(std::vector<std::shared_ptr<Module>> layers) : Module("Sequential") {
    for (size_t i = 0; i < layers.size(); ++i) items_.push_back(register_module(std::to_string(i), layers[i]));
  }
  TensorList Forward(const TensorList& in) override {
    TensorList x = in;
    for (auto& m : items_) x = (*m)(x);
    return x;
  }
  size_t size() const { return items_.size(); }
  std::shared_ptr<Module> at(size_t i) const { return items_.at(i); }

 private:
  std::vector<std::shared_ptr<Module>> items_;
};

class ModuleList : public Module {
 public:
  ModuleList() : Module("ModuleList") {}
  explicit ModuleList(std::vector<std::shared_ptr<Module>> layers) : Module("ModuleList") {
    for (auto& l : layers) push_back(l);
  }
  void push_back(std::shared_ptr<Module> m) { items_.push_back(register_module(std::to_string(items_.size()), std::move(m))); }
  size_t size() const { return items_.size(); }
  std::shared_ptr<Module> at(size_t i) const { return items_.at(i); }
  auto begin() const { return items_.begin(); }
  auto end() const { return items_.end(); }

 private:
  std::vector<std::shared_ptr<Module>> items_;
};

class ModuleDict : public Module {
 public:
  ModuleDict() : Module("ModuleDict") {}
  void insert(const std::string& name, std::shared_ptr<Module> m) { register_module(name, std::move(m)); }
  std::shared_ptr<Module> at(const std::string& name) const { return mutable_module(name); }
};

}  // namespace nn
}  // namespace itb
