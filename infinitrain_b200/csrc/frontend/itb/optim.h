// Optimizers of the C++ frontend (reference: infini_train/include/optimizer.h, src/optimizer.cc:23-105):
// Step / ZeroGrad / StateDict / LoadStateDict, positional state keys adam.m.<i>, adam.v.<i>, adam.t.
// On a B200 one fused launch per parameter updates the fp32 weight and writes its bf16 shadow (the raw
// launch leaves the tensor's version alone, so the shadow stays marked fresh).
#pragma once
#include <cmath>
#include <functional>
#include <memory>

#include "ops.h"

namespace itb {
namespace optim {

class Optimizer {
 public:
  explicit Optimizer(TensorList params) : params_(std::move(params)) {}
  virtual ~Optimizer() = default;
  virtual void Step() = 0;
  virtual void ZeroGrad(bool set_to_none = true) {
    for (auto& p : params_) {
      if (!p.grad().defined()) continue;
      if (set_to_none) p.mutable_grad() = Tensor();
      else p.mutable_grad().zero_();
    }
  }
  virtual std::map<std::string, Tensor> StateDict() const { return {}; }
  virtual void LoadStateDict(const std::map<std::string, Tensor>&) {}
  const TensorList& params() const { return params_; }

 protected:
  TensorList params_;
};

// Builds an optimizer over a parameter list that is only known later (a ZeRO shard: DistributedOptimizer).
using OptimizerCreator = std::function<std::unique_ptr<Optimizer>(TensorList)>;

class SGD : public Optimizer {
 public:
  SGD(TensorList params, double lr) : Optimizer(std::move(params)), lr_(lr) {}
  // reference: optimizers::SGD::Create(lr), include/optimizer.h:35-46
  static OptimizerCreator Create(double lr) {
    return [lr](TensorList params) -> std::unique_ptr<Optimizer> { return std::make_unique<SGD>(std::move(params), lr); };
  }
  void Step() override {
    ITB_PROFILE("sgd.Step", params_.empty() ? Tensor() : params_[0]);
    torch::NoGradGuard g;
    for (auto& p : params_) {
      if (!p.grad().defined()) continue;
#ifdef ITB_WITH_CUDA
      if (p.is_cuda() && p.scalar_type() == torch::kFloat32 && p.is_contiguous()) {
        Tensor grad = ops::fused::contig(p.grad());
        Tensor shadow = ops::fused::shadow_of(p);
        ops::fused::check(itb_sgd(p.data_ptr<float>(), grad.data_ptr(), ops::fused::code(grad), shadow.data_ptr(), p.numel(),
                                  static_cast<float>(lr_), 1.0f, ops::fused::stream()), "sgd");
        continue;
      }
#endif
      p.add_(p.grad().to(p.scalar_type()), -lr_);
    }
  }
  void set_lr(double lr) { lr_ = lr; }

 private:
  double lr_;
};

// Adam with bias correction; weight_decay > 0 gives AdamW (decoupled decay).  The step counter
// advances on every Step, also for parameters without a gradient.
class Adam : public Optimizer {
 public:
  Adam(TensorList params, double lr, double beta1 = 0.9, double beta2 = 0.999, double eps = 1e-8, double weight_decay = 0.0)
      : Optimizer(std::move(params)), lr_(lr), b1_(beta1), b2_(beta2), eps_(eps), wd_(weight_decay) {
    for (auto& p : params_) {
      m_.push_back(torch::zeros_like(p, p.options().requires_grad(false)));
      v_.push_back(torch::zeros_like(p, p.options().requires_grad(false)));
    }
  }
  // reference: optimizers::Adam::Create(lr, beta1, beta2, eps), include/optimizer.h:48-68
  static OptimizerCreator Create(double lr = 1e-3, double beta1 = 0.9, double beta2 = 0.999, double eps = 1e-8, double weight_decay = 0.0) {
    return [=](TensorList params) -> std::unique_ptr<Optimizer> {
      return std::make_unique<Adam>(std::move(params), lr, beta1, beta2, eps, weight_decay);
    };
  }
  void Step() override {
    ITB_PROFILE("adam.Step", params_.empty() ? Tensor() : params_[0]);
    torch::NoGradGuard g;
    ++t_;
    double bc1 = 1.0 - std::pow(b1_, t_), bc2 = 1.0 - std::pow(b2_, t_);
    for (size_t i = 0; i < params_.size(); ++i) {
      Tensor& p = params_[i];
      if (!p.grad().defined()) continue;
      if (m_[i].device() != p.device()) {
        m_[i] = m_[i].to(p.device());
        v_[i] = v_[i].to(p.device());
      }
#ifdef ITB_WITH_CUDA
      if (p.is_cuda() && p.scalar_type() == torch::kFloat32 && p.is_contiguous()) {
        Tensor grad = ops::fused::contig(p.grad());
        Tensor shadow = ops::fused::shadow_of(p);
        ops::fused::check(itb_adamw(p.data_ptr<float>(), grad.data_ptr(), ops::fused::code(grad), m_[i].data_ptr<float>(),
                                    v_[i].data_ptr<float>(), shadow.data_ptr(), p.numel(), static_cast<float>(lr_),
                                    static_cast<float>(b1_), static_cast<float>(b2_), static_cast<float>(eps_),
                                    static_cast<float>(wd_), static_cast<float>(bc1), static_cast<float>(bc2), 1.0f, nullptr,
                                    ops::fused::stream()), "adamw");
        continue;
      }
#endif
      Tensor grad = p.grad().to(p.scalar_type());
      m_[i].mul_(b1_).add_(grad, 1.0 - b1_);
      v_[i].mul_(b2_).addcmul_(grad, grad, 1.0 - b2_);
      Tensor update = (m_[i] / bc1) / ((v_[i] / bc2).sqrt() + eps_);
      if (wd_ != 0.0) update = update + wd_ * p;
      p.add_(update, -lr_);
    }
  }
  std::map<std::string, Tensor> StateDict() const override {
    std::map<std::string, Tensor> out;
    for (size_t i = 0; i < params_.size(); ++i) {
      out["adam.m." + std::to_string(i)] = m_[i];
      out["adam.v." + std::to_string(i)] = v_[i];
    }
    out["adam.t"] = torch::tensor(static_cast<int64_t>(t_), torch::kInt64);
    return out;
  }
  void LoadStateDict(const std::map<std::string, Tensor>& sd) override {
    torch::NoGradGuard g;
    for (size_t i = 0; i < params_.size(); ++i) {
      m_[i].copy_(sd.at("adam.m." + std::to_string(i)));
      v_[i].copy_(sd.at("adam.v." + std::to_string(i)));
    }
    t_ = sd.at("adam.t").item<int64_t>();
  }
  int64_t t() const { return t_; }
  void set_lr(double lr) { lr_ = lr; }

 private:
  double lr_, b1_, b2_, eps_, wd_;
  std::vector<Tensor> m_, v_;
  int64_t t_ = 0;
};

}  // namespace optim
}  // namespace itb
