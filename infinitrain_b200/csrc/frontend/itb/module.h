// C++ frontend on libtorch: the Module tree.
//
// A program written against the reference's C++ API (infini_train/include/nn/modules/module.h:42-97:
// Parameters / Buffers / StateDict / LoadStateDict / Forward / To / Apply / NamedModules / Register*Hook)
// finds the same names here.  Tensors are torch::Tensor (autograd, devices, dtypes and CPU math come
// from libtorch); the hot ops on a B200 are this library's sm_100a kernels (ops.h).
#pragma once
#include <torch/torch.h>

#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_set>
#include <utility>
#include <vector>

namespace itb {

using Tensor = torch::Tensor;
using TensorList = std::vector<Tensor>;

namespace autograd {
using NoGradGuard = torch::NoGradGuard;   // the reference's autograd::NoGradGuard
}  // namespace autograd

// Handle of a registered hook; Remove() unregisters it (reference: include/common/hook.h:7-28).
class HookHandle {
 public:
  explicit HookHandle(std::function<void()> remove) : remove_(std::move(remove)) {}
  void Remove() {
    if (remove_) remove_();
    remove_ = nullptr;
  }

 private:
  std::function<void()> remove_;
};

class Module;

// Process-wide module hooks: they run for every module's call, around the module's own hooks
// (reference: include/utils/global_module_hook_registry.h:19-52 and src/nn/modules/module.cc:198-266;
// the precision checker and the profiler hang their per-module work here).  Registration and the calls
// take a snapshot under a mutex, so ranks that run as threads of one process may register and call
// concurrently.
class GlobalModuleHookRegistry {
 public:
  using ModuleForwardPreHook = std::function<void(Module*, const TensorList&)>;
  using ModuleForwardHook = std::function<void(Module*, const TensorList&, const TensorList&)>;
  // hook(module, gradients w.r.t. the outputs, gradients w.r.t. the inputs); the second list holds the
  // entries that exist when the hook runs (libtorch shows a module's backward one output at a time)
  using ModuleFullBackwardHook = std::function<void(Module*, const TensorList&, const TensorList&)>;

  static GlobalModuleHookRegistry& Instance() {
    static GlobalModuleHookRegistry r;
    return r;
  }
  std::shared_ptr<HookHandle> RegisterModuleForwardPreHook(ModuleForwardPreHook h) { return add(&pre_, std::move(h)); }
  std::shared_ptr<HookHandle> RegisterModuleForwardHook(ModuleForwardHook h) { return add(&post_, std::move(h)); }
  std::shared_ptr<HookHandle> RegisterModuleFullBackwardHook(ModuleFullBackwardHook h) { return add(&bwd_, std::move(h)); }

  void CallModuleForwardPreHooks(Module* m, const TensorList& in) {
    for (auto& h : snapshot(pre_)) h(m, in);
  }
  void CallModuleForwardHooks(Module* m, const TensorList& in, const TensorList& out) {
    for (auto& h : snapshot(post_)) h(m, in, out);
  }
  void CallModuleFullBackwardHooks(Module* m, const TensorList& grad_outputs, const TensorList& grad_inputs) {
    for (auto& h : snapshot(bwd_)) h(m, grad_outputs, grad_inputs);
  }
  bool HasModuleBackwardHooks() const {
    std::lock_guard<std::mutex> lock(mu_);
    return !bwd_.empty();
  }
  bool empty() const {
    std::lock_guard<std::mutex> lock(mu_);
    return pre_.empty() && post_.empty() && bwd_.empty();
  }

 private:
  template <class H>
  std::shared_ptr<HookHandle> add(std::map<int, H>* where, H h) {
    std::lock_guard<std::mutex> lock(mu_);
    int id = next_++;
    (*where)[id] = std::move(h);
    return std::make_shared<HookHandle>([this, where, id] {
      std::lock_guard<std::mutex> l(mu_);
      where->erase(id);
    });
  }
  template <class H>
  std::vector<H> snapshot(const std::map<int, H>& from) const {
    std::lock_guard<std::mutex> lock(mu_);
    std::vector<H> out;
    out.reserve(from.size());
    for (auto& [id, h] : from) out.push_back(h);
    return out;
  }
  mutable std::mutex mu_;
  std::map<int, ModuleForwardPreHook> pre_;
  std::map<int, ModuleForwardHook> post_;
  std::map<int, ModuleFullBackwardHook> bwd_;
  int next_ = 0;
};

class Module : public std::enable_shared_from_this<Module> {
 public:
  using PreHook = std::function<void(Module*, const TensorList&)>;
  using PostHook = std::function<void(Module*, const TensorList&, const TensorList&)>;

  Module() : type_("Module") {}
  explicit Module(std::string type) : type_(std::move(type)) {}
  virtual ~Module() = default;

  const std::string& type() const { return type_; }

  // Parameters of this module and its children, each tensor once (weight tying keeps one entry).
  virtual TensorList Parameters() const {
    TensorList out;
    std::unordered_set<const void*> seen;
    CollectParameters(&out, &seen);
    return out;
  }
  virtual TensorList Buffers() const {
    TensorList out;
    for (const auto& [name, t] : buffers_) out.push_back(t);
    for (const auto& [name, m] : modules_)
      for (auto& t : m->Buffers()) out.push_back(t);
    return out;
  }
  std::vector<std::pair<std::string, Tensor>> NamedParameters(const std::string& prefix = "") const {
    std::vector<std::pair<std::string, Tensor>> out;
    for (const auto& name : param_order_) out.emplace_back(prefix + name, parameters_.at(name));
    for (const auto& name : module_order_) {
      auto sub = modules_.at(name)->NamedParameters(prefix + name + ".");
      out.insert(out.end(), sub.begin(), sub.end());
    }
    return out;
  }

  // Pre-order list of (path, module), every module once.
  std::vector<std::pair<std::string, std::shared_ptr<Module>>> NamedModules(const std::string& prefix = "") {
    std::vector<std::pair<std::string, std::shared_ptr<Module>>> out;
    std::unordered_set<Module*> seen;
    CollectModules(prefix, &out, &seen);
    return out;
  }
  std::shared_ptr<Module> mutable_module(const std::string& name) const { return modules_.at(name); }
  // Swaps a direct child for another module under the same name (LoRA injection, merge-and-unload).
  void replace_module(const std::string& name, std::shared_ptr<Module> m) {
    TORCH_CHECK(modules_.count(name), "replace_module: no child named '", name, "'");
    modules_[name] = std::move(m);
  }
  const std::vector<std::string>& child_names() const { return module_order_; }
  bool has_module(const std::string& name) const { return modules_.count(name) != 0; }
  Tensor& parameter(const std::string& name) { return parameters_.at(name); }
  Tensor& mutable_parameter(const std::string& name) { return parameters_.at(name); }   // the reference's name
  // this module and every module below it, pre-order, each once (reference: Module::modules())
  std::vector<std::shared_ptr<Module>> modules() {
    std::vector<std::shared_ptr<Module>> out;
    for (auto& [path, m] : NamedModules()) out.push_back(m);
    return out;
  }
  const Tensor& parameter(const std::string& name) const { return parameters_.at(name); }
  bool has_parameter(const std::string& name) const { return parameters_.count(name) != 0; }

  // name -> tensor over parameters and buffers, dotted paths.
  std::map<std::string, Tensor> StateDict(const std::string& prefix = "") const {
    std::map<std::string, Tensor> out;
    for (const auto& [name, t] : parameters_) out[prefix + name] = t;
    for (const auto& [name, t] : buffers_) out[prefix + name] = t;
    for (const auto& [name, m] : modules_) {
      auto sub = m->StateDict(prefix + name + ".");
      out.insert(sub.begin(), sub.end());
    }
    return out;
  }
  // Strict on missing keys, shapes and dtypes; keys the module does not have are ignored.
  void LoadStateDict(const std::map<std::string, Tensor>& state_dict) {
    torch::NoGradGuard no_grad;
    for (auto& [name, dst] : StateDict()) {
      auto it = state_dict.find(name);
      TORCH_CHECK(it != state_dict.end(), "LoadStateDict: missing key '", name, "'");
      TORCH_CHECK(it->second.sizes() == dst.sizes(), "LoadStateDict: shape mismatch for '", name, "'");
      TORCH_CHECK(it->second.scalar_type() == dst.scalar_type(), "LoadStateDict: dtype mismatch for '", name, "'");
      Tensor t = dst;
      t.copy_(it->second);
    }
  }

  virtual TensorList Forward(const TensorList& inputs) {
    TORCH_CHECK(false, "Forward is not implemented for module type ", type_);
  }
  // Order of a call (the reference's, module.cc:198-266): global pre-hooks, the module's pre-hooks,
  // Forward, the module's post-hooks, global post-hooks; backward hooks are attached to the outputs.
  TensorList operator()(const TensorList& inputs) {
    auto& global = GlobalModuleHookRegistry::Instance();
    const bool any_global = !global.empty();
    if (any_global) global.CallModuleForwardPreHooks(this, inputs);
    for (auto& [id, h] : pre_hooks_) h(this, inputs);
    TensorList outputs = Forward(inputs);
    for (auto& [id, h] : post_hooks_) h(this, inputs, outputs);
    if (any_global) global.CallModuleForwardHooks(this, inputs, outputs);
    const bool global_bwd = any_global && global.HasModuleBackwardHooks();
    if (!backward_hooks_.empty() || !backward_pre_hooks_.empty() || global_bwd) {
      // the gradient that reaches output i during backward is shown to the hooks registered now:
      // pre-hooks first, then the module's backward hooks, then the process-wide ones
      for (size_t i = 0; i < outputs.size(); ++i) {
        if (!outputs[i].defined() || !outputs[i].requires_grad()) continue;
        auto pre = backward_pre_hooks_;
        auto hooks = backward_hooks_;
        const size_t n_out = outputs.size();
        outputs[i].register_hook([this, pre, hooks, i, n_out, global_bwd](const Tensor& grad) {
          for (auto& [id, h] : pre) h(this, i, grad);
          for (auto& [id, h] : hooks) h(this, i, grad);
          if (global_bwd) {
            TensorList grad_outputs(n_out);
            grad_outputs[i] = grad;
            GlobalModuleHookRegistry::Instance().CallModuleFullBackwardHooks(this, grad_outputs, {});
          }
        });
      }
    }
    return outputs;
  }
  Tensor operator()(const Tensor& x) { return (*this)(TensorList{x})[0]; }

  // Moves parameters and buffers in place (the tensors keep their identity, so tied weights, optimizer
  // references and hooks survive; the reference re-creates every parameter, module.cc:269-285).
  virtual void To(torch::Device device) {
    torch::NoGradGuard no_grad;
    Apply([&](Module* m) {
      for (auto& [name, t] : m->parameters_)
        if (t.device() != device) t.set_data(t.to(device));
      for (auto& [name, t] : m->buffers_)
        if (t.device() != device) t.set_data(t.to(device));
    });
  }
  virtual void To(torch::Dtype dtype) {
    torch::NoGradGuard no_grad;
    Apply([&](Module* m) {
      for (auto& [name, t] : m->parameters_)
        if (t.is_floating_point() && t.scalar_type() != dtype) t.set_data(t.to(dtype));
    });
  }
  void Apply(const std::function<void(Module*)>& fn) {
    for (const auto& name : module_order_) modules_.at(name)->Apply(fn);
    fn(this);
  }

  std::shared_ptr<HookHandle> RegisterForwardPreHook(PreHook hook) {
    int id = next_hook_++;
    pre_hooks_[id] = std::move(hook);
    return std::make_shared<HookHandle>([this, id] { pre_hooks_.erase(id); });
  }
  std::shared_ptr<HookHandle> RegisterForwardPostHook(PostHook hook) {
    int id = next_hook_++;
    post_hooks_[id] = std::move(hook);
    return std::make_shared<HookHandle>([this, id] { post_hooks_.erase(id); });
  }

  // hook(module, output index, gradient w.r.t. that output), called during backward (the reference's
  // RegisterBackwardPostHook records the same tensors as "GradOutputs")
  using BackwardHook = std::function<void(Module*, size_t, const Tensor&)>;
  std::shared_ptr<HookHandle> RegisterBackwardPostHook(BackwardHook hook) {
    int id = next_hook_++;
    backward_hooks_[id] = std::move(hook);
    return std::make_shared<HookHandle>([this, id] { backward_hooks_.erase(id); });
  }

  // Runs before the module's backward hooks, on the same gradient (reference:
  // Module::RegisterBackwardPreHook, module.cc:321-324).
  std::shared_ptr<HookHandle> RegisterBackwardPreHook(BackwardHook hook) {
    int id = next_hook_++;
    backward_pre_hooks_[id] = std::move(hook);
    return std::make_shared<HookHandle>([this, id] { backward_pre_hooks_.erase(id); });
  }

  void set_requires_grad(bool on) {
    for (auto& p : Parameters()) p.set_requires_grad(on);
  }

 protected:
  // A subclass that specialises an existing layer type (tensor-parallel linears) names itself.
  void set_type(std::string type) { type_ = std::move(type); }
  Tensor& register_parameter(const std::string& name, Tensor t, bool requires_grad = true) {
    if (!parameters_.count(name)) param_order_.push_back(name);
    t.set_requires_grad(requires_grad);
    parameters_[name] = std::move(t);
    return parameters_[name];
  }
  // Shares another module's parameter under this module's name (weight tying).
  void alias_parameter(const std::string& name, const Tensor& existing) {
    if (!parameters_.count(name)) param_order_.push_back(name);
    parameters_[name] = existing;
  }
  Tensor& register_buffer(const std::string& name, Tensor t) {
    buffers_[name] = std::move(t);
    return buffers_[name];
  }
  template <class M>
  std::shared_ptr<M> register_module(const std::string& name, std::shared_ptr<M> m) {
    if (!modules_.count(name)) module_order_.push_back(name);
    modules_[name] = m;
    return m;
  }

 private:
  void CollectParameters(TensorList* out, std::unordered_set<const void*>* seen) const {
    for (const auto& name : param_order_) {
      const Tensor& t = parameters_.at(name);
      if (seen->insert(t.unsafeGetTensorImpl()).second) out->push_back(t);
    }
    for (const auto& name : module_order_) modules_.at(name)->CollectParameters(out, seen);
  }
  void CollectModules(const std::string& prefix, std::vector<std::pair<std::string, std::shared_ptr<Module>>>* out,
                      std::unordered_set<Module*>* seen) {
    if (!seen->insert(this).second) return;
    out->emplace_back(prefix, shared_from_this());
    for (const auto& name : module_order_)
      modules_.at(name)->CollectModules(prefix.empty() ? name : prefix + "." + name, out, seen);
  }

  std::string type_;
  std::map<std::string, Tensor> parameters_, buffers_;
  std::map<std::string, std::shared_ptr<Module>> modules_;
  std::vector<std::string> param_order_, module_order_;   // registration order
  std::map<int, PreHook> pre_hooks_;
  std::map<int, PostHook> post_hooks_;
  std::map<int, std::function<void(Module*, size_t, const Tensor&)>> backward_hooks_, backward_pre_hooks_;
  int next_hook_ = 0;
};

}  // namespace itb
