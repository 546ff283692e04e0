// Free-function collectives and the single-process, multi-device DataParallel of the C++ frontend.
//
// Reference: infini_train/src/nn/parallel/parallel_functional.cc:16-143 (AllReduce / AllGather /
// ReduceScatter / Send / Recv on the default group; Scatter / Gather / BroadcastCoalescedReshape /
// Replicate), src/nn/parallel/data_parallel.cc:22-100 (scatter the batch, replicate the module, run the
// replicas in threads, gather the outputs) and src/autograd/comm.cc:13-124 (the backward of those steps:
// gradients of the replicas are reduce-added onto the source module).
//
// The examples train with one process per GPU (ddp.h); this module is the reference's older
// "parameter server" form, kept because programs written against it exist.  Two things differ from the
// reference, on purpose:
//   * a replica is BUILT by a factory the caller passes (the layers of this frontend keep handles to their
//     parameter tensors, so a replica is a module object of its own, built once); every forward refreshes
//     the replicas' parameter VALUES from the source module, which is what "replicate each forward" means;
//   * the reduce-add of the replicas' gradients starts in a post-accumulate hook of each replica parameter
//     and lands on the source parameters when the backward pass ends, so it also holds when libtorch's
//     engine runs the per-device parts of backward in threads of its own.
#pragma once
#include <torch/csrc/autograd/engine.h>

#include <exception>
#include <mutex>
#include <thread>

#include "module.h"
#include "ops.h"
#include "process_group.h"

namespace itb {
namespace parallel {
namespace function {

inline std::shared_ptr<ProcessGroup> group_or_default(const std::shared_ptr<ProcessGroup>& pg) {
  if (pg) return pg;
  auto d = ProcessGroupFactory::Instance().GetDefaultProcessGroup();
  TORCH_CHECK(d, "no process group given and no default group exists");
  return d;
}
inline std::shared_ptr<Work> AllReduce(Tensor& t, ReduceOp op = ReduceOp::kSum, std::shared_ptr<ProcessGroup> pg = nullptr,
                                       bool async_op = false) {
  return group_or_default(pg)->AllReduce(t, op, async_op);
}
inline std::shared_ptr<Work> AllGather(Tensor& out, const Tensor& in, std::shared_ptr<ProcessGroup> pg = nullptr,
                                       bool async_op = false) {
  return group_or_default(pg)->AllGather(out, in, async_op);
}
inline std::shared_ptr<Work> ReduceScatter(Tensor& out, const Tensor& in, ReduceOp op = ReduceOp::kSum,
                                           std::shared_ptr<ProcessGroup> pg = nullptr, bool async_op = false) {
  return group_or_default(pg)->ReduceScatter(out, in, op, async_op);
}
inline std::shared_ptr<Work> Send(const TensorList& ts, int dst, std::shared_ptr<ProcessGroup> pg = nullptr, bool async_op = false) {
  return group_or_default(pg)->Send(ts, dst, async_op);
}
inline std::shared_ptr<Work> Recv(TensorList& ts, int src, std::shared_ptr<ProcessGroup> pg = nullptr, bool async_op = false) {
  return group_or_default(pg)->Recv(ts, src, async_op);
}

// ---- one process, several devices
// result[d][i] = chunk d of input i along `dim`, on device d.  With fewer chunks than devices (a batch
// smaller than the device count) the trailing devices get no entry: result.size() is the chunk count.
// The copies are differentiable, so a gradient w.r.t. a chunk flows back into the unsplit input.
inline std::vector<TensorList> Scatter(const TensorList& inputs, const std::vector<torch::Device>& devices, int64_t dim = 0) {
  TORCH_CHECK(!devices.empty(), "Scatter: no devices");
  std::vector<TensorList> out;
  for (size_t i = 0; i < inputs.size(); ++i) {
    auto chunks = inputs[i].chunk(static_cast<int64_t>(devices.size()), dim);
    if (i == 0) out.resize(chunks.size());
    TORCH_CHECK(chunks.size() == out.size(), "Scatter: the inputs split into different numbers of chunks");
    for (size_t d = 0; d < chunks.size(); ++d) out[d].push_back(chunks[d].to(devices[d]));
  }
  return out;
}
// result[i] = concatenation over devices of outputs[d][i] along `dim`, on `target`.
inline TensorList Gather(const std::vector<TensorList>& outputs, torch::Device target, int64_t dim = 0) {
  TORCH_CHECK(!outputs.empty(), "Gather: nothing to gather");
  TensorList out;
  for (size_t i = 0; i < outputs[0].size(); ++i) {
    TensorList parts;
    for (const auto& per_device : outputs) {
      TORCH_CHECK(per_device.size() == outputs[0].size(), "Gather: the replicas returned different numbers of outputs");
      // a replica that returned a scalar (a loss) contributes one element
      Tensor t = per_device[i].dim() == 0 ? per_device[i].unsqueeze(0) : per_device[i];
      parts.push_back(t.to(target));
    }
    out.push_back(torch::cat(parts, dim));
  }
  return out;
}
// result[d][i] = tensor i on device d (detached copies: values only).
inline std::vector<TensorList> BroadcastCoalescedReshape(const TensorList& tensors, const std::vector<torch::Device>& devices) {
  std::vector<TensorList> out(devices.size());
  for (size_t d = 0; d < devices.size(); ++d)
    for (const Tensor& t : tensors) out[d].push_back(t.detach().to(devices[d], /*non_blocking=*/false, /*copy=*/true));
  return out;
}

using ModuleFactory = std::function<std::shared_ptr<Module>()>;

// Copies the parameter and buffer values of `network` into `replica` (same structure), in place.
inline void RefreshReplica(const std::shared_ptr<Module>& network, const std::shared_ptr<Module>& replica) {
  torch::NoGradGuard no_grad;
  auto src = network->StateDict();
  for (auto& [name, dst] : replica->StateDict()) {
    auto it = src.find(name);
    TORCH_CHECK(it != src.end(), "replica has a tensor the source module lacks: ", name);
    TORCH_CHECK(it->second.sizes() == dst.sizes(), "replica tensor ", name, " has another shape than the source's");
    Tensor t = dst;
    t.copy_(it->second);
  }
}

// One module per device: device 0 keeps `network` itself, the others get a module built by `make`, moved to
// their device and filled with the source's values.
inline std::vector<std::shared_ptr<Module>> Replicate(const std::shared_ptr<Module>& network, const ModuleFactory& make,
                                                      const std::vector<torch::Device>& devices) {
  std::vector<std::shared_ptr<Module>> out;
  for (size_t d = 0; d < devices.size(); ++d) {
    if (d == 0) {
      out.push_back(network);
      continue;
    }
    auto r = make();
    r->To(devices[d]);
    RefreshReplica(network, r);
    out.push_back(r);
  }
  return out;
}

}  // namespace function

class DataParallel : public Module {
 public:
  static constexpr const char* kType = "DataParallel";
  static constexpr const char* kModuleName = "module";

  // `module` lives on devices[0] (it is moved there); `make` builds a module of the same structure for
  // each further device.  Inputs are split along `dim`, outputs are joined along it on devices[0].
  DataParallel(std::shared_ptr<Module> module, function::ModuleFactory make, std::vector<torch::Device> devices, int64_t dim = 0)
      : Module(kType), make_(std::move(make)), devices_(std::move(devices)), dim_(dim) {
    TORCH_CHECK(!devices_.empty(), "DataParallel: no devices");
    module->To(devices_[0]);
    register_module(kModuleName, module);
  }

  const std::vector<torch::Device>& devices() const { return devices_; }
  std::shared_ptr<Module> module() const { return mutable_module(kModuleName); }
  int64_t replica_forwards() const { return replica_forwards_; }

  TensorList Forward(const TensorList& inputs) override {
    auto source = module();
    for (const Tensor& p : source->Parameters())
      TORCH_CHECK(p.device() == devices_[0], "DataParallel: the module's parameters must be on ", devices_[0], ", found one on ",
                  p.device());
    auto scattered = function::Scatter(inputs, devices_, dim_);
    if (devices_.size() == 1 || scattered.size() == 1) return (*source)(scattered[0]);
    EnsureReplicas(source);
    for (size_t d = 1; d < scattered.size(); ++d) function::RefreshReplica(source, replicas_[d]);

    const size_t n = scattered.size();
    std::vector<TensorList> outputs(n);
    std::vector<std::exception_ptr> errors(n);
    const bool grad_on = torch::GradMode::is_enabled();
    const auto autocast = autocast_state();
    auto worker = [&](size_t d) {
      try {
        // grad mode and the autocast state are thread-local: the replica threads take the caller's
        torch::AutoGradMode mode(grad_on);
        autocast_state() = autocast;
        c10::OptionalDeviceGuard guard(devices_[d]);
        outputs[d] = (*replicas_[d])(scattered[d]);
      } catch (...) {
        errors[d] = std::current_exception();
      }
    };
    std::vector<std::thread> threads;
    for (size_t d = 1; d < n; ++d) threads.emplace_back(worker, d);
    worker(0);
    for (auto& t : threads) t.join();
    for (auto& e : errors)
      if (e) std::rethrow_exception(e);
    replica_forwards_ += static_cast<int64_t>(n);
    return function::Gather(outputs, devices_[0], dim_);
  }

 private:
  // Gradients of the replicas, summed per source parameter on the source's device while backward runs,
  // and added onto the source's .grad once the whole backward pass has finished (a callback the autograd
  // engine runs at the end of the pass, in the thread that called backward).  Folding at the end keeps the
  // engine's own accumulation into the source parameter and this sum from touching .grad at the same time
  // when the engine runs each device's part of backward in a thread of its own.
  struct Pending {
    std::mutex mu;
    TensorList masters, sums;
    bool queued = false;
    void Fold() {
      std::lock_guard<std::mutex> lock(mu);
      torch::NoGradGuard no_grad;
      for (size_t i = 0; i < masters.size(); ++i) {
        if (!sums[i].defined()) continue;
        if (masters[i].grad().defined()) masters[i].mutable_grad().add_(sums[i]);
        else masters[i].mutable_grad() = sums[i];
        sums[i] = Tensor();
      }
      queued = false;
    }
  };
  struct ReduceAddHook : torch::autograd::PostAccumulateGradHook {
    ReduceAddHook(std::shared_ptr<Pending> s, size_t i) : state(std::move(s)), index(i) {}
    void operator()(const torch::autograd::Variable& replica_param) override {
      Tensor p = replica_param;
      if (!p.grad().defined()) return;
      torch::NoGradGuard no_grad;
      Tensor g = p.grad().to(state->masters[index].device());
      if (g.is_same(p.grad())) g = g.clone();
      p.mutable_grad() = Tensor();
      std::lock_guard<std::mutex> lock(state->mu);
      Tensor& sum = state->sums[index];
      if (sum.defined()) sum.add_(g);
      else sum = g;
      if (!state->queued) {
        state->queued = true;
        auto s = state;
        torch::autograd::Engine::get_default_engine().queue_callback([s] { s->Fold(); });
      }
    }
    std::shared_ptr<Pending> state;
    size_t index;
  };
  void EnsureReplicas(const std::shared_ptr<Module>& source) {
    if (!replicas_.empty()) return;
    replicas_ = function::Replicate(source, make_, devices_);
    auto masters = source->Parameters();
    pending_->masters = masters;
    pending_->sums.assign(masters.size(), Tensor());
    for (size_t d = 1; d < replicas_.size(); ++d) {
      auto params = replicas_[d]->Parameters();
      TORCH_CHECK(params.size() == masters.size(), "DataParallel: the factory built a module with ", params.size(),
                  " parameters, the source has ", masters.size());
      for (size_t i = 0; i < params.size(); ++i) {
        TORCH_CHECK(params[i].sizes() == masters[i].sizes(), "DataParallel: parameter ", i, " of the replica has another shape");
        params[i].set_requires_grad(masters[i].requires_grad());
        if (!masters[i].requires_grad()) continue;
        // the replica's gradient moves onto the source parameter's as soon as autograd has accumulated it
        torch::autograd::impl::set_post_acc_grad_hooks(params[i], std::make_unique<ReduceAddHook>(pending_, i));
      }
    }
  }

  function::ModuleFactory make_;
  std::vector<torch::Device> devices_;
  int64_t dim_;
  std::vector<std::shared_ptr<Module>> replicas_;
  std::shared_ptr<Pending> pending_ = std::make_shared<Pending>();
  int64_t replica_forwards_ = 0;
};

}  // namespace parallel
}  // namespace itb
