// Data parallelism for the C++ frontend with gradient communication overlapped with backward:
// DistributedDataParallel in its three modes, the Reducer, the flat parameter / gradient buffers and
// the ZeRO-1/2 DistributedOptimizer.
//
// Reference: infini_train/src/nn/parallel/ddp/distributed_data_parallel.cc:40-165 (modes),
// reducer.cc:56-438 (size-capped buckets in reverse parameter order, 1 MB then 25 MB; per-parameter
// ready hooks; in-order asynchronous all-reduce(avg); finalisation waits on every Work),
// param_and_grad_buffer.cc:149-531 (flat buffers, parameters packed in reverse, 64-element parameter
// starts, bucket ends padded to lcm(dp, 128), buckets of >= 1 M elements, reduce-scatter to the owner
// shard, all-gather of the updated shards), distributed_optimizer.cc:34-137 (one optimizer over the
// rank's shard pieces; Step = finish gradient sync -> base step -> parameter sync).
//
// Gradients live in ONE flat fp32 buffer per model (parameter.grad is a view of it), so a bucket is a
// contiguous message; the ready signal is libtorch's post-accumulate-grad hook on every parameter.
#pragma once
#include <torch/csrc/autograd/function_hook.h>
#include <torch/csrc/autograd/variable.h>

#include <set>

#include "optim.h"
#include "process_group.h"
#define ITB_PLANNERS_INLINE inline
#include "../../runtime/planners.cpp"

namespace itb {
namespace parallel {

struct DistributedDataParallelConfig {
  int first_bucket_cap_mb = 1, normal_bucket_cap_mb = 25;   // Reducer (ZeRO-0)
  bool gradient_bucketing_enabled = true;
  bool overlap_grad_reduce = true;
  int zero_stage = 0;
  bool average_in_collective = true;
  int64_t bucket_size_in_elements = 1000000;               // flat buffers (ZeRO >= 1)
  bool pad_buckets_for_high_nccl_busbw = false;
};

// One flat fp32 parameter buffer and one flat fp32 gradient buffer; every parameter's data and grad
// become views of them.
class ParamAndGradBuffer {
 public:
  struct Bucket {
    int64_t start = 0, end = 0, unpadded = 0;
    std::vector<size_t> params;      // indices into params()
    Tensor param_data, grad_data;    // views [start, end)
  };
  ParamAndGradBuffer(TensorList params, int dp_size, int dp_rank, bool shard, int64_t bucket_elems = 1000000, bool pad_busbw = false)
      : params_(std::move(params)), dp_size_(dp_size), dp_rank_(dp_rank) {
    TORCH_CHECK(!params_.empty(), "ParamAndGradBuffer needs at least one parameter");
    std::vector<int64_t> numels;
    for (auto& p : params_) {
      TORCH_CHECK(p.scalar_type() == torch::kFloat32, "flat buffers hold fp32 parameters");
      numels.push_back(p.numel());
    }
    layout_ = PlanFlatLayout(numels, dp_size, shard, bucket_elems, pad_busbw);
    auto opts = params_[0].options().requires_grad(false);
    param_buffer = torch::zeros({layout_.numel}, opts);
    grad_buffer = torch::zeros({layout_.numel}, opts);
    buckets_.resize(layout_.bucket_start.size());
    torch::NoGradGuard ng;
    for (size_t i = 0; i < params_.size(); ++i) {
      const int64_t s = layout_.param_start[i], e = layout_.param_end[i];
      Tensor view = param_buffer.narrow(0, s, e - s).view(params_[i].sizes());
      view.copy_(params_[i]);
      params_[i].set_data(view);
      params_[i].mutable_grad() = grad_buffer.narrow(0, s, e - s).view(params_[i].sizes());
      buckets_[layout_.param_bucket[i]].params.push_back(i);
    }
    for (size_t b = 0; b < buckets_.size(); ++b) {
      buckets_[b].start = layout_.bucket_start[b], buckets_[b].end = layout_.bucket_end[b];
      buckets_[b].unpadded = layout_.bucket_unpadded[b];
      buckets_[b].param_data = param_buffer.narrow(0, buckets_[b].start, buckets_[b].end - buckets_[b].start);
      buckets_[b].grad_data = grad_buffer.narrow(0, buckets_[b].start, buckets_[b].end - buckets_[b].start);
    }
  }
  const TensorList& params() const { return params_; }
  std::vector<Bucket>& buckets() { return buckets_; }
  const FlatLayoutResult& layout() const { return layout_; }
  // [start, end) of `rank`'s shard inside bucket b (bucket-relative)
  std::pair<int64_t, int64_t> shard_range(size_t b, int rank) const {
    const int64_t n = (buckets_[b].end - buckets_[b].start) / dp_size_;
    return {rank * n, (rank + 1) * n};
  }
  void zero_grads() { grad_buffer.zero_(); }
  // After ZeroGrad(set_to_none) dropped them: the grad views point into the buffer again.
  void rebind_grads() {
    for (size_t i = 0; i < params_.size(); ++i)
      if (!params_[i].grad().defined())
        params_[i].mutable_grad() =
            grad_buffer.narrow(0, layout_.param_start[i], layout_.param_end[i] - layout_.param_start[i]).view(params_[i].sizes());
  }
  int dp_size() const { return dp_size_; }
  int dp_rank() const { return dp_rank_; }
  Tensor param_buffer, grad_buffer;

 private:
  TensorList params_;
  int dp_size_, dp_rank_;
  FlatLayoutResult layout_;
  std::vector<Bucket> buckets_;
};

// Reverse-order, size-capped bucket assignment of the Reducer: the first bucket closes at
// `first_cap` bytes so that communication starts early, the others at `cap` bytes; a bucket may
// exceed its cap by one tensor (reference: reducer.cc:56-139).  Returns parameter indices per bucket.
inline std::vector<std::vector<size_t>> ComputeBucketAssignmentBySize(const TensorList& params, int64_t first_cap, int64_t cap) {
  std::vector<std::vector<size_t>> out(1);
  int64_t bytes = 0;
  for (size_t k = params.size(); k-- > 0;) {
    out.back().push_back(k);
    bytes += params[k].numel() * params[k].element_size();
    if (bytes >= (out.size() == 1 ? first_cap : cap) && k > 0) {
      out.emplace_back();
      bytes = 0;
    }
  }
  if (out.back().empty()) out.pop_back();
  return out;
}

// The wrapper module.  Modes, as in the reference:
//   * gradient_bucketing_enabled = false: one all-reduce(avg) per parameter, from its ready hook;
//   * ZeRO-0 (default): Reducer buckets, all-reduced asynchronously as backward fills them;
//   * ZeRO-1 / 2: flat buffers; every bucket is reduce-scattered to its owner shard as soon as its
//     last gradient arrives; DistributedOptimizer updates the shards and all-gathers the parameters.
// Call FinishGradSync() after the last backward of a step (DistributedOptimizer::Step does).
class DistributedDataParallel : public Module {
 public:
  DistributedDataParallel(std::shared_ptr<Module> module, std::shared_ptr<ProcessGroup> pg, DistributedDataParallelConfig config = {})
      : Module("DistributedDataParallel"), config_(config), pg_(std::move(pg)) {
    TORCH_CHECK(config_.zero_stage >= 0 && config_.zero_stage <= 2, "ZeRO-3 (parameter partitioning) is not supported");
    module_ = register_module("module", std::move(module));
    const int dp = pg_ ? pg_->size() : 1;
    {
      torch::NoGradGuard g;   // replicas start from rank 0's parameters
      if (dp > 1)
        for (auto& p : module_->Parameters()) {
          Tensor flat = p.detach().contiguous().view({-1}).clone();
          pg_->BroadCast(flat, 0);
          p.copy_(flat.view(p.sizes()));
        }
    }
    for (auto& p : module_->Parameters())
      if (p.requires_grad()) trainable_.push_back(p);
    if (trainable_.empty()) return;
    const bool flat_ok = std::all_of(trainable_.begin(), trainable_.end(), [](const Tensor& p) { return p.scalar_type() == torch::kFloat32; });
    if (!config_.gradient_bucketing_enabled || !flat_ok) {
      per_param_ = true;
    } else {
      buffer_ = std::make_unique<ParamAndGradBuffer>(trainable_, dp, pg_ ? pg_->rank() : 0, config_.zero_stage >= 1,
                                                     config_.bucket_size_in_elements, config_.pad_buckets_for_high_nccl_busbw);
      if (config_.zero_stage == 0) {
        // Reducer buckets are runs of consecutive parameters in reverse order: contiguous slices of
        // the flat gradient buffer (it is packed in the same order).
        auto idx = ComputeBucketAssignmentBySize(trainable_, int64_t(config_.first_bucket_cap_mb) << 20, int64_t(config_.normal_bucket_cap_mb) << 20);
        for (auto& ids : idx) {
          Group g;
          int64_t lo = buffer_->layout().numel, hi = 0;
          for (size_t i : ids) {
            lo = std::min(lo, buffer_->layout().param_start[i]);
            hi = std::max(hi, buffer_->layout().param_end[i]);
            owner_[i] = groups_.size();
          }
          g.grads = buffer_->grad_buffer.narrow(0, lo, hi - lo);
          g.expected = ids.size();
          groups_.push_back(std::move(g));
        }
      } else {
        for (size_t b = 0; b < buffer_->buckets().size(); ++b) {
          Group g;
          g.grads = buffer_->buckets()[b].grad_data;
          g.expected = buffer_->buckets()[b].params.size();
          g.bucket = static_cast<int>(b);
          for (size_t i : buffer_->buckets()[b].params) owner_[i] = groups_.size();
          groups_.push_back(std::move(g));
        }
      }
    }
    for (size_t i = 0; i < trainable_.size(); ++i)
      torch::autograd::impl::set_post_acc_grad_hooks(trainable_[i], std::make_unique<ReadyHook>(this, i));
  }
  ~DistributedDataParallel() override {
    for (auto& p : trainable_) torch::autograd::impl::set_post_acc_grad_hooks(p, nullptr);
  }
  TensorList Forward(const TensorList& in) override {
    if (buffer_) buffer_->rebind_grads();
    finished_ = false;
    return (*module_)(in);
  }
  std::shared_ptr<Module> module() const { return module_; }
  const DistributedDataParallelConfig& config() const { return config_; }
  ParamAndGradBuffer* buffer() const { return buffer_.get(); }
  std::shared_ptr<ProcessGroup> process_group() const { return pg_; }
  size_t num_buckets() const { return groups_.size(); }
  int64_t launches_during_backward() const { return launched_in_backward_; }

  // Gradient accumulation: backward passes before the last micro-batch only add into the buffers.
  void set_sync(bool on) { sync_enabled_ = on; }

  // Launches what has not been launched (parameters that received no gradient this step), then
  // makes the current stream wait for every collective.  Idempotent within a step.
  void FinishGradSync() {
    if (finished_) return;
    finished_ = true;
    if (!pg_ || pg_->size() == 1 || per_param_) {
      Reset();
      return;
    }
    for (size_t g = 0; g < groups_.size(); ++g)
      if (!groups_[g].launched) Launch(g, /*in_backward=*/false);
    for (auto& g : groups_)
      if (g.work) {
        g.work->WaitNonBlocking();
        g.work.reset();
      }
    Reset();
  }
  void ZeroGrad() {
    finished_ = false;
    if (buffer_) {
      buffer_->zero_grads();
      buffer_->rebind_grads();   // an optimizer's ZeroGrad may have dropped the views
    } else
      for (auto& p : trainable_) p.mutable_grad() = Tensor();
  }

 private:
  struct Group {
    Tensor grads;            // contiguous slice of the flat gradient buffer
    size_t expected = 0, ready = 0;
    int bucket = -1;         // ZeRO: index into buffer()->buckets()
    bool launched = false;
    std::shared_ptr<Work> work;
  };
  struct ReadyHook : torch::autograd::PostAccumulateGradHook {
    ReadyHook(DistributedDataParallel* d, size_t i) : ddp(d), index(i) {}
    void operator()(const torch::autograd::Variable&) override { ddp->OnGradReady(index); }
    DistributedDataParallel* ddp;
    size_t index;
  };
  void OnGradReady(size_t i) {
    finished_ = false;
    if (!sync_enabled_ || !pg_ || pg_->size() == 1) return;
    if (per_param_) {
      Tensor g = trainable_[i].mutable_grad();
      if (!g.defined()) return;
      Tensor flat = g.is_contiguous() ? g : g.contiguous();
      pg_->AllReduce(flat, ReduceOp::kAvg);
      if (!g.is_contiguous()) g.copy_(flat);
      return;
    }
    if (!config_.overlap_grad_reduce || !seen_.insert(i).second) return;
    Group& g = groups_[owner_.at(i)];
    if (++g.ready < g.expected) return;
    // buckets leave in order (the order every rank launches them in)
    while (next_ < groups_.size() && groups_[next_].ready >= groups_[next_].expected) Launch(next_++, /*in_backward=*/true);
  }
  void Launch(size_t gi, bool in_backward) {
    Group& g = groups_[gi];
    g.launched = true;
    const ReduceOp op = config_.average_in_collective ? ReduceOp::kAvg : ReduceOp::kSum;
    if (config_.zero_stage == 0) {
      g.work = pg_->AllReduce(g.grads, op, /*async_op=*/true);
    } else {
      auto r = buffer_->shard_range(static_cast<size_t>(g.bucket), pg_->rank());
      Tensor shard = g.grads.narrow(0, r.first, r.second - r.first);
      g.work = pg_->ReduceScatter(shard, g.grads, op, /*async_op=*/true);
    }
    if (in_backward) ++launched_in_backward_;
  }
  void Reset() {
    for (auto& g : groups_) g.ready = 0, g.launched = false;
    seen_.clear();
    next_ = 0;
  }

  DistributedDataParallelConfig config_;
  std::shared_ptr<Module> module_;
  std::shared_ptr<ProcessGroup> pg_;
  TensorList trainable_;
  std::unique_ptr<ParamAndGradBuffer> buffer_;
  std::vector<Group> groups_;
  std::map<size_t, size_t> owner_;     // parameter index -> group
  std::set<size_t> seen_;
  size_t next_ = 0;
  bool per_param_ = false, sync_enabled_ = true, finished_ = false;
  int64_t launched_in_backward_ = 0;
};

// ZeRO-1 / ZeRO-2: the base optimizer sees ONE tensor per bucket -- this rank's contiguous 1/dp slice
// of the flat parameter buffer, with the matching slice of the reduce-scattered gradients -- so the
// optimizer state exists only for the shard.  Step = finish the gradient sync -> update the shards ->
// all-gather every bucket's shards into the full parameter buffer.
class DistributedOptimizer : public optim::Optimizer {
 public:
  using Creator = optim::OptimizerCreator;
  DistributedOptimizer(const Creator& creator, std::vector<DistributedDataParallel*> chunks) : optim::Optimizer({}), chunks_(std::move(chunks)) {
    TensorList shards;
    for (auto* ddp : chunks_) {
      TORCH_CHECK(ddp->config().zero_stage >= 1 && ddp->buffer(), "DistributedOptimizer needs zero_stage >= 1");
      auto* buf = ddp->buffer();
      for (size_t b = 0; b < buf->buckets().size(); ++b) {
        auto r = buf->shard_range(b, buf->dp_rank());
        Tensor p = buf->buckets()[b].param_data.narrow(0, r.first, r.second - r.first);
        p.set_requires_grad(true);
        p.mutable_grad() = buf->buckets()[b].grad_data.narrow(0, r.first, r.second - r.first);
        shards.push_back(p);
      }
      for (auto& p : buf->params()) params_.push_back(p);
    }
    base_ = creator(shards);
    shards_ = shards;
  }
  void ZeroGrad(bool = true) override {
    for (auto* ddp : chunks_) ddp->ZeroGrad();
  }
  void Step() override {
    for (auto* ddp : chunks_) ddp->FinishGradSync();
    base_->Step();
    // parameter sync: every rank's updated shard into everybody's full buffer
    std::vector<std::shared_ptr<Work>> works;
    size_t k = 0;
    for (auto* ddp : chunks_) {
      auto pg = ddp->process_group();
      auto* buf = ddp->buffer();
      for (size_t b = 0; b < buf->buckets().size(); ++b, ++k) {
        if (!pg || pg->size() == 1) continue;
        Tensor shard = shards_[k].detach();
        works.push_back(pg->AllGather(buf->buckets()[b].param_data, shard, /*async_op=*/true));
      }
    }
    for (auto& w : works) w->WaitNonBlocking();
    // the buffer changed under the parameters' views: anything cached per parameter version (the
    // bf16 copies of the weights) must see a new version
    for (auto& p : params_) torch::autograd::impl::bump_version(p);
  }
  std::map<std::string, Tensor> StateDict() const override { return base_->StateDict(); }
  void LoadStateDict(const std::map<std::string, Tensor>& sd) override { base_->LoadStateDict(sd); }
  optim::Optimizer* base() const { return base_.get(); }

 private:
  std::vector<DistributedDataParallel*> chunks_;
  std::unique_ptr<optim::Optimizer> base_;
  TensorList shards_;
};

// Elastic resume: the state of a ZeRO optimizer that `old_states.size()` data-parallel ranks saved, re-cut for
// rank `new_rank` of a job with `new_dp` data-parallel ranks (same model, same tensor / pipeline coordinates).
// A saved state holds, per family of keys "<prefix>.<k>" (adam.m, adam.v), rank r's contiguous 1/dp slice of
// flat bucket k; the bucket layout depends on dp (bucket ends are padded to lcm(dp, 128)), so the slices are
// put back into the old flat layout, moved parameter by parameter into the new one and cut again.  Keys without
// a bucket index (adam.t) are taken from the first rank.  `chunk_numels[c]` lists the parameter sizes of the
// c-th wrapped module chunk in the order its ParamAndGradBuffer was built from.  The reference resumes only on
// the topology that saved (checkpoint_manager.cc:56-63).
inline std::map<std::string, Tensor> ReshardZeroState(const std::vector<std::map<std::string, Tensor>>& old_states,
                                                      const std::vector<std::vector<int64_t>>& chunk_numels, int new_dp, int new_rank,
                                                      int64_t bucket_elems = 1000000, bool pad_busbw = false) {
  TORCH_CHECK(!old_states.empty() && new_dp >= 1 && new_rank >= 0 && new_rank < new_dp, "ReshardZeroState: bad arguments");
  const int old_dp = static_cast<int>(old_states.size());
  std::map<std::string, Tensor> out;
  std::set<std::string> families;
  for (const auto& [key, t] : old_states[0]) {
    const size_t dot = key.rfind('.');
    const bool indexed = dot != std::string::npos && dot + 1 < key.size() &&
                         key.find_first_not_of("0123456789", dot + 1) == std::string::npos;
    if (indexed) families.insert(key.substr(0, dot));
    else out[key] = t.clone();
  }
  for (const auto& family : families) {
    size_t k_old = 0, k_new = 0;
    for (const auto& numels : chunk_numels) {
      const FlatLayoutResult lo = PlanFlatLayout(numels, old_dp, true, bucket_elems, pad_busbw);
      const FlatLayoutResult ln = PlanFlatLayout(numels, new_dp, true, bucket_elems, pad_busbw);
      Tensor flat_old, flat_new;
      for (size_t b = 0; b < lo.bucket_start.size(); ++b) {
        const int64_t n = (lo.bucket_end[b] - lo.bucket_start[b]) / old_dp;
        for (int r = 0; r < old_dp; ++r) {
          auto it = old_states[r].find(family + "." + std::to_string(k_old + b));
          TORCH_CHECK(it != old_states[r].end(), "ReshardZeroState: rank ", r, " has no ", family, ".", k_old + b);
          TORCH_CHECK(it->second.numel() == n, "ReshardZeroState: ", family, ".", k_old + b, " of rank ", r, " holds ", it->second.numel(),
                      " elements, the layout of ", old_dp, " ranks gives ", n, " (was the checkpoint written by another model?)");
          if (!flat_old.defined()) {
            flat_old = torch::zeros({lo.numel}, it->second.options().device(torch::kCPU));
            flat_new = torch::zeros({ln.numel}, flat_old.options());
          }
          flat_old.narrow(0, lo.bucket_start[b] + r * n, n).copy_(it->second.view({-1}));
        }
      }
      for (size_t i = 0; i < numels.size(); ++i)
        flat_new.narrow(0, ln.param_start[i], numels[i]).copy_(flat_old.narrow(0, lo.param_start[i], numels[i]));
      for (size_t b = 0; b < ln.bucket_start.size(); ++b) {
        const int64_t n = (ln.bucket_end[b] - ln.bucket_start[b]) / new_dp;
        out[family + "." + std::to_string(k_new + b)] = flat_new.narrow(0, ln.bucket_start[b] + new_rank * n, n).clone();
      }
      k_old += lo.bucket_start.size(), k_new += ln.bucket_start.size();
    }
  }
  return out;
}

}  // namespace parallel
}  // namespace itb
