// Pipeline parallelism for the C++ frontend: runs a GPipe or interleaved-1F1B task list over the
// chunks of layers that this stage owns, moving activations forward and their gradients backward
// between neighbouring stages.
//
// Reference: infini_train/src/nn/parallel/pp/pipeline_schedule.cc:27-329 (the task tables, printed once
// by the first stage; per task: receive, run the chunk, send), pipeline_stage.cc (the chunks of one
// stage), send_recv.cc:19-136 (ISend / IRecv as autograd functions), pipeline_parallel.cc:42-115
// (GetStageInfo, TrainStep).  The task tables come from the same planner the Python package uses
// (GpipeSchedule / Interleaved1F1BSchedule).
//
// Transfers are organised by STEP of the task table, not by task: after the tasks of step b every
// stage runs one exchange that holds its sends of what step b produced and its receives of what the
// neighbours produced in step b, all in one batched point-to-point call.  Two neighbours that owe each
// other a tensor in the same step (an activation one way, a gradient the other, the steady state of
// 1F1B) therefore cannot block one another, and an exchange of step b depends only on exchanges of
// earlier steps, whatever the transport's buffering.  A tensor that arrives before its consumer's
// step waits in a small map.
#pragma once
#include <functional>
#include <tuple>

#include "ddp.h"
#include "process_group.h"

namespace itb {
namespace parallel {

struct PipelineConfig {
  int num_stages = 1, stage = 0, vpp = 1, num_micro_batches = 1;
  std::string schedule = "1f1b";                 // "gpipe" | "1f1b"
  std::vector<int64_t> boundary_shape;           // activation of one micro-batch between chunks: [B_mb, T (/ sp), C]
  torch::Dtype boundary_dtype = torch::kFloat32;
  torch::Device device = torch::Device(torch::kCPU);
};

// Text table of a schedule, one row per step and one column per stage ("F3.1" = forward of micro-batch
// 3 on local chunk 1).
inline std::string FormatScheduleTable(const std::vector<PipeTask>& tasks, int num_stages) {
  int steps = 0;
  for (const auto& t : tasks) steps = std::max(steps, t.step + 1);
  std::vector<std::vector<std::string>> cell(steps, std::vector<std::string>(num_stages));
  for (const auto& t : tasks) {
    std::string& c = cell[t.step][t.stage];
    if (!c.empty()) c += ",";
    c += std::string(t.is_forward ? "F" : "B") + std::to_string(t.microbatch) + "." + std::to_string(t.local_chunk);
  }
  std::ostringstream os;
  os << "step";
  for (int s = 0; s < num_stages; ++s) os << " | stage " << s;
  os << "\n";
  for (int b = 0; b < steps; ++b) {
    os << b;
    for (int s = 0; s < num_stages; ++s) os << " | " << (cell[b][s].empty() ? "-" : cell[b][s]);
    os << "\n";
  }
  return os.str();
}

class PipelineParallel {
 public:
  // chunk_fn(local chunk, input) -> output.  The input of the first chunk of the first stage is the
  // micro-batch's token ids; the output of the last chunk of the last stage goes to the loss.
  using ChunkFn = std::function<Tensor(int64_t, const Tensor&)>;
  using LossFn = std::function<Tensor(const Tensor&, const Tensor&)>;
  // Called before every backward task with (local chunk, whether it is that chunk's last backward of
  // the step): the place to switch gradient synchronisation on.
  using BackwardNotice = std::function<void(int64_t, bool)>;

  PipelineParallel(PipelineConfig config, ChunkFn chunk_fn, std::shared_ptr<ProcessGroup> pg)
      : cfg_(std::move(config)), chunk_fn_(std::move(chunk_fn)), pg_(std::move(pg)) {
    TORCH_CHECK(cfg_.num_stages >= 1 && cfg_.stage >= 0 && cfg_.stage < cfg_.num_stages, "bad pipeline coordinates");
    TORCH_CHECK(cfg_.num_stages == 1 || pg_, "a pipeline of several stages needs a process group");
    TORCH_CHECK(cfg_.schedule == "gpipe" || cfg_.schedule == "1f1b", "schedule must be gpipe or 1f1b");
    tasks_ = cfg_.schedule == "gpipe" ? GpipeSchedule(cfg_.num_micro_batches, cfg_.num_stages, cfg_.vpp)
                                      : Interleaved1F1BSchedule(cfg_.num_micro_batches, cfg_.num_stages, cfg_.vpp);
    for (const auto& t : tasks_) num_steps_ = std::max(num_steps_, t.step + 1);
    // what every step produces for another chunk: (step, is activation, micro-batch, consumer's global chunk)
    std::map<Key, int> consumer_step;
    for (const auto& t : tasks_) consumer_step[Key{t.is_forward, t.microbatch, t.global_chunk}] = t.step;
    for (const auto& t : tasks_) {
      if (t.is_forward && !t.is_last_chunk) AddMessage(t, /*act=*/true, t.global_chunk + 1, consumer_step);
      if (!t.is_forward && !t.is_first_chunk) AddMessage(t, /*act=*/false, t.global_chunk - 1, consumer_step);
    }
  }
  const std::vector<PipeTask>& tasks() const { return tasks_; }
  std::string ScheduleTable() const { return FormatScheduleTable(tasks_, cfg_.num_stages); }
  int64_t exchanges() const { return exchanges_; }

  // One optimizer step on one batch (reference: PipelineParallel::TrainStep -> PipelineSchedule::Step,
  // pp/pipeline_schedule.cc:275-295): the batch is cut into `num_micro_batches` equal parts along dimension 0
  // (the input on the first stage, the target on the last; the other stages may pass undefined tensors),
  // gradients are cleared, the schedule runs, the optimizer steps.  Returns the mean loss on the last stage.
  double TrainStep(const Tensor& input, const Tensor& target, optim::Optimizer& optimizer, const LossFn& loss_fn,
                   const BackwardNotice& notice = {}) {
    const int n = cfg_.num_micro_batches;
    auto split = [n](const Tensor& t, const char* what) {
      std::vector<Tensor> parts(n);
      if (!t.defined()) return parts;
      TORCH_CHECK(t.size(0) % n == 0, "TrainStep: the ", what, " batch of ", t.size(0), " does not split into ", n, " micro-batches");
      auto chunks = t.split(t.size(0) / n, 0);
      for (int i = 0; i < n; ++i) parts[i] = chunks[i];
      return parts;
    };
    optimizer.ZeroGrad();
    const double loss = StepMicroBatches(split(input, "input"), split(target, "target"), loss_fn, notice);
    optimizer.Step();
    return loss;
  }

  // One optimizer step's worth of micro-batches.  `inputs` matter on the first stage, `targets` on the
  // last; returns the mean loss over the micro-batches on the last stage, 0 elsewhere.
  double StepMicroBatches(const std::vector<Tensor>& inputs, const std::vector<Tensor>& targets, const LossFn& loss_fn,
                          const BackwardNotice& notice = {}) {
    const int n = cfg_.num_micro_batches, me = cfg_.stage;
    std::map<int64_t, int> last_bwd;
    for (const auto& t : tasks_)
      if (t.stage == me && !t.is_forward) last_bwd[t.local_chunk] = std::max(last_bwd[t.local_chunk], t.step * n + t.microbatch);
    std::map<Key, Arrived> inbox;
    std::map<std::pair<int64_t, int>, std::pair<Tensor, Tensor>> saved;   // (local chunk, micro-batch) -> (input leaf, output)
    std::vector<std::pair<std::shared_ptr<Work>, TensorList>> in_flight;
    Tensor total = torch::zeros({}, torch::dtype(torch::kFloat32).device(cfg_.device));
    size_t cursor = 0;
    for (int b = 0; b < num_steps_; ++b) {
      std::map<Key, Tensor> outbox;
      for (; cursor < tasks_.size() && tasks_[cursor].step == b; ++cursor) {
        const PipeTask& t = tasks_[cursor];
        if (t.stage != me) continue;
        const auto slot = std::make_pair(static_cast<int64_t>(t.local_chunk), t.microbatch);
        if (t.is_forward) {
          Tensor x_in, out;
          if (t.is_first_chunk) {
            out = chunk_fn_(t.local_chunk, inputs.at(t.microbatch));
          } else {
            x_in = Take(&inbox, Key{true, t.microbatch, t.global_chunk});
            x_in.set_requires_grad(true);
            out = chunk_fn_(t.local_chunk, x_in);
          }
          saved[slot] = {x_in, out};
          if (!t.is_last_chunk) outbox[Key{true, t.microbatch, t.global_chunk + 1}] = out.detach().to(cfg_.boundary_dtype).contiguous();
        } else {
          auto it = saved.find(slot);
          TORCH_CHECK(it != saved.end(), "backward of a micro-batch whose forward did not run here");
          auto [x_in, out] = it->second;
          saved.erase(it);
          if (notice) notice(t.local_chunk, t.step * n + t.microbatch == last_bwd[t.local_chunk]);
          if (t.is_last_chunk) {
            Tensor loss = loss_fn(out, targets.at(t.microbatch)) / static_cast<double>(n);
            total += loss.detach().to(torch::kFloat32);
            loss.backward();
          } else {
            Tensor g = Take(&inbox, Key{false, t.microbatch, t.global_chunk});
            out.backward(g.to(out.scalar_type()));
          }
          if (!t.is_first_chunk) {
            TORCH_CHECK(x_in.grad().defined(), "no gradient reached the input of chunk ", t.global_chunk);
            outbox[Key{false, t.microbatch, t.global_chunk - 1}] = x_in.grad().to(cfg_.boundary_dtype).contiguous();
          }
        }
      }
      Exchange(b, &outbox, &inbox, &in_flight);
    }
    for (auto& f : in_flight) f.first->WaitNonBlocking();
    TORCH_CHECK(inbox.empty() && saved.empty(), "pipeline step ended with undelivered tensors");
    return total.item<float>();
  }

 private:
  using Key = std::tuple<bool, int, int>;   // (activation?, micro-batch, consumer's global chunk)
  struct Message {
    Key key;
    int src_stage, dst_stage;
  };
  struct Arrived {
    Tensor tensor;
    std::shared_ptr<Work> work;
  };
  void AddMessage(const PipeTask& t, bool act, int consumer_chunk, const std::map<Key, int>& consumer_step) {
    const Key key{act, t.microbatch, consumer_chunk};
    auto it = consumer_step.find(Key{act, t.microbatch, consumer_chunk});
    TORCH_CHECK(it != consumer_step.end() && it->second > t.step, "schedule consumes a tensor before the step after its production");
    if (static_cast<int>(messages_.size()) <= t.step) messages_.resize(t.step + 1);
    messages_[t.step].push_back(Message{key, t.stage, consumer_chunk % cfg_.num_stages});
  }
  Tensor Take(std::map<Key, Arrived>* inbox, const Key& key) {
    auto it = inbox->find(key);
    TORCH_CHECK(it != inbox->end(), "pipeline: a tensor this task needs has not been received");
    if (it->second.work) it->second.work->WaitNonBlocking();
    Tensor t = it->second.tensor;
    inbox->erase(it);
    return t;
  }
  // Sends of what this stage produced in step b and receives of what the others produced for it,
  // in the order of the task table on both sides.
  void Exchange(int b, std::map<Key, Tensor>* outbox, std::map<Key, Arrived>* inbox,
                std::vector<std::pair<std::shared_ptr<Work>, TensorList>>* in_flight) {
    if (b >= static_cast<int>(messages_.size())) return;
    std::vector<P2POp> ops;
    TensorList sent;
    std::vector<Key> received;
    for (const Message& m : messages_[b]) {
      if (m.src_stage == cfg_.stage && m.dst_stage == cfg_.stage) {   // one stage holds both chunks (a single-stage ring)
        (*inbox)[m.key] = Arrived{outbox->at(m.key), nullptr};
      } else if (m.src_stage == cfg_.stage) {
        ops.push_back(P2POp{true, outbox->at(m.key), m.dst_stage});
        sent.push_back(ops.back().tensor);
      } else if (m.dst_stage == cfg_.stage) {
        Tensor buf = torch::empty(cfg_.boundary_shape, torch::dtype(cfg_.boundary_dtype).device(cfg_.device));
        ops.push_back(P2POp{false, buf, m.src_stage});
        received.push_back(m.key);
        (*inbox)[m.key] = Arrived{buf, nullptr};
      }
    }
    if (ops.empty()) return;
    auto work = pg_->BatchSendRecv(ops, /*async_op=*/true);
    ++exchanges_;
    for (const Key& k : received) (*inbox)[k].work = work;
    if (!sent.empty()) in_flight->emplace_back(work, sent);   // the payloads live until the step's end
  }

  PipelineConfig cfg_;
  ChunkFn chunk_fn_;
  std::shared_ptr<ProcessGroup> pg_;
  std::vector<PipeTask> tasks_;
  std::vector<std::vector<Message>> messages_;   // by producing step
  int num_steps_ = 0;
  int64_t exchanges_ = 0;
};

}  // namespace parallel
}  // namespace itb
