// Data parallelism for the C++ frontend: one process per device, rendezvous through a TCP store
// (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT, as set by infini_run or torchrun),
// gradients averaged bucket by bucket after backward (reference: DistributedDataParallel + Reducer,
// infini_train/src/nn/parallel/ddp/{distributed_data_parallel,reducer}.cc: 25 MB buckets in reverse
// parameter order, average over the group).
//
// Two transports behind one interface: NCCL on GPUs (under ITB_WITH_CUDA; the unique id travels
// through the store, collectives run on the current stream) and, for CPU ranks and tests, the store
// itself (every rank publishes its buffer, all sum the buffers in rank order: slow, deterministic).
#pragma once
#include <torch/csrc/distributed/c10d/TCPStore.hpp>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "module.h"
#ifdef ITB_WITH_CUDA
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAFunctions.h>
#include <nccl.h>
#endif

namespace itb {
namespace dist {

struct Env {
  int rank = 0, world = 1, local_rank = 0, port = 29500;
  std::string addr = "127.0.0.1";
  static Env FromEnvironment() {
    Env e;
    auto geti = [](const char* k, int d) { const char* v = std::getenv(k); return v && *v ? std::atoi(v) : d; };
    e.rank = geti("RANK", 0), e.world = geti("WORLD_SIZE", 1), e.local_rank = geti("LOCAL_RANK", e.rank);
    e.port = geti("MASTER_PORT", 29500);
    if (const char* a = std::getenv("MASTER_ADDR")) e.addr = a;
    return e;
  }
};

class Comm {
 public:
  virtual ~Comm() = default;
  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual void AllReduceSum(Tensor& flat) = 0;        // in place, contiguous fp32
  virtual void Broadcast(Tensor& flat, int root) = 0;  // in place, contiguous
  virtual void Barrier() = 0;
};

inline c10::intrusive_ptr<c10d::TCPStore> MakeStore(const Env& env, int timeout_s = 300) {
  c10d::TCPStoreOptions o;
  o.port = static_cast<uint16_t>(env.port);
  o.isServer = env.rank == 0;
  o.numWorkers = env.world;
  o.timeout = std::chrono::milliseconds(1000LL * timeout_s);
  return c10::make_intrusive<c10d::TCPStore>(env.addr, o);
}

// Collectives through the store, for CPU ranks.
class StoreComm : public Comm {
 public:
  StoreComm(const Env& env, c10::intrusive_ptr<c10d::TCPStore> store) : env_(env), store_(std::move(store)) {}
  int rank() const override { return env_.rank; }
  int world() const override { return env_.world; }
  void AllReduceSum(Tensor& flat) override {
    TORCH_CHECK(flat.is_contiguous() && !flat.is_cuda(), "StoreComm: contiguous CPU tensor required");
    const int64_t n = reduce_seq_++;
    Publish(Key("ar", n, env_.rank), flat);
    Tensor sum = torch::zeros_like(flat);
    for (int r = 0; r < env_.world; ++r) sum += Fetch(Key("ar", n, r), flat);   // rank order: bit-identical on every rank
    flat.copy_(sum);
    // every rank publishes in every all-reduce, so once this rank is in number n all ranks have
    // finished reading number n - 2
    if (n >= 2) store_->deleteKey(Key("ar", n - 2, env_.rank));
  }
  void Broadcast(Tensor& flat, int root) override {
    TORCH_CHECK(flat.is_contiguous() && !flat.is_cuda(), "StoreComm: contiguous CPU tensor required");
    const int64_t n = bcast_seq_++;
    const std::string key = Key("bc", n, root), ack = key + "/ack";
    if (env_.rank == root) {
      Publish(key, flat);
      pending_.push_back(key);
      // the root may run ahead of its readers: drop a buffer only when all of them acknowledged it
      while (!pending_.empty() && store_->add(pending_.front() + "/ack", 0) >= env_.world - 1) {
        store_->deleteKey(pending_.front());
        pending_.erase(pending_.begin());
      }
    } else {
      flat.copy_(Fetch(key, flat));
      store_->add(ack, 1);
    }
  }
  void Barrier() override {
    const std::string key = "itb/bar/" + std::to_string(barrier_seq_++);
    store_->add(key, 1);
    while (store_->add(key, 0) < env_.world) std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }

 private:
  static std::string Key(const char* kind, int64_t n, int r) {
    return std::string("itb/") + kind + "/" + std::to_string(n) + "/" + std::to_string(r);
  }
  void Publish(const std::string& key, const Tensor& t) {
    const uint8_t* p = static_cast<const uint8_t*>(t.data_ptr());
    store_->set(key, std::vector<uint8_t>(p, p + t.nbytes()));
  }
  Tensor Fetch(const std::string& key, const Tensor& like) {
    auto bytes = store_->get(key);   // blocks until the key exists
    TORCH_CHECK(bytes.size() == like.nbytes(), "StoreComm: ranks disagree on the size of ", key);
    Tensor t = torch::empty_like(like);
    std::memcpy(t.data_ptr(), bytes.data(), bytes.size());
    return t;
  }
  Env env_;
  c10::intrusive_ptr<c10d::TCPStore> store_;
  int64_t reduce_seq_ = 0, bcast_seq_ = 0, barrier_seq_ = 0;
  std::vector<std::string> pending_;
};

#ifdef ITB_WITH_CUDA
// NCCL over NVLink / NVSwitch; collectives are enqueued on the caller's current stream.
class NcclComm : public Comm {
 public:
  NcclComm(const Env& env, c10::intrusive_ptr<c10d::TCPStore> store) : env_(env) {
    ncclUniqueId id;
    if (env.rank == 0) {
      Check(ncclGetUniqueId(&id), "ncclGetUniqueId");
      const uint8_t* p = reinterpret_cast<const uint8_t*>(&id);
      store->set("itb/nccl_id", std::vector<uint8_t>(p, p + sizeof(id)));
    } else {
      auto bytes = store->get("itb/nccl_id");
      TORCH_CHECK(bytes.size() == sizeof(id), "bad NCCL id in the store");
      std::memcpy(&id, bytes.data(), sizeof(id));
    }
    Check(ncclCommInitRank(&comm_, env.world, id, env.rank), "ncclCommInitRank");
  }
  ~NcclComm() override {
    if (comm_) ncclCommDestroy(comm_);
  }
  int rank() const override { return env_.rank; }
  int world() const override { return env_.world; }
  void AllReduceSum(Tensor& flat) override {
    TORCH_CHECK(flat.is_cuda() && flat.is_contiguous() && flat.scalar_type() == torch::kFloat32, "NcclComm: fp32 CUDA tensor");
    Check(ncclAllReduce(flat.data_ptr(), flat.data_ptr(), flat.numel(), ncclFloat, ncclSum, comm_,
                        at::cuda::getCurrentCUDAStream().stream()), "ncclAllReduce");
  }
  void Broadcast(Tensor& flat, int root) override {
    TORCH_CHECK(flat.is_cuda() && flat.is_contiguous(), "NcclComm: contiguous CUDA tensor");
    Check(ncclBroadcast(flat.data_ptr(), flat.data_ptr(), flat.nbytes(), ncclChar, root, comm_,
                        at::cuda::getCurrentCUDAStream().stream()), "ncclBroadcast");
  }
  void Barrier() override {
    Tensor t = torch::zeros({1}, torch::dtype(torch::kFloat32).device(torch::kCUDA));
    AllReduceSum(t);
    at::cuda::getCurrentCUDAStream().synchronize();
  }

 private:
  static void Check(ncclResult_t r, const char* what) { TORCH_CHECK(r == ncclSuccess, what, ": ", ncclGetErrorString(r)); }
  Env env_;
  ncclComm_t comm_ = nullptr;
};
#endif

inline std::shared_ptr<Comm> MakeComm(const Env& env, torch::Device device) {
  auto store = MakeStore(env);
#ifdef ITB_WITH_CUDA
  if (device.is_cuda()) {
    c10::cuda::set_device(device.has_index() ? device.index() : static_cast<c10::DeviceIndex>(env.local_rank));
    return std::make_shared<NcclComm>(env, store);
  }
#endif
  TORCH_CHECK(!device.is_cuda(), "this build has no CUDA support");
  return std::make_shared<StoreComm>(env, store);
}

// Wraps a module for data parallelism: parameters start equal to rank 0's, and SyncGradients()
// (call it after the last backward of a step) leaves the group average in every parameter's grad.
class DistributedDataParallel : public Module {
 public:
  static constexpr int64_t kBucketBytes = 25 << 20;
  DistributedDataParallel(std::shared_ptr<Module> module, std::shared_ptr<Comm> comm)
      : Module("DistributedDataParallel"), comm_(std::move(comm)) {
    module_ = register_module("module", std::move(module));
    torch::NoGradGuard g;
    for (auto& p : module_->Parameters()) {
      Tensor flat = p.detach().contiguous().view({-1});
      comm_->Broadcast(flat, 0);
      p.copy_(flat.view(p.sizes()));
    }
    // buckets of trainable parameters in reverse order (the order gradients become ready)
    auto params = module_->Parameters();
    int64_t bytes = 0;
    buckets_.emplace_back();
    for (auto it = params.rbegin(); it != params.rend(); ++it) {
      if (!it->requires_grad()) continue;
      if (bytes > 0 && bytes + it->numel() * 4 > kBucketBytes) {
        buckets_.emplace_back();
        bytes = 0;
      }
      buckets_.back().push_back(*it);
      bytes += it->numel() * 4;
    }
  }
  TensorList Forward(const TensorList& in) override { return (*module_)(in); }
  std::shared_ptr<Module> module() const { return module_; }
  size_t num_buckets() const { return buckets_.size(); }

  void SyncGradients() {
    torch::NoGradGuard g;
    const double inv = 1.0 / comm_->world();
    for (auto& bucket : buckets_) {
      TensorList grads;
      for (auto& p : bucket)
        grads.push_back((p.grad().defined() ? p.grad() : torch::zeros_like(p)).to(torch::kFloat32).reshape({-1}));
      if (grads.empty()) continue;
      Tensor flat = torch::cat(grads).contiguous();
      comm_->AllReduceSum(flat);
      flat.mul_(inv);
      int64_t off = 0;
      for (auto& p : bucket) {
        Tensor piece = flat.narrow(0, off, p.numel()).view(p.sizes());
        if (p.grad().defined()) p.mutable_grad().copy_(piece);
        else p.mutable_grad() = piece.clone();
        off += p.numel();
      }
    }
  }

 private:
  std::shared_ptr<Module> module_;
  std::shared_ptr<Comm> comm_;
  std::vector<TensorList> buckets_;
};

}  // namespace dist
}  // namespace itb
