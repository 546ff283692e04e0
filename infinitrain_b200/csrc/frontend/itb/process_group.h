// Process groups for the C++ frontend: collectives and point-to-point transfers among a subset of the
// job's ranks, with the completion handle (`Work`) of the asynchronous forms.
//
// Reference: infini_train/src/nn/parallel/process_group.cc:118-249 (per-group high-priority
// communication stream; ready event on the compute stream -> collective on the communication stream ->
// done event; a synchronous call makes the compute stream wait on the done event, an asynchronous one
// returns the Work), work.cc:37-141 (WaitBlocking with a time-out, WaitNonBlocking, IsCompleted,
// IsSuccess), process_group.h:40-72 (AllReduce / AllGather / ReduceScatter / Send / Recv / BroadCast),
// and the group names "TP<i>" / "DP<i>" / "PP<i>" of the factory.
//
// Two transports behind one interface:
//   * NcclProcessGroup (under ITB_WITH_CUDA): one NCCL communicator per group, its unique id published
//     through the job's TCP store; collectives run on the group's own stream with the event protocol
//     above, so backward keeps computing while a bucket is reduced.
//   * StoreProcessGroup: CPU ranks exchange buffers through the TCP store itself (every rank publishes
//     its contribution, everybody combines them in group-rank order: slow, deterministic, and enough
//     to run every parallel strategy of the framework on a machine without GPUs).
#pragma once
#include <torch/csrc/distributed/c10d/FileStore.hpp>
#include <torch/csrc/distributed/c10d/TCPStore.hpp>

#include <atomic>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>

#include "module.h"
#include "parallel_env.h"
#include "profiler.h"
#ifdef ITB_WITH_CUDA
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <nccl.h>
#endif

namespace itb {
namespace parallel {

enum class ReduceOp { kSum, kAvg, kMax, kMin, kProd };

// Completion handle of an asynchronous collective.
class Work {
 public:
  virtual ~Work() = default;
  // Host waits until the operation has finished; false when `timeout_ms` (> 0) ran out first.
  virtual bool WaitBlocking(int64_t timeout_ms = 0) = 0;
  // The caller's current stream waits (on the device) for the operation; the host does not block.
  virtual bool WaitNonBlocking() = 0;
  virtual bool IsCompleted() const = 0;
  virtual bool IsSuccess() const { return IsCompleted() && error().empty(); }
  virtual void Synchronize() { WaitBlocking(0); }
  virtual std::string error() const { return std::string(); }
};

// A Work that was complete when it was returned (CPU transport, synchronous calls).
class CompletedWork : public Work {
 public:
  bool WaitBlocking(int64_t) override { return true; }
  bool WaitNonBlocking() override { return true; }
  bool IsCompleted() const override { return true; }
};

// One transfer of a batched point-to-point exchange.
struct P2POp {
  bool is_send;
  Tensor tensor;   // contiguous; a receive fills it in place
  int peer;        // group rank
};

class ProcessGroup {
 public:
  ProcessGroup(std::string name, std::vector<int> ranks, int my_global_rank) : name_(std::move(name)), ranks_(std::move(ranks)) {
    group_rank_ = -1;
    for (size_t i = 0; i < ranks_.size(); ++i)
      if (ranks_[i] == my_global_rank) group_rank_ = static_cast<int>(i);
    TORCH_CHECK(group_rank_ >= 0, "rank ", my_global_rank, " is not a member of group ", name_);
  }
  virtual ~ProcessGroup() = default;
  const std::string& name() const { return name_; }
  int size() const { return static_cast<int>(ranks_.size()); }
  int rank() const { return group_rank_; }                 // this process's rank inside the group
  const std::vector<int>& ranks() const { return ranks_; }  // global ranks, by group rank
  int GetGroupRank(int global_rank) const {
    for (size_t i = 0; i < ranks_.size(); ++i)
      if (ranks_[i] == global_rank) return static_cast<int>(i);
    return -1;
  }

  // In place on a contiguous tensor.
  virtual std::shared_ptr<Work> AllReduce(Tensor& t, ReduceOp op = ReduceOp::kSum, bool async_op = false) = 0;
  // out = concatenation of every rank's `in` by group rank (out.numel() == size() * in.numel()).
  virtual std::shared_ptr<Work> AllGather(Tensor& out, const Tensor& in, bool async_op = false) = 0;
  // out = this rank's slice of the reduction of every rank's `in` (in.numel() == size() * out.numel()).
  virtual std::shared_ptr<Work> ReduceScatter(Tensor& out, const Tensor& in, ReduceOp op = ReduceOp::kSum, bool async_op = false) = 0;
  virtual std::shared_ptr<Work> BroadCast(Tensor& t, int src_group_rank = 0, bool async_op = false) = 0;
  virtual std::shared_ptr<Work> Send(const TensorList& ts, int dst_group_rank, bool async_op = false) = 0;
  virtual std::shared_ptr<Work> Recv(TensorList& ts, int src_group_rank, bool async_op = false) = 0;
  // All transfers of `ops` progress together (one NCCL group), so two ranks that each send to and
  // receive from the other in one exchange cannot block one another.  Transfers between one pair of
  // ranks match in list order.
  virtual std::shared_ptr<Work> BatchSendRecv(std::vector<P2POp>& ops, bool async_op = false) = 0;
  virtual void Barrier() = 0;

  // ---- rooted collectives (reference: src/nn/parallel/process_group.cc:251-401, the legacy DataParallel's
  // transport), built from the calls above so that every transport has them; NCCL overrides Reduce.
  // The reduction of every rank's `t` lands in `t` on dst; the other ranks' tensors keep their values.
  virtual std::shared_ptr<Work> Reduce(Tensor& t, int dst_group_rank, ReduceOp op = ReduceOp::kSum, bool async_op = false) {
    Tensor tmp = t.clone();
    auto w = AllReduce(tmp, op, false);
    if (rank() == dst_group_rank) t.copy_(tmp);
    (void)async_op;
    return w;
  }
  // Sums every tensor of the list onto dst, one reduction per tensor.
  void ReduceAddCoalesced(TensorList& ts, int dst_group_rank) {
    for (Tensor& t : ts) Reduce(t, dst_group_rank, ReduceOp::kSum, false);
  }
  // out = chunk rank() of src's `in` split along `dim` into size() equal parts; `in` is read on src only.
  void Scatter(Tensor& out, const Tensor& in, int src_group_rank, int64_t dim = 0) {
    std::vector<P2POp> ops;
    TensorList chunks;
    if (rank() == src_group_rank) {
      TORCH_CHECK(in.size(dim) % size() == 0, "Scatter: dimension ", dim, " of size ", in.size(dim), " does not split over ", size(), " ranks");
      for (auto& c : in.chunk(size(), dim)) chunks.push_back(c.contiguous());
      for (int r = 0; r < size(); ++r) {
        if (r == rank()) out.copy_(chunks[r]);
        else ops.push_back(P2POp{true, chunks[r], r});
      }
    } else {
      TORCH_CHECK(out.is_contiguous(), "Scatter: contiguous output required");
      ops.push_back(P2POp{false, out, src_group_rank});
    }
    if (!ops.empty()) BatchSendRecv(ops, false);
  }
  // On dst: the concatenation of every rank's `t` along `dim`, by group rank; an undefined tensor elsewhere.
  Tensor Gather(const Tensor& t, int dst_group_rank, int64_t dim = 0) {
    std::vector<P2POp> ops;
    Tensor mine = t.contiguous();
    if (rank() != dst_group_rank) {
      ops.push_back(P2POp{true, mine, dst_group_rank});
      BatchSendRecv(ops, false);
      return Tensor();
    }
    TensorList parts(size());
    for (int r = 0; r < size(); ++r) {
      parts[r] = r == rank() ? mine : torch::empty_like(mine);
      if (r != rank()) ops.push_back(P2POp{false, parts[r], r});
    }
    if (!ops.empty()) BatchSendRecv(ops, false);
    return torch::cat(parts, dim);
  }
  // 0 = healthy; a transport error code otherwise (NCCL: the communicator's asynchronous error).
  virtual int AsyncError() { return 0; }
  // Failure handling (fault_tolerance.h).  Abort() may be called from another thread than the one inside a
  // collective: it makes this group's pending and future calls end with an error instead of waiting for a
  // peer that is gone.  A group waits abortably (in short slices, looking at the flag) once set_abortable(true)
  // has been called; without it a wait costs one store round trip less.
  virtual void Abort() { aborted_ = true; }
  bool aborted() const { return aborted_; }
  void set_abortable(bool on) { abortable_ = on; }

 protected:
  void CheckNotAborted() const { TORCH_CHECK(!aborted_, "process group ", name_, " was aborted (a peer failed)"); }
  std::string name_;
  std::vector<int> ranks_;
  int group_rank_;
  std::atomic<bool> aborted_{false}, abortable_{false};
};

inline Tensor Combine(const Tensor& acc, const Tensor& next, ReduceOp op) {
  switch (op) {
    case ReduceOp::kSum:
    case ReduceOp::kAvg: return acc + next;
    case ReduceOp::kMax: return torch::maximum(acc, next);
    case ReduceOp::kMin: return torch::minimum(acc, next);
    case ReduceOp::kProd: return acc * next;
  }
  return acc;
}

// ------------------------------------------------------------------ CPU ranks through the TCP store
class StoreProcessGroup : public ProcessGroup {
 public:
  StoreProcessGroup(std::string name, std::vector<int> ranks, int my_global_rank, c10::intrusive_ptr<c10d::Store> store)
      : ProcessGroup(std::move(name), std::move(ranks), my_global_rank), store_(std::move(store)) {}

  std::shared_ptr<Work> AllReduce(Tensor& t, ReduceOp op, bool) override {
    ITB_PROFILE("pg.AllReduce(" + name_ + ")", false);
    Check(t);
    const int64_t n = seq_++;
    Publish(Key("c", n, rank()), t);
    Tensor acc = Fetch(Key("c", n, 0), t);
    for (int r = 1; r < size(); ++r) acc = Combine(acc, Fetch(Key("c", n, r), t), op);
    if (op == ReduceOp::kAvg) acc = acc / size();
    t.copy_(acc);
    Retire(n);
    return done();
  }
  std::shared_ptr<Work> AllGather(Tensor& out, const Tensor& in, bool) override {
    ITB_PROFILE("pg.AllGather(" + name_ + ")", false);
    Check(out), Check(in);
    TORCH_CHECK(out.numel() == in.numel() * size(), "AllGather: output must hold one input per rank");
    const int64_t n = seq_++;
    Publish(Key("c", n, rank()), in);
    Tensor flat = out.view({size(), -1});
    for (int r = 0; r < size(); ++r) flat[r].copy_(Fetch(Key("c", n, r), in).view({-1}));
    Retire(n);
    return done();
  }
  std::shared_ptr<Work> ReduceScatter(Tensor& out, const Tensor& in, ReduceOp op, bool) override {
    ITB_PROFILE("pg.ReduceScatter(" + name_ + ")", false);
    Check(out), Check(in);
    TORCH_CHECK(in.numel() == out.numel() * size(), "ReduceScatter: input must hold one output per rank");
    const int64_t n = seq_++;
    Publish(Key("c", n, rank()), in);
    Tensor acc;
    for (int r = 0; r < size(); ++r) {
      Tensor piece = Fetch(Key("c", n, r), in).view({size(), -1})[rank()];
      acc = r == 0 ? piece.clone() : Combine(acc, piece, op);
    }
    if (op == ReduceOp::kAvg) acc = acc / size();
    out.view({-1}).copy_(acc);
    Retire(n);
    return done();
  }
  std::shared_ptr<Work> BroadCast(Tensor& t, int src, bool) override {
    ITB_PROFILE("pg.BroadCast(" + name_ + ")", false);
    Check(t);
    const int64_t n = seq_++;
    const std::string key = Key("c", n, src), ack = key + "/ack";
    if (rank() == src) {
      // the source waits for every reader: nothing else holds it back, and its buffer must outlive them
      Publish(key, t);
      while (store_->add(ack, 0) < size() - 1) {
        CheckNotAborted();
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      store_->deleteKey(key);
      store_->deleteKey(ack);
    } else {
      t.copy_(Fetch(key, t));
      store_->add(ack, 1);
    }
    return done();
  }
  std::shared_ptr<Work> Send(const TensorList& ts, int dst, bool) override {
    for (const Tensor& t : ts) {
      Check(t);
      Publish(P2PKey(rank(), dst, send_seq_[dst]++), t);
    }
    return done();
  }
  std::shared_ptr<Work> Recv(TensorList& ts, int src, bool) override {
    for (Tensor& t : ts) {
      Check(t);
      const std::string key = P2PKey(src, rank(), recv_seq_[src]++);
      t.copy_(Fetch(key, t));
      store_->deleteKey(key);
    }
    return done();
  }
  std::shared_ptr<Work> BatchSendRecv(std::vector<P2POp>& ops, bool) override {
    for (auto& op : ops)   // publishing never blocks, so every send goes out before the first receive waits
      if (op.is_send) Send({op.tensor}, op.peer, false);
    for (auto& op : ops)
      if (!op.is_send) {
        TensorList one = {op.tensor};
        Recv(one, op.peer, false);
      }
    return done();
  }
  void Barrier() override {
    const std::string key = "itb/pg/" + name_ + "/bar/" + std::to_string(barrier_seq_++);
    store_->add(key, 1);
    while (store_->add(key, 0) < size()) {
      CheckNotAborted();
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
  }

 private:
  static void Check(const Tensor& t) { TORCH_CHECK(t.is_contiguous() && !t.is_cuda(), "StoreProcessGroup: contiguous CPU tensor required"); }
  static std::shared_ptr<Work> done() { return std::make_shared<CompletedWork>(); }
  std::string Key(const char* kind, int64_t n, int r) const {
    return "itb/pg/" + name_ + "/" + kind + "/" + std::to_string(n) + "/" + std::to_string(r);
  }
  std::string P2PKey(int src, int dst, int64_t n) const {
    return "itb/pg/" + name_ + "/p2p/" + std::to_string(src) + ">" + std::to_string(dst) + "/" + std::to_string(n);
  }
  void Publish(const std::string& key, const Tensor& t) {
    const uint8_t* p = static_cast<const uint8_t*>(t.data_ptr());
    store_->set(key, std::vector<uint8_t>(p, p + t.nbytes()));
  }
  Tensor Fetch(const std::string& key, const Tensor& like) {
    if (abortable_) {
      // wait in slices so that Abort() from the watchdog thread ends the wait
      const auto t0 = std::chrono::steady_clock::now();
      while (!store_->check({key})) {
        CheckNotAborted();
        TORCH_CHECK(std::chrono::steady_clock::now() - t0 < store_->getTimeout(), "StoreProcessGroup ", name_, ": no rank published ", key);
        std::this_thread::sleep_for(std::chrono::microseconds(200));
      }
    }
    CheckNotAborted();
    auto bytes = store_->get(key);   // blocks until the key exists
    TORCH_CHECK(bytes.size() == like.nbytes(), "StoreProcessGroup ", name_, ": ranks disagree on the size of ", key);
    Tensor t = torch::empty_like(like);
    std::memcpy(t.data_ptr(), bytes.data(), bytes.size());
    return t;
  }
  // Every rank takes part in every numbered collective, so once this rank is in number n all ranks
  // have finished reading number n - 2: this rank's buffer of that collective can go.
  void Retire(int64_t n) {
    mine_.push_back(Key("c", n, rank()));
    while (mine_.size() > 2) {
      store_->deleteKey(mine_.front());
      mine_.erase(mine_.begin());
    }
  }
  c10::intrusive_ptr<c10d::Store> store_;
  int64_t seq_ = 0, barrier_seq_ = 0;
  std::map<int, int64_t> send_seq_, recv_seq_;
  std::vector<std::string> mine_;
};

#ifdef ITB_WITH_CUDA
// ------------------------------------------------------------------ NCCL over NVLink / NVSwitch
// Work of a collective enqueued on the group's stream: a CUDA event recorded behind it.
class CudaWork : public Work {
 public:
  CudaWork(ncclComm_t comm, std::shared_ptr<std::atomic<bool>> comm_gone) : comm_(comm), comm_gone_(std::move(comm_gone)) {}
  void record(const c10::cuda::CUDAStream& s) { done_.record(s); }
  bool WaitBlocking(int64_t timeout_ms) override {
    const auto t0 = std::chrono::steady_clock::now();
    while (!done_.query()) {
      if (timeout_ms > 0 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) return false;
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    return true;
  }
  bool WaitNonBlocking() override {
    done_.block(at::cuda::getCurrentCUDAStream());
    return true;
  }
  bool IsCompleted() const override { return done_.query(); }
  std::string error() const override {
    ncclResult_t st = ncclSuccess;
    if (comm_gone_ && *comm_gone_) return "the communicator was aborted";
    if (comm_ && ncclCommGetAsyncError(comm_, &st) == ncclSuccess && st != ncclSuccess && st != ncclInProgress)
      return ncclGetErrorString(st);
    return std::string();
  }

 private:
  ncclComm_t comm_;
  std::shared_ptr<std::atomic<bool>> comm_gone_;   // set by the group's Abort(): comm_ must not be touched any more
  at::cuda::CUDAEvent done_;
};

class NcclProcessGroup : public ProcessGroup {
 public:
  NcclProcessGroup(std::string name, std::vector<int> ranks, int my_global_rank, c10::intrusive_ptr<c10d::Store> store)
      : ProcessGroup(std::move(name), std::move(ranks), my_global_rank),
        stream_(c10::cuda::getStreamFromPool(/*isHighPriority=*/true)) {
    ncclUniqueId id;
    const std::string key = "itb/nccl_id/" + name_;
    if (rank() == 0) {
      Check(ncclGetUniqueId(&id), "ncclGetUniqueId");
      const uint8_t* p = reinterpret_cast<const uint8_t*>(&id);
      store->set(key, std::vector<uint8_t>(p, p + sizeof(id)));
    } else {
      auto bytes = store->get(key);
      TORCH_CHECK(bytes.size() == sizeof(id), "bad NCCL id in the store for group ", name_);
      std::memcpy(&id, bytes.data(), sizeof(id));
    }
    Check(ncclCommInitRank(&comm_, size(), id, rank()), "ncclCommInitRank");
  }
  ~NcclProcessGroup() override {
    if (comm_ && !*comm_gone_) ncclCommDestroy(comm_);
  }
  // ncclCommAbort ends the communicator's kernels that wait for a peer and frees it; the group is unusable afterwards.
  void Abort() override {
    if (aborted_.exchange(true)) return;
    *comm_gone_ = true;
    if (comm_) ncclCommAbort(comm_);
  }
  std::shared_ptr<Work> AllReduce(Tensor& t, ReduceOp op, bool async_op) override {
    return Run(async_op, {t}, [&](cudaStream_t s) {
      return ncclAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), Dtype(t), Op(op), comm_, s);
    });
  }
  std::shared_ptr<Work> AllGather(Tensor& out, const Tensor& in, bool async_op) override {
    TORCH_CHECK(out.numel() == in.numel() * size(), "AllGather: output must hold one input per rank");
    return Run(async_op, {out, in}, [&](cudaStream_t s) {
      return ncclAllGather(in.data_ptr(), out.data_ptr(), in.numel(), Dtype(in), comm_, s);
    });
  }
  std::shared_ptr<Work> ReduceScatter(Tensor& out, const Tensor& in, ReduceOp op, bool async_op) override {
    TORCH_CHECK(in.numel() == out.numel() * size(), "ReduceScatter: input must hold one output per rank");
    return Run(async_op, {out, in}, [&](cudaStream_t s) {
      return ncclReduceScatter(in.data_ptr(), out.data_ptr(), out.numel(), Dtype(in), Op(op), comm_, s);
    });
  }
  std::shared_ptr<Work> BroadCast(Tensor& t, int src, bool async_op) override {
    return Run(async_op, {t}, [&](cudaStream_t s) {
      return ncclBroadcast(t.data_ptr(), t.data_ptr(), t.nbytes(), ncclChar, src, comm_, s);
    });
  }
  std::shared_ptr<Work> Reduce(Tensor& t, int dst, ReduceOp op, bool async_op) override {
    return Run(async_op, {t}, [&](cudaStream_t s) {
      return ncclReduce(t.data_ptr(), t.data_ptr(), t.numel(), Dtype(t), Op(op), dst, comm_, s);
    });
  }
  std::shared_ptr<Work> Send(const TensorList& ts, int dst, bool async_op) override {
    return Run(async_op, ts, [&](cudaStream_t s) {
      ncclResult_t r = ncclGroupStart();
      for (const Tensor& t : ts)
        if (r == ncclSuccess) r = ncclSend(t.data_ptr(), t.nbytes(), ncclChar, dst, comm_, s);
      ncclResult_t e = ncclGroupEnd();
      return r != ncclSuccess ? r : e;
    });
  }
  std::shared_ptr<Work> Recv(TensorList& ts, int src, bool async_op) override {
    return Run(async_op, ts, [&](cudaStream_t s) {
      ncclResult_t r = ncclGroupStart();
      for (Tensor& t : ts)
        if (r == ncclSuccess) r = ncclRecv(t.data_ptr(), t.nbytes(), ncclChar, src, comm_, s);
      ncclResult_t e = ncclGroupEnd();
      return r != ncclSuccess ? r : e;
    });
  }
  std::shared_ptr<Work> BatchSendRecv(std::vector<P2POp>& ops, bool async_op) override {
    TensorList touched;
    for (auto& op : ops) touched.push_back(op.tensor);
    if (ops.empty()) return std::make_shared<CompletedWork>();
    return Run(async_op, touched, [&](cudaStream_t s) {
      ncclResult_t r = ncclGroupStart();
      for (auto& op : ops) {
        if (r != ncclSuccess) break;
        r = op.is_send ? ncclSend(op.tensor.data_ptr(), op.tensor.nbytes(), ncclChar, op.peer, comm_, s)
                       : ncclRecv(op.tensor.data_ptr(), op.tensor.nbytes(), ncclChar, op.peer, comm_, s);
      }
      ncclResult_t e = ncclGroupEnd();
      return r != ncclSuccess ? r : e;
    });
  }
  void Barrier() override {
    Tensor t = torch::zeros({1}, torch::dtype(torch::kFloat32).device(torch::kCUDA));
    AllReduce(t, ReduceOp::kSum, false);
    at::cuda::getCurrentCUDAStream().synchronize();
  }
  int AsyncError() override {
    if (*comm_gone_) return static_cast<int>(ncclInternalError);
    ncclResult_t st = ncclSuccess;
    ncclCommGetAsyncError(comm_, &st);
    return st == ncclInProgress ? 0 : static_cast<int>(st);
  }

 private:
  template <class F>
  std::shared_ptr<Work> Run(bool async_op, const TensorList& touched, F&& enqueue) {
    ITB_PROFILE("pg.nccl(" + name_ + ")", true);
    CheckNotAborted();
    for (const Tensor& t : touched) TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "NcclProcessGroup: contiguous CUDA tensors");
    auto compute = at::cuda::getCurrentCUDAStream();
    at::cuda::CUDAEvent ready;
    ready.record(compute);
    ready.block(stream_);                       // the communication stream starts after the producers
    for (const Tensor& t : touched)             // the caching allocator must not recycle them under the collective
      c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), stream_);
    Check(enqueue(stream_.stream()), "NCCL collective");
    auto work = std::make_shared<CudaWork>(comm_, comm_gone_);
    work->record(stream_);
    if (!async_op) work->WaitNonBlocking();     // the compute stream waits; the host never does
    return work;
  }
  static ncclDataType_t Dtype(const Tensor& t) {
    switch (t.scalar_type()) {
      case torch::kFloat32: return ncclFloat;
      case torch::kBFloat16: return ncclBfloat16;
      case torch::kFloat16: return ncclHalf;
      case torch::kFloat64: return ncclDouble;
      case torch::kInt64: return ncclInt64;
      case torch::kInt32: return ncclInt32;
      case torch::kUInt8: return ncclUint8;
      case torch::kInt8: return ncclInt8;
      default: TORCH_CHECK(false, "NCCL has no type for ", t.scalar_type());
    }
  }
  static ncclRedOp_t Op(ReduceOp op) {
    switch (op) {
      case ReduceOp::kSum: return ncclSum;
      case ReduceOp::kAvg: return ncclAvg;
      case ReduceOp::kMax: return ncclMax;
      case ReduceOp::kMin: return ncclMin;
      case ReduceOp::kProd: return ncclProd;
    }
    return ncclSum;
  }
  static void Check(ncclResult_t r, const char* what) { TORCH_CHECK(r == ncclSuccess, what, ": ", ncclGetErrorString(r)); }
  ncclComm_t comm_ = nullptr;
  std::shared_ptr<std::atomic<bool>> comm_gone_ = std::make_shared<std::atomic<bool>>(false);
  c10::cuda::CUDAStream stream_;
};
#endif  // ITB_WITH_CUDA

// ------------------------------------------------------------------ factory
// One store per job (a TCP store that rank 0 serves, or a shared file), one process group per name.  Init() creates the
// "default" group over every rank; DP / TP / PP groups of this rank come from the layout.
class ProcessGroupFactory {
 public:
  static ProcessGroupFactory& Instance() {
    static ProcessGroupFactory f;
    return f;
  }
  void Init(torch::Device device, int timeout_s = 300) {
    if (store_) return;
    GlobalEnv& e = env();
    device_ = device;
    // Rendezvous: a file every rank can reach (ITB_RDZV_FILE, for jobs whose nodes share a file system and
    // have no address to agree on; the reference exchanges its communicator ids through files in the same
    // way, src/core/ccl/ccl_utils.cc:14-53), else the TCP store served by rank 0 at MASTER_ADDR:MASTER_PORT.
    const char* file = std::getenv("ITB_RDZV_FILE");
    if (file && *file) {
      store_ = c10::make_intrusive<c10d::FileStore>(file, e.world);
      store_->setTimeout(std::chrono::milliseconds(1000LL * timeout_s));
    } else {
      c10d::TCPStoreOptions o;
      const char* port = std::getenv("MASTER_PORT");
      const char* addr = std::getenv("MASTER_ADDR");
      o.port = static_cast<uint16_t>(port && *port ? std::atoi(port) : 29500);
      o.isServer = e.rank == 0;
      o.numWorkers = e.world;
      o.timeout = std::chrono::milliseconds(1000LL * timeout_s);
      store_ = c10::make_intrusive<c10d::TCPStore>(addr && *addr ? addr : "127.0.0.1", o);
    }
#ifdef ITB_WITH_CUDA
    if (device.is_cuda()) c10::cuda::set_device(device.has_index() ? device.index() : static_cast<c10::DeviceIndex>(e.local_rank));
#endif
    std::vector<int> all(e.world);
    for (int i = 0; i < e.world; ++i) all[i] = i;
    GetOrCreate("default", all);
  }
  bool initialized() const { return static_cast<bool>(store_); }
  c10::intrusive_ptr<c10d::Store> store() const { return store_; }

  std::shared_ptr<ProcessGroup> GetOrCreate(const std::string& name, const std::vector<int>& ranks) {
    auto it = groups_.find(name);
    if (it != groups_.end()) return it->second;
    TORCH_CHECK(store_, "ProcessGroupFactory::Init has not been called");
    std::shared_ptr<ProcessGroup> g;
#ifdef ITB_WITH_CUDA
    if (device_.is_cuda()) g = std::make_shared<NcclProcessGroup>(name, ranks, env().rank, store_);
#endif
    if (!g) {
      TORCH_CHECK(!device_.is_cuda(), "this build has no CUDA support");
      g = std::make_shared<StoreProcessGroup>(name, ranks, env().rank, store_);
    }
    g->set_abortable(abortable_);
    std::lock_guard<std::mutex> lock(mu_);
    groups_[name] = g;
    return g;
  }
  // Every group of the job, those created later included, waits in short slices so that Abort() (from a
  // watchdog thread) ends a wait for a peer that is gone.
  void SetAbortable(bool on) {
    abortable_ = on;
    for (auto& g : AllGroups()) g->set_abortable(on);
  }
  std::shared_ptr<ProcessGroup> Get(const std::string& name) const {
    auto it = groups_.find(name);
    return it == groups_.end() ? nullptr : it->second;
  }
  std::shared_ptr<ProcessGroup> GetDefaultProcessGroup() const { return Get("default"); }
  // Every group created so far (what a watchdog aborts when a peer fails).
  std::vector<std::shared_ptr<ProcessGroup>> AllGroups() const {
    std::vector<std::shared_ptr<ProcessGroup>> out;
    std::lock_guard<std::mutex> lock(mu_);
    for (auto& [name, g] : groups_) out.push_back(g);
    return out;
  }
  // The group of this rank along one axis, or null when the axis has one rank.
  std::shared_ptr<ProcessGroup> AxisGroup(Axis axis) {
    if (env().layout.size(axis) <= 1 || !store_) return nullptr;
    return GetOrCreate(env().GroupName(axis), env().GroupRanks(axis));
  }
  std::shared_ptr<ProcessGroup> tp_group() { return AxisGroup(Axis::kTP); }
  std::shared_ptr<ProcessGroup> dp_group() { return AxisGroup(Axis::kDP); }
  std::shared_ptr<ProcessGroup> pp_group() { return AxisGroup(Axis::kPP); }
  // Rank 0 serves the store: it leaves last, once every other rank has said that it needs the
  // store no more (or after `wait_s` seconds, when one of them died).
  void Shutdown(int wait_s = 30) {
    groups_.clear();
    if (store_ && env().world > 1) {
      try {
        if (env().rank != 0) {
          store_->add("itb/shutdown", 1);
        } else {
          const auto t0 = std::chrono::steady_clock::now();
          while (store_->add("itb/shutdown", 0) < env().world - 1 && std::chrono::steady_clock::now() - t0 < std::chrono::seconds(wait_s))
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
        }
      } catch (const std::exception&) {   // the server may be gone already: nothing left to order
      }
    }
    store_.reset();
  }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  std::map<std::string, std::shared_ptr<ProcessGroup>> groups_;
  mutable std::mutex mu_;   // AllGroups() may be called from a watchdog thread while the training thread creates a group
  bool abortable_ = false;
  torch::Device device_ = torch::Device(torch::kCPU);
};

inline std::shared_ptr<ProcessGroup> tp_group() { return ProcessGroupFactory::Instance().tp_group(); }
inline std::shared_ptr<ProcessGroup> dp_group() { return ProcessGroupFactory::Instance().dp_group(); }
inline std::shared_ptr<ProcessGroup> pp_group() { return ProcessGroupFactory::Instance().pp_group(); }

}  // namespace parallel
}  // namespace itb
