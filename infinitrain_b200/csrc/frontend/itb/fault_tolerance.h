// Failure detection on the host for the C++ frontend: step heartbeats through the job's store, a
// watchdog thread per rank, coordinated abort of the process groups, and host-side fault injection.
//
// The reference has none of this: a lost peer leaves every other rank inside a collective for ever (only
// Work::WaitBlocking(timeout) and the NCCL async-error query exist, infini_train/src/nn/parallel/work.cc:37-73,
// src/core/ccl/cuda/nccl_impl.cc:63-69).  Here
//   * every rank publishes "<step>:<wall seconds>" under <prefix>/<rank> after each step;
//   * a thread per rank reads the peers' entries every `poll_s` and, when one is older than `timeout_s`, when a
//     peer has posted an abort reason, or when the store itself stops answering, records a FailureReport,
//     posts the abort reason for everybody else and calls Abort() on the process groups it was given (CPU
//     ranks: a wait inside a collective ends with an error; NCCL: ncclCommAbort), so that the training thread
//     comes back and finds the report at its next Heartbeat::Step();
//     A heartbeat is a sign of progress, not only of life: a rank that sits in a collective, writes a large
//     checkpoint or waits at a barrier does not beat, so `timeout_s` has to exceed the longest time a healthy
//     step (with everything that happens between two steps) can take;
//   * faults are injected on the host only (FaultInjector, ITB_FAULT="<rank>:<step>:<kind>[:<arg>]", kinds
//     raise / exit / stall / mute), before the step launches anything, so no kernel or collective of the
//     faulty rank is in flight when it goes away.  Nothing here makes a device fault, trap or hang.
#pragma once
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <fstream>
#include <functional>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "process_group.h"

namespace itb {
namespace utils {

// A peer stopped sending heartbeats, asked for an abort, or the store went away.
struct RankFailure : std::runtime_error {
  using std::runtime_error::runtime_error;
};
// A bounded wait inside a kernel ran out; the status word holds the code of the wait.
struct KernelTimeout : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct FailureReport {
  std::string kind;   // "stale_heartbeat" | "peer_abort" | "store_lost"
  int rank = -1;      // the rank the report is about
  std::string detail;
  int64_t step = -1;
  std::string str() const { return "rank " + std::to_string(rank) + ": " + kind + (detail.empty() ? "" : " " + detail); }
};

inline double wall_seconds() {
  return std::chrono::duration<double>(std::chrono::system_clock::now().time_since_epoch()).count();
}

class Heartbeat {
 public:
  using OnFailure = std::function<void(const FailureReport&)>;
  // The groups to abort are asked for when a failure is seen: groups are created on first use, some of them
  // after the watchdog has started.  They must wait abortably (ProcessGroup::set_abortable, or
  // ProcessGroupFactory::SetAbortable for every group of the job) for Abort() to end a wait of theirs.
  using Groups = std::function<std::vector<std::shared_ptr<parallel::ProcessGroup>>()>;

  Heartbeat(c10::intrusive_ptr<c10d::Store> store, int rank, int world, double timeout_s = 60.0, double poll_s = 0.5,
            Groups groups = nullptr, OnFailure on_failure = nullptr, std::string prefix = "itb/hb")
      : store_(std::move(store)), rank_(rank), world_(world), timeout_s_(timeout_s), poll_s_(poll_s), groups_(std::move(groups)),
        on_failure_(std::move(on_failure)), prefix_(std::move(prefix)), started_(wall_seconds()) {}
  ~Heartbeat() { Stop(); }
  Heartbeat(const Heartbeat&) = delete;
  Heartbeat& operator=(const Heartbeat&) = delete;

  // ---- publishing
  void Beat(int64_t step) {
    step_ = step;
    if (!muted_) Set(Key(rank_), std::to_string(step) + ":" + std::to_string(wall_seconds()));
  }
  // Once per training step: publishes the heartbeat; throws RankFailure in the calling (training) thread when
  // the watchdog has seen a failure.
  void Step(int64_t step) {
    ThrowIfFailed();
    Beat(step);
  }
  // Blocks until every peer has published a heartbeat of `step` or later; RankFailure when one has not within
  // `timeout_s` (default: the watchdog's).  Called before the first collective of a step it turns "a peer is
  // gone" into an exception instead of a collective that never returns.
  void WaitPeers(int64_t step, double timeout_s = -1.0) {
    const double deadline = wall_seconds() + (timeout_s < 0 ? timeout_s_ : timeout_s);
    std::vector<int> pending;
    for (int r = 0; r < world_; ++r)
      if (r != rank_) pending.push_back(r);
    while (!pending.empty()) {
      ThrowIfFailed();
      if (auto abort = PeerAbort()) {
        Fail(*abort);
        continue;
      }
      std::vector<int> still;
      for (int r : pending) {
        auto hb = Read(Key(r));
        if (!hb || hb->first < step) still.push_back(r);
      }
      pending.swap(still);
      if (pending.empty()) break;
      if (wall_seconds() > deadline) {
        FailureReport rep{"stale_heartbeat", pending[0], "did not reach step " + std::to_string(step) + " within the time limit", step};
        try {
          RequestAbort("rank " + std::to_string(pending[0]) + " did not reach step " + std::to_string(step));
        } catch (const std::exception&) {
        }
        Fail(rep);
        continue;
      }
      std::this_thread::sleep_for(std::chrono::duration<double>(std::min(0.01, poll_s_)));
    }
  }
  // Tells every rank to stop (they see it at their next watchdog poll).
  void RequestAbort(const std::string& reason) { Set(prefix_ + "/abort", std::to_string(rank_) + ":" + reason); }

  // ---- watching
  Heartbeat& Start() {
    Beat(step_);
    stop_ = false;
    thread_ = std::thread([this] { Watch(); });
    return *this;
  }
  void Stop() {
    stop_ = true;
    if (thread_.joinable()) thread_.join();
  }
  // One pass over the store (the watchdog thread calls this; tests may call it directly with a clock of theirs).
  std::optional<FailureReport> Scan(double now = -1.0) {
    if (now < 0) now = wall_seconds();
    try {
      if (auto abort = PeerAbort()) return abort;
      for (int r = 0; r < world_; ++r) {
        if (r == rank_) continue;
        auto hb = Read(Key(r));
        if (!hb) {
          // never seen: stale only once the grace period since this rank's own start has passed
          if (now - started_ > timeout_s_) return FailureReport{"stale_heartbeat", r, "no heartbeat was ever published", step_};
          continue;
        }
        if (now - hb->second > timeout_s_)
          return FailureReport{"stale_heartbeat", r,
                               "last heartbeat at step " + std::to_string(hb->first) + ", " + std::to_string(now - hb->second) + " s ago",
                               hb->first};
      }
    } catch (const std::exception& e) {
      return FailureReport{"store_lost", 0, std::string("the job's store does not answer: ") + e.what(), step_};
    }
    return std::nullopt;
  }
  std::optional<FailureReport> failure() const {
    std::lock_guard<std::mutex> lock(mu_);
    return failure_;
  }
  void set_muted(bool on) { muted_ = on; }   // fault injection: keep running, stop beating
  int rank() const { return rank_; }

 private:
  std::string Key(int r) const { return prefix_ + "/" + std::to_string(r); }
  void Set(const std::string& key, const std::string& value) { store_->set(key, std::vector<uint8_t>(value.begin(), value.end())); }
  // (step, wall seconds) of an entry, or nothing when the key does not exist yet
  std::optional<std::pair<int64_t, double>> Read(const std::string& key) {
    auto raw = Raw(key);
    if (!raw) return std::nullopt;
    auto colon = raw->find(':');
    return std::make_pair<int64_t, double>(std::stoll(raw->substr(0, colon)), colon == std::string::npos ? 0.0 : std::stod(raw->substr(colon + 1)));
  }
  std::optional<std::string> Raw(const std::string& key) {
    if (!store_->check({key})) return std::nullopt;
    auto bytes = store_->get(key);
    return std::string(bytes.begin(), bytes.end());
  }
  std::optional<FailureReport> PeerAbort() {
    auto raw = Raw(prefix_ + "/abort");
    if (!raw) return std::nullopt;
    auto colon = raw->find(':');
    int who = std::stoi(raw->substr(0, colon));
    if (who == rank_) return std::nullopt;
    return FailureReport{"peer_abort", who, colon == std::string::npos ? "" : raw->substr(colon + 1), step_};
  }
  void ThrowIfFailed() const {
    std::lock_guard<std::mutex> lock(mu_);
    if (failure_) throw RankFailure(failure_->str());
  }
  void Fail(const FailureReport& rep) {
    std::lock_guard<std::mutex> lock(mu_);
    if (!failure_) failure_ = rep;
  }
  void Watch() {
    auto next = std::chrono::steady_clock::now();
    while (!stop_) {
      next += std::chrono::duration_cast<std::chrono::steady_clock::duration>(std::chrono::duration<double>(poll_s_));
      while (!stop_ && std::chrono::steady_clock::now() < next) std::this_thread::sleep_for(std::chrono::milliseconds(5));
      if (stop_) return;
      auto rep = Scan();
      if (!rep) continue;
      Fail(*rep);
      if (on_failure_) on_failure_(*rep);
      else DefaultOnFailure(*rep);
      return;
    }
  }
  void DefaultOnFailure(const FailureReport& rep) {
    if (rep.kind == "stale_heartbeat") {
      try {
        RequestAbort(rep.kind + " of rank " + std::to_string(rep.rank));
      } catch (const std::exception&) {
      }
    }
    if (groups_)
      for (auto& g : groups_())
        if (g) g->Abort();
  }

  c10::intrusive_ptr<c10d::Store> store_;
  int rank_, world_;
  double timeout_s_, poll_s_;
  Groups groups_;
  OnFailure on_failure_;
  std::string prefix_;
  double started_;
  std::atomic<int64_t> step_{-1};
  std::atomic<bool> muted_{false}, stop_{false};
  mutable std::mutex mu_;
  std::optional<FailureReport> failure_;
  std::thread thread_;
};

// Raises KernelTimeout when a device status word is non-zero; `status` reads the word.
inline void CheckKernelStatus(const std::function<int()>& status, const std::string& what = "kernel") {
  const int code = status();
  if (code != 0) throw KernelTimeout(what + ": a bounded device-side wait gave up (code " + std::to_string(code) + ")");
}

// ITB_FAULT="<rank>:<step>:<kind>[:<arg>]" with kind one of
//   raise -- the rank throws std::runtime_error at that step;
//   exit  -- the rank leaves the process with _exit(arg or 17) between two steps;
//   stall -- the rank sleeps `arg` seconds (a straggler);
//   mute  -- the rank keeps training but stops publishing heartbeats.
// MaybeFire(step) is called by the training loop before it launches anything for the step.
class FaultInjector {
 public:
  explicit FaultInjector(int rank, const char* spec = nullptr, Heartbeat* heartbeat = nullptr, bool on_cuda = false)
      : rank_(rank), heartbeat_(heartbeat), on_cuda_(on_cuda) {
    const char* env = spec ? spec : std::getenv("ITB_FAULT");
    if (!env || !*env) return;
    // a fault from the environment belongs to a job's first attempt: the attempt that the launcher starts after it
    // (ITB_RESTART_COUNT > 0) must be able to get past the step
    const char* restarted = std::getenv("ITB_RESTART_COUNT");
    if (!spec && restarted && std::atoi(restarted) > 0) return;
    std::vector<std::string> parts;
    std::string s(env);
    size_t begin = 0;
    while (true) {
      size_t colon = s.find(':', begin);
      parts.push_back(s.substr(begin, colon == std::string::npos ? std::string::npos : colon - begin));
      if (colon == std::string::npos) break;
      begin = colon + 1;
    }
    if (parts.size() < 3) throw std::invalid_argument("ITB_FAULT wants <rank>:<step>:<kind>[:<arg>], got '" + s + "'");
    target_rank_ = std::stoi(parts[0]), step_ = std::stoll(parts[1]), kind_ = parts[2];
    if (parts.size() > 3) arg_ = parts[3];
    if (kind_ != "raise" && kind_ != "exit" && kind_ != "stall" && kind_ != "mute")
      throw std::invalid_argument("unknown fault kind '" + kind_ + "'");
  }
  bool armed() const { return !kind_.empty() && rank_ == target_rank_; }
  const std::string& kind() const { return kind_; }
  bool fired() const { return fired_; }
  // A process may be ended by the injector when it has no CUDA context, or when neither NCCL nor this framework's
  // kernels use NVLink multicast (NCCL_NVLS_ENABLE=0 and ITB_NVLS=0): a rank that dies while its memory is bound
  // to a multicast object faults its peers' GPUs.
  bool ExitAllowed() const {
    if (!on_cuda_) return true;
    const char* a = std::getenv("ITB_NVLS");
    const char* b = std::getenv("NCCL_NVLS_ENABLE");
    return a && std::string(a) == "0" && b && std::string(b) == "0";
  }
  void MaybeFire(int64_t step) {
    if (fired_ || !armed() || step != step_) return;
    fired_ = true;
    if (kind_ == "raise") throw std::runtime_error("injected fault on rank " + std::to_string(rank_) + " at step " + std::to_string(step));
    if (kind_ == "exit") {
      if (!ExitAllowed())
        throw std::runtime_error("ITB_FAULT ...:exit refused: this process holds CUDA memory that may be bound to an NVLink multicast "
                                 "object; rerun on CPU ranks, or with ITB_NVLS=0 and NCCL_NVLS_ENABLE=0");
      std::_Exit(arg_.empty() ? 17 : std::stoi(arg_));
    }
    if (kind_ == "stall") std::this_thread::sleep_for(std::chrono::duration<double>(arg_.empty() ? 1.0 : std::stod(arg_)));
    if (kind_ == "mute" && heartbeat_) heartbeat_->set_muted(true);
  }

 private:
  int rank_, target_rank_ = -1;
  int64_t step_ = -1;
  std::string kind_, arg_;
  Heartbeat* heartbeat_;
  bool on_cuda_, fired_ = false;
};

// Flips `nbytes` bytes of a file in place (checkpoint-corruption tests).
inline void CorruptFile(const std::string& path, int64_t offset = 0, int64_t nbytes = 8) {
  std::fstream f(path, std::ios::in | std::ios::out | std::ios::binary);
  if (!f.is_open()) throw std::runtime_error("cannot open " + path);
  f.seekg(offset);
  std::string data(static_cast<size_t>(nbytes), '\0');
  f.read(data.data(), nbytes);
  data.resize(static_cast<size_t>(f.gcount()));
  for (char& c : data) c = static_cast<char>(~c);
  f.clear();
  f.seekp(offset);
  f.write(data.data(), static_cast<std::streamsize>(data.size()));
}

}  // namespace utils
}  // namespace itb
