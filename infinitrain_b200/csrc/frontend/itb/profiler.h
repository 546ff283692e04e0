// Profiler of the C++ frontend: one record per op (forward and, on the fused path, backward), per
// optimizer step and per collective, with host time, device time and the memory pool's peak; records
// carry a tag ("Step_9"); a per-tag table and a flat record log, one pair of files per rank.
//
// Reference: infini_train/include/profiler.h:40-97 and src/profiler.cc:41-313 (StartRecord / EndRecord
// around every dispatched kernel with a device synchronisation on both sides, device time from a pair
// of events, nested calls ignored through a depth counter, Report sorted by one of eight keys,
// PrintRecords, SetTag, Reset).  There the profiler is a build mode (PROFILE_MODE); here it is a
// run-time switch, off by default: a disabled range costs one load and one branch.  Like the
// reference's, an enabled profiler serialises the device around every record: its numbers are shares
// of a step, not a benchmark.  Beyond the reference: every record is also an NVTX range (CUDA build; a
// no-op unless a tool is attached) and the records export as a Chrome trace (chrome://tracing, Perfetto).
#pragma once
#include <torch/torch.h>

#include <algorithm>
#include <chrono>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#ifdef ITB_WITH_CUDA
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <nvtx3/nvToolsExt.h>   // header-only: loads the tool's injection library when one is attached
#endif

namespace itb {
namespace utils {

struct KernelCallRecord {
  std::string tag, name, device;
  int64_t rank = 0;
  double host_us = 0, device_us = 0, start_us = 0;
  int64_t max_device_mem_usage_mb = 0;
};

class Profiler {
 public:
  enum class SortBy { HostTimeTotal, HostTimePercentage, HostTimeAverage, DeviceTimeTotal, DeviceTimePercentage,
                      DeviceTimeAverage, Count, NotSorted };
  static Profiler& Instance() {
    static Profiler p;
    return p;
  }
  void Enable(int64_t rank = 0) {
    rank_ = rank;
    enabled_ = true;
  }
  void Disable() { enabled_ = false; }
  bool enabled() const { return enabled_; }
  void SetTag(const std::string& tag) { tag_ = tag; }
  void Reset() {
    std::lock_guard<std::mutex> g(mu_);
    records_.clear();
  }
  const std::vector<KernelCallRecord>& records() const { return records_; }

  // One open record per thread; a range opened inside another is part of the outer one.
  void StartRecord(const std::string& name, bool cuda) {
    if (!enabled_) return;
    State& s = state();
    if (s.depth++ > 0) return;
    s.name = name, s.cuda = cuda;
#ifdef ITB_WITH_CUDA
    nvtxRangePushA(name.c_str());
    if (cuda) {
      at::cuda::getCurrentCUDAStream().synchronize();
      s.begin = std::make_unique<at::cuda::CUDAEvent>(cudaEventDefault);
      s.end = std::make_unique<at::cuda::CUDAEvent>(cudaEventDefault);
      s.begin->record(at::cuda::getCurrentCUDAStream());
    }
#endif
    s.t0 = std::chrono::steady_clock::now();
  }
  void EndRecord() {
    if (!enabled_) return;
    State& s = state();
    if (s.depth == 0 || --s.depth > 0) return;
    KernelCallRecord r;
    r.host_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - s.t0).count();
    r.start_us = std::chrono::duration<double, std::micro>(s.t0 - origin_).count();
    r.tag = tag_, r.name = s.name, r.device = s.cuda ? "cuda" : "cpu", r.rank = rank_;
#ifdef ITB_WITH_CUDA
    if (s.cuda) {
      s.end->record(at::cuda::getCurrentCUDAStream());
      s.end->synchronize();
      r.device_us = s.begin->elapsed_time(*s.end) * 1e3;
      const auto st = c10::cuda::CUDACachingAllocator::getDeviceStats(c10::cuda::current_device());
      r.max_device_mem_usage_mb = static_cast<int64_t>(st.reserved_bytes[0].peak >> 20);
    }
    nvtxRangePop();
#endif
    std::lock_guard<std::mutex> g(mu_);
    records_.push_back(std::move(r));
  }

  // Per tag: name, count, host total / average, device total / average / share, peak memory.
  void Report(std::ostream& os, SortBy sort_by = SortBy::DeviceTimeTotal) const {
    struct Agg {
      int64_t count = 0;
      double host = 0, dev = 0;
      int64_t peak = 0;
    };
    std::vector<std::string> tags;
    for (const auto& r : records_)
      if (std::find(tags.begin(), tags.end(), r.tag) == tags.end()) tags.push_back(r.tag);
    for (const auto& tag : tags) {
      std::map<std::string, Agg> agg;
      std::vector<std::string> order;
      double host_all = 0, dev_all = 0;
      for (const auto& r : records_) {
        if (r.tag != tag) continue;
        if (!agg.count(r.name)) order.push_back(r.name);
        Agg& a = agg[r.name];
        a.count++, a.host += r.host_us, a.dev += r.device_us;
        a.peak = std::max(a.peak, r.max_device_mem_usage_mb);
        host_all += r.host_us, dev_all += r.device_us;
      }
      auto key = [&](const std::string& n) {
        const Agg& a = agg.at(n);
        switch (sort_by) {
          case SortBy::HostTimeTotal:
          case SortBy::HostTimePercentage: return a.host;
          case SortBy::HostTimeAverage: return a.host / a.count;
          case SortBy::DeviceTimeTotal:
          case SortBy::DeviceTimePercentage: return a.dev;
          case SortBy::DeviceTimeAverage: return a.dev / a.count;
          case SortBy::Count: return static_cast<double>(a.count);
          default: return 0.0;
        }
      };
      if (sort_by != SortBy::NotSorted)
        std::stable_sort(order.begin(), order.end(), [&](const std::string& x, const std::string& y) { return key(x) > key(y); });
      os << "Tag: " << tag << "\n"
         << std::left << std::setw(32) << "Name" << std::right << std::setw(8) << "Count" << std::setw(16) << "Host Total(us)"
         << std::setw(14) << "Host Avg(us)" << std::setw(10) << "Host %" << std::setw(18) << "Device Total(us)" << std::setw(16)
         << "Device Avg(us)" << std::setw(10) << "Device %" << std::setw(14) << "Peak Mem(MB)" << "\n";
      os << std::fixed << std::setprecision(2);
      for (const auto& n : order) {
        const Agg& a = agg.at(n);
        os << std::left << std::setw(32) << n << std::right << std::setw(8) << a.count << std::setw(16) << a.host << std::setw(14)
           << a.host / a.count << std::setw(9) << (host_all > 0 ? 100 * a.host / host_all : 0.0) << "%" << std::setw(18) << a.dev
           << std::setw(16) << a.dev / a.count << std::setw(9) << (dev_all > 0 ? 100 * a.dev / dev_all : 0.0) << "%" << std::setw(14)
           << a.peak << "\n";
      }
      os << "\n";
    }
  }
  void Report(const std::string& path, SortBy sort_by = SortBy::DeviceTimeTotal) const {
    std::ofstream f(path);
    TORCH_CHECK(f.is_open(), "cannot write ", path);
    Report(f, sort_by);
  }
  void PrintRecords(std::ostream& os) const {
    os << std::fixed << std::setprecision(2);
    for (const auto& r : records_)
      os << r.tag << "\t" << r.rank << "\t" << r.name << "\t" << r.device << "\thost_us=" << r.host_us << "\tdevice_us=" << r.device_us
         << "\tpeak_mb=" << r.max_device_mem_usage_mb << "\n";
  }
  void PrintRecords(const std::string& path) const {
    std::ofstream f(path);
    TORCH_CHECK(f.is_open(), "cannot write ", path);
    PrintRecords(f);
  }
  // Complete ("X") events, one per record, in the Trace Event format: pid = rank, tid 0 = host spans (start
  // and host duration), tid 1 = device spans (same start, device duration), args carry the tag and the peak.
  void ExportChromeTrace(std::ostream& os) const {
    auto esc = [](const std::string& in) {
      std::string out;
      for (char c : in) {
        if (c == '"' || c == '\\') out.push_back('\\');
        out.push_back(c);
      }
      return out;
    };
    os << std::fixed << std::setprecision(3) << "{\"displayTimeUnit\": \"ms\", \"traceEvents\": [";
    bool first = true;
    for (const auto& r : records_) {
      for (int lane = 0; lane < (r.device == "cuda" ? 2 : 1); ++lane) {
        os << (first ? "\n" : ",\n") << "{\"name\": \"" << esc(r.name) << "\", \"cat\": \"" << (lane ? "device" : "host")
           << "\", \"ph\": \"X\", \"pid\": " << r.rank << ", \"tid\": " << lane << ", \"ts\": " << r.start_us << ", \"dur\": "
           << (lane ? r.device_us : r.host_us) << ", \"args\": {\"tag\": \"" << esc(r.tag) << "\", \"peak_mb\": "
           << r.max_device_mem_usage_mb << "}}";
        first = false;
      }
    }
    os << "\n]}\n";
  }
  void ExportChromeTrace(const std::string& path) const {
    std::ofstream f(path);
    TORCH_CHECK(f.is_open(), "cannot write ", path);
    ExportChromeTrace(f);
  }

 private:
  struct State {
    int depth = 0;
    std::string name;
    bool cuda = false;
    std::chrono::steady_clock::time_point t0;
#ifdef ITB_WITH_CUDA
    std::unique_ptr<at::cuda::CUDAEvent> begin, end;
#endif
  };
  static State& state() {
    thread_local State s;
    return s;
  }
  bool enabled_ = false;
  int64_t rank_ = 0;
  std::string tag_ = "Untagged";
  std::vector<KernelCallRecord> records_;
  std::mutex mu_;
  std::chrono::steady_clock::time_point origin_ = std::chrono::steady_clock::now();
};

// RAII range; `like` decides the device the record is timed on.
class ProfileRange {
 public:
  ProfileRange(const char* name, const torch::Tensor& like) : active_(Profiler::Instance().enabled()) {
    if (active_) Profiler::Instance().StartRecord(name, like.defined() && like.is_cuda());
  }
  ProfileRange(const std::string& name, bool cuda) : active_(Profiler::Instance().enabled()) {
    if (active_) Profiler::Instance().StartRecord(name, cuda);
  }
  ~ProfileRange() {
    if (active_) Profiler::Instance().EndRecord();
  }
  ProfileRange(const ProfileRange&) = delete;
  ProfileRange& operator=(const ProfileRange&) = delete;

 private:
  bool active_;
};

}  // namespace utils
}  // namespace itb

#define ITB_PROFILE_CAT2(a, b) a##b
#define ITB_PROFILE_CAT(a, b) ITB_PROFILE_CAT2(a, b)
#define ITB_PROFILE(name, like) ::itb::utils::ProfileRange ITB_PROFILE_CAT(itb_profile_range_, __LINE__)(name, like)
