// Per-module tensor records for cross-framework alignment (reference: infini_train/src/utils/
// precision_checker.cc:281-473): one line per module output and per gradient that reaches a module
// output, `<context> <name>[_<n>]_<forward|backward> tensor[<i>]: dtype= shape= min= max= mean=
// [first six, ...] [NaN:n Inf:m]`, optional .npy dumps `rank_<r>/<name>[_<n>]_<stage>.npy`, module
// names = state-dict paths.  The Python layer and the reference write the same records, so the three
// logs and dump folders can be compared file by file.  While the checker is on, the Transformer runs
// un-fused through its modules' call operators so that every module computes what its namesake in the
// reference computes.  Format `simple` only.
#pragma once
#include <cstdio>
#include <ctime>
#include <filesystem>
#include <fstream>
#include <sstream>

#include "module.h"

namespace itb {
namespace utils {

class PrecisionChecker {
 public:
  static PrecisionChecker& Instance() {
    static PrecisionChecker c;
    return c;
  }
  bool enabled() const { return level_ > 0; }
  // "level=1,format=simple,path=./out,save_tensors=true"
  void Init(const std::string& config, int rank = 0) {
    std::string path = "./log_precision_check";
    std::stringstream ss(config);
    std::string kv;
    while (std::getline(ss, kv, ',')) {
      auto eq = kv.find('=');
      if (eq == std::string::npos) continue;
      std::string k = kv.substr(0, eq), v = kv.substr(eq + 1);
      if (k == "level") level_ = std::stoi(v);
      else if (k == "path") path = v;
      else if (k == "save_tensors") save_ = v == "true" || v == "1";
      else if (k == "format") TORCH_CHECK(v == "simple", "the C++ precision checker writes the simple format only");
    }
    if (level_ <= 0) return;
    rank_ = rank;
    char stamp[32];
    std::time_t now = std::time(nullptr);
    std::strftime(stamp, sizeof(stamp), "%Y%m%d_%H%M%S", std::localtime(&now));
    dir_ = (std::filesystem::path(path) / stamp).string();
    std::filesystem::create_directories(dir_);
    log_.open(dir_ + "/precision_check_rank_" + std::to_string(rank) + ".log");
  }
  const std::string& output_path() const { return dir_; }
  void ResetCounters() { counters_.clear(); }

  // Hooks every module under `root`: paths as names, the root by its type.
  void Attach(const std::shared_ptr<Module>& root) {
    if (!enabled()) return;
    for (auto& [path, m] : root->NamedModules()) {
      std::string name = path.empty() ? m->type() : path;
      Module* raw = m.get();
      handles_.push_back(raw->RegisterForwardPostHook([this, name](Module*, const TensorList&, const TensorList& out) {
        for (size_t i = 0; i < out.size(); ++i) Record("forward", name, i, out[i]);
      }));
      handles_.push_back(raw->RegisterBackwardPostHook(
          [this, name](Module*, size_t i, const Tensor& grad) { Record("backward", name, i, grad); }));
    }
  }

  void Record(const std::string& stage, const std::string& name, size_t i, const Tensor& t) {
    if (!enabled() || !t.defined() || !t.is_floating_point()) return;
    int n = counters_[name + "_" + stage]++;
    std::string log_name = name + (n > 0 ? "_" + std::to_string(n) : "") + "_" + stage;
    Tensor f = t.detach().to(torch::kCPU, torch::kFloat32).contiguous();
    Tensor flat = f.reshape({-1});
    std::ostringstream os;
    os << "[GAS-0] [L-0] " << log_name << " tensor[" << i << "]: dtype=" << DtypeName(t) << " shape=(";
    for (int64_t d = 0; d < t.dim(); ++d) os << (d ? "," : "") << t.size(d);
    os << ") ";
    if (flat.numel() == 0) {
      os << "min=0 max=0 mean=0 [] [NaN:0 Inf:0]";
    } else {
      os << "min=" << flat.min().item<float>() << " max=" << flat.max().item<float>()
         << " mean=" << static_cast<float>(flat.to(torch::kFloat64).mean().item<double>()) << " [";
      const float* p = flat.data_ptr<float>();
      for (int64_t j = 0; j < std::min<int64_t>(6, flat.numel()); ++j) os << (j ? ", " : "") << p[j];
      if (flat.numel() > 6) os << ", ...";
      os << "] [NaN:" << torch::isnan(flat).sum().item<int64_t>() << " Inf:" << torch::isinf(flat).sum().item<int64_t>() << "]";
    }
    log_ << os.str() << std::endl;
    if (save_) SaveNpy(f, dir_ + "/rank_" + std::to_string(rank_), log_name + ".npy");
  }

 private:
  static const char* DtypeName(const Tensor& t) {
    switch (t.scalar_type()) {
      case torch::kFloat32: return "float32";
      case torch::kBFloat16: return "bfloat16";
      case torch::kFloat16: return "float16";
      case torch::kFloat64: return "float64";
      default: return "other";
    }
  }
  // NumPy .npy version 1.0, little-endian fp32, C order
  static void SaveNpy(const Tensor& f32, const std::string& dir, const std::string& file) {
    std::filesystem::create_directories(dir);
    std::ostringstream shape;
    for (int64_t d = 0; d < f32.dim(); ++d) shape << f32.size(d) << (f32.dim() == 1 || d + 1 < f32.dim() ? "," : "");
    std::string header = "{'descr': '<f4', 'fortran_order': False, 'shape': (" + shape.str() + "), }";
    size_t total = 10 + header.size() + 1;
    header += std::string((64 - total % 64) % 64, ' ') + "\n";
    std::ofstream out(dir + "/" + file, std::ios::binary);
    const char magic[8] = {'\x93', 'N', 'U', 'M', 'P', 'Y', 1, 0};
    out.write(magic, 8);
    uint16_t len = static_cast<uint16_t>(header.size());
    out.write(reinterpret_cast<const char*>(&len), 2);
    out.write(header.data(), header.size());
    out.write(static_cast<const char*>(f32.data_ptr()), f32.numel() * 4);
  }
  int level_ = 0, rank_ = 0;
  bool save_ = false;
  std::string dir_;
  std::ofstream log_;
  std::map<std::string, int> counters_;
  std::vector<std::shared_ptr<HookHandle>> handles_;
};

// True while module outputs are being recorded: the Transformer then takes its un-fused path.
inline bool aligned_mode() { return PrecisionChecker::Instance().enabled(); }

}  // namespace utils
}  // namespace itb
