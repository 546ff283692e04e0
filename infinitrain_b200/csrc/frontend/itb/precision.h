// Per-module tensor records for cross-framework alignment (reference: infini_train/src/utils/
// precision_checker.cc:281-473): one line per module output and per gradient that reaches a module
// output, `<context> <name>[_<n>]_<forward|backward> tensor[<i>]: dtype= shape= min= max= mean=
// [first six, ...] [NaN:n Inf:m]`, optional .npy dumps `rank_<r>/<name>[_<n>]_<stage>.npy`, module
// names = state-dict paths.  The Python layer and the reference write the same records, so the three
// logs and dump folders can be compared file by file.  While the checker is on, the Transformer runs
// un-fused through its modules' call operators so that every module computes what its namesake in the
// reference computes.  Formats: `simple` (statistics and the first six values) and `md5` (digest of the fp32
// bytes, after rounding to multiples of `md5_tolerance` when one is given: equal digests then mean "equal within
// the tolerance", precision_checker.cc:249-279).  Levels: 1 = modules, 2 = modules and functions (every op of
// ops.h records its tensor inputs, its output and the gradient that reaches its output under
// `<Name>Function_forward / _backward`, precision_checker.cc:420-446).
#pragma once
#include <array>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <filesystem>
#include <fstream>
#include <sstream>

#include "module.h"
#include "ops.h"

namespace itb {
namespace utils {

// MD5 (RFC 1321) of a byte range, as 32 lowercase hex digits.
inline std::string MD5Hex(const void* data, size_t size) {
  static const uint32_t K[64] = {
      0xd76aa478, 0xe8c7b756, 0x242070db, 0xc1bdceee, 0xf57c0faf, 0x4787c62a, 0xa8304613, 0xfd469501, 0x698098d8, 0x8b44f7af, 0xffff5bb1,
      0x895cd7be, 0x6b901122, 0xfd987193, 0xa679438e, 0x49b40821, 0xf61e2562, 0xc040b340, 0x265e5a51, 0xe9b6c7aa, 0xd62f105d, 0x02441453,
      0xd8a1e681, 0xe7d3fbc8, 0x21e1cde6, 0xc33707d6, 0xf4d50d87, 0x455a14ed, 0xa9e3e905, 0xfcefa3f8, 0x676f02d9, 0x8d2a4c8a, 0xfffa3942,
      0x8771f681, 0x6d9d6122, 0xfde5380c, 0xa4beea44, 0x4bdecfa9, 0xf6bb4b60, 0xbebfbc70, 0x289b7ec6, 0xeaa127fa, 0xd4ef3085, 0x04881d05,
      0xd9d4d039, 0xe6db99e5, 0x1fa27cf8, 0xc4ac5665, 0xf4292244, 0x432aff97, 0xab9423a7, 0xfc93a039, 0x655b59c3, 0x8f0ccc92, 0xffeff47d,
      0x85845dd1, 0x6fa87e4f, 0xfe2ce6e0, 0xa3014314, 0x4e0811a1, 0xf7537e82, 0xbd3af235, 0x2ad7d2bb, 0xeb86d391};
  static const int R[64] = {7, 12, 17, 22, 7, 12, 17, 22, 7, 12, 17, 22, 7, 12, 17, 22, 5, 9,  14, 20, 5, 9,  14, 20, 5, 9,  14, 20, 5, 9,  14, 20,
                            4, 11, 16, 23, 4, 11, 16, 23, 4, 11, 16, 23, 4, 11, 16, 23, 6, 10, 15, 21, 6, 10, 15, 21, 6, 10, 15, 21, 6, 10, 15, 21};
  uint32_t h[4] = {0x67452301, 0xefcdab89, 0x98badcfe, 0x10325476};
  auto block = [&](const uint8_t* p) {
    uint32_t w[16];
    for (int i = 0; i < 16; ++i) w[i] = uint32_t(p[4 * i]) | uint32_t(p[4 * i + 1]) << 8 | uint32_t(p[4 * i + 2]) << 16 | uint32_t(p[4 * i + 3]) << 24;
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3];
    for (int i = 0; i < 64; ++i) {
      uint32_t f;
      int g;
      if (i < 16) f = (b & c) | (~b & d), g = i;
      else if (i < 32) f = (d & b) | (~d & c), g = (5 * i + 1) % 16;
      else if (i < 48) f = b ^ c ^ d, g = (3 * i + 5) % 16;
      else f = c ^ (b | ~d), g = (7 * i) % 16;
      const uint32_t x = a + f + K[i] + w[g];
      a = d, d = c, c = b;
      b = b + ((x << R[i]) | (x >> (32 - R[i])));
    }
    h[0] += a, h[1] += b, h[2] += c, h[3] += d;
  };
  const uint8_t* bytes = static_cast<const uint8_t*>(data);
  size_t done = 0;
  for (; done + 64 <= size; done += 64) block(bytes + done);
  uint8_t tail[128] = {0};
  const size_t rest = size - done;
  if (rest) std::memcpy(tail, bytes + done, rest);
  tail[rest] = 0x80;
  const size_t padded = rest < 56 ? 64 : 128;
  const uint64_t bits = static_cast<uint64_t>(size) * 8;
  for (int i = 0; i < 8; ++i) tail[padded - 8 + i] = static_cast<uint8_t>(bits >> (8 * i));
  block(tail);
  if (padded == 128) block(tail + 64);
  char out[33];
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) std::snprintf(out + 8 * i + 2 * j, 3, "%02x", (h[i] >> (8 * j)) & 0xff);
  return std::string(out, 32);
}

// Digest of a tensor's values as fp32; with a tolerance the values are first rounded to its multiples (double
// arithmetic, halves away from zero, back to fp32), the reference's quantisation bit for bit.
inline std::string ComputeMD5(const Tensor& t, double tolerance = 0.0) {
  Tensor f = t.detach().to(torch::kCPU, torch::kFloat32).contiguous();
  if (tolerance > 0) {
    Tensor x = f.to(torch::kFloat64) * (1.0 / tolerance);
    f = (torch::sign(x) * torch::floor(torch::abs(x) + 0.5) * tolerance).to(torch::kFloat32).contiguous();
  }
  return MD5Hex(f.data_ptr(), static_cast<size_t>(f.numel()) * 4);
}

class PrecisionChecker {
 public:
  static PrecisionChecker& Instance() {
    static PrecisionChecker c;
    return c;
  }
  bool enabled() const { return level_ > 0; }
  int level() const { return level_; }
  // Where in the step the records are made: micro-batch (gradient accumulation step), layer, a name; part of
  // every record ("[GAS-g] [L-l] name ...", precision_check_context.cc:22-29).
  void SetContext(int gas_step, int layer = 0, const std::string& layer_name = "") {
    gas_ = gas_step, layer_ = layer, layer_name_ = layer_name;
  }
  // "level=1,format=simple|md5,path=./out,save_tensors=true,md5_tolerance=1e-3"
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
      else if (k == "md5_tolerance") md5_tolerance_ = std::stod(v);
      else if (k == "format") {
        TORCH_CHECK(v == "simple" || v == "md5", "precision_check: format is simple or md5, not '", v, "'");
        md5_ = v == "md5";
      }
    }
    if (level_ <= 0) return;
    rank_ = rank;
    char stamp[32];
    std::time_t now = std::time(nullptr);
    std::strftime(stamp, sizeof(stamp), "%Y%m%d_%H%M%S", std::localtime(&now));
    dir_ = (std::filesystem::path(path) / stamp).string();
    std::filesystem::create_directories(dir_);
    log_.open(dir_ + "/precision_check_rank_" + std::to_string(rank) + ".log");
    if (level_ >= 2) InstallFunctionHooks();
  }
  // Level 2: the ops of ops.h call this for their tensor arguments and their result.
  void InstallFunctionHooks() {
    ops::function_hook() = [this](const char* name, const TensorList& inputs, const Tensor& output) {
      const std::string n = std::string(name) + "Function";
      size_t i = 0;
      for (const Tensor& t : inputs)
        if (t.defined()) Record("forward", n, i++, t);
      Record("forward", n, 0, output);
      if (output.defined() && output.requires_grad())
        output.register_hook([this, n](const Tensor& grad) { Record("backward", n, 0, grad); });
    };
  }
  void RemoveFunctionHooks() { ops::function_hook() = nullptr; }
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
    os << "[GAS-" << gas_ << "] [L-" << layer_ << "] " << (layer_name_.empty() ? "" : layer_name_ + " ") << log_name << " tensor[" << i
       << "]: dtype=" << DtypeName(t) << " shape=(";
    for (int64_t d = 0; d < t.dim(); ++d) os << (d ? "," : "") << t.size(d);
    os << ") ";
    if (md5_) {
      os << "md5=" << ComputeMD5(f, md5_tolerance_);
    } else if (flat.numel() == 0) {
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
  int level_ = 0, rank_ = 0, gas_ = 0, layer_ = 0;
  std::string layer_name_;
  bool save_ = false, md5_ = false;
  double md5_tolerance_ = 0.0;
  std::string dir_;
  std::ofstream log_;
  std::map<std::string, int> counters_;
  std::vector<std::shared_ptr<HookHandle>> handles_;
};

// True while module outputs are being recorded: the Transformer then takes its un-fused path.
inline bool aligned_mode() { return PrecisionChecker::Instance().enabled(); }

}  // namespace utils
}  // namespace itb
