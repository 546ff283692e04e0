// Python bindings of the host runtime: checkpoint file IO, llm.c token files with a prefetching
// batch assembler, planners.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <torch/extension.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <fstream>
#include <mutex>
#include <thread>

#include "runtime.h"

namespace {

// ------------------------------------------------------------------ checkpoint state-dict files
// Layout (little endian): uint32 magic 0x54504B43, uint32 version 1, uint32 count, then per tensor
// { uint32 name_len, name, int8 dtype code, uint32 ndim, int64 dims[ndim], uint64 bytes, raw data }.
constexpr uint32_t kCkptMagic = 0x54504B43, kCkptVersion = 1;

int8_t dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kBool: return 0;
    case at::kByte: return 1;
    case at::kChar: return 2;
    case at::kUInt16: return 3;
    case at::kShort: return 4;
    case at::kUInt32: return 5;
    case at::kInt: return 6;
    case at::kUInt64: return 7;
    case at::kLong: return 8;
    case at::kBFloat16: return 9;
    case at::kHalf: return 10;
    case at::kFloat: return 11;
    case at::kDouble: return 12;
    default: TORCH_CHECK(false, "checkpoint: unsupported dtype ", t);
  }
}
at::ScalarType dtype_from_code(int8_t c) {
  static const at::ScalarType table[13] = {at::kBool,  at::kByte,   at::kChar, at::kUInt16,   at::kShort,
                                           at::kUInt32, at::kInt,   at::kUInt64, at::kLong,   at::kBFloat16,
                                           at::kHalf,  at::kFloat, at::kDouble};
  TORCH_CHECK(c >= 0 && c < 13, "checkpoint: bad dtype code ", int(c));
  return table[c];
}

void save_state_dict(const std::string& path, const std::vector<std::string>& names,
                     const std::vector<at::Tensor>& tensors) {
  TORCH_CHECK(names.size() == tensors.size(), "save_state_dict: names / tensors mismatch");
  const std::string tmp = path + ".tmp";
  {
    std::ofstream ofs(tmp, std::ios::binary);
    TORCH_CHECK(ofs.is_open(), "Failed to open checkpoint file: ", tmp);
    uint32_t count = static_cast<uint32_t>(names.size());
    ofs.write(reinterpret_cast<const char*>(&kCkptMagic), 4);
    ofs.write(reinterpret_cast<const char*>(&kCkptVersion), 4);
    ofs.write(reinterpret_cast<const char*>(&count), 4);
    for (size_t i = 0; i < names.size(); ++i) {
      at::Tensor t = tensors[i].detach().to(at::kCPU).contiguous();
      uint32_t len = static_cast<uint32_t>(names[i].size());
      ofs.write(reinterpret_cast<const char*>(&len), 4);
      ofs.write(names[i].data(), len);
      int8_t code = dtype_code(t.scalar_type());
      ofs.write(reinterpret_cast<const char*>(&code), 1);
      uint32_t ndim = static_cast<uint32_t>(t.dim());
      ofs.write(reinterpret_cast<const char*>(&ndim), 4);
      for (int64_t d : t.sizes()) ofs.write(reinterpret_cast<const char*>(&d), 8);
      uint64_t bytes = static_cast<uint64_t>(t.numel()) * t.element_size();
      ofs.write(reinterpret_cast<const char*>(&bytes), 8);
      ofs.write(static_cast<const char*>(t.data_ptr()), static_cast<std::streamsize>(bytes));
    }
    TORCH_CHECK(ofs.good(), "write failed: ", tmp);
  }
  TORCH_CHECK(std::rename(tmp.c_str(), path.c_str()) == 0, "rename failed: ", path);
}

std::vector<std::pair<std::string, at::Tensor>> load_state_dict(const std::string& path) {
  std::ifstream ifs(path, std::ios::binary);
  TORCH_CHECK(ifs.is_open(), "Failed to open checkpoint file: ", path);
  uint32_t magic = 0, version = 0, count = 0;
  ifs.read(reinterpret_cast<char*>(&magic), 4);
  ifs.read(reinterpret_cast<char*>(&version), 4);
  ifs.read(reinterpret_cast<char*>(&count), 4);
  TORCH_CHECK(ifs.good() && magic == kCkptMagic, "Invalid checkpoint magic: ", path);
  TORCH_CHECK(version == kCkptVersion, "Unsupported checkpoint version: ", path);
  std::vector<std::pair<std::string, at::Tensor>> out;
  for (uint32_t i = 0; i < count; ++i) {
    uint32_t len = 0;
    ifs.read(reinterpret_cast<char*>(&len), 4);
    TORCH_CHECK(ifs.good() && len < (1u << 20), "Corrupt checkpoint (name length): ", path);
    std::string name(len, '\0');
    ifs.read(name.data(), len);
    int8_t code = 0;
    ifs.read(reinterpret_cast<char*>(&code), 1);
    uint32_t ndim = 0;
    ifs.read(reinterpret_cast<char*>(&ndim), 4);
    TORCH_CHECK(ifs.good() && ndim <= 16, "Corrupt checkpoint (rank): ", path);
    std::vector<int64_t> dims(ndim);
    for (auto& d : dims) ifs.read(reinterpret_cast<char*>(&d), 8);
    uint64_t bytes = 0;
    ifs.read(reinterpret_cast<char*>(&bytes), 8);
    at::Tensor t = torch::empty(dims, torch::dtype(dtype_from_code(code)));
    TORCH_CHECK(bytes == static_cast<uint64_t>(t.numel()) * t.element_size(),
                "Tensor bytes mismatch for key: ", name);
    ifs.read(static_cast<char*>(t.data_ptr()), static_cast<std::streamsize>(bytes));
    TORCH_CHECK(ifs.good() || (ifs.eof() && i + 1 == count && ifs.gcount() == (std::streamsize)bytes),
                "Truncated checkpoint: ", path);
    out.emplace_back(std::move(name), std::move(t));
  }
  return out;
}

// ------------------------------------------------------------------ llm.c token file + batcher
// File: 1024-byte header (int32 magic 20240520 -> uint16 tokens, 20240801 -> uint32 tokens; int32
// version; int32 num_tokens), then the tokens.  Sample i is x = tok[i*T, i*T+T), y = x shifted by 1.
class TokenFile {
 public:
  explicit TokenFile(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    TORCH_CHECK(fd_ >= 0, "cannot open token file: ", path);
    struct stat st;
    TORCH_CHECK(fstat(fd_, &st) == 0, "fstat failed: ", path);
    size_ = static_cast<size_t>(st.st_size);
    TORCH_CHECK(size_ >= 1024, "token file too small: ", path);
    base_ = static_cast<const uint8_t*>(mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
    TORCH_CHECK(base_ != MAP_FAILED, "mmap failed: ", path);
    const int32_t* h = reinterpret_cast<const int32_t*>(base_);
    magic_ = h[0];
    version_ = h[1];
    num_tokens_ = h[2];
    if (magic_ == 20240520) bytes_per_token_ = 2;
    else if (magic_ == 20240801) bytes_per_token_ = 4;
    else TORCH_CHECK(false, "unknown token file magic ", magic_);
    TORCH_CHECK(1024 + static_cast<size_t>(num_tokens_) * bytes_per_token_ <= size_, "token file truncated: ", path);
  }
  ~TokenFile() {
    if (base_ && base_ != MAP_FAILED) munmap(const_cast<uint8_t*>(base_), size_);
    if (fd_ >= 0) ::close(fd_);
  }
  int64_t num_tokens() const { return num_tokens_; }
  int64_t magic() const { return magic_; }
  int64_t version() const { return version_; }
  inline int64_t token(int64_t i) const {
    const uint8_t* p = base_ + 1024 + i * bytes_per_token_;
    if (bytes_per_token_ == 2) { uint16_t v; std::memcpy(&v, p, 2); return v; }
    uint32_t v; std::memcpy(&v, p, 4); return v;
  }
  // x[b, t] = tok[(first + b) * T + t], y shifted by one token.
  void fill(int64_t first_sample, int64_t B, int64_t T, int64_t* x, int64_t* y) const {
    for (int64_t b = 0; b < B; ++b) {
      const int64_t s = (first_sample + b) * T;
      for (int64_t t = 0; t < T; ++t) {
        x[b * T + t] = token(s + t);
        y[b * T + t] = token(s + t + 1);
      }
    }
  }

 private:
  int fd_ = -1;
  size_t size_ = 0;
  const uint8_t* base_ = nullptr;
  int32_t magic_ = 0, version_ = 0, num_tokens_ = 0;
  int bytes_per_token_ = 2;
};

// Assembles batches on a background thread into a ring of (pinned when CUDA is present) host
// buffers; `next()` hands out the oldest ready batch.  Batch k of this loader covers samples
// [(start_batch + k * stride) * B, ... + B): rank r of dp ranks uses start_batch = r, stride = dp.
class TokenBatcher {
 public:
  TokenBatcher(std::shared_ptr<TokenFile> file, int64_t B, int64_t T, int64_t start_batch, int64_t stride,
               int64_t depth, bool pin)
      : file_(std::move(file)), B_(B), T_(T), start_(start_batch), stride_(stride), depth_(depth) {
    TORCH_CHECK(B > 0 && T > 0 && stride > 0 && depth >= 3, "TokenBatcher: bad arguments (depth >= 3)");
    num_samples_ = file_->num_tokens() / T - 1;   // the last sample needs one token of look-ahead
    TORCH_CHECK(num_samples_ >= B, "token file holds fewer samples than one batch");
    num_batches_ = num_samples_ / B;
    auto opts = torch::dtype(torch::kInt64).pinned_memory(pin);
    for (int64_t i = 0; i < depth_; ++i) {
      xs_.push_back(torch::empty({B, T}, opts));
      ys_.push_back(torch::empty({B, T}, opts));
    }
    worker_ = std::thread([this] { this->run(); });
  }
  ~TokenBatcher() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
  }
  int64_t num_batches() const { return num_batches_; }
  // Returns (x, y) host tensors that stay valid until two further calls of next().
  std::pair<at::Tensor, at::Tensor> next() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [this] { return produced_ > consumed_ || stop_; });
    const int64_t slot = consumed_ % depth_;
    ++consumed_;
    lk.unlock();
    cv_.notify_all();
    return {xs_[slot], ys_[slot]};
  }
  void skip(int64_t n) {
    for (int64_t i = 0; i < n; ++i) next();
  }

 private:
  void run() {
    int64_t k = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        // the two batches handed out last may still be read by the consumer: never refill them
        cv_.wait(lk, [this] { return stop_ || produced_ - consumed_ < depth_ - 2; });
        if (stop_) return;
      }
      const int64_t batch = (start_ + k * stride_) % num_batches_;
      const int64_t slot = produced_ % depth_;
      file_->fill(batch * B_, B_, T_, xs_[slot].data_ptr<int64_t>(), ys_[slot].data_ptr<int64_t>());
      ++k;
      {
        std::lock_guard<std::mutex> g(mu_);
        ++produced_;
      }
      cv_.notify_all();
    }
  }
  std::shared_ptr<TokenFile> file_;
  int64_t B_, T_, start_, stride_, depth_;
  int64_t num_samples_ = 0, num_batches_ = 0;
  std::vector<at::Tensor> xs_, ys_;
  std::thread worker_;
  std::mutex mu_;
  std::condition_variable cv_;
  int64_t produced_ = 0, consumed_ = 0;
  bool stop_ = false;
};

}  // namespace

void bind_runtime(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("save_state_dict", &save_state_dict, py::call_guard<py::gil_scoped_release>());
  m.def("load_state_dict", &load_state_dict, py::call_guard<py::gil_scoped_release>());
  py::class_<TokenFile, std::shared_ptr<TokenFile>>(m, "TokenFile")
      .def(py::init<const std::string&>())
      .def_property_readonly("num_tokens", &TokenFile::num_tokens)
      .def_property_readonly("magic", &TokenFile::magic)
      .def_property_readonly("version", &TokenFile::version)
      .def("token", &TokenFile::token)
      .def("sample", [](const TokenFile& f, int64_t i, int64_t T) {
        auto x = torch::empty({T}, torch::kInt64), y = torch::empty({T}, torch::kInt64);
        f.fill(i, 1, T, x.data_ptr<int64_t>(), y.data_ptr<int64_t>());
        return std::make_pair(x, y);
      });
  py::class_<TokenBatcher>(m, "TokenBatcher")
      .def(py::init<std::shared_ptr<TokenFile>, int64_t, int64_t, int64_t, int64_t, int64_t, bool>(),
           py::arg("file"), py::arg("batch"), py::arg("seq_len"), py::arg("start_batch") = 0,
           py::arg("stride") = 1, py::arg("depth") = 4, py::arg("pin") = false)
      .def_property_readonly("num_batches", &TokenBatcher::num_batches)
      .def("next", &TokenBatcher::next, py::call_guard<py::gil_scoped_release>())
      .def("skip", &TokenBatcher::skip, py::call_guard<py::gil_scoped_release>());
  m.def("plan_flat_layout", [](const std::vector<int64_t>& numels, int64_t dp, bool shard, int64_t bucket,
                               bool pad) {
    itb::FlatLayoutResult r = itb::PlanFlatLayout(numels, dp, shard, bucket, pad);
    return py::make_tuple(r.param_start, r.param_end, r.param_bucket, r.bucket_start, r.bucket_end,
                          r.bucket_unpadded, r.numel, r.numel_unpadded);
  });
  auto to_py = [](const std::vector<itb::PipeTask>& v) {
    py::list out;
    for (const auto& t : v)
      out.append(py::make_tuple(t.step, t.microbatch, t.global_chunk, t.local_chunk, t.is_forward, t.stage,
                                t.is_last_chunk, t.is_first_chunk));
    return out;
  };
  m.def("gpipe_schedule", [to_py](int n, int s, int v) { return to_py(itb::GpipeSchedule(n, s, v)); });
  m.def("interleaved_1f1b_schedule",
        [to_py](int n, int s, int v) { return to_py(itb::Interleaved1F1BSchedule(n, s, v)); });
}
