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
#include "token_io.h"

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
using itb::TokenFile;

// The prefetching ring of token_io.h over (pinned when asked) host tensors.
class TokenBatcher {
 public:
  TokenBatcher(std::shared_ptr<TokenFile> file, int64_t B, int64_t T, int64_t start_batch, int64_t stride,
               int64_t depth, bool pin) {
    TORCH_CHECK(depth >= 3, "TokenBatcher: bad arguments (depth >= 3)");
    auto opts = torch::dtype(torch::kInt64).pinned_memory(pin);
    std::vector<int64_t*> xp, yp;
    for (int64_t i = 0; i < depth; ++i) {
      xs_.push_back(torch::empty({B, T}, opts));
      ys_.push_back(torch::empty({B, T}, opts));
      xp.push_back(xs_.back().data_ptr<int64_t>());
      yp.push_back(ys_.back().data_ptr<int64_t>());
    }
    ring_ = std::make_unique<itb::BatchRing>(std::move(file), B, T, start_batch, stride, std::move(xp), std::move(yp));
  }
  int64_t num_batches() const { return ring_->num_batches(); }
  // Returns (x, y) host tensors that stay valid until two further calls of next().
  std::pair<at::Tensor, at::Tensor> next() {
    const int64_t slot = ring_->next_slot();
    return {xs_[slot], ys_[slot]};
  }
  void skip(int64_t n) {
    for (int64_t i = 0; i < n; ++i) ring_->next_slot();
  }

 private:
  std::vector<at::Tensor> xs_, ys_;          // declared before the ring: its worker writes into them
  std::unique_ptr<itb::BatchRing> ring_;
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
