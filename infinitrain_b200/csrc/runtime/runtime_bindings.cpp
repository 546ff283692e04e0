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
#include "state_dict_io.h"
#include "token_io.h"

namespace {

using itb::load_state_dict;
using itb::save_state_dict;

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
