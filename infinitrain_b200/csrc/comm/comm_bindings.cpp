// Python bindings of the multi-GPU kernels.  Pointers of peers' buffers come from
// torch.distributed._symmetric_memory as integers; the status word is owned by the caller.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <vector>

#include "comm.h"

namespace {

ItbPeerPtrs to_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK(v.size() <= kItbMaxRanks, "at most ", int(kItbMaxRanks), " ranks per NVLink group");
  ItbPeerPtrs p{};
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}
void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "infinitrain_b200 NVLink kernel '", what, "' failed with code ", rc);
}

void nvl_allreduce_scale(const std::vector<int64_t>& bufs, int64_t mc, const std::vector<int64_t>& flags,
                         int64_t off, int64_t n, int64_t rank, int64_t world, int64_t ch0, int64_t epoch,
                         double scale, at::Tensor& err, const c10::optional<at::Tensor>& epoch_ctr) {
  ItbPeerPtrs b = to_ptrs(bufs), f = to_ptrs(flags);
  check(itb_nvl_allreduce_scale(&b, reinterpret_cast<void*>(mc), &f, off, n, rank, world, ch0, epoch,
                                static_cast<float>(scale), err.data_ptr<int>(),
                                epoch_ctr.has_value() ? epoch_ctr->data_ptr<int>() : nullptr,
                                at::cuda::getCurrentCUDAStream().stream()),
        "allreduce_scale");
}

void nvl_rs_adamw_bcast(const std::vector<int64_t>& grads, int64_t mc_grads,
                        const std::vector<int64_t>& params, int64_t mc_params,
                        const std::vector<int64_t>& shadows, int64_t mc_shadows, at::Tensor& m,
                        at::Tensor& v, const std::vector<int64_t>& flags, int64_t off, int64_t n,
                        int64_t rank, int64_t world, int64_t ch0, int64_t epoch, double lr, double b1,
                        double b2, double eps, double wd, double bc1, double bc2, double grad_scale,
                        at::Tensor& err, const c10::optional<at::Tensor>& epoch_ctr,
                        const c10::optional<at::Tensor>& dev_hyper) {
  ItbPeerPtrs g = to_ptrs(grads), p = to_ptrs(params), s = to_ptrs(shadows), f = to_ptrs(flags);
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && m.is_contiguous() &&
                  v.is_contiguous() && m.numel() * world == n && v.numel() * world == n,
              "rs_adamw: m and v must be fp32 shard-sized state");
  ItbAdamHyper h{static_cast<float>(lr),  static_cast<float>(b1),        static_cast<float>(b2),
                 static_cast<float>(eps), static_cast<float>(wd),        static_cast<float>(1.0 / bc1),
                 static_cast<float>(1.0 / bc2), static_cast<float>(grad_scale)};
  check(itb_nvl_rs_adamw_bcast(&g, reinterpret_cast<const void*>(mc_grads), &p,
                               reinterpret_cast<void*>(mc_params), &s,
                               reinterpret_cast<void*>(mc_shadows), m.data_ptr<float>(),
                               v.data_ptr<float>(), &f, off, n, rank, world, ch0, epoch, &h,
                               err.data_ptr<int>(),
                               epoch_ctr.has_value() ? epoch_ctr->data_ptr<int>() : nullptr,
                               dev_hyper.has_value() ? dev_hyper->data_ptr<float>() : nullptr,
                               at::cuda::getCurrentCUDAStream().stream()),
        "rs_adamw_bcast");
}

}  // namespace

void bind_comm(pybind11::module_& m) {
  m.attr("MAX_RANKS") = static_cast<int>(kItbMaxRanks);
  m.attr("MAX_COMM_BLOCKS") = static_cast<int>(kItbMaxCommBlocks);
  m.def("comm_blocks", [](int64_t n) { return itb_comm_blocks(n); });
  m.def("nvl_allreduce_scale", &nvl_allreduce_scale);
  m.def("nvl_rs_adamw_bcast", &nvl_rs_adamw_bcast);
}
