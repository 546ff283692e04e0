// Python bindings of the multi-GPU kernels.  Pointers of peers' buffers come from
// torch.distributed._symmetric_memory as integers; the status word is owned by the caller.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <vector>

#include "../kernels/kernels.h"
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

ItbPeerPtrs dict_ptrs(const pybind11::dict& d, const char* key) {
  if (!d.contains(key)) return ItbPeerPtrs{};
  return to_ptrs(d[key].cast<std::vector<int64_t>>());
}
template <typename T>
T* dict_tensor_ptr(const pybind11::dict& d, const char* key) {
  if (!d.contains(key) || d[key].is_none()) return nullptr;
  return static_cast<T*>(d[key].cast<at::Tensor>().data_ptr());
}
int dict_int(const pybind11::dict& d, const char* key, int dflt) {
  return d.contains(key) ? d[key].cast<int>() : dflt;
}

// One tensor-parallel GEMM launch; `tp` carries the ItbTpArgs fields by name (tensors for this
// GPU's counters and operands, lists of integers for symmetric-memory pointer tables).
void tp_gemm(const at::Tensor& a, bool a_mn, const at::Tensor& b, bool b_mn, int64_t M, int64_t N, int64_t K,
             const c10::optional<at::Tensor>& c, const c10::optional<at::Tensor>& c2,
             const c10::optional<at::Tensor>& bias, const c10::optional<at::Tensor>& aux, int64_t flags,
             const pybind11::dict& tp, at::Tensor& err) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                  a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1,
              "tp_gemm: 2-D bf16 CUDA operands with contiguous rows required");
  TORCH_CHECK(a_mn ? (a.size(0) == K && a.size(1) == M) : (a.size(0) == M && a.size(1) == K), "tp_gemm: A shape");
  TORCH_CHECK(b_mn ? (b.size(0) == K && b.size(1) == N) : (b.size(0) == N && b.size(1) == K), "tp_gemm: B shape");
  ItbGemmArgs g{};
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.A = a.data_ptr();
  g.lda = a.stride(0);
  g.a_mn_major = a_mn;
  g.B = b.data_ptr();
  g.ldb = b.stride(0);
  g.b_mn_major = b_mn;
  if (c.has_value()) {
    TORCH_CHECK(c->scalar_type() == at::kBFloat16 && c->dim() == 2 && c->size(0) == M && c->size(1) >= N &&
                    c->stride(1) == 1,
                "tp_gemm: C must be bf16 [M, >=N]");
    g.C = c->data_ptr();
    g.ldc = c->stride(0);
  }
  if (flags & kGemmGeluDual) {
    TORCH_CHECK(c.has_value() && c2.has_value() && c2->scalar_type() == at::kBFloat16 && c2->stride(0) == c->stride(0),
                "tp_gemm: gelu dual output needs a bf16 C2 with C's layout");
    g.C2 = c2->data_ptr();
  }
  if (flags & kGemmBias) {
    TORCH_CHECK(bias.has_value() && bias->scalar_type() == at::kFloat && bias->numel() >= N, "tp_gemm: fp32 bias");
    g.bias = static_cast<const float*>(bias->data_ptr());
  }
  if (flags & kGemmDGelu) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && aux->stride(1) == 1, "tp_gemm: bf16 aux");
    g.aux = aux->data_ptr();
    g.ld_aux = aux->stride(0);
  }
  g.flags = static_cast<int>(flags);
  g.err = err.data_ptr<int>();

  ItbTpArgs t{};
  t.mode = dict_int(tp, "mode", 0);
  t.rank = dict_int(tp, "rank", 0);
  t.world = dict_int(tp, "world", 0);
  t.T = dict_int(tp, "T", 0);
  t.Tl = dict_int(tp, "Tl", 0);
  t.batch = dict_int(tp, "batch", 0);
  t.started = dict_ptrs(tp, "started");
  t.launch_ctr = dict_tensor_ptr<int>(tp, "launch_ctr");
  t.cta_done = dict_tensor_ptr<unsigned>(tp, "cta_done");
  TORCH_CHECK(t.launch_ctr && t.cta_done, "tp_gemm: launch_ctr and cta_done are required");
  if (t.mode & kItbTpPush) {
    at::Tensor src = tp["push_src"].cast<at::Tensor>();
    TORCH_CHECK(src.scalar_type() == at::kBFloat16 && src.is_contiguous() && src.dim() == 2 &&
                    src.size(0) == static_cast<int64_t>(t.batch) * t.Tl,
                "tp_gemm: push_src must be a contiguous bf16 [batch * Tl, cols] shard");
    t.push_src = src.data_ptr();
    t.push_cols = static_cast<int>(src.size(1));
    t.gather = dict_ptrs(tp, "gather");
    t.gather_mc = reinterpret_cast<void*>(tp.contains("gather_mc") ? tp["gather_mc"].cast<int64_t>() : 0);
    t.push_arrive = dict_ptrs(tp, "push_arrive");
    t.push_total = dict_tensor_ptr<int>(tp, "push_total");
    t.push_lag = dict_int(tp, "push_lag", 1 << 24);
    TORCH_CHECK(t.push_total, "tp_gemm: push_total is required");
  }
  if (t.mode & kItbTpGateA) {
    t.gate_arrive = reinterpret_cast<const int*>(tp["gate_arrive"].cast<int64_t>());
    t.gate_total = dict_tensor_ptr<int>(tp, "gate_total");
    t.gate_includes_this_launch = dict_int(tp, "gate_includes_this_launch", 1);
    TORCH_CHECK(t.gate_arrive && t.gate_total, "tp_gemm: gate counters are required");
  }
  if (t.mode & kItbTpScatter) {
    t.slab = dict_ptrs(tp, "slab");
    t.rs_arrive = dict_ptrs(tp, "rs_arrive");
    t.rs_total = dict_tensor_ptr<int>(tp, "rs_total");
    t.rs_lag = dict_int(tp, "rs_lag", 1 << 24);
    const int64_t rows_local = static_cast<int64_t>(t.batch) * t.Tl;
    if (t.mode & kItbTpBroadcast) {
      t.ar_out = dict_ptrs(tp, "ar_out");
      t.ar_mc = reinterpret_cast<void*>(tp.contains("ar_mc") ? tp["ar_mc"].cast<int64_t>() : 0);
      t.ar_arrive = dict_ptrs(tp, "ar_arrive");
      t.ar_total = dict_tensor_ptr<int>(tp, "ar_total");
      t.ar_lag = dict_int(tp, "ar_lag", 1 << 24);
      TORCH_CHECK(t.ar_total, "tp_gemm: ar_total is required");
    } else {
      at::Tensor out = tp["rs_out"].cast<at::Tensor>();
      TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.size(0) == rows_local && out.size(1) == N &&
                      (out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat),
                  "tp_gemm: rs_out must be [batch * Tl, N] bf16 or fp32");
      t.rs_out = out.data_ptr();
      t.rs_ld_out = out.stride(0);
      t.rs_out_f32 = out.scalar_type() == at::kFloat;
    }
    t.rs_bias = dict_tensor_ptr<const float>(tp, "rs_bias");
    if (tp.contains("rs_residual") && !tp["rs_residual"].is_none()) {
      at::Tensor res = tp["rs_residual"].cast<at::Tensor>();
      TORCH_CHECK(res.scalar_type() == at::kBFloat16 && res.dim() == 2 && res.stride(1) == 1 &&
                      res.size(0) == rows_local && res.size(1) == N,
                  "tp_gemm: rs_residual must be bf16 [batch * Tl, N]");
      t.rs_residual = res.data_ptr();
      t.rs_ld_res = res.stride(0);
    }
    TORCH_CHECK(t.rs_total, "tp_gemm: rs_total is required");
  }
  check(itb_tp_gemm(&g, &t, at::cuda::getCurrentCUDAStream().stream()), "tp_gemm");
}

void nvl_ce_merge(const std::vector<int64_t>& bufs, const std::vector<int64_t>& flags, const at::Tensor& lse_local,
                  const at::Tensor& row_loss, const at::Tensor& t_local, int64_t vocab_valid, at::Tensor& lse_out,
                  at::Tensor& loss_out, int64_t rows_cap, int64_t rank, int64_t world, int64_t ch0, at::Tensor& err,
                  at::Tensor& epoch_ctr) {
  TORCH_CHECK(lse_local.scalar_type() == at::kFloat && row_loss.scalar_type() == at::kFloat &&
                  t_local.scalar_type() == at::kLong && lse_out.scalar_type() == at::kFloat &&
                  loss_out.scalar_type() == at::kFloat && lse_local.is_contiguous() && row_loss.is_contiguous() &&
                  t_local.is_contiguous() && lse_out.is_contiguous() && loss_out.is_contiguous(),
              "nvl_ce_merge: contiguous fp32 statistics and int64 targets required");
  const int64_t rows = lse_local.numel();
  TORCH_CHECK(row_loss.numel() == rows && t_local.numel() == rows && lse_out.numel() == rows && loss_out.numel() == rows,
              "nvl_ce_merge: one entry per row");
  ItbPeerPtrs b = to_ptrs(bufs), f = to_ptrs(flags);
  check(itb_nvl_ce_merge(&b, &f, lse_local.data_ptr<float>(), row_loss.data_ptr<float>(), reinterpret_cast<const long long*>(t_local.data_ptr<int64_t>()),
                         static_cast<int>(vocab_valid), lse_out.data_ptr<float>(), loss_out.data_ptr<float>(),
                         static_cast<int>(rows), static_cast<int>(rows_cap), static_cast<int>(rank),
                         static_cast<int>(world), static_cast<int>(ch0), err.data_ptr<int>(), epoch_ctr.data_ptr<int>(),
                         at::cuda::getCurrentCUDAStream().stream()),
        "ce_merge");
}

void wait_flag(const at::Tensor& flag, int64_t target, int64_t limit, int64_t code, at::Tensor& err) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt && err.is_cuda() && err.scalar_type() == at::kInt,
              "wait_flag: int32 CUDA tensors required");
  check(itb_wait_flag(flag.data_ptr<int>(), static_cast<int>(target), static_cast<unsigned>(limit),
                      static_cast<int>(code), err.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream()),
        "wait_flag");
}

void tp_wait(int64_t arrive_ptr, const at::Tensor& total, int64_t world, at::Tensor& err) {
  check(itb_tp_wait(reinterpret_cast<const int*>(arrive_ptr), total.data_ptr<int>(), static_cast<int>(world),
                    err.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream()),
        "tp_wait");
}

}  // namespace

void bind_comm(pybind11::module_& m) {
  m.attr("MAX_RANKS") = static_cast<int>(kItbMaxRanks);
  m.attr("MAX_COMM_BLOCKS") = static_cast<int>(kItbMaxCommBlocks);
  m.def("comm_blocks", [](int64_t n) { return itb_comm_blocks(n); });
  m.def("nvl_allreduce_scale", &nvl_allreduce_scale);
  m.def("nvl_rs_adamw_bcast", &nvl_rs_adamw_bcast);
  m.attr("TP_PUSH") = static_cast<int>(kItbTpPush);
  m.attr("TP_GATE_A") = static_cast<int>(kItbTpGateA);
  m.attr("TP_SCATTER") = static_cast<int>(kItbTpScatter);
  m.attr("TP_BROADCAST") = static_cast<int>(kItbTpBroadcast);
  m.def("tp_gemm", &tp_gemm);
  m.def("tp_wait", &tp_wait);
  m.def("wait_flag", &wait_flag);
  m.def("nvl_ce_merge", &nvl_ce_merge);
  m.def("tp_gemm_ctas", [](int64_t M, int64_t N) { return itb_tp_gemm_ctas(static_cast<int>(M), static_cast<int>(N)); });
}
