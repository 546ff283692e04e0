// The device runtime (itb/runtime.h: streams with priorities, events, raw memory from the tensors'
// pool, copies, the device guard) and the reference-named tensor functions (itb/tensor_api.h), on the
// CPU and, in the CUDA pass, on cuda:0.  Reference surface: infini_train/include/core/runtime/
// device_guard.h:59-143 and include/tensor.h:62-223.
#define ITB_TEST_WITH_TORCH
#include "itb_test.h"

#include <algorithm>
#include <filesystem>
#include <fstream>
#include <sstream>

#include <torch/csrc/distributed/c10d/HashStore.hpp>

#include "itb/itb.h"

using itb::Tensor;
using itbtest::device;
namespace core = itb::core;
namespace ta = itb::tensor_api;

ITB_TEST_P(Runtime, StreamsEventsAndOrdering) {
  core::Runtime& rt = core::Runtime::For(device());
  EXPECT(rt.Type() == device().type() && rt.DeviceCount() >= 1);
  int low = 1, high = 1;
  rt.GetStreamPriorityRange(&low, &high);
  EXPECT(high <= low);
  core::Stream cur = rt.GetStream(device());
  core::Stream side = rt.CreateStreamWithPriority(device(), high);
  // the pools keep fewer levels than the device offers: a high-priority request gets the highest there is
  EXPECT(side.priority() <= 0 && (high == 0 || side.priority() < 0) && side.priority() >= high);
  EXPECT(side.device().type() == device().type());
  core::Event a, b, untimed(core::EventFlag::kDisableTiming);
  EXPECT(rt.EventQuery(&a) == core::RuntimeStatus::kError);   // never recorded
  EXPECT_THROWS(rt.StreamWaitEvent(side, &a));
  rt.EventRecord(&a, cur);
  Tensor x = torch::ones({1 << 16}, torch::dtype(torch::kFloat32).device(device()));
  for (int i = 0; i < 8; ++i) x = x * 1.0001f + 0.5f;
  rt.EventRecord(&b, cur);
  rt.StreamWaitEvent(side, &b);          // work queued on `side` from here on sees x
  EXPECT(rt.EventSynchronize(&b) == core::RuntimeStatus::kSuccess);
  EXPECT(rt.EventQuery(&a) == core::RuntimeStatus::kSuccess);
  EXPECT(rt.EventElapsedTime(&a, &b) >= 0.0f);
  rt.EventRecord(&untimed, cur);
  EXPECT_THROWS(rt.EventElapsedTime(&a, &untimed));
  rt.SynchronizeStream(side);
  rt.SynchronizeDevice(device());
}

ITB_TEST_P(Runtime, RawMemoryAndCopies) {
  core::Runtime& rt = core::Runtime::For(device());
  const size_t n = 1 << 14;
  std::vector<float> host(n), back(n, 0.f);
  for (size_t i = 0; i < n; ++i) host[i] = static_cast<float>(i) * 0.25f;
  rt.ResetMemPoolHighWatermarks(device());
  void *p = nullptr, *q = nullptr;
  rt.Malloc(&p, n * sizeof(float));
  core::Stream s = rt.CreateStream(device());
  rt.MallocAsync(&q, n * sizeof(float), s);
  EXPECT(p && q && p != q && reinterpret_cast<uintptr_t>(p) % 64 == 0);
  rt.Memcpy(p, host.data(), n * sizeof(float), core::MemcpyKind::kH2D);
  core::Event copied;
  rt.EventRecord(&copied, rt.GetStream(device()));
  rt.StreamWaitEvent(s, &copied);
  rt.MemcpyAsync(q, p, n * sizeof(float), core::MemcpyKind::kD2D, s);
  rt.SynchronizeStream(s);
  rt.Memcpy(back.data(), q, n * sizeof(float), core::MemcpyKind::kD2H);
  EXPECT(back == host);
  if (rt.is_cuda()) EXPECT(rt.GetMemPoolPeakMB(device()).second >= rt.GetMemPoolPeakMB(device()).first);
  rt.FreeAsync(q, s);
  rt.Free(p);
  rt.Free(nullptr);
}

ITB_TEST_P(Runtime, DeviceGuardRestoresTheDevice) {
  core::Runtime& rt = core::Runtime::For(device());
  const torch::Device before = rt.GetDevice();
  {
    core::DeviceGuard g(device());
    EXPECT(g.original_device() == before && g.current_device().type() == device().type());
    if (rt.is_cuda() && rt.DeviceCount() > 1) {
      g.SetDevice(torch::Device(torch::kCUDA, 1));
      EXPECT(rt.GetDevice().index() == 1);
    }
  }
  EXPECT(rt.GetDevice() == before);
}

ITB_TEST_P(TensorApi, ReferenceNamesComputeWhatTheirTorchFormsDo) {
  torch::manual_seed(3);
  Tensor a = torch::randn({4, 6}).to(device()), b = torch::randn({4, 6}).to(device());
  EXPECT(ta::Dims(a) == (std::vector<int64_t>{4, 6}) && ta::NumElements(a) == 24 && ta::SizeInBytes(a) == 96);
  EXPECT(torch::equal(ta::Add(ta::Mul(a, 2.0f), b), a * 2.0f + b));
  EXPECT(torch::equal(ta::And(ta::Gt(a, 0.f), ta::Le(b, a)), (a > 0).logical_and(b <= a)));
  EXPECT(torch::allclose(ta::Matmul(a, ta::Transpose(b, 0, 1)), a.matmul(b.t())));
  EXPECT(torch::equal(ta::Max(a, 1, true), std::get<0>(a.max(1, true))));
  EXPECT(ta::Split(a, 4, 1).size() == 2 && ta::Slice(a, 1, 0, 6, 2).size(1) == 3);
  EXPECT(torch::equal(ta::MaskedFill(a, ta::Lt(a, 0.f), 0.f), a.clamp_min(0.f)));
  EXPECT(torch::allclose(ta::Outer(ta::Flatten(a), ta::Flatten(b)).sum(), a.sum() * b.sum(), 1e-3, 1e-3));
  Tensor w = ta::RequiresGrad(torch::ones({6}).to(device()));
  ta::Backward(ta::Sum(ta::Mul(ta::Matmul(a, w), ta::Matmul(a, w)), 0));
  EXPECT(torch::allclose(w.grad(), 2.0f * a.t().matmul(a.matmul(w.detach())), 1e-4, 1e-4));
  ta::ZeroGrad(w);
  EXPECT(!w.grad().defined());
  Tensor f = ta::MakeTensor({3, 2}, torch::kFloat32, device());
  ta::Fill(f, 1.5);
  Tensor g = torch::zeros({3, 2}, torch::kFloat64);
  ta::CopyFrom(g, f);                                   // across devices and dtypes
  EXPECT(g.sum().item<double>() == 9.0);
}

ITB_TEST(TensorApi, SaveAsNpyWritesAVersionOneFile) {
  Tensor t = torch::arange(6, torch::kFloat32).view({2, 3});
  const std::string path = "itb_test_core.npy";
  ta::SaveAsNpy(t, path);
  std::ifstream in(path, std::ios::binary);
  std::string bytes((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  EXPECT(bytes.size() > 64 && bytes.compare(1, 5, "NUMPY") == 0 && bytes[6] == 1);
  EXPECT(bytes.find("'shape': (2,3)") != std::string::npos && bytes.find("'<f4'") != std::string::npos);
  const size_t data = 10 + (static_cast<unsigned char>(bytes[8]) | (static_cast<unsigned char>(bytes[9]) << 8));
  EXPECT(data % 64 == 0 && bytes.size() == data + 24);
  float last;
  std::memcpy(&last, bytes.data() + data + 20, 4);
  EXPECT(last == 5.0f);
  std::remove(path.c_str());
}

ITB_TEST_P(Profiler, RecordsOpsOncePerOuterRangeAndReportsPerTag) {
  auto& prof = itb::utils::Profiler::Instance();
  prof.Reset();
  torch::manual_seed(1);
  Tensor x = torch::randn({8, 16}).to(device()), w = torch::randn({32, 16}).to(device()).set_requires_grad(true);
  itb::ops::linear(x, w);                      // disabled: nothing is recorded
  EXPECT(prof.records().empty());
  prof.Enable(3);
  prof.SetTag("Step_1");
  {
    ITB_PROFILE("outer", x);
    itb::ops::linear(x, w);                    // nested in "outer": part of it
  }
  Tensor y = itb::ops::linear(x, w);
  itb::ops::layernorm(y, torch::ones({32}).to(device()), c10::nullopt);
  prof.SetTag("Step_2");
  itb::ops::linear(x, w).sum().backward();
  prof.Disable();
  std::vector<std::string> names;
  for (const auto& r : prof.records()) names.push_back(r.tag + ":" + r.name);
  EXPECT(names.size() >= 4 && names[0] == "Step_1:outer" && names[1] == "Step_1:linear" && names[2] == "Step_1:layernorm");
  EXPECT(names[3] == "Step_2:linear");
  for (const auto& r : prof.records()) EXPECT(r.rank == 3 && r.host_us >= 0 && r.device == (device().is_cuda() ? "cuda" : "cpu"));
  if (device().is_cuda()) EXPECT(prof.records()[1].device_us > 0);
  std::ostringstream rep, rec;
  prof.Report(rep, itb::utils::Profiler::SortBy::Count);
  prof.PrintRecords(rec);
  EXPECT(rep.str().find("Tag: Step_1") != std::string::npos && rep.str().find("Tag: Step_2") != std::string::npos);
  EXPECT(rep.str().find("Device Avg(us)") != std::string::npos && rec.str().find("Step_2\t3\tlinear") != std::string::npos);
  // Chrome trace: one host span per record (and one device span on cuda), rank as the process id
  std::ostringstream trace;
  prof.ExportChromeTrace(trace);
  const std::string tj = trace.str();
  size_t spans = 0;
  for (size_t at = tj.find("\"ph\": \"X\""); at != std::string::npos; at = tj.find("\"ph\": \"X\"", at + 1)) ++spans;
  EXPECT(spans == prof.records().size() * (device().is_cuda() ? 2 : 1));
  EXPECT(tj.find("\"traceEvents\": [") != std::string::npos && tj.find("\"name\": \"outer\"") != std::string::npos);
  EXPECT(tj.find("\"pid\": 3") != std::string::npos && tj.find("\"tag\": \"Step_2\"") != std::string::npos);
  EXPECT(tj.rfind("]}") != std::string::npos && std::count(tj.begin(), tj.end(), '{') == std::count(tj.begin(), tj.end(), '}'));
  prof.Reset();
  EXPECT(prof.records().empty());
}

ITB_TEST(Data, LoadersStackConsecutiveSamplesAndRanksStrideOverBatches) {
  // 7 samples of (i, 10 i): batch size 2 gives three full batches, the ragged one is dropped
  auto ds = std::make_shared<itb::data::TensorDataset>(torch::arange(7, torch::kFloat32).view({7, 1}), torch::arange(7, torch::kFloat32) * 10);
  itb::data::DataLoader loader(ds, 2);
  EXPECT(loader.num_batches() == 3);
  std::vector<float> firsts;
  for (auto it = loader.begin(); it != loader.end(); ++it) {
    auto [x, y] = *it;
    EXPECT(x.size(0) == 2 && x.size(1) == 1 && y.size(0) == 2);
    EXPECT(y[1].item<float>() == 10 * x[1][0].item<float>());
    firsts.push_back(x[0][0].item<float>());
  }
  EXPECT((firsts == std::vector<float>{0, 2, 4}));
  itb::data::DistributedDataLoader r0(ds, 2, 0, 2), r1(ds, 2, 1, 2);
  std::vector<size_t> b0, b1;
  for (auto it = r0.begin(); it < r0.end(); it++) b0.push_back(it.BatchIndex());
  for (auto it = r1.begin(); it < r1.end(); it++) b1.push_back(it.BatchIndex());
  EXPECT((b0 == std::vector<size_t>{0, 2}) && (b1 == std::vector<size_t>{1}));
  EXPECT_THROWS(*loader.end());
  EXPECT_THROWS(itb::data::DistributedDataLoader(ds, 2, 2, 2));
}

ITB_TEST(Data, TokenFileSamplesShiftTheTargetByOneToken) {
  const std::string path = "itb_test_tokens.bin";
  {
    std::ofstream f(path, std::ios::binary);
    int32_t header[256] = {20240520, 1, 11};
    f.write(reinterpret_cast<const char*>(header), sizeof(header));
    for (uint16_t t = 0; t < 11; ++t) {
      uint16_t v = static_cast<uint16_t>(100 + t);
      f.write(reinterpret_cast<const char*>(&v), 2);
    }
  }
  itb::data::TinyShakespeareDataset ds(path, 4);
  EXPECT(ds.Size() == 2);                         // (11 - 1) / 4
  auto [x, y] = ds[1];
  EXPECT(x[0].item<int64_t>() == 104 && x[3].item<int64_t>() == 107 && y[0].item<int64_t>() == 105 && y[3].item<int64_t>() == 108);
  EXPECT_THROWS(ds[2]);
  std::remove(path.c_str());
}

ITB_TEST(DataTypes, SizesNamesPromotionAndTorchMapping) {
  using itb::DataType;
  const DataType all[] = {DataType::kBOOL, DataType::kUINT8, DataType::kINT8, DataType::kUINT16, DataType::kINT16, DataType::kUINT32,
                          DataType::kINT32, DataType::kUINT64, DataType::kINT64, DataType::kBFLOAT16, DataType::kFLOAT16,
                          DataType::kFLOAT32, DataType::kFLOAT64};
  for (DataType t : all) {
    EXPECT(itb::FromTorch(itb::ToTorch(t)) == t);
    EXPECT(itb::DataTypeSize(t) == torch::elementSize(itb::ToTorch(t)));
    EXPECT(itb::PromoteDataTypes(t, t) == t);
  }
  EXPECT(std::string(itb::DataTypeDesc(DataType::kBFLOAT16)) == "bfloat16");
  EXPECT(itb::PromoteDataTypes(DataType::kFLOAT16, DataType::kBFLOAT16) == DataType::kFLOAT32);
  EXPECT(itb::PromoteDataTypes(DataType::kINT64, DataType::kBFLOAT16) == DataType::kBFLOAT16);
  EXPECT(itb::PromoteDataTypes(DataType::kINT32, DataType::kINT64) == DataType::kINT64);
  EXPECT(itb::PromoteDataTypes(DataType::kFLOAT32, DataType::kFLOAT64) == DataType::kFLOAT64);
  itb::Scalar a(2.75), b(true), c(int64_t(-3)), d(uint64_t(7));
  EXPECT(a.To<int>() == 2 && b.To<double>() == 1.0 && c.To<float>() == -3.0f && d.kind() == itb::Scalar::Kind::kUInt64);
  Tensor t = torch::zeros({2});
  t.fill_(a.ToTorch());
  EXPECT(t[1].item<float>() == 2.75f);
}

// ---- process-wide module hooks, backward pre-hooks
ITB_TEST(Hooks, GlobalRegistryRunsAroundTheModulesOwnHooksAndHandlesRemoveThem) {
  using namespace itb::nn;
  auto net = std::make_shared<Sequential>(std::vector<std::shared_ptr<itb::Module>>{
      std::make_shared<Linear>(4, 3), std::make_shared<Sigmoid>(), std::make_shared<Linear>(3, 2)});
  std::vector<std::string> order;
  auto& reg = itb::GlobalModuleHookRegistry::Instance();
  auto h1 = reg.RegisterModuleForwardPreHook([&](itb::Module* m, const itb::TensorList&) { order.push_back("gpre:" + m->type()); });
  auto h2 = reg.RegisterModuleForwardHook(
      [&](itb::Module* m, const itb::TensorList&, const itb::TensorList& out) { order.push_back("gpost:" + m->type() + ":" + std::to_string(out.size())); });
  int backward_calls = 0;
  auto h3 = reg.RegisterModuleFullBackwardHook([&](itb::Module*, const itb::TensorList& grad_outputs, const itb::TensorList&) {
    EXPECT(grad_outputs.size() == 1 && grad_outputs[0].defined());
    ++backward_calls;
  });
  auto local_pre = net->RegisterForwardPreHook([&](itb::Module*, const itb::TensorList&) { order.push_back("pre"); });
  auto local_post = net->RegisterForwardPostHook([&](itb::Module*, const itb::TensorList&, const itb::TensorList&) { order.push_back("post"); });
  std::vector<std::string> bwd_order;
  auto bpre = net->RegisterBackwardPreHook([&](itb::Module*, size_t, const Tensor&) { bwd_order.push_back("bpre"); });
  auto bpost = net->RegisterBackwardPostHook([&](itb::Module*, size_t, const Tensor&) { bwd_order.push_back("bpost"); });
  EXPECT(reg.HasModuleBackwardHooks());

  Tensor x = torch::randn({5, 4});
  Tensor y = (*net)(x);
  // the Sequential itself, then its three children; the module's own hooks sit inside the global ones
  EXPECT(order.size() == 2 + 2 + 3 * 2);
  EXPECT(order[0] == "gpre:Sequential" && order[1] == "pre");
  EXPECT(order[2] == "gpre:Linear" && order[3] == "gpost:Linear:1");
  EXPECT(order[order.size() - 2] == "post" && order.back() == "gpost:Sequential:1");
  y.sum().backward();
  EXPECT(backward_calls == 4);               // every module whose output needed a gradient
  EXPECT(bwd_order.size() == 2 && bwd_order[0] == "bpre" && bwd_order[1] == "bpost");

  h1->Remove(), h2->Remove(), h3->Remove();
  EXPECT(reg.empty() && !reg.HasModuleBackwardHooks());
  order.clear();
  backward_calls = 0;
  (*net)(x).sum().backward();
  EXPECT(order.size() == 2 && order[0] == "pre" && order[1] == "post" && backward_calls == 0);
}

// ---- nn::function
ITB_TEST_P(Functional, ReferenceNamesAndTheReferencesResultTypes) {
  namespace F = itb::nn::function;
  auto opt = torch::dtype(torch::kFloat32).device(device());
  Tensor a = torch::arange(12, opt).reshape({3, 4}) - 5.0f;
  EXPECT(torch::equal(F::Tril(a), a.tril()) && torch::equal(F::Triu(a, 1), a.triu(1)));
  EXPECT(F::Ones({2, 3}).sum().item<float>() == 6.0f);
  EXPECT(torch::allclose(F::Pow(2.0f, a), torch::pow(2.0, a)) && torch::allclose(F::Pow(a, 2.0f), a * a));
  EXPECT(torch::allclose(F::Softmax(a, -1).sum(-1), torch::ones({3}, opt)));
  EXPECT(torch::equal(F::Slice(a, {1, 0}, {3, 4}, {1, 2}), a.slice(0, 1, 3).slice(1, 0, 4, 2)));
  EXPECT_THROWS(F::Slice(a, {0}, {1}, {1}));
  EXPECT(F::Stack({a, a}, 0).sizes() == torch::IntArrayRef({2, 3, 4}) && F::Concat({a, a}, 1).sizes() == torch::IntArrayRef({3, 8}));
  EXPECT(torch::equal(F::Max(a, 1), std::get<0>(a.max(1))) && torch::equal(F::Mean(a, 0, true), a.mean(0, true)));
  // comparisons: 0 / 1 in the input's dtype, also for a half-precision input
  Tensor lt = F::Lt(a, 0.0f);
  EXPECT(lt.scalar_type() == torch::kFloat32 && lt.sum().item<float>() == 5.0f);
  Tensor h = a.to(torch::kBFloat16);
  EXPECT(F::Ge(h, h).scalar_type() == torch::kBFloat16 && F::Equals(h, h).to(torch::kFloat32).sum().item<float>() == 12.0f);
  EXPECT(torch::equal(F::And(F::Gt(a, -2.0f), F::Le(a, 2.0f)), ((a > -2) & (a <= 2)).to(torch::kFloat32)));
  EXPECT(torch::equal(F::Or(F::Lt(a, -4.0f), F::Gt(a, 5.0f)), ((a < -4) | (a > 5)).to(torch::kFloat32)));
  // masks aligned to the trailing or to the leading dimensions
  Tensor t3 = torch::ones({2, 3, 4}, opt);
  Tensor tail = torch::zeros({3, 4}, opt);
  tail[0][0] = 1;
  EXPECT(F::Mask(t3, tail, -1.0f).sum().item<float>() == 24.0f - 2 * 2.0f);
  Tensor lead = torch::zeros({2}, opt);
  lead[1] = 1;
  EXPECT(F::Mask(t3, lead, 0.0f).sum().item<float>() == 12.0f);
  EXPECT_THROWS(F::Mask(t3, torch::zeros({5}, opt), 0.0f));
  // top-k scatter
  Tensor vals = torch::tensor({{1.0f, 2.0f}, {3.0f, 4.0f}}, opt);
  Tensor idx = torch::tensor({{0, 3}, {2, 1}}, torch::dtype(torch::kLong).device(device()));
  Tensor sc = F::Scatter(vals, idx, {2, 4});
  EXPECT(torch::equal(sc, torch::tensor({{1.0f, 0.0f, 0.0f, 2.0f}, {0.0f, 4.0f, 3.0f, 0.0f}}, opt)));
  EXPECT(torch::equal(F::Gather(sc, 1, idx), vals));
}

// ---- single-process DataParallel and its helpers
namespace {
std::shared_ptr<itb::Module> TinyNet() {
  using namespace itb::nn;
  return std::make_shared<Sequential>(std::vector<std::shared_ptr<itb::Module>>{
      std::make_shared<Linear>(6, 5), std::make_shared<Sigmoid>(), std::make_shared<Linear>(5, 3)});
}
}  // namespace

ITB_TEST(DataParallel, ScatterGatherAndBroadcastHelpers) {
  namespace pf = itb::parallel::function;
  std::vector<torch::Device> cpus(3, torch::Device(torch::kCPU));
  Tensor x = torch::arange(14, torch::kFloat32).reshape({7, 2}).set_requires_grad(true);
  auto parts = pf::Scatter({x}, cpus, 0);
  EXPECT(parts.size() == 3 && parts[0][0].size(0) == 3 && parts[2][0].size(0) == 1);
  auto two = pf::Scatter({torch::zeros({2, 2})}, cpus, 0);
  EXPECT(two.size() == 2);                                   // fewer chunks than devices
  Tensor back = pf::Gather(parts, cpus[0], 0)[0];
  EXPECT(torch::equal(back, x));
  (back * 2).sum().backward();
  EXPECT(torch::equal(x.grad(), torch::full({7, 2}, 2.0f)));  // the split and the join are differentiable
  auto copies = pf::BroadcastCoalescedReshape({x, back}, cpus);
  EXPECT(copies.size() == 3 && copies[1].size() == 2 && torch::equal(copies[2][0], x));
  EXPECT(copies[1][0].data_ptr() != x.data_ptr() && !copies[1][0].requires_grad());
  auto net = TinyNet();
  auto reps = pf::Replicate(net, TinyNet, cpus);
  EXPECT(reps.size() == 3 && reps[0] == net && reps[1] != net);
  auto a = net->StateDict(), b = reps[2]->StateDict();
  for (auto& [k, v] : a) EXPECT(torch::equal(v, b.at(k)) && v.data_ptr() != b.at(k).data_ptr());
}

ITB_TEST(DataParallel, ReplicasGiveTheOneModuleGradientsAndFollowItsUpdates) {
  itb::nn::ManualSeed(7);
  auto single = TinyNet();
  auto wrapped_inner = TinyNet();
  wrapped_inner->LoadStateDict(single->StateDict());
  std::vector<torch::Device> cpus(3, torch::Device(torch::kCPU));
  auto dp = std::make_shared<itb::parallel::DataParallel>(wrapped_inner, TinyNet, cpus);
  EXPECT(dp->Parameters().size() == single->Parameters().size());   // the replicas are not parameters of the wrapper
  itb::optim::SGD opt_single(single->Parameters(), 0.1), opt_dp(dp->Parameters(), 0.1);
  Tensor x = torch::randn({8, 6}), y = torch::randint(0, 3, {8});
  for (int step = 0; step < 3; ++step) {
    opt_single.ZeroGrad(), opt_dp.ZeroGrad();
    Tensor l1 = itb::ops::cross_entropy((*single)(x), y);
    Tensor l2 = itb::ops::cross_entropy((*dp)(x), y);
    EXPECT(std::fabs(l1.item<float>() - l2.item<float>()) < 1e-6f);
    l1.backward(), l2.backward();
    auto g1 = single->Parameters(), g2 = dp->Parameters();
    for (size_t i = 0; i < g1.size(); ++i) EXPECT(torch::allclose(g1[i].grad(), g2[i].grad(), 1e-5, 1e-6));
    opt_single.Step(), opt_dp.Step();
  }
  EXPECT(dp->replica_forwards() == 9);
  // a batch of one runs on the source module alone; without grad mode nothing is recorded
  EXPECT((*dp)(x.slice(0, 0, 1)).sizes() == torch::IntArrayRef({1, 3}) && dp->replica_forwards() == 9);
  {
    torch::NoGradGuard g;
    EXPECT(!(*dp)(x).requires_grad());
  }
  // an error inside one replica's thread comes back to the caller
  EXPECT_THROWS((*dp)(torch::randn({8, 5})));
}

// ---- LoRA utilities by path and by state dict
ITB_TEST(LoRA, ReplaceByPathBaseParametersAndStateDictLoading) {
  namespace lora = itb::nn::lora;
  auto net = TinyNet();
  lora::LoRAConfig cfg;
  cfg.rank = 2, cfg.alpha = 4.0f;
  cfg.target_modules = lora::ParseLoRATargetModules("0");
  lora::GetLoRAModel(net, cfg);
  EXPECT(lora::LoRAModules(net).size() == 1);
  EXPECT(lora::GetLoRAParameters(net).size() == 2 && lora::GetBaseParameters(net).size() == 4);
  for (auto& p : lora::GetBaseParameters(net)) EXPECT(!p.requires_grad());
  auto sd = lora::LoRAStateDict(net);
  std::map<std::string, Tensor> incoming;
  for (auto& [k, v] : sd) incoming[k] = torch::full_like(v, 0.5f);
  incoming["nowhere.lora_A"] = torch::zeros({1});
  lora::LoadLoRAStateDict(net, incoming);                      // the unknown name is reported, not fatal
  for (auto& [k, v] : lora::LoRAStateDict(net)) EXPECT(v.mean().item<float>() == 0.5f);
  incoming.begin()->second = torch::zeros({1, 1});
  EXPECT_THROWS(lora::LoadLoRAStateDict(net, incoming));
  auto fresh = std::make_shared<itb::nn::Linear>(6, 5);
  lora::ReplaceModuleByPath(net, "0", fresh);
  EXPECT(lora::LoRAModules(net).empty() && net->mutable_module("0") == fresh);
  EXPECT_THROWS(lora::ReplaceModuleByPath(net, "7.weight", fresh));
  EXPECT_THROWS(lora::ReplaceModuleByPath(net, "", fresh));
}

// ---- IDX files
ITB_TEST(Data, IdxFilesAndTheMnistDataset) {
  const std::string dir = itbtest::temp_dir("mnist");
  auto be32 = [](std::ofstream& f, uint32_t v) {
    unsigned char b[4] = {static_cast<unsigned char>(v >> 24), static_cast<unsigned char>(v >> 16), static_cast<unsigned char>(v >> 8),
                          static_cast<unsigned char>(v)};
    f.write(reinterpret_cast<const char*>(b), 4);
  };
  const int n = 5;
  for (const char* prefix : {"train", "t10k"}) {
    std::ofstream img(dir + "/" + prefix + "-images-idx3-ubyte", std::ios::binary), lab(dir + "/" + prefix + "-labels-idx1-ubyte", std::ios::binary);
    be32(img, 0x00000803), be32(img, n), be32(img, 28), be32(img, 28);
    be32(lab, 0x00000801), be32(lab, n);
    for (int i = 0; i < n; ++i) {
      std::vector<unsigned char> px(28 * 28, static_cast<unsigned char>(51 * i));
      img.write(reinterpret_cast<const char*>(px.data()), px.size());
      unsigned char l = static_cast<unsigned char>(i * 2);
      lab.write(reinterpret_cast<const char*>(&l), 1);
    }
  }
  itb::data::MNISTDataset ds(dir, true);
  EXPECT(ds.Size() == 5);
  auto [x, y] = ds[3];
  EXPECT(x.sizes() == torch::IntArrayRef({28, 28}) && x.scalar_type() == torch::kFloat32 && y.scalar_type() == torch::kUInt8);
  EXPECT(std::fabs(x[0][0].item<float>() - 153.0f / 255.0f) < 1e-6f && y.item<uint8_t>() == 6);
  itb::data::DataLoader loader(std::make_shared<itb::data::MNISTDataset>(dir, false), 2);
  auto [bx, by] = *loader.begin();
  EXPECT(bx.sizes() == torch::IntArrayRef({2, 28, 28}) && by.sizes() == torch::IntArrayRef({2}));
  // uint8 class indices go straight into the loss
  Tensor loss = itb::ops::cross_entropy(torch::zeros({2, 10}), by);
  EXPECT(std::fabs(loss.item<float>() - std::log(10.0f)) < 1e-5f);
  // a file that is not IDX, and one shorter than its header says
  { std::ofstream bad(dir + "/bad", std::ios::binary); bad << "nope, not idx"; }
  EXPECT_THROWS(itb::data::ReadIdxFile(dir + "/bad"));
  { std::ofstream cut(dir + "/short", std::ios::binary); be32(cut, 0x00000801); be32(cut, 100); cut << "abc"; }
  EXPECT_THROWS(itb::data::ReadIdxFile(dir + "/short"));
  EXPECT_THROWS(itb::data::ReadIdxFile(dir + "/absent"));
}

// ---- failure detection on the host: heartbeats, watchdog, abort, fault injection
ITB_TEST(FaultTolerance, WatchdogSeesAStalePeerAndAbortsTheGroupsOfItsRank) {
  using itb::utils::Heartbeat;
  auto store = c10::make_intrusive<c10d::HashStore>();
  // a group that only records that it was aborted
  struct Probe : itb::parallel::ProcessGroup {
    Probe() : ProcessGroup("probe", {0, 1}, 0) {}
    using W = std::shared_ptr<itb::parallel::Work>;
    W AllReduce(Tensor&, itb::parallel::ReduceOp, bool) override { return nullptr; }
    W AllGather(Tensor&, const Tensor&, bool) override { return nullptr; }
    W ReduceScatter(Tensor&, const Tensor&, itb::parallel::ReduceOp, bool) override { return nullptr; }
    W BroadCast(Tensor&, int, bool) override { return nullptr; }
    W Send(const itb::TensorList&, int, bool) override { return nullptr; }
    W Recv(itb::TensorList&, int, bool) override { return nullptr; }
    W BatchSendRecv(std::vector<itb::parallel::P2POp>&, bool) override { return nullptr; }
    void Barrier() override {}
  };
  auto group = std::make_shared<Probe>();
  Heartbeat a(store, 0, 2, /*timeout_s=*/0.3, /*poll_s=*/0.05, [&] { return std::vector<std::shared_ptr<itb::parallel::ProcessGroup>>{group}; });
  Heartbeat b(store, 1, 2, 0.3, 0.05);
  a.Start();
  b.Beat(0);
  for (int step = 1; step <= 3; ++step) {          // both alive: no report
    a.Step(step), b.Step(step);
    std::this_thread::sleep_for(std::chrono::milliseconds(60));
  }
  EXPECT(!a.failure() && !group->aborted());
  // rank 1 falls silent; rank 0 goes on beating
  const auto t0 = std::chrono::steady_clock::now();
  while (!a.failure() && std::chrono::steady_clock::now() - t0 < std::chrono::seconds(5)) {
    a.Beat(4);
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
  EXPECT(a.failure() && a.failure()->kind == "stale_heartbeat" && a.failure()->rank == 1 && a.failure()->step == 3);
  EXPECT(group->aborted());
  EXPECT_THROWS(a.Step(5));
  // rank 0 posted the reason: rank 1 reads it as a peer's abort, on a scan of its own and in WaitPeers
  auto seen = b.Scan();
  EXPECT(seen && seen->kind == "peer_abort" && seen->rank == 0 && seen->detail.find("stale_heartbeat of rank 1") != std::string::npos);
  EXPECT_THROWS(b.WaitPeers(9, 0.2));
  a.Stop();
}

ITB_TEST(FaultTolerance, ScanClockGracePeriodAndWaitPeers) {
  using itb::utils::Heartbeat;
  auto store = c10::make_intrusive<c10d::HashStore>();
  Heartbeat a(store, 0, 3, 10.0, 0.05), b(store, 1, 3, 10.0, 0.05), c(store, 2, 3, 10.0, 0.05);
  const double now = itb::utils::wall_seconds();
  EXPECT(!a.Scan(now));                                   // nobody has beaten yet, inside the grace period
  auto late = a.Scan(now + 11.0);
  EXPECT(late && late->kind == "stale_heartbeat" && late->detail == "no heartbeat was ever published");
  b.Beat(4), c.Beat(5);
  EXPECT(!a.Scan(now + 5.0));
  auto stale = a.Scan(now + 20.0);
  EXPECT(stale && stale->rank == 1 && stale->step == 4);
  a.WaitPeers(4, 1.0);                                    // both peers are at step 4 or later
  std::thread slow([&] {
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    b.Beat(5);
  });
  a.WaitPeers(5, 2.0);                                    // returns once rank 1 arrives
  slow.join();
  bool threw = false;
  try {
    a.WaitPeers(6, 0.15);
  } catch (const itb::utils::RankFailure& e) {
    threw = std::string(e.what()).find("did not reach step 6") != std::string::npos;
  }
  EXPECT(threw);
  // a status word of a kernel: zero passes, anything else is a timeout of a bounded wait
  itb::utils::CheckKernelStatus([] { return 0; });
  EXPECT_THROWS(itb::utils::CheckKernelStatus([] { return 7; }, "probe"));
}

ITB_TEST(FaultTolerance, InjectorFiresOnceOnItsRankAndStepAndRefusesToEndACudaRankUnderMulticast) {
  using itb::utils::FaultInjector;
  FaultInjector none(0, "");
  EXPECT(!none.armed());
  none.MaybeFire(1);
  FaultInjector other(0, "1:3:raise");
  EXPECT(!other.armed());
  other.MaybeFire(3);                                      // another rank's fault
  FaultInjector raise(1, "1:3:raise");
  raise.MaybeFire(2);
  EXPECT(!raise.fired());
  EXPECT_THROWS(raise.MaybeFire(3));
  raise.MaybeFire(3);                                      // once only
  auto store = c10::make_intrusive<c10d::HashStore>();
  itb::utils::Heartbeat hb(store, 0, 1);
  FaultInjector mute(0, "0:2:mute", &hb);
  hb.Beat(1);
  mute.MaybeFire(2);
  hb.Beat(2);                                              // muted: the store keeps step 1
  auto raw = store->get("itb/hb/0");
  EXPECT(std::string(raw.begin(), raw.end()).rfind("1:", 0) == 0);
  FaultInjector stall(0, "0:1:stall:0.05");
  const auto t0 = std::chrono::steady_clock::now();
  stall.MaybeFire(1);
  EXPECT(std::chrono::steady_clock::now() - t0 >= std::chrono::milliseconds(45));
  EXPECT_THROWS(FaultInjector(0, "0:1"));
  EXPECT_THROWS(FaultInjector(0, "0:1:explode"));
  // a CUDA rank may be ended only with NVLink multicast off in NCCL and in this framework's kernels
  unsetenv("ITB_NVLS"), unsetenv("NCCL_NVLS_ENABLE");
  FaultInjector gpu_exit(0, "0:1:exit", nullptr, /*on_cuda=*/true);
  EXPECT(!gpu_exit.ExitAllowed());
  EXPECT_THROWS(gpu_exit.MaybeFire(1));
  setenv("ITB_NVLS", "0", 1), setenv("NCCL_NVLS_ENABLE", "0", 1);
  EXPECT(FaultInjector(0, "0:1:exit", nullptr, true).ExitAllowed());
  unsetenv("ITB_NVLS"), unsetenv("NCCL_NVLS_ENABLE");
  EXPECT(FaultInjector(0, "0:1:exit").ExitAllowed());     // CPU rank
}

ITB_TEST(FaultTolerance, ACorruptedCheckpointIsRefusedByTheLoader) {
  const std::string dir = itbtest::temp_dir("corrupt");
  std::map<std::string, Tensor> sd = {{"w", torch::arange(12, torch::kFloat32).view({3, 4})}, {"b", torch::ones({4})}};
  itb::io::SaveStateDict(dir + "/model.ckpt", sd);
  auto back = itb::io::LoadStateDict(dir + "/model.ckpt");
  EXPECT(torch::equal(back.at("w"), sd.at("w")));
  itb::utils::CorruptFile(dir + "/model.ckpt", 0, 4);      // the magic number
  EXPECT_THROWS(itb::io::LoadStateDict(dir + "/model.ckpt"));
  itb::utils::CorruptFile(dir + "/model.ckpt", 0, 4);      // flipping twice restores the file
  EXPECT(torch::equal(itb::io::LoadStateDict(dir + "/model.ckpt").at("b"), sd.at("b")));
  EXPECT_THROWS(itb::utils::CorruptFile(dir + "/absent", 0, 4));
}

ITB_TEST(Init, FansGainsBoundsAndGenerators) {
  namespace init = itb::nn::init;
  Tensor w = torch::empty({6, 4, 3});
  auto fans = init::CalculateFanInAndFanOut(w);
  EXPECT(fans.first == 12 && fans.second == 18);
  EXPECT_THROWS(init::CalculateFanInAndFanOut(torch::empty({5})));
  EXPECT_NEAR(init::CalculateGain(init::NonLinearityType::kLeakyReLU, std::sqrt(5.0f)), std::sqrt(1.0f / 3.0f), 1e-6);
  EXPECT_NEAR(init::CalculateGain(init::NonLinearityType::kReLU), std::sqrt(2.0f), 1e-6);
  EXPECT(init::CalculateGain(init::NonLinearityType::kSigmoid) == 1.0f && init::CalculateGain(init::NonLinearityType::kTanh) > 1.6f);
  // Linear's default: every value inside 1 / sqrt(fan_in), and the range is used
  Tensor big = torch::empty({64, 100});
  init::KaimingUniform(big);
  EXPECT(big.abs().max().item<float>() <= 0.1f + 1e-6f && big.abs().max().item<float>() > 0.09f);
  init::KaimingUniform(big, 0.0f, init::KaimingMode::kFanOut, init::NonLinearityType::kReLU);
  const float bound = std::sqrt(3.0f) * std::sqrt(2.0f) / 8.0f;
  EXPECT(big.abs().max().item<float>() <= bound + 1e-6f && big.abs().max().item<float>() > 0.9f * bound);
  // a generator of the caller's: the same seed gives the same draws and leaves the global stream alone
  itb::nn::ManualSeed(99);
  Tensor g1 = torch::empty({8}), g2 = torch::empty({8}), a = torch::empty({8}), b = torch::empty({8});
  init::Normal(g1, 0.0f, 1.0f);
  itb::nn::ManualSeed(99);
  std::mt19937 own(7), same(7);
  init::Uniform(a, -1.0f, 1.0f, &own);
  init::Uniform(b, -1.0f, 1.0f, &same);
  init::Normal(g2, 0.0f, 1.0f);
  EXPECT(torch::equal(a, b) && torch::equal(g1, g2));
  init::Ones(a), init::Zeros(b);
  EXPECT(a.sum().item<float>() == 8.0f && b.abs().sum().item<float>() == 0.0f);
  EXPECT(torch::equal(init::Arange(2, 6), torch::tensor({2, 3, 4, 5}, torch::kInt64)));
}

ITB_TEST(ApiNames, CreatorsModulesListAndGuards) {
  using namespace itb::nn;
  auto net = std::make_shared<Sequential>(std::vector<std::shared_ptr<itb::Module>>{std::make_shared<Linear>(3, 2), std::make_shared<Sigmoid>()});
  EXPECT(net->modules().size() == 3 && net->modules()[0] == net);
  EXPECT(net->at(0)->mutable_parameter("weight").data_ptr() == net->at(0)->parameter("weight").data_ptr());
  // optimizer creators: the parameter list arrives later
  auto sgd = itb::optim::SGD::Create(0.5)(net->Parameters());
  auto adam = itb::optim::Adam::Create(1e-2, 0.9, 0.95)(net->Parameters());
  Tensor before = net->Parameters()[0].clone();
  (*net)(torch::ones({4, 3})).sum().backward();
  sgd->Step();
  EXPECT(!torch::equal(before, net->Parameters()[0].detach()));
  adam->Step();
  EXPECT(adam->StateDict().count("adam.t") == 1 && adam->StateDict().at("adam.t").item<int64_t>() == 1);
  {
    itb::autograd::NoGradGuard guard;
    EXPECT(!(*net)(torch::ones({1, 3})).requires_grad());
  }
  EXPECT((*net)(torch::ones({1, 3})).requires_grad());
}

ITB_TEST(Checkpoint, NewestCompleteStepSkipsWhatAFailureLeftHalfWritten) {
  const std::string root = itbtest::temp_dir("ckpts");
  EXPECT(itb::io::NewestCompleteCheckpointStep(root + "/absent") == 0 && itb::io::ListCheckpoints(root).empty());
  for (int64_t step : {2, 4, 6}) {
    const std::string dir = itb::io::CheckpointDirOfStep(root, step);
    std::filesystem::create_directories(dir + "/rank_000001");
    std::ofstream(dir + "/model.ckpt") << "x";
    if (step == 6) continue;                              // the job died before this step's state file was written
    itb::io::TrainerState st;
    st.global_step = step;
    itb::io::SaveTrainerState(dir + "/trainer_state.json", st);
    if (step == 2) itb::io::SaveTrainerState(dir + "/rank_000001/trainer_state.json", st);
  }
  std::filesystem::create_directories(root + "/checkpoint_step_notanumber");
  auto all = itb::io::ListCheckpoints(root);
  EXPECT(all.size() == 3 && all.front().first == 2 && all.back().first == 6);
  EXPECT(itb::io::NewestCompleteCheckpointStep(root) == 4);
  EXPECT(itb::io::NewestCompleteCheckpointStep(root, /*global_rank=*/1) == 2);
  EXPECT(itb::io::NewestCompleteCheckpointStep(root, 3) == 0);
  std::ofstream(itb::io::CheckpointDirOfStep(root, 4) + "/trainer_state.json") << "{ \"global_step\": 3 }";   // another step's file
  EXPECT(itb::io::NewestCompleteCheckpointStep(root) == 2);
  EXPECT(!std::filesystem::exists(itb::io::CheckpointDirOfStep(root, 2) + "/trainer_state.json.tmp"));
  EXPECT(itb::io::PruneCheckpoints(root, 1) == 2 && itb::io::ListCheckpoints(root).size() == 1);
}

ITB_TEST_MAIN()
