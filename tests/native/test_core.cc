// The device runtime (itb/runtime.h: streams with priorities, events, raw memory from the tensors'
// pool, copies, the device guard) and the reference-named tensor functions (itb/tensor_api.h), on the
// CPU and, in the CUDA pass, on cuda:0.  Reference surface: infini_train/include/core/runtime/
// device_guard.h:59-143 and include/tensor.h:62-223.
#define ITB_TEST_WITH_TORCH
#include "itb_test.h"

#include <fstream>
#include <sstream>

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

ITB_TEST_MAIN()
