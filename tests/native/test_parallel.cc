// The parallel stack of the C++ frontend with the ranks of a job played by threads of one process:
// every thread owns its process-group objects (CPU transport through one in-process TCP store), its
// replica of the model and its optimizer, exactly as a rank process would.  Covers the rank layout and
// group names (reference: infini_train/src/nn/parallel/global.cc:22-112), the stage partition
// (pp/pipeline_parallel.cc:42-77), every collective and the batched point-to-point exchange
// (process_group.cc:118-249), the Reducer's bucket assignment and overlap (ddp/reducer.cc:56-438),
// ZeRO-1 state partitioning (ddp/distributed_optimizer.cc:34-137) and the pipeline schedules
// (pp/pipeline_schedule.cc:27-329) against the same computation done by one rank.

#define ITB_TEST_WITH_TORCH
#include "itb_test.h"

#include <atomic>
#include <thread>

#include "itb/itb.h"

using itb::Tensor;
using itb::TensorList;
namespace par = itb::parallel;

namespace {

// The server store asks the system for a free port (port 0) and the clients read it back: a number computed here
// can fall into the range the system hands to outgoing connections and meet a socket that still lingers there.
//
// Runs fn(rank, group) on `world` threads; the group spans all of them.  Exceptions of any rank fail
// the calling test.
void run_ranks(int world, const std::function<void(int, std::shared_ptr<par::ProcessGroup>)>& fn) {
  c10d::TCPStoreOptions server;
  server.port = 0;
  server.isServer = true;
  server.numWorkers = c10::nullopt;
  server.waitWorkers = false;
  server.timeout = std::chrono::milliseconds(60000);
  auto master = c10::make_intrusive<c10d::TCPStore>("127.0.0.1", server);
  server.port = master->getPort();
  std::vector<std::string> errors(world);
  std::vector<std::thread> threads;
  std::vector<int> ranks(world);
  for (int i = 0; i < world; ++i) ranks[i] = i;
  for (int r = 0; r < world; ++r)
    threads.emplace_back([&, r] {
      try {
        c10d::TCPStoreOptions client = server;
        client.isServer = false;
        auto store = c10::make_intrusive<c10d::TCPStore>("127.0.0.1", client);
        auto pg = std::make_shared<par::StoreProcessGroup>("world", ranks, r, store);
        fn(r, pg);
        pg->Barrier();
      } catch (const std::exception& e) {
        errors[r] = e.what();
      }
    });
  for (auto& t : threads) t.join();
  for (int r = 0; r < world; ++r)
    if (!errors[r].empty()) throw itbtest::Failure("rank " + std::to_string(r) + ": " + errors[r]);
}

double max_abs_diff(const Tensor& a, const Tensor& b) { return (a.detach() - b.detach()).abs().max().item<double>(); }

// A small residual MLP block standing in for a transformer layer.
struct Block : itb::Module {
  Block(int64_t width, int64_t seed) : itb::Module("Block") {
    auto gen = at::detail::createCPUGenerator(static_cast<uint64_t>(seed));   // the global generator is shared by the rank threads
    w1 = register_parameter("w1", torch::randn({4 * width, width}, gen) * 0.2);
    b1 = register_parameter("b1", torch::randn({4 * width}, gen) * 0.1);
    w2 = register_parameter("w2", torch::randn({width, 4 * width}, gen) * 0.2);
  }
  Tensor forward(const Tensor& x) { return x + torch::matmul(torch::tanh(torch::matmul(x, w1.t()) + b1), w2.t()); }
  TensorList Forward(const TensorList& in) override { return {forward(in[0])}; }
  Tensor w1, b1, w2;
};
struct Stack : itb::Module {
  Stack(int64_t layers, int64_t width, int64_t first_seed = 100) : itb::Module("Stack") {
    for (int64_t i = 0; i < layers; ++i) blocks.push_back(register_module("b" + std::to_string(i), std::make_shared<Block>(width, first_seed + i)));
  }
  Tensor forward(Tensor x) {
    for (auto& b : blocks) x = b->forward(x);
    return x;
  }
  TensorList Forward(const TensorList& in) override { return {forward(in[0])}; }
  std::vector<std::shared_ptr<Block>> blocks;
};

}  // namespace

// ------------------------------------------------------------------ layout, names, stage partition
// A rank that waits inside a collective for a peer that never arrives comes back with an error once
// another thread (the watchdog of fault_tolerance.h) aborts its group; later calls fail at once.
ITB_TEST(ProcessGroup, AbortEndsAWaitForAPeerThatIsGone) {
  c10d::TCPStoreOptions server;
  server.port = 0;   // any free port
  server.isServer = true;
  server.numWorkers = c10::nullopt;
  server.waitWorkers = false;
  server.timeout = std::chrono::milliseconds(60000);
  auto store = c10::make_intrusive<c10d::TCPStore>("127.0.0.1", server);
  auto pg = std::make_shared<par::StoreProcessGroup>("lonely", std::vector<int>{0, 1}, 0, store);
  pg->set_abortable(true);
  std::string error;
  std::atomic<bool> returned{false};
  std::thread rank0([&] {
    try {
      Tensor t = torch::ones({4});
      pg->AllReduce(t, par::ReduceOp::kSum, false);   // rank 1 never publishes its part
    } catch (const std::exception& e) {
      error = e.what();
    }
    returned = true;
  });
  std::this_thread::sleep_for(std::chrono::milliseconds(150));
  EXPECT(!returned);                          // still waiting
  const auto t0 = std::chrono::steady_clock::now();
  pg->Abort();
  rank0.join();
  EXPECT(std::chrono::steady_clock::now() - t0 < std::chrono::seconds(2));
  EXPECT(error.find("was aborted") != std::string::npos && pg->aborted());
  Tensor again = torch::ones({4});
  EXPECT_THROWS(pg->AllReduce(again, par::ReduceOp::kSum, false));
  EXPECT_THROWS(pg->Barrier());
}

// The slices that `dp` ranks hold of a per-parameter state, cut directly from the flat layout of that size.
static std::vector<std::map<std::string, Tensor>> ShardedState(const std::vector<std::vector<Tensor>>& chunks, int dp, int64_t bucket_elems) {
  std::vector<std::map<std::string, Tensor>> out(dp);
  size_t k = 0;
  for (const auto& values : chunks) {
    std::vector<int64_t> numels;
    for (const auto& v : values) numels.push_back(v.numel());
    auto lay = itb::PlanFlatLayout(numels, dp, true, bucket_elems, false);
    Tensor flat = torch::zeros({lay.numel});
    for (size_t i = 0; i < values.size(); ++i) flat.narrow(0, lay.param_start[i], numels[i]).copy_(values[i].view({-1}));
    for (size_t b = 0; b < lay.bucket_start.size(); ++b, ++k) {
      const int64_t n = (lay.bucket_end[b] - lay.bucket_start[b]) / dp;
      for (int r = 0; r < dp; ++r) {
        out[r]["adam.m." + std::to_string(k)] = flat.narrow(0, lay.bucket_start[b] + r * n, n).clone();
        out[r]["adam.v." + std::to_string(k)] = flat.narrow(0, lay.bucket_start[b] + r * n, n).clone() * 2;
        out[r]["adam.t"] = torch::tensor(static_cast<int64_t>(17), torch::kInt64);
      }
    }
  }
  return out;
}

ITB_TEST(ZeroReshard, StateOfOneDataParallelSizeRecutForAnotherEqualsCuttingItDirectly) {
  // two module chunks, several buckets each (buckets close at 300 elements), sizes that need padding
  std::vector<std::vector<Tensor>> chunks(2);
  int64_t seed = 0;
  for (int64_t n : {130, 257, 64, 301, 7, 190}) chunks[0].push_back(torch::arange(n, torch::kFloat32) + 1000.0f * static_cast<float>(++seed));
  for (int64_t n : {512, 33, 95}) chunks[1].push_back(torch::arange(n, torch::kFloat32) + 1000.0f * static_cast<float>(++seed));
  std::vector<std::vector<int64_t>> numels(2);
  for (int c = 0; c < 2; ++c)
    for (const auto& v : chunks[c]) numels[c].push_back(v.numel());
  for (auto [old_dp, new_dp] : std::vector<std::pair<int, int>>{{4, 2}, {2, 4}, {3, 8}, {8, 1}, {1, 3}}) {
    auto old_states = ShardedState(chunks, old_dp, 300);
    auto want = ShardedState(chunks, new_dp, 300);
    for (int r = 0; r < new_dp; ++r) {
      auto got = par::ReshardZeroState(old_states, numels, new_dp, r, 300);
      EXPECT(got.size() == want[r].size());
      for (const auto& [key, t] : want[r]) {
        EXPECT(got.count(key) == 1);
        EXPECT(got.at(key).sizes() == t.sizes() && torch::equal(got.at(key), t));
      }
    }
  }
  // a state written for another model is refused with the size that was expected
  auto other = ShardedState(chunks, 2, 300);
  numels[0][0] += 1000;
  EXPECT_THROWS(par::ReshardZeroState(other, numels, 4, 0, 300));
}

ITB_TEST(Layout3D, TensorParallelRanksAreAdjacentThenDataThenPipeline) {
  par::Layout l;
  l.tp = 2, l.dp = 2, l.pp = 2;
  EXPECT(l.world() == 8);
  EXPECT(l.RankOf(1, 0, 0) == 1 && l.RankOf(0, 1, 0) == 2 && l.RankOf(0, 0, 1) == 4);
  EXPECT((l.GroupRanks(par::Axis::kTP, 5) == std::vector<int>{4, 5}));
  EXPECT((l.GroupRanks(par::Axis::kDP, 5) == std::vector<int>{5, 7}));
  EXPECT((l.GroupRanks(par::Axis::kPP, 5) == std::vector<int>{1, 5}));
  EXPECT(l.GroupName(par::Axis::kTP, 5) == "TP2" && l.GroupName(par::Axis::kDP, 5) == "DP3" && l.GroupName(par::Axis::kPP, 5) == "PP1");
  for (int r = 0; r < 8; ++r) {
    int t, d, p;
    l.CoordOf(r, &t, &d, &p);
    EXPECT(l.RankOf(t, d, p) == r);
  }
  par::GlobalEnv e;
  EXPECT_THROWS(e.Init(8, 0, 3, false, 1));
  e.Init(8, 6, 2, true, 2, 2);
  EXPECT(e.dp() == 2 && e.tp_rank == 0 && e.dp_rank == 1 && e.pp_rank == 1 && e.sp() == 2 && e.vpp == 2);
  EXPECT(e.ProcessGroupOverview().find("TP3 (dp=1, tp=-, pp=1): [6, 7]") != std::string::npos);
}

ITB_TEST(Layout3D, ReferenceNamedAccessorsReadTheSameState) {
  namespace g = par::global;
  par::GlobalEnv saved = par::env();
  par::env().Init(/*world=*/16, /*rank=*/13, /*tp=*/2, /*sp=*/true, /*pp=*/2, /*vpp=*/3);
  EXPECT(g::GetWorldSize() == 16 && g::GetGlobalProcRank() == 13 && g::GetNthreadPerProc() == 1);
  EXPECT(g::GetTensorParallelSize() == 2 && g::GetDataParallelSize() == 4 && g::GetPipelineParallelSize() == 2);
  EXPECT(g::GetSequenceParallelEnabled() && g::GetSequenceParallelSize() == 2 && g::GetVirtualPipelineParallelSize() == 3);
  int dp = -1, tp = -1, pp = -1;
  g::GetCoordOf(13, dp, tp, pp);                       // TP fastest, then DP, then PP: 13 = 1 + 2 * (2 + 4 * 1)
  EXPECT(tp == 1 && dp == 2 && pp == 1 && g::GetRankOf(dp, tp, pp) == 13);
  EXPECT(g::GetGroupRanks(par::Axis::kDP, 13) == (std::vector<int>{9, 11, 13, 15}));
  EXPECT(g::GetGroupRanks(par::Axis::kTP, 2, 0, 1) == (std::vector<int>{12, 13}));
  EXPECT(g::GetGroupId(par::Axis::kTP, 13) == 6 && g::GetGroupId(par::Axis::kPP, 2, 1, 0) == g::GetGroupId(par::Axis::kPP, 13));
  EXPECT(g::ProcessGroupOverview().find("world_size = 16") != std::string::npos);
  par::env() = saved;
}

ITB_TEST(Layout3D, RankCountsProcessesAndThreads) {
  par::Rank r(2, 1, 4, 2);                       // process 2 of 4, thread 1 of 2
  EXPECT(r.GlobalRank() == 5 && r.IsParallel() && !r.IsMainRank() && !r.IsLastRank());
  EXPECT(par::Rank(3, 1, 4, 2).IsLastRank() && par::Rank(0, 0, 1, 1).IsMainRank() && !par::Rank(0, 0, 1, 1).IsParallel());
}

ITB_TEST(StagePartition, RoundRobinChunksAndRemainderToTheFirstChunks) {
  auto s0 = par::GetStageInfo(10, 2, 0, 2), s1 = par::GetStageInfo(10, 2, 1, 2);   // 4 chunks: 3 3 2 2
  EXPECT((s0.layer_ranges_per_chunk == std::vector<std::pair<int, int>>{{0, 3}, {6, 8}}));
  EXPECT((s1.layer_ranges_per_chunk == std::vector<std::pair<int, int>>{{3, 6}, {8, 10}}));
  EXPECT(s0.is_first_stage && !s0.is_last_stage && s1.is_last_stage);
  EXPECT_THROWS(par::GetStageInfo(3, 2, 0, 2));
}

// ------------------------------------------------------------------ collectives
ITB_TEST(StoreGroup, CollectivesAndPointToPoint) {
  const int W = 4;
  run_ranks(W, [&](int r, std::shared_ptr<par::ProcessGroup> pg) {
    EXPECT(pg->size() == W && pg->rank() == r);
    Tensor t = torch::full({5}, static_cast<float>(r + 1));
    pg->AllReduce(t, par::ReduceOp::kSum);
    EXPECT_NEAR(t[0].item<float>(), 10.0, 0);
    t = torch::full({5}, static_cast<float>(r + 1));
    pg->AllReduce(t, par::ReduceOp::kAvg);
    EXPECT_NEAR(t[3].item<float>(), 2.5, 0);
    t = torch::full({2}, static_cast<float>(r));
    pg->AllReduce(t, par::ReduceOp::kMax);
    EXPECT_NEAR(t[0].item<float>(), 3.0, 0);
    Tensor mine = torch::arange(3, torch::kFloat32) + 10 * r, all = torch::empty({W * 3});
    pg->AllGather(all, mine);
    for (int q = 0; q < W; ++q) EXPECT_NEAR(all[3 * q + 2].item<float>(), 10 * q + 2, 0);
    Tensor in = torch::arange(W * 2, torch::kFloat32) * (r + 1), out = torch::empty({2});
    pg->ReduceScatter(out, in, par::ReduceOp::kSum);
    EXPECT_NEAR(out[1].item<float>(), (2 * r + 1) * 10.0, 0);
    for (int src = 0; src < W; ++src) {   // back-to-back broadcasts from every rank
      Tensor b = torch::full({4}, r == src ? 7.0f + src : -1.0f);
      pg->BroadCast(b, src);
      EXPECT_NEAR(b[2].item<float>(), 7.0 + src, 0);
    }
    // a ring exchange in ONE batched call: everybody sends right and receives from the left
    Tensor send = torch::full({3}, static_cast<float>(r)), recv = torch::empty({3});
    std::vector<par::P2POp> ops = {{true, send, (r + 1) % W}, {false, recv, (r + W - 1) % W}};
    auto work = pg->BatchSendRecv(ops, true);
    EXPECT(work->WaitBlocking(1000) && work->IsCompleted() && work->IsSuccess());
    EXPECT_NEAR(recv[0].item<float>(), (r + W - 1) % W, 0);
    // two messages between one pair arrive in the order they were sent
    if (r == 0) {
      pg->Send({torch::full({1}, 1.0f)}, 1);
      pg->Send({torch::full({1}, 2.0f)}, 1);
    } else if (r == 1) {
      TensorList a = {torch::empty({1})}, b = {torch::empty({1})};
      pg->Recv(a, 0);
      pg->Recv(b, 0);
      EXPECT(a[0].item<float>() == 1.0f && b[0].item<float>() == 2.0f);
    }
  });
}

ITB_TEST(StoreGroup, RootedCollectivesReduceScatterGather) {
  run_ranks(4, [](int rank, std::shared_ptr<par::ProcessGroup> pg) {
    // Reduce: the sum lands on rank 2 only
    Tensor t = torch::full({3}, static_cast<float>(rank + 1));
    pg->Reduce(t, 2, par::ReduceOp::kSum, false);
    EXPECT(t[0].item<float>() == (rank == 2 ? 10.0f : static_cast<float>(rank + 1)));
    TensorList pair = {torch::full({2}, 1.0f), torch::full({1}, static_cast<float>(rank))};
    pg->ReduceAddCoalesced(pair, 0);
    if (rank == 0) EXPECT(pair[0][0].item<float>() == 4.0f && pair[1][0].item<float>() == 6.0f);
    // Scatter from rank 1 along dimension 1, then Gather the pieces back on rank 3 along the same dimension
    Tensor full = rank == 1 ? torch::arange(24, torch::kFloat32).view({3, 8}) : Tensor();
    Tensor piece = torch::empty({3, 2});
    pg->Scatter(piece, rank == 1 ? full : torch::empty({0}), 1, 1);
    EXPECT(torch::equal(piece, torch::arange(24, torch::kFloat32).view({3, 8}).slice(1, 2 * rank, 2 * rank + 2)));
    Tensor back = pg->Gather(piece, 3, 1);
    if (rank == 3) EXPECT(torch::equal(back, torch::arange(24, torch::kFloat32).view({3, 8})));
    else EXPECT(!back.defined());
  });
}

ITB_TEST(StoreGroup, RanksThatDisagreeOnASizeGetAnErrorNotAHang) {
  bool threw = false;
  try {
    run_ranks(2, [&](int r, std::shared_ptr<par::ProcessGroup> pg) {
      Tensor t = torch::zeros({r == 0 ? 4 : 5});
      pg->AllReduce(t);
    });
  } catch (const itbtest::Failure& f) {
    threw = std::string(f.what()).find("disagree on the size") != std::string::npos;
  }
  EXPECT(threw);
}

// ------------------------------------------------------------------ data parallel
ITB_TEST(Reducer, BucketsAreCutInReverseOrderWithASmallFirstBucket) {
  TensorList params;
  for (int64_t n : {300000, 200000, 100, 400000, 50000}) params.push_back(torch::zeros({n}));   // fp32: 4 bytes each
  auto b = par::ComputeBucketAssignmentBySize(params, 1 << 20, 2 << 20);
  // reverse order: 50000 (0.2 MB), 400000 (1.6 MB) -> first bucket closes past 1 MB; then 100, 200000, 300000 (2 MB)
  EXPECT(b.size() == 2);
  EXPECT((b[0] == std::vector<size_t>{4, 3}));
  EXPECT((b[1] == std::vector<size_t>{2, 1, 0}));
}

ITB_TEST(FlatBuffers, ParametersAndGradientsBecomeViewsOfOneBuffer) {
  auto model = std::make_shared<Stack>(2, 8);
  Tensor before = model->blocks[1]->w2.detach().clone();
  par::ParamAndGradBuffer buf(model->Parameters(), 2, 0, /*shard=*/true, /*bucket_elems=*/300);
  EXPECT(max_abs_diff(model->blocks[1]->w2, before) == 0.0);
  EXPECT(buf.buckets().size() >= 2);
  const float* base = buf.param_buffer.data_ptr<float>();
  for (auto& p : model->Parameters()) {
    EXPECT(p.data_ptr<float>() >= base && p.data_ptr<float>() + p.numel() <= base + buf.param_buffer.numel());
    EXPECT((p.data_ptr<float>() - base) % 64 == 0);
    EXPECT(p.grad().defined());
  }
  Tensor x = torch::randn({3, 8});
  model->forward(x).sum().backward();
  EXPECT(buf.grad_buffer.abs().sum().item<float>() > 0);   // autograd accumulated into the views
  auto r = buf.shard_range(0, 1);
  EXPECT(r.second - r.first == (buf.buckets()[0].end - buf.buckets()[0].start) / 2);
}

// Two data-parallel replicas on different batches against one rank on both batches: same update,
// and most buckets leave while backward is still running.
static void data_parallel_case(int zero_stage, bool overlap) {
  const int W = 2;
  const int64_t width = 16, layers = 6;
  torch::manual_seed(7);
  Tensor xs = torch::randn({W, 4, width}), ys = torch::randn({W, 4, width});
  auto ref = std::make_shared<Stack>(layers, width);
  itb::optim::Adam ref_opt(ref->Parameters(), 1e-2);
  for (int step = 0; step < 3; ++step) {
    ref_opt.ZeroGrad();
    for (int r = 0; r < W; ++r) ((ref->forward(xs[r]) - ys[r]).pow(2).mean() / W).backward();
    ref_opt.Step();
  }
  std::vector<Tensor> finals(W);
  std::vector<int64_t> during(W), buckets(W);
  run_ranks(W, [&](int r, std::shared_ptr<par::ProcessGroup> pg) {
    auto model = std::make_shared<Stack>(layers, width, r == 0 ? 100 : 500);   // rank 1 starts elsewhere: the wrapper must broadcast
    par::DistributedDataParallelConfig cfg;
    cfg.zero_stage = zero_stage, cfg.overlap_grad_reduce = overlap;
    cfg.first_bucket_cap_mb = 0, cfg.normal_bucket_cap_mb = 0;   // a bucket per parameter: many launches to order
    cfg.bucket_size_in_elements = 2000;
    par::DistributedDataParallel ddp(model, pg, cfg);
    std::unique_ptr<itb::optim::Optimizer> opt;
    auto make = [](TensorList p) -> std::unique_ptr<itb::optim::Optimizer> { return std::make_unique<itb::optim::Adam>(std::move(p), 1e-2); };
    if (zero_stage >= 1) opt = std::make_unique<par::DistributedOptimizer>(make, std::vector<par::DistributedDataParallel*>{&ddp});
    else opt = make(model->Parameters());
    for (int step = 0; step < 3; ++step) {
      opt->ZeroGrad();
      ddp.ZeroGrad();
      (ddp(xs[r]) - ys[r]).pow(2).mean().backward();
      ddp.FinishGradSync();
      opt->Step();
    }
    if (zero_stage >= 1) {   // the optimizer state covers this rank's half of every bucket only
      int64_t state = 0, all = 0;
      for (auto& [k, v] : opt->StateDict())
        if (k.rfind("adam.m.", 0) == 0) state += v.numel();
      for (auto& p : model->Parameters()) all += p.numel();
      EXPECT(state * W >= all && state * W <= all + 4096);
    }
    TensorList flat;
    for (auto& p : model->Parameters()) flat.push_back(p.detach().reshape({-1}));
    finals[r] = torch::cat(flat);
    during[r] = ddp.launches_during_backward();
    buckets[r] = static_cast<int64_t>(ddp.num_buckets());
  });
  TensorList flat;
  for (auto& p : ref->Parameters()) flat.push_back(p.detach().reshape({-1}));
  Tensor want = torch::cat(flat);
  for (int r = 0; r < W; ++r) EXPECT(max_abs_diff(finals[r], want) < 2e-6);
  EXPECT(buckets[0] > 1);
  if (overlap) EXPECT(during[0] == 3 * buckets[0]);   // every bucket of every step left from a ready hook
  else EXPECT(during[0] == 0);
}
ITB_TEST(DataParallel, ReducerOverlapsAndMatchesOneRank) { data_parallel_case(0, true); }
ITB_TEST(DataParallel, WithoutOverlapEverythingLeavesAtTheEnd) { data_parallel_case(0, false); }
ITB_TEST(DataParallel, ZeroOnePartitionsTheOptimizerState) { data_parallel_case(1, true); }
ITB_TEST(DataParallel, ZeroTwo) { data_parallel_case(2, true); }

ITB_TEST(DataParallel, AccumulationSyncsOnlyOnTheLastMicroBatch) {
  const int W = 2;
  torch::manual_seed(3);
  Tensor xs = torch::randn({W, 2, 3, 8});
  auto ref = std::make_shared<Stack>(2, 8);
  for (int r = 0; r < W; ++r)
    for (int m = 0; m < 2; ++m) (ref->forward(xs[r][m]).pow(2).mean() / (2 * W)).backward();
  std::vector<double> err(W);
  run_ranks(W, [&](int r, std::shared_ptr<par::ProcessGroup> pg) {
    auto model = std::make_shared<Stack>(2, 8);
    par::DistributedDataParallel ddp(model, pg);
    ddp.ZeroGrad();
    for (int m = 0; m < 2; ++m) {
      ddp.set_sync(m == 1);
      (ddp(xs[r][m]).pow(2).mean() / 2).backward();
      if (m == 0) EXPECT(ddp.launches_during_backward() == 0);
    }
    ddp.FinishGradSync();
    err[r] = max_abs_diff(model->blocks[0]->w1.grad(), ref->blocks[0]->w1.grad());
  });
  EXPECT(err[0] < 1e-6 && err[1] < 1e-6);
}

// ------------------------------------------------------------------ pipeline
// Stages are threads; every stage holds the chunks GetStageInfo gives it.  The parameter gradients
// must equal those of the whole stack run on one rank over the same micro-batches.
static void pipeline_case(const std::string& schedule, int S, int vpp, int n) {
  const int64_t width = 8, layers = 2 * S * vpp + 1, B = 2;
  torch::manual_seed(11);
  Tensor xs = torch::randn({n, B, width}), ys = torch::randn({n, B, width});
  auto ref = std::make_shared<Stack>(layers, width);
  double ref_loss = 0;
  for (int m = 0; m < n; ++m) {
    Tensor l = (ref->forward(xs[m]) - ys[m]).pow(2).mean() / n;
    ref_loss += l.item<double>();
    l.backward();
  }
  std::vector<double> err(S, 1.0), loss(S, 0.0);
  run_ranks(S, [&](int s, std::shared_ptr<par::ProcessGroup> pg) {
    auto info = par::GetStageInfo(static_cast<int>(layers), S, s, vpp);
    auto full = std::make_shared<Stack>(layers, width);   // same seeds: block i is layer i
    par::PipelineConfig pc;
    pc.num_stages = S, pc.stage = s, pc.vpp = vpp, pc.num_micro_batches = n, pc.schedule = schedule;
    pc.boundary_shape = {B, width};
    par::PipelineParallel pipe(pc, [&](int64_t ci, const Tensor& in) {
      Tensor x = in;
      for (int i = info.layer_ranges_per_chunk[ci].first; i < info.layer_ranges_per_chunk[ci].second; ++i) x = full->blocks[i]->forward(x);
      return x;
    }, pg);
    std::vector<Tensor> in, tg;
    for (int m = 0; m < n; ++m) in.push_back(xs[m]), tg.push_back(ys[m]);
    std::vector<std::pair<int64_t, bool>> notices;
    loss[s] = pipe.StepMicroBatches(in, tg, [](const Tensor& out, const Tensor& y) { return (out - y).pow(2).mean(); },
                                    [&](int64_t lc, bool last) { notices.emplace_back(lc, last); });
    double e = 0;
    for (const auto& r : info.layer_ranges_per_chunk)
      for (int i = r.first; i < r.second; ++i) {
        e = std::max(e, max_abs_diff(full->blocks[i]->w1.grad(), ref->blocks[i]->w1.grad()));
        e = std::max(e, max_abs_diff(full->blocks[i]->w2.grad(), ref->blocks[i]->w2.grad()));
      }
    err[s] = e;
    int lasts = 0;
    for (auto& nt : notices) lasts += nt.second;
    EXPECT(static_cast<int>(notices.size()) == n * vpp && lasts == vpp);   // one "last backward" per local chunk
    if (S > 1) EXPECT(pipe.exchanges() > 0);
  });
  for (int s = 0; s < S; ++s) EXPECT(err[s] < 1e-6);
  EXPECT_NEAR(loss[S - 1], ref_loss, 1e-6);
  if (S > 1) EXPECT(loss[0] == 0.0);
}
ITB_TEST(Pipeline, GpipeTwoStages) { pipeline_case("gpipe", 2, 1, 4); }
ITB_TEST(Pipeline, OneFOneBThreeStages) { pipeline_case("1f1b", 3, 1, 5); }
ITB_TEST(Pipeline, InterleavedTwoStagesTwoChunks) { pipeline_case("1f1b", 2, 2, 4); }
ITB_TEST(Pipeline, InterleavedFourStagesTwoChunksGpipe) { pipeline_case("gpipe", 4, 2, 3); }
ITB_TEST(Pipeline, OneStageWithChunksNeedsNoGroup) { pipeline_case("1f1b", 1, 3, 2); }

// TrainStep = split the batch, clear gradients, run the schedule, step the optimizer: two stages trained for
// three steps end with the weights of the whole stack trained on one rank with the same batches.
ITB_TEST(Pipeline, TrainStepSplitsTheBatchAndStepsTheOptimizer) {
  const int S = 2, n = 4;
  const int64_t width = 8, layers = 4, B = 2;
  torch::manual_seed(5);
  Tensor xs = torch::randn({3, n * B, width}), ys = torch::randn({3, n * B, width});
  auto ref = std::make_shared<Stack>(layers, width);
  itb::optim::SGD ref_opt(ref->Parameters(), 0.1);
  std::vector<double> ref_losses;
  for (int step = 0; step < 3; ++step) {
    ref_opt.ZeroGrad();
    double total = 0;
    for (int m = 0; m < n; ++m) {
      Tensor l = (ref->forward(xs[step].slice(0, m * B, (m + 1) * B)) - ys[step].slice(0, m * B, (m + 1) * B)).pow(2).mean() / n;
      total += l.item<double>();
      l.backward();
    }
    ref_losses.push_back(total);
    ref_opt.Step();
  }
  std::vector<double> err(S, 1.0);
  std::vector<std::vector<double>> losses(S);
  run_ranks(S, [&](int s, std::shared_ptr<par::ProcessGroup> pg) {
    auto info = par::GetStageInfo(static_cast<int>(layers), S, s, 1);
    auto full = std::make_shared<Stack>(layers, width);
    itb::TensorList mine;
    for (int i = info.layer_ranges_per_chunk[0].first; i < info.layer_ranges_per_chunk[0].second; ++i)
      for (auto& p : full->blocks[i]->Parameters()) mine.push_back(p);
    itb::optim::SGD opt(mine, 0.1);
    par::PipelineConfig pc;
    pc.num_stages = S, pc.stage = s, pc.vpp = 1, pc.num_micro_batches = n, pc.schedule = "1f1b";
    pc.boundary_shape = {B, width};
    par::PipelineParallel pipe(pc, [&](int64_t ci, const Tensor& in) {
      Tensor x = in;
      for (int i = info.layer_ranges_per_chunk[ci].first; i < info.layer_ranges_per_chunk[ci].second; ++i) x = full->blocks[i]->forward(x);
      return x;
    }, pg);
    for (int step = 0; step < 3; ++step)
      losses[s].push_back(pipe.TrainStep(s == 0 ? xs[step] : Tensor(), s == S - 1 ? ys[step] : Tensor(), opt,
                                         [](const Tensor& out, const Tensor& y) { return (out - y).pow(2).mean(); }));
    double e = 0;
    for (int i = info.layer_ranges_per_chunk[0].first; i < info.layer_ranges_per_chunk[0].second; ++i)
      e = std::max(e, max_abs_diff(full->blocks[i]->w1, ref->blocks[i]->w1));
    err[s] = e;
    if (s == 0) EXPECT_THROWS(pipe.TrainStep(torch::randn({7, width}), Tensor(), opt, [](const Tensor& o, const Tensor&) { return o.sum(); }));
  });
  for (int s = 0; s < S; ++s) EXPECT(err[s] < 1e-6);
  for (int step = 0; step < 3; ++step) EXPECT_NEAR(losses[S - 1][step], ref_losses[step], 1e-6);
}

ITB_TEST(Pipeline, EveryTensorIsConsumedAfterTheStepThatProducesIt) {
  // the constructor checks the property the step-wise exchange relies on; sweep the planner
  for (const char* kind : {"gpipe", "1f1b"})
    for (int S : {1, 2, 3, 4, 8})
      for (int vpp : {1, 2, 3})
        for (int n : {1, 2, 4, 8, 9}) {
          if (S == 1) continue;
          par::PipelineConfig pc;
          pc.num_stages = S, pc.stage = 0, pc.vpp = vpp, pc.num_micro_batches = n, pc.schedule = kind;
          par::PipelineParallel pipe(pc, [](int64_t, const Tensor& x) { return x; }, std::make_shared<par::StoreProcessGroup>("x", std::vector<int>{0}, 0, nullptr));
          EXPECT(static_cast<int>(pipe.tasks().size()) == 2 * n * S * vpp);
        }
  par::PipelineConfig pc;
  pc.num_stages = 2, pc.vpp = 1, pc.num_micro_batches = 2;
  par::PipelineParallel pipe(pc, [](int64_t, const Tensor& x) { return x; }, std::make_shared<par::StoreProcessGroup>("x", std::vector<int>{0}, 0, nullptr));
  EXPECT(pipe.ScheduleTable().find("F0.0") != std::string::npos);
}

ITB_TEST_MAIN()
