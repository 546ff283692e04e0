// The framework-free host runtime (csrc/runtime: flat-buffer layout planner, pipeline schedule
// generators) against the partitioning rules of the reference, as worked examples:
// infini_train/src/nn/parallel/ddp/param_and_grad_buffer.cc:425-531 (reverse packing, 64-element
// parameter starts, bucket end padded to lcm(dp, 128), buckets of >= 1 M elements) and
// pp/pipeline_schedule.cc:86-192 (GPipe and interleaved 1F1B task lists).
#include "itb_test.h"

#include <map>
#include <numeric>
#include <set>

#include "runtime.h"

ITB_TEST(Layout, ReversePackingAlignmentAndShardableBuckets) {
  const std::vector<int64_t> numels = {130, 4096, 77, 250000, 1200000, 64, 900000, 31};
  for (int64_t dp : {1, 2, 3, 8}) {
    itb::FlatLayoutResult r = itb::PlanFlatLayout(numels, dp, true, 1000000, false);
    EXPECT(r.param_start.size() == numels.size());
    for (size_t i = 0; i < numels.size(); ++i) {
      EXPECT(r.param_end[i] - r.param_start[i] == numels[i]);
      EXPECT(r.param_start[i] % 64 == 0);
      if (i > 0) EXPECT(r.param_end[i] <= r.param_start[i - 1]);     // later parameters come first
      const int64_t b = r.param_bucket[i];
      EXPECT(r.bucket_start[b] <= r.param_start[i] && r.param_end[i] <= r.bucket_end[b]);
    }
    const int64_t l = std::lcm<int64_t>(dp, 128);
    for (size_t b = 0; b < r.bucket_start.size(); ++b) {
      EXPECT((r.bucket_end[b] - r.bucket_start[b]) % dp == 0);
      EXPECT(r.bucket_end[b] % l == 0);
      if (b > 0) EXPECT(r.bucket_start[b] == r.bucket_end[b - 1]);
      if (b + 1 < r.bucket_start.size()) EXPECT(r.bucket_unpadded[b] >= 1000000);   // only the last may be short
    }
    EXPECT(r.bucket_end.back() == r.numel);
  }
}

ITB_TEST(Layout, UnshardedBuffersArePackedTightly) {
  itb::FlatLayoutResult r = itb::PlanFlatLayout({10, 20, 30}, 1, false, 1000000, false);
  EXPECT(r.numel == 60 && r.numel_unpadded == 60 && r.bucket_start.size() == 1);
  EXPECT(r.param_start[2] == 0 && r.param_start[1] == 30 && r.param_start[0] == 50);
}

ITB_TEST(Layout, BusBandwidthPaddingRoundsBucketsTo64Ki) {
  itb::FlatLayoutResult r = itb::PlanFlatLayout({1200000, 1200000}, 8, true, 1000000, true);
  for (size_t b = 0; b < r.bucket_end.size(); ++b) EXPECT(r.bucket_end[b] % (1 << 16) == 0);
}

static void check_schedule(const std::vector<itb::PipeTask>& tasks, int n, int stages, int vpp) {
  EXPECT(static_cast<int>(tasks.size()) == 2 * n * stages * vpp);
  std::map<std::pair<int, int>, int> fwd_pos, bwd_pos;
  for (size_t i = 0; i < tasks.size(); ++i) {
    const itb::PipeTask& t = tasks[i];
    EXPECT(t.stage == t.global_chunk % stages && t.local_chunk == t.global_chunk / stages);
    EXPECT(t.is_first_chunk == (t.global_chunk == 0) && t.is_last_chunk == (t.global_chunk == stages * vpp - 1));
    const auto key = std::make_pair(t.microbatch, t.global_chunk);
    if (t.is_forward) {
      EXPECT(!fwd_pos.count(key));
      if (t.global_chunk > 0) EXPECT(fwd_pos.count(std::make_pair(t.microbatch, t.global_chunk - 1)));
      fwd_pos[key] = static_cast<int>(i);
    } else {
      EXPECT(fwd_pos.count(key) && !bwd_pos.count(key));               // a backward never precedes its forward
      if (t.global_chunk < stages * vpp - 1) EXPECT(bwd_pos.count(std::make_pair(t.microbatch, t.global_chunk + 1)));
      bwd_pos[key] = static_cast<int>(i);
    }
  }
  EXPECT(static_cast<int>(fwd_pos.size()) == n * stages * vpp && bwd_pos.size() == fwd_pos.size());
}

ITB_TEST(Schedule, GPipeAndInterleaved1F1BAreCompleteAndCausal) {
  for (int vpp : {1, 2, 3})
    for (int stages : {2, 4})
      for (int n : {4, 8}) {
        check_schedule(itb::GpipeSchedule(n, stages, vpp), n, stages, vpp);
        check_schedule(itb::Interleaved1F1BSchedule(n, stages, vpp), n, stages, vpp);
      }
}

ITB_TEST(Schedule, GPipeRunsEveryForwardBeforeAnyBackward) {
  bool seen_backward = false;
  for (const itb::PipeTask& t : itb::GpipeSchedule(4, 2, 1)) {
    if (!t.is_forward) seen_backward = true;
    else EXPECT(!seen_backward);
  }
}

ITB_TEST(Schedule, OneFOneBBoundsTheForwardsInFlightPerStage) {
  // Under 1F1B the number of forwards a stage holds without their backward depends on the pipeline's
  // depth, not on the number of micro-batches (GPipe holds all n): with the reference's generator it is
  // 2 (S - 1 - stage) on stage `stage`, at least 1.
  const int stages = 4, vpp = 1;
  for (int stage = 0; stage < stages; ++stage) {
    int peaks[2] = {0, 0};
    for (int k = 0; k < 2; ++k) {
      const int n = k ? 16 : 8;
      int live = 0;
      for (const itb::PipeTask& t : itb::Interleaved1F1BSchedule(n, stages, vpp)) {
        if (t.stage != stage) continue;
        live += t.is_forward ? 1 : -1;
        peaks[k] = std::max(peaks[k], live);
      }
      EXPECT(live == 0);
    }
    EXPECT(peaks[0] == peaks[1]);
    EXPECT(peaks[0] == std::max(1, 2 * (stages - 1 - stage)));
  }
  int live = 0, peak = 0;
  for (const itb::PipeTask& t : itb::GpipeSchedule(16, stages, vpp)) {
    if (t.stage != 0) continue;
    live += t.is_forward ? 1 : -1;
    peak = std::max(peak, live);
  }
  EXPECT(peak == 16);
}

ITB_TEST_MAIN()
