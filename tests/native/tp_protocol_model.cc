// Host-threads model of the synchronisation protocol of the fused tensor-parallel GEMM launches
// (one thread per rank, std::atomic in place of the system-scope flag words):
//
//   * at its start, launch e of rank r publishes started[d][r] = e + 1 on every rank d;
//   * before writing into a workspace last used `lag` launches ago, a rank waits until every rank
//     has begun launch e - lag + 1 (started >= e - lag + 2): whatever read the workspace after its
//     previous use -- inside that launch or between that launch and the next -- is then over;
//   * a rank writes its slot of the workspace on every rank, then adds one arrival per rank;
//   * a consumer waits for the cumulative arrival count of every source and reads all slots, either
//     inside the launch ("gated" workspaces) or right before its next launch ("deferred": the
//     re-gathered activation that a later plain GEMM reads).
//
// The check: whenever a rank reads a slot it must hold the epoch of the launch being consumed.  A
// writer that got ahead (a wrong lag rule) would show up as a newer epoch in a slot.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

constexpr int kRanks = 4, kLaunches = 3000, kBuffers = 3;
#ifndef ITB_MODEL_SLACK
#define ITB_MODEL_SLACK 0   // 1 = wait for one launch less than the rule asks (negative control)
#endif

struct Workspace {
  std::atomic<int> slot[kRanks];        // epoch of the data each source wrote
  std::atomic<int> arrive[kRanks];      // cumulative arrivals per source
};
struct RankMem {
  std::atomic<int> started[kRanks];
  Workspace ws[kBuffers];
};
static RankMem mem[kRanks];
static std::atomic<int> failures{0};

// which workspace launch e uses, and whether its data is consumed after the launch (deferred)
static int buffer_of(int e) {
  if (e % 7 == 3) return buffer_of(e - 1);      // back-to-back reuse: nothing but the rule protects it
  return (e % 5 == 4) ? 2 : (e % 2);
}
static bool deferred(int e) { return buffer_of(e) == 2; }

static void consume(int r, int e, std::mt19937& rng) {
  // a slow reader: the moment a wrong rule would let a fast writer overwrite the workspace
  if (rng() % 8 == 0) std::this_thread::sleep_for(std::chrono::microseconds(50 + rng() % 250));
  Workspace& w = mem[r].ws[buffer_of(e)];
  for (int s = 0; s < kRanks; ++s) {
    const int got = w.slot[s].load(std::memory_order_acquire);
    if (got != e) {
      failures.fetch_add(1);
      std::fprintf(stderr, "rank %d consuming launch %d found epoch %d in slot %d\n", r, e, got, s);
    }
  }
}

static void rank_main(int r) {
  std::mt19937 rng(1234 + r);
  int last_use[kBuffers], uses[kBuffers];
  for (int b = 0; b < kBuffers; ++b) last_use[b] = -1, uses[b] = 0;
  int pending_deferred = -1;
  for (int e = 0; e < kLaunches; ++e) {
    if (rng() % 64 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));
    // work between launches: the deferred consumer of the previous launch (a plain GEMM in the stream)
    if (pending_deferred >= 0) {
      const int b = buffer_of(pending_deferred);
      for (int s = 0; s < kRanks; ++s)
        while (mem[r].ws[b].arrive[s].load(std::memory_order_acquire) < uses[b]) std::this_thread::yield();
      consume(r, pending_deferred, rng);
      pending_deferred = -1;
    }
    // ---- launch e begins
    for (int d = 0; d < kRanks; ++d) mem[d].started[r].store(e + 1, std::memory_order_release);
    const int b = buffer_of(e);
    const int lag = last_use[b] < 0 ? (1 << 24) : e - last_use[b];
    for (int d = 0; d < kRanks; ++d)
      while (mem[r].started[d].load(std::memory_order_acquire) < e - lag + 2 - ITB_MODEL_SLACK) std::this_thread::yield();
    for (int d = 0; d < kRanks; ++d) {
      mem[d].ws[b].slot[r].store(e, std::memory_order_relaxed);
      mem[d].ws[b].arrive[r].fetch_add(1, std::memory_order_release);
    }
    last_use[b] = e;
    ++uses[b];
    if (deferred(e)) {
      pending_deferred = e;             // read after the launch, before the next one begins
    } else {
      for (int s = 0; s < kRanks; ++s)
        while (mem[r].ws[b].arrive[s].load(std::memory_order_acquire) < uses[b]) std::this_thread::yield();
      consume(r, e, rng);
    }
  }
}

int main() {
  for (auto& m : mem) {
    for (auto& s : m.started) s.store(0);
    for (auto& w : m.ws)
      for (int i = 0; i < kRanks; ++i) w.slot[i].store(-1), w.arrive[i].store(0);
  }
  std::vector<std::thread> threads;
  for (int r = 0; r < kRanks; ++r) threads.emplace_back(rank_main, r);
  for (auto& t : threads) t.join();
  if (failures.load()) {
    std::fprintf(stderr, "%d protocol violations\n", failures.load());
    return 1;
  }
  std::puts("protocol model ok");
  return 0;
}
