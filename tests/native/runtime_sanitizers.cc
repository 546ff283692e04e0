// Exercises the framework-free parts of the host runtime (layout and schedule planners, llm.c token
// file reader, prefetching batch ring) so that they can run under ThreadSanitizer and
// AddressSanitizer / UBSan.  Exit code 0 = every check held.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

#include "runtime.h"
#include "token_io.h"

#define REQUIRE(cond)                                                         \
  do {                                                                        \
    if (!(cond)) {                                                            \
      std::fprintf(stderr, "REQUIRE failed: %s (line %d)\n", #cond, __LINE__); \
      std::exit(1);                                                           \
    }                                                                         \
  } while (0)

static void check_layout() {
  const std::vector<int64_t> numels = {130, 4096, 77, 250000, 1200000, 64, 900000, 31};
  for (int64_t dp : {1, 2, 3, 8}) {
    itb::FlatLayoutResult r = itb::PlanFlatLayout(numels, dp, true, 1000000, false);
    REQUIRE(r.param_start.size() == numels.size());
    int64_t prev_end = r.numel;
    for (size_t i = 0; i < numels.size(); ++i) {       // reverse packing: later parameters come first
      REQUIRE(r.param_end[i] - r.param_start[i] == numels[i]);
      REQUIRE(r.param_start[i] % 64 == 0);
      if (i > 0) REQUIRE(r.param_end[i] <= r.param_start[i - 1]);
      const int64_t b = r.param_bucket[i];
      REQUIRE(r.bucket_start[b] <= r.param_start[i] && r.param_end[i] <= r.bucket_end[b]);
      prev_end = r.param_start[i];
    }
    (void)prev_end;
    for (size_t b = 0; b < r.bucket_start.size(); ++b) {
      REQUIRE((r.bucket_end[b] - r.bucket_start[b]) % dp == 0);
      REQUIRE(r.bucket_end[b] % 128 == 0);
      if (b > 0) REQUIRE(r.bucket_start[b] == r.bucket_end[b - 1]);
    }
    REQUIRE(r.bucket_end.back() == r.numel);
  }
}

static void check_schedule(const std::vector<itb::PipeTask>& tasks, int n, int stages, int vpp) {
  REQUIRE(static_cast<int>(tasks.size()) == 2 * n * stages * vpp);
  std::map<std::pair<int, int>, int> fwd_pos;
  for (size_t i = 0; i < tasks.size(); ++i) {
    const itb::PipeTask& t = tasks[i];
    REQUIRE(t.stage == t.global_chunk % stages && t.local_chunk == t.global_chunk / stages);
    const auto key = std::make_pair(t.microbatch, t.global_chunk);
    if (t.is_forward) {
      REQUIRE(!fwd_pos.count(key));
      if (t.global_chunk > 0) REQUIRE(fwd_pos.count(std::make_pair(t.microbatch, t.global_chunk - 1)));
      fwd_pos[key] = static_cast<int>(i);
    } else {
      REQUIRE(fwd_pos.count(key));      // a backward never precedes its forward
    }
  }
}

static std::string write_tokens(int n_tokens) {
  char path[] = "/tmp/itb_tokens_XXXXXX";
  const int fd = mkstemp(path);
  REQUIRE(fd >= 0);
  std::vector<int32_t> header(256, 0);
  header[0] = 20240520;
  header[1] = 1;
  header[2] = n_tokens;
  std::vector<uint16_t> toks(static_cast<size_t>(n_tokens));
  for (int i = 0; i < n_tokens; ++i) toks[static_cast<size_t>(i)] = static_cast<uint16_t>((i * 7 + 3) % 50257);
  REQUIRE(write(fd, header.data(), 1024) == 1024);
  REQUIRE(write(fd, toks.data(), toks.size() * 2) == static_cast<ssize_t>(toks.size() * 2));
  close(fd);
  return path;
}

static void check_ring() {
  const int64_t B = 4, T = 32, depth = 4;
  const std::string path = write_tokens(B * T * 40 + 1);
  auto file = std::make_shared<itb::TokenFile>(path);
  REQUIRE(file->num_tokens() == B * T * 40 + 1 && file->token(5) == (5 * 7 + 3));
  std::vector<std::vector<int64_t>> xs(depth, std::vector<int64_t>(B * T)), ys(depth, std::vector<int64_t>(B * T));
  std::vector<int64_t*> xp, yp;
  for (auto& v : xs) xp.push_back(v.data());
  for (auto& v : ys) yp.push_back(v.data());
  {
    itb::BatchRing ring(file, B, T, /*start_batch=*/1, /*stride=*/2, xp, yp);
    std::vector<int64_t> want_x(B * T), want_y(B * T);
    int64_t held[2] = {-1, -1}, held_batch[2] = {-1, -1};
    for (int64_t k = 0; k < 200; ++k) {
      const int64_t slot = ring.next_slot();
      const int64_t batch = (1 + k * 2) % ring.num_batches();
      file->fill(batch * B, B, T, want_x.data(), want_y.data());
      REQUIRE(xs[slot] == want_x && ys[slot] == want_y);
      // the slot handed out one call ago must still hold its batch
      if (held[0] >= 0) {
        file->fill(held_batch[0] * B, B, T, want_x.data(), want_y.data());
        REQUIRE(xs[held[0]] == want_x);
      }
      held[1] = held[0];
      held_batch[1] = held_batch[0];
      held[0] = slot;
      held_batch[0] = batch;
    }
  }   // destructor joins the worker while batches are pending
  bool threw = false;
  try {
    itb::BatchRing bad(file, B, T, 0, 1, {xp[0], xp[1]}, {yp[0], yp[1]});
  } catch (const std::runtime_error&) {
    threw = true;
  }
  REQUIRE(threw);
  threw = false;
  try {
    itb::TokenFile missing("/tmp/itb_no_such_token_file");
  } catch (const std::runtime_error&) {
    threw = true;
  }
  REQUIRE(threw);
  std::remove(path.c_str());
}

int main() {
  check_layout();
  for (int vpp : {1, 2})
    for (int stages : {2, 4}) {
      check_schedule(itb::GpipeSchedule(8, stages, vpp), 8, stages, vpp);
      check_schedule(itb::Interleaved1F1BSchedule(8, stages, vpp), 8, stages, vpp);
    }
  check_ring();
  std::puts("runtime checks ok");
  return 0;
}
