// Topology of a training job for the C++ frontend: world size and rank from the launcher's
// environment, the three parallel axes and the rank layout.
//
// Reference: infini_train/src/nn/parallel/global.cc:22-112 -- world = tp * dp * pp, three-axis layout
// with TP varying fastest, then DP, then PP (so that a tensor-parallel group sits on adjacent GPUs),
// `RankOf / CoordOf / GroupRanks`, group names "TP<i>" / "DP<i>" / "PP<i>".  The reference keeps the
// per-thread ranks in thread-local variables because it runs one thread per GPU; here a process IS a
// rank, so the state is one process-wide object.
#pragma once
#include <cstdlib>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace itb {
namespace parallel {

enum class Axis { kTP = 0, kDP = 1, kPP = 2 };

struct Layout {
  int tp = 1, dp = 1, pp = 1;
  int world() const { return tp * dp * pp; }
  int RankOf(int tp_rank, int dp_rank, int pp_rank) const { return tp_rank + tp * (dp_rank + dp * pp_rank); }
  void CoordOf(int rank, int* tp_rank, int* dp_rank, int* pp_rank) const {
    *tp_rank = rank % tp;
    *dp_rank = (rank / tp) % dp;
    *pp_rank = rank / (tp * dp);
  }
  int size(Axis a) const { return a == Axis::kTP ? tp : (a == Axis::kDP ? dp : pp); }
  // Ranks of the group of `rank` along `axis`, ordered by their coordinate on that axis.
  std::vector<int> GroupRanks(Axis axis, int rank) const {
    int c[3];
    CoordOf(rank, &c[0], &c[1], &c[2]);
    std::vector<int> out;
    for (int i = 0; i < size(axis); ++i) {
      int d[3] = {c[0], c[1], c[2]};
      d[static_cast<int>(axis)] = i;
      out.push_back(RankOf(d[0], d[1], d[2]));
    }
    return out;
  }
  // Index of that group among the groups of its axis (the <i> of "TP<i>"): the lowest rank of every
  // group, in increasing order.
  int GroupId(Axis axis, int rank) const {
    const int lowest = GroupRanks(axis, rank)[0];
    int id = 0;
    for (int r = 0; r < lowest; ++r)
      if (GroupRanks(axis, r)[0] == r) ++id;
    return id;
  }
  std::string GroupName(Axis axis, int rank) const {
    static const char* kNames[3] = {"TP", "DP", "PP"};
    return std::string(kNames[static_cast<int>(axis)]) + std::to_string(GroupId(axis, rank));
  }
};

// Process-wide parallel state.  InitAllEnv() reads RANK / WORLD_SIZE / LOCAL_RANK (set by infini_run
// or torchrun; the reference's names GLOBAL_PROC_RANK / PROC_WORLD_SIZE / LOCAL_PROC_RANK are
// honoured too) and derives dp = world / (tp * pp).
struct GlobalEnv {
  int world = 1, rank = 0, local_rank = 0;
  Layout layout;
  int tp_rank = 0, dp_rank = 0, pp_rank = 0;
  int vpp = 1;
  bool sequence_parallel = false;
  bool initialized = false;

  static GlobalEnv& Instance() {
    static GlobalEnv g;
    return g;
  }
  static int EnvInt(const char* a, const char* b, int dflt) {
    for (const char* k : {a, b}) {
      const char* v = k ? std::getenv(k) : nullptr;
      if (v && *v) return std::atoi(v);
    }
    return dflt;
  }
  void Init(int world_size, int my_rank, int tensor_parallel, bool seq_parallel, int pipeline_parallel, int virtual_pp = 1,
            int my_local_rank = -1) {
    if (tensor_parallel < 1 || pipeline_parallel < 1 || virtual_pp < 1 || world_size % (tensor_parallel * pipeline_parallel))
      throw std::invalid_argument("world size must be a multiple of tensor_parallel * pipeline_parallel");
    world = world_size, rank = my_rank, local_rank = my_local_rank < 0 ? my_rank : my_local_rank;
    layout.tp = tensor_parallel, layout.pp = pipeline_parallel, layout.dp = world_size / (tensor_parallel * pipeline_parallel);
    layout.CoordOf(rank, &tp_rank, &dp_rank, &pp_rank);
    vpp = virtual_pp;
    sequence_parallel = seq_parallel && tensor_parallel > 1;
    initialized = true;
  }
  void InitAllEnv(int tensor_parallel = 1, bool seq_parallel = false, int pipeline_parallel = 1, int virtual_pp = 1) {
    const int w = EnvInt("WORLD_SIZE", "PROC_WORLD_SIZE", 1), r = EnvInt("RANK", "GLOBAL_PROC_RANK", 0);
    Init(w, r, tensor_parallel, seq_parallel, pipeline_parallel, virtual_pp, EnvInt("LOCAL_RANK", "LOCAL_PROC_RANK", r));
  }
  int tp() const { return layout.tp; }
  int dp() const { return layout.dp; }
  int pp() const { return layout.pp; }
  int sp() const { return sequence_parallel ? layout.tp : 1; }
  std::vector<int> GroupRanks(Axis a) const { return layout.GroupRanks(a, rank); }
  std::string GroupName(Axis a) const { return layout.GroupName(a, rank); }

  // Human-readable overview of every group (reference: global.cc:196-257).
  std::string ProcessGroupOverview() const {
    std::ostringstream os;
    os << "\n=== Parallel Communication Groups ===\nworld_size = " << world << ", config: {DP=" << dp() << ", TP=" << tp()
       << ", PP=" << pp() << "}, order: {TP -> DP -> PP}\n";
    const Axis axes[3] = {Axis::kDP, Axis::kTP, Axis::kPP};
    const char* names[3] = {"DP", "TP", "PP"};
    for (int a = 0; a < 3; ++a) {
      if (layout.size(axes[a]) == 1) {
        os << "[" << names[a] << "] size=1, unenabled\n";
        continue;
      }
      os << "[" << names[a] << "] size=" << layout.size(axes[a]) << ", num_groups=" << world / layout.size(axes[a]) << "\n";
      for (int r = 0; r < world; ++r) {
        auto g = layout.GroupRanks(axes[a], r);
        if (g[0] != r) continue;
        os << "  - " << layout.GroupName(axes[a], r) << " (dp=";
        int t, d, p;
        layout.CoordOf(r, &t, &d, &p);
        os << (axes[a] == Axis::kDP ? "-" : std::to_string(d)) << ", tp=" << (axes[a] == Axis::kTP ? "-" : std::to_string(t))
           << ", pp=" << (axes[a] == Axis::kPP ? "-" : std::to_string(p)) << "): [";
        for (size_t i = 0; i < g.size(); ++i) os << (i ? ", " : "") << g[i];
        os << "]\n";
      }
    }
    return os.str();
  }
};

inline GlobalEnv& env() { return GlobalEnv::Instance(); }

// The reference's free-function accessors (include/nn/parallel/global.h:90-160) over the same state.  A worker is
// a process here, so the thread count per process is 1 and the process ranks are the ranks; coordinates keep the
// reference's (dp, tp, pp) argument order.
namespace global {
inline void InitAllEnv(int /*nthread_per_process*/, int tensor_parallel_size, bool sequence_parallel_enabled, int pipeline_parallel_size,
                       int virtual_pipeline_parallel_size = 1) {
  env().InitAllEnv(tensor_parallel_size, sequence_parallel_enabled, pipeline_parallel_size, virtual_pipeline_parallel_size);
}
inline int GetNnodes() { return GlobalEnv::EnvInt("NNODES", nullptr, 1); }
inline int GetWorldSize() { return env().world; }
inline int GetNprocPerNode() { return GlobalEnv::EnvInt("LOCAL_WORLD_SIZE", "NPROC_PER_NODE", env().world); }
inline int GetNthreadPerProc() { return 1; }
inline int GetGlobalProcRank() { return env().rank; }
inline int GetLocalProcRank() { return env().local_rank; }
inline int GetTensorParallelSize() { return env().tp(); }
inline int GetSequenceParallelSize() { return env().sp(); }
inline bool GetSequenceParallelEnabled() { return env().sequence_parallel; }
inline int GetDataParallelSize() { return env().dp(); }
inline int GetPipelineParallelSize() { return env().pp(); }
inline int GetVirtualPipelineParallelSize() { return env().vpp; }
inline int GetRankOf(int dp, int tp, int pp) { return env().layout.RankOf(tp, dp, pp); }
inline void GetCoordOf(int rank, int& dp, int& tp, int& pp) { env().layout.CoordOf(rank, &tp, &dp, &pp); }
inline int GetGroupId(Axis target, int rank) { return env().layout.GroupId(target, rank); }
inline int GetGroupId(Axis target, int dp, int tp, int pp) { return GetGroupId(target, GetRankOf(dp, tp, pp)); }
inline std::vector<int> GetGroupRanks(Axis target, int rank) { return env().layout.GroupRanks(target, rank); }
inline std::vector<int> GetGroupRanks(Axis target, int dp, int tp, int pp) { return GetGroupRanks(target, GetRankOf(dp, tp, pp)); }
inline std::string ProcessGroupOverview() { return env().ProcessGroupOverview(); }
}  // namespace global

// Who this worker is among the job's workers (reference: include/nn/parallel/rank.h).  The reference
// counts processes on the node and threads inside a process (one thread per GPU); here a worker is a
// process, so thread_rank is 0 and thread_size 1 unless a program sets them for threads of its own.
class Rank {
 public:
  Rank(int process_rank, int thread_rank, int process_size, int thread_size)
      : process_rank_(process_rank), thread_rank_(thread_rank), process_size_(process_size), thread_size_(thread_size) {}
  static Rank Current() { return Rank(env().rank, 0, env().world, 1); }
  int process_rank() const { return process_rank_; }
  int thread_rank() const { return thread_rank_; }
  int process_size() const { return process_size_; }
  int thread_size() const { return thread_size_; }
  int GlobalRank() const { return process_rank_ * thread_size_ + thread_rank_; }
  bool IsParallel() const { return process_size_ * thread_size_ > 1; }
  bool IsMainRank() const { return GlobalRank() == 0; }
  bool IsLastRank() const { return GlobalRank() == process_size_ * thread_size_ - 1; }

 private:
  int process_rank_, thread_rank_, process_size_, thread_size_;
};

// Which layers a pipeline stage holds (reference: pipeline_parallel.cc:42-77).  The model is cut into
// pp * vpp chunks of consecutive layers; the first (layers % chunks) chunks get one layer more; stage s
// owns the chunks local * pp + s, local = 0 .. vpp - 1 (round robin, so that consecutive chunks sit on
// consecutive stages and the last stage hands over to the first between rounds).
struct StageInfo {
  bool is_first_stage = true, is_last_stage = true;
  std::vector<std::pair<int, int>> layer_ranges_per_chunk;   // [start, end) of every chunk this stage owns
};
inline StageInfo GetStageInfo(int total_layers, int pp_size, int pp_rank, int chunks_per_stage = 1) {
  if (pp_size < 1 || chunks_per_stage < 1 || pp_rank < 0 || pp_rank >= pp_size)
    throw std::invalid_argument("GetStageInfo: bad pipeline coordinates");
  const int chunks = pp_size * chunks_per_stage;
  if (total_layers < chunks) throw std::invalid_argument("fewer layers than pipeline chunks");
  const int base = total_layers / chunks, rem = total_layers % chunks;
  StageInfo info;
  info.is_first_stage = pp_rank == 0;
  info.is_last_stage = pp_rank == pp_size - 1;
  for (int local = 0; local < chunks_per_stage; ++local) {
    const int g = local * pp_size + pp_rank;
    const int start = g * base + (g < rem ? g : rem);
    info.layer_ranges_per_chunk.emplace_back(start, start + base + (g < rem ? 1 : 0));
  }
  return info;
}

}  // namespace parallel
}  // namespace itb
