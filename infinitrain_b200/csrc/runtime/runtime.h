// Host runtime of the native layer: checkpoint file IO, llm.c token files with a prefetching batch
// assembler, and planners (flat-buffer layout, pipeline schedules) used by the Python layer.
#pragma once
#include <stdint.h>

#include <string>
#include <utility>
#include <vector>

namespace itb {

// ---------------------------------------------------------------- flat-buffer layout planner
struct FlatLayoutResult {
  std::vector<int64_t> param_start, param_end, param_bucket;   // per parameter, input order
  std::vector<int64_t> bucket_start, bucket_end, bucket_unpadded;
  int64_t numel = 0, numel_unpadded = 0;
};
// Parameters are packed in reverse order; with `shard` every parameter starts at a multiple of 64
// elements and a bucket end is padded to lcm(dp_size, 128) (and 2^16 when pad_for_busbw); a bucket
// closes once it holds >= bucket_size elements.
FlatLayoutResult PlanFlatLayout(const std::vector<int64_t>& numels, int64_t dp_size, bool shard,
                                int64_t bucket_size, bool pad_for_busbw);

// ---------------------------------------------------------------- pipeline schedules
struct PipeTask {
  int step, microbatch, global_chunk, local_chunk, stage;
  bool is_forward, is_first_chunk, is_last_chunk;
};
std::vector<PipeTask> GpipeSchedule(int n, int num_stages, int vpp);
std::vector<PipeTask> Interleaved1F1BSchedule(int n, int num_stages, int vpp);

}  // namespace itb
