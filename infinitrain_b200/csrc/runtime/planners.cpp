// Flat-buffer layout and pipeline schedule planners (pure host code).  Compiled as a translation unit
// of the extension; a header-only user (the C++ frontend) defines ITB_PLANNERS_INLINE as `inline` and
// includes this file.
#pragma once
#ifndef ITB_PLANNERS_INLINE
#define ITB_PLANNERS_INLINE
#endif
#include <algorithm>
#include <numeric>

#include "runtime.h"

namespace itb {

static inline int64_t pad_to(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

ITB_PLANNERS_INLINE FlatLayoutResult PlanFlatLayout(const std::vector<int64_t>& numels, int64_t dp_size, bool shard,
                                int64_t bucket_size, bool pad_for_busbw) {
  FlatLayoutResult r;
  const size_t n = numels.size();
  r.param_start.assign(n, 0);
  r.param_end.assign(n, 0);
  r.param_bucket.assign(n, 0);
  int64_t pstart = 0, pend = 0, bstart = 0, bucket = 0;
  int open = 0;
  auto close = [&](int64_t end_unpadded) {
    r.bucket_unpadded.push_back(end_unpadded - bstart);
    int64_t bend = end_unpadded;
    if (shard) {
      int64_t l = std::lcm<int64_t>(dp_size, 128);
      if (pad_for_busbw) l = std::lcm<int64_t>(l, int64_t(1) << 16);
      bend = pad_to(end_unpadded, l);
    }
    r.bucket_start.push_back(bstart);
    r.bucket_end.push_back(bend);
    bstart = bend;
    ++bucket;
    open = 0;
    return bend;
  };
  for (size_t k = n; k-- > 0;) {
    if (shard) pstart = pad_to(pstart, 64);
    pend = pstart + numels[k];
    r.param_start[k] = pstart;
    r.param_end[k] = pend;
    r.param_bucket[k] = bucket;
    ++open;
    if (pend - bstart >= bucket_size)
      pstart = close(pend);
    else
      pstart = pend;
  }
  if (open) close(pend);
  r.numel = r.bucket_end.empty() ? 0 : r.bucket_end.back();
  r.numel_unpadded = std::accumulate(r.bucket_unpadded.begin(), r.bucket_unpadded.end(), int64_t(0));
  return r;
}

static inline PipeTask make_task(int step, int mb, int g, int stages, int chunks, bool fwd) {
  return PipeTask{step, mb, g, g / stages, g % stages, fwd, g == 0, g == chunks - 1};
}

ITB_PLANNERS_INLINE std::vector<PipeTask> GpipeSchedule(int n, int stages, int vpp) {
  std::vector<PipeTask> out;
  const int chunks = stages * vpp, total = n + chunks - 1;
  for (int step = 0; step < total; ++step)
    for (int mb = 0; mb < n; ++mb) {
      int g = step - mb;
      if (g >= 0 && g < chunks) out.push_back(make_task(step, mb, g, stages, chunks, true));
    }
  for (int step = 0; step < total; ++step)
    for (int mb = 0; mb < n; ++mb) {
      int g = (total - 1 - step) - mb;
      if (g >= 0 && g < chunks) out.push_back(make_task(step + total, mb, g, stages, chunks, false));
    }
  std::stable_sort(out.begin(), out.end(), [](const PipeTask& a, const PipeTask& b) {
    return a.step != b.step ? a.step < b.step : a.local_chunk < b.local_chunk;
  });
  return out;
}

ITB_PLANNERS_INLINE std::vector<PipeTask> Interleaved1F1BSchedule(int n, int stages, int vpp) {
  std::vector<PipeTask> out;
  if (n <= 0 || stages <= 0 || vpp <= 0) return out;
  const int chunks = stages * vpp, warm = chunks - 1, total = 2 * warm + n;
  for (int step = 0; step < warm; ++step)
    for (int mb = 0; mb < n; ++mb) {
      int g = step - mb;
      if (g >= 0 && g < chunks) out.push_back(make_task(step, mb, g, stages, chunks, true));
    }
  for (int step = warm; step < warm + n; ++step)
    for (int mb = 0; mb < n; ++mb) {
      int g = step - mb;
      if (g >= 0 && g < chunks) out.push_back(make_task(step, mb, g, stages, chunks, true));
      int gb = (chunks - 1) - ((step - warm) - mb);
      if (gb >= 0 && gb < chunks) out.push_back(make_task(step, mb, gb, stages, chunks, false));
    }
  for (int step = warm + n; step < total; ++step)
    for (int mb = 0; mb < n; ++mb) {
      int gb = (chunks - 1) - ((step - warm) - mb);
      if (gb >= 0 && gb < chunks) out.push_back(make_task(step, mb, gb, stages, chunks, false));
    }
  return out;
}

}  // namespace itb
