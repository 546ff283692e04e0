// Device code of the CTA-pair GEMM (tcgen05 cta_group::2), shared by the single-GPU launcher
// (gemm_tcgen05_2cta.cu) and the tensor-parallel launcher (comm/tp_gemm.cu), which compiles the same
// pipeline with the kTp hooks enabled: a prologue that pushes this rank's activation shard into every
// rank's gathered buffer, loads of A gated on the arrival of the shard they read, an epilogue that
// scatters partial output rows to their owner rank, and a closing phase that sums the partials.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "gemm_epilogue.cuh"
#include "kernels.h"

namespace itb {
namespace pair {

constexpr int BMC = 128;        // rows of A per CTA (pair: 256)
constexpr int BNC = 128;        // columns of B per CTA (pair: 256)
constexpr int BN = 256;
constexpr int BK = 64;
#ifndef ITB_PAIR_STAGES
#define ITB_PAIR_STAGES 5
#endif
constexpr int kStages = ITB_PAIR_STAGES;
constexpr int kSlotsPerWarp = kStages >= 6 ? 2 : 4;
constexpr int kThreads = 192;
constexpr int kABytes = BMC * BK * 2;
constexpr int kBBytes = BNC * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;                 // 32 KB
constexpr int kSlotBytes = 32 * 128;                           // 32 rows x 64 bf16, 128-byte swizzle
constexpr int kWarpStaging = kSlotsPerWarp * kSlotBytes;       // two sets of (C, C2 / operand) slots
constexpr int kStagingOffset = kStages * kStageBytes;
constexpr int kBarOffset = kStagingOffset + 4 * kWarpStaging;
constexpr int kSmemTotal = kBarOffset + (2 * kStages + 4 + 4) * 8 + 16;
constexpr uint32_t kTmemCols = 512;                            // two 256-column accumulators

// ---- tensor-parallel hooks -------------------------------------------------------------------
// Rows of the full activation are (b, t) pairs, row = b * T + t; under sequence parallelism rank s
// holds t in [s * Tl, (s + 1) * Tl) of every b as local row b * Tl + (t - s * Tl).
enum { kTpPush = 1, kTpGateA = 2, kTpScatter = 4, kTpBroadcast = 8 };
constexpr int kTpMaxRanks = 8;
constexpr unsigned kTpSpinLimit = 1u << 23;     // polls with a short sleep: seconds of skew

struct TpDev {
  int mode;                 // kTpPush | kTpGateA | kTpScatter
  int rank, world;
  int T, Tl, batch;
  // every launch of a context: `started[r]` on each rank holds 1 + the index of the latest launch
  // rank r has begun; a buffer last used `lag` launches ago is free once every rank has begun the
  // launch after that use
  int* started[kTpMaxRanks];
  int* launch_ctr;          // this GPU: number of launches so far
  unsigned* cta_done;       // this GPU: CTAs that have finished (self-resetting)
  int* err;
  // push: local shard [batch * Tl, push_cols] bf16 -> rows of every rank's gathered buffer
  const uint4* push_src;
  int push_row_vecs;        // 16-byte vectors per row
  uint4* gather[kTpMaxRanks];
  uint4* gather_mc;         // multicast address of the gathered buffer, or null
  int* push_arrive[kTpMaxRanks];   // counters [world] on each rank: warps of rank s that have pushed
  int* push_total;          // this GPU: arrivals per source that the pushes so far add up to
  int push_lag;
  // gate: loads of A wait for the shard they read
  const int* gate_arrive;   // this GPU's counters of the gated buffer
  const int* gate_total;
  int gate_includes_this_launch;
  // scatter: partial rows go to slab [rank] of their owner; the owner sums the slabs
  __nv_bfloat16* slab[kTpMaxRanks];     // [world][batch * Tl, N] bf16 on each rank
  int* rs_arrive[kTpMaxRanks];     // counters [world] on each rank: warp-tiles rank s has delivered
  int* rs_total;            // this GPU: arrivals per source that the launches so far add up to
  int rs_lag;
  void* rs_out;             // [batch * Tl, N]
  long long rs_ld_out;
  int rs_out_f32;
  const float* rs_bias;
  const __nv_bfloat16* rs_residual;
  long long rs_ld_res;
  // broadcast (with scatter): the summed rows go to every rank's full [batch * T, N] bf16 buffer
  // instead of rs_out, which turns the reduce-scatter into an all-reduce
  __nv_bfloat16* ar_out[kTpMaxRanks];
  uint4* ar_mc;             // multicast address of that buffer, or null
  int* ar_arrive[kTpMaxRanks];     // counters [world] on each rank: CTAs of rank s that have delivered
  int* ar_total;            // this GPU: arrivals per source that the launches so far add up to
  int ar_lag;
};

__device__ __forceinline__ void tp_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int tp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_red_release_sys(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Waits until *p - target >= 0 (wrap-safe).  False when the limit ran out.
__device__ __forceinline__ bool tp_wait_ge(const int* p, int target) {
  for (unsigned i = 0; i < kTpSpinLimit; ++i) {
    if (tp_ld_acquire_sys(p) - target >= 0) return true;
    if (i > 16) __nanosleep(200);
  }
  return false;
}

template <bool A_MN, bool B_MN, bool kTp>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_c2,
                      const __grid_constant__ CUtensorMap tma_e, const GemmDev p, const TpDev tp) {
  if constexpr (kTp) {
    // an earlier launch gave up on a peer: do not wait for it again (the status word was written
    // before this launch began, so both CTAs of a pair read the same value)
    if (*static_cast<volatile int*>(p.err) != 0) return;
  }
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* operand_bar = tmem_empty + 2;         // one per epilogue warp: residual / aux tile landed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(operand_bar + 4);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const bool leader = cta == 0;
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);     // leader: its own arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty_bar[s], 1);    // one commit from the leader's MMA warp
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);    // one commit
      mbar_init(&tmem_empty[i], 8);   // 4 epilogue warps of each CTA (used on the leader only)
    }
    for (int i = 0; i < 4; ++i) mbar_init(&operand_bar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();      // both CTAs' barriers are initialised before any remote signal
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  int tp_launch = 0;
  if constexpr (kTp) {
    tp_launch = *tp.launch_ctr;
    if (blockIdx.x == 0 && threadIdx.x < tp.world)
      tp_st_release_sys(tp.started[threadIdx.x] + tp.rank, tp_launch + 1);
  }
  const int total_tiles = p.tiles_m * p.tiles_n * p.split_k;
  const int kb_per_split = (p.k_blocks + p.split_k - 1) / p.split_k;
  constexpr int kGroupM = 8;
  auto decode_tile = [&](int t, int& tm, int& tn, int& kb0, int& kb1) {
    int ks = t % p.split_k;
    int t2 = t / p.split_k;
    int width = kGroupM * p.tiles_n;
    int group = t2 / width;
    int first_m = group * kGroupM;
    int gsz = min(p.tiles_m - first_m, kGroupM);
    int in_group = t2 - group * width;
    tm = first_m + in_group % gsz;
    tn = in_group / gsz;
    if constexpr (kTp) {
      // visit the shards in ring order: a gated GEMM starts with the rows this rank already holds,
      // a scattering GEMM ends with the rows it keeps
      const int nb = tp.Tl / 256, per = tp.batch * nb;
      const int j = tm / per, rem = tm - j * per;
      const int b = rem / nb, blk = rem - b * nb;
      const int sh = (tp.rank + j + ((tp.mode & kTpScatter) ? 1 : 0)) % tp.world;
      tm = (b * tp.T + sh * tp.Tl) / 256 + blk;
    }
    kb0 = ks * kb_per_split;
    kb1 = min(p.k_blocks, kb0 + kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t gate_seen = 0;
      // (probe without loads: nothing holds the leader back for the peer's sake, so the peer's producer
      // could miss a barrier phase; it has no part in that run)
      if ((p.flags & kGemmProbeNoLoad) && !leader) ok = false;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        int tm, tn, kb0, kb1;
        decode_tile(t, tm, tn, kb0, kb1);
        const int row0 = tm * 256 + cta * BMC;     // this CTA's rows of A
        const int col0 = tn * 256 + cta * BNC;     // this CTA's columns of B
        if constexpr (kTp) {
          if (tp.mode & kTpGateA) {
            const int sh = ((tm * 256) % tp.T) / tp.Tl;
            if (!((gate_seen >> sh) & 1u)) {
              const int target = *tp.gate_total + (tp.gate_includes_this_launch ? static_cast<int>(gridDim.x) * 4 : 0);
              if (!tp_wait_ge(tp.gate_arrive + sh, target)) {
                atomicCAS(p.err, 0, 121);
                *abort_flag = 1;
                ok = false;
                break;
              }
              gate_seen |= 1u << sh;
              // the shard was written with ordinary stores; the loads below go through the async proxy
              asm volatile("fence.proxy.async;" ::: "memory");
            }
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1) || *abort_flag) {
            atomicCAS(p.err, 0, 111);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          // every load of the pair completes on the LEADER's barrier
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
          if (p.flags & kGemmProbeNoLoad) {
            if (leader) mbar_arrive(&full_bar[stage]);
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, bar, kb * BK, row0);
          } else {
#pragma unroll
            for (int i = 0; i < BMC / 64; ++i)
              tma_load_2d_pair(sa + i * (64 * BK * 2), &tma_a, bar, row0 + i * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, bar, kb * BK, col0);
          } else {
#pragma unroll
            for (int i = 0; i < BNC / 64; ++i)
              tma_load_2d_pair(sb + i * (64 * BK * 2), &tma_b, bar, col0 + i * 64, kb * BK);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    // ONE thread runs the whole loop: wait for a stage, issue its four MMAs, release it with one
    // commit that arrives on both CTAs' barriers.  No tcgen05 fence inside the k-loop (the operands
    // arrive through the async proxy and the barrier wait orders them); the fence after a thread
    // synchronisation is only needed where the epilogue warps hand an accumulator back.
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16_f32(256, BN, A_MN, B_MN);
      const bool probe_no_mma = p.flags & kGemmProbeNoMma;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase0 = 0, acc_phase1 = 0;
      int local = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++local) {
        int tm, tn, kb0, kb1;
        decode_tile(t, tm, tn, kb0, kb1);
        const int acc = local & 1;
        if (kb1 <= kb0) continue;
        const uint32_t ap = acc ? acc_phase1 : acc_phase0;
        if (!mbar_wait(&tmem_empty[acc], ap ^ 1) || *abort_flag) {
          atomicCAS(p.err, 0, 112);
          *abort_flag = 1;
          break;
        }
        if (acc) acc_phase1 ^= 1; else acc_phase0 ^= 1;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicCAS(p.err, 0, 113);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
          const uint64_t adesc0 = A_MN ? make_smem_desc_sw128(sa, 64 * BK * 2, 1024)
                                       : make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc0 = B_MN ? make_smem_desc_sw128(sb, 64 * BK * 2, 1024)
                                       : make_smem_desc_sw128(sb, 16, 1024);
          if (!probe_no_mma) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adesc = adesc0 + (A_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              const uint64_t bdesc = bdesc0 + (B_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              umma_f16_ss_pair(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
          }
          // free this stage in both CTAs
          umma_commit_pair_mc(smem_u32(&empty_bar[stage]), 3);
          if (kb == kb1 - 1) umma_commit_pair_mc(smem_u32(&tmem_full[acc]), 3);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps per CTA)
    const int q = warp & 3;
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    uint8_t* wstage = smem + kStagingOffset + q * kWarpStaging;
    const bool has_operand = p.flags & (kGemmResidual | kGemmDGelu);
    const bool dual = p.flags & kGemmGeluDual;
    uint32_t operand_phase = 0;
    int group = 0;
    bool tp_ok = true;
    if constexpr (kTp) {
      if (tp.mode & (kTpPush | kTpScatter)) {
        // the buffers written below are free once every rank has begun the launch that follows
        // their previous use
        int lag = 1 << 24;
        if (tp.mode & kTpPush) lag = min(lag, tp.push_lag);
        if (tp.mode & kTpScatter) lag = min(lag, tp.rs_lag);
        if (tp.mode & kTpBroadcast) lag = min(lag, tp.ar_lag);
        bool ok = true;
        if (lane < tp.world) ok = tp_wait_ge(tp.started[tp.rank] + lane, tp_launch - lag + 2);
        tp_ok = __all_sync(0xffffffffu, ok);
        if (!tp_ok) {
          if (lane == 0) atomicCAS(p.err, 0, 122);
          *abort_flag = 1;
        }
      }
      if ((tp.mode & kTpPush) && tp_ok) {
        const long long total = static_cast<long long>(tp.batch) * tp.Tl * tp.push_row_vecs;
        const long long stride = static_cast<long long>(gridDim.x) * 128;
        for (long long v = static_cast<long long>(blockIdx.x) * 128 + (warp - 2) * 32 + lane; v < total; v += stride) {
          const long long l = v / tp.push_row_vecs;
          const int cv = static_cast<int>(v - l * tp.push_row_vecs);
          const int b = static_cast<int>(l / tp.Tl), t = static_cast<int>(l - static_cast<long long>(b) * tp.Tl);
          const long long dst = (static_cast<long long>(b) * tp.T + tp.rank * tp.Tl + t) * tp.push_row_vecs + cv;
          const uint4 u = __ldg(tp.push_src + v);
          if (tp.gather_mc) {
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(tp.gather_mc + dst),
                         "f"(__uint_as_float(u.x)), "f"(__uint_as_float(u.y)), "f"(__uint_as_float(u.z)),
                         "f"(__uint_as_float(u.w))
                         : "memory");
          } else {
            for (int d = 0; d < tp.world; ++d) tp.gather[(tp.rank + d) % tp.world][dst] = u;
          }
        }
        __threadfence_system();
        __syncwarp();
        if (lane < tp.world) tp_red_release_sys(tp.push_arrive[lane] + tp.rank, 1);
      }
    }
    for (int t = pair_id; t < total_tiles && tp_ok; t += num_pairs, ++local) {
      int tm, tn, kb0, kb1;
      decode_tile(t, tm, tn, kb0, kb1);
      const int acc = local & 1;
      if (kb1 <= kb0) continue;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc]) || *abort_flag) {
        if (lane == 0) atomicCAS(p.err, 0, 114);
        *abort_flag = 1;
        break;
      }
      acc_phase[acc] ^= 1;
      tc_fence_after_sync();
      const int row0 = tm * 256 + cta * BMC + q * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (p.staged == 2) {
        // fp32 output: 32 columns per slot; store, or add into C (split-K partial sums / accumulation)
        const bool add = p.flags & (kGemmAtomic | kGemmAccum);
#pragma unroll 1
        for (int c = 0; c < BN; c += 64, ++group) {
          const int col0 = tn * BN + c;
          if (col0 >= p.N) break;
          uint8_t* s0 = wstage + (group & 1) * (2 * kSlotBytes);
          uint8_t* s1 = s0 + kSlotBytes;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr0 + c, r0);
          tmem_ld_32x32(taddr0 + c + 32, r1);
          tmem_ld_wait();
          float v0[32], v1[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v0[j] = __uint_as_float(r0[j]), v1[j] = __uint_as_float(r1[j]);
          if (p.flags & kGemmBias) {
            add_bias32(p, col0, v0);
            add_bias32(p, col0 + 32, v1);
          }
          stage_put32_f32(s0, lane, v0);
          stage_put32_f32(s1, lane, v1);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.M) {
            const bool second = col0 + 32 < p.N;
            if (add) {
              tma_reduce_add_2d(&tma_c, s0, col0, row0);
              if (second) tma_reduce_add_2d(&tma_c, s1, col0 + 32, row0);
            } else {
              tma_store_2d(&tma_c, s0, col0, row0);
              if (second) tma_store_2d(&tma_c, s1, col0 + 32, row0);
            }
            tma_store_commit();
          }
        }
      } else if (p.staged) {
        bool ok = true;
#pragma unroll 1
        for (int c = 0; c < BN && ok; c += 64, ++group) {
          const int col0 = tn * BN + c;
          if (col0 >= p.N) break;
          uint8_t* s0 = wstage + (group & 1) * ((kSlotsPerWarp / 2) * kSlotBytes);
          uint8_t* s1 = s0 + kSlotBytes;
          // the slots of this set were last read by the store group issued two groups ago
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          if (has_operand && lane == 0) {
            mbar_expect_tx(&operand_bar[q], kSlotBytes);
            tma_load_2d(s1, &tma_e, &operand_bar[q], col0, row0);
          }
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr0 + c, r0);
          tmem_ld_32x32(taddr0 + c + 32, r1);
          tmem_ld_wait();
          float v0[32], v1[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v0[j] = __uint_as_float(r0[j]), v1[j] = __uint_as_float(r1[j]);
          if (p.flags & kGemmBias) {
            add_bias32(p, col0, v0);
            add_bias32(p, col0 + 32, v1);
          }
          if (has_operand) {
            if (!mbar_wait(&operand_bar[q], operand_phase) || *abort_flag) {
              if (lane == 0) atomicCAS(p.err, 0, 115);
              *abort_flag = 1;
              ok = false;
            }
            operand_phase ^= 1;
            if (p.flags & kGemmDGelu) {
              stage_fold32<true>(s1, lane, 0, v0);
              stage_fold32<true>(s1, lane, 1, v1);
            } else {
              stage_fold32<false>(s1, lane, 0, v0);
              stage_fold32<false>(s1, lane, 1, v1);
            }
          }
          if (dual) {
            stage_put32_gelu(s0, s1, lane, 0, v0);
            stage_put32_gelu(s0, s1, lane, 1, v1);
          } else {
            stage_put32(s0, lane, 0, v0);
            stage_put32(s0, lane, 1, v1);
          }
          fence_proxy_async_smem();
          __syncwarp();
          bool scattered = false;
          if constexpr (kTp) {
            if (tp.mode & kTpScatter) {
              // coalesced 16-byte stores of the slot into this rank's slab on the owner of the rows
              scattered = true;
              const int sh = (row0 % tp.T) / tp.Tl;
              const long long lrow0 = static_cast<long long>(row0 / tp.T) * tp.Tl + (row0 % tp.T) - sh * tp.Tl;
              __nv_bfloat16* dst = tp.slab[sh] + (static_cast<long long>(tp.rank) * tp.batch * tp.Tl + lrow0) * p.N;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int idx = i * 32 + lane, r = idx >> 3, pos = idx & 7;
                const int col = col0 + ((pos ^ (r & 7)) << 3);
                if (col < p.N)
                  *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * p.N + col) =
                      *reinterpret_cast<const uint4*>(s0 + r * 128 + pos * 16);
              }
            }
          }
          if (!scattered && lane == 0 && ok && row0 < p.M) {
            tma_store_2d(&tma_c, s0, col0, row0);
            if (dual) tma_store_2d(&tma_c2, s1, col0, row0);
            tma_store_commit();
          }
        }
        if constexpr (kTp) {
          if (tp.mode & kTpScatter) {
            __threadfence_system();
            __syncwarp();
            if (lane == 0) tp_red_release_sys(tp.rs_arrive[(row0 % tp.T) / tp.Tl] + tp.rank, 1);
          }
        }
        if (!ok) break;
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int col0 = tn * BN + c;
          if (col0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr0 + c, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          gemm_epilogue_chunk(p, row, row_ok, col0, v);
        }
      }
      // hand the accumulator back to the leader's MMA warp: one arrival per warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
    }
    if (lane == 0) tma_store_wait<0>();   // shared memory stays allocated until the stores have left
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();      // the peer may still signal this CTA's barriers until it gets here
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if constexpr (kTp) {
    if (tp.mode & kTpScatter) {
      // every rank's partial rows for this rank have to be in the slabs before they are summed
      __shared__ int tail_ok;
      if (threadIdx.x == 0) tail_ok = (*abort_flag == 0);
      __syncthreads();
      const int rows = tp.batch * tp.Tl;
      if (threadIdx.x < tp.world) {
        const int per_launch = (rows / 256) * p.tiles_n * 8;
        if (!tp_wait_ge(tp.rs_arrive[tp.rank] + threadIdx.x, *tp.rs_total + per_launch)) {
          atomicCAS(p.err, 0, 123);
          tail_ok = 0;
        }
      }
      __syncthreads();
      if (tail_ok) {
        const int nv = p.N >> 3;
        const long long total = static_cast<long long>(rows) * nv;
        const uint4* slabs = reinterpret_cast<const uint4*>(tp.slab[tp.rank]);
        for (long long v = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; v < total;
             v += static_cast<long long>(gridDim.x) * kThreads) {
          const long long row = v / nv;
          const int c8 = static_cast<int>(v - row * nv);
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
          for (int src = 0; src < tp.world; ++src) {
            const uint4 u = __ldcg(slabs + static_cast<long long>(src) * total + v);
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += __bfloat162float(b[e]);
          }
          if (tp.rs_bias) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += __ldg(tp.rs_bias + c8 * 8 + e);
          }
          if (tp.rs_residual) {
            const uint4 u = *reinterpret_cast<const uint4*>(tp.rs_residual + row * tp.rs_ld_res + c8 * 8);
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += __bfloat162float(b[e]);
          }
          if (tp.mode & kTpBroadcast) {
            // local row -> row of the full activation; every rank receives the 16 bytes
            const long long bb = row / tp.Tl, tt = row - bb * tp.Tl;
            const long long idx = (bb * tp.T + tp.rank * tp.Tl + tt) * nv + c8;     // in 16-byte units
            const uint4 u = pack8_bf16(acc);
            if (tp.ar_mc) {
              asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(tp.ar_mc + idx),
                           "f"(__uint_as_float(u.x)), "f"(__uint_as_float(u.y)), "f"(__uint_as_float(u.z)),
                           "f"(__uint_as_float(u.w))
                           : "memory");
            } else {
              for (int d = 0; d < tp.world; ++d)
                reinterpret_cast<uint4*>(tp.ar_out[(tp.rank + d) % tp.world])[idx] = u;
            }
          } else if (tp.rs_out_f32) {
            float* o = static_cast<float*>(tp.rs_out) + row * tp.rs_ld_out + c8 * 8;
            *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
          } else {
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(tp.rs_out) + row * tp.rs_ld_out + c8 * 8) =
                pack8_bf16(acc);
          }
        }
      }
    }
    if (tp.mode & kTpBroadcast) {
      // this CTA's share of the summed rows has left: count it on every rank
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < tp.world) tp_red_release_sys(tp.ar_arrive[threadIdx.x] + tp.rank, 1);
    }
    // the last CTA to get here advances this GPU's counters for the next launch
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned prev = atomicAdd(tp.cta_done, 1u);
      if (prev == gridDim.x - 1) {
        *tp.cta_done = 0;
        *tp.launch_ctr = tp_launch + 1;
        if (tp.mode & kTpPush) *tp.push_total += static_cast<int>(gridDim.x) * 4;
        if (tp.mode & kTpScatter) *tp.rs_total += (tp.batch * tp.Tl / 256) * p.tiles_n * 8;
        if (tp.mode & kTpBroadcast) *tp.ar_total += static_cast<int>(gridDim.x);
        __threadfence();
      }
    }
  }
}

}  // namespace pair
}  // namespace itb
