// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs computes one 256 x 256
// output tile.  Each CTA stages its own 128 rows of A and its own 128 columns of B per k-block
// (32 KB instead of the 48 KB a single-CTA 128 x 256 tile needs for the same work per CTA), so the
// shared-memory fill traffic per FLOP drops by a third and the ring is 5 stages deep; the MMA of
// shape 256 x 256 x 16 is issued by one thread of the even CTA for both, each CTA keeps its half of
// the accumulator in its own TMEM and runs its own epilogue.  Same operand layouts and epilogues as
// the single-CTA kernel (gemm_tcgen05.cu); the reference has only cuBLAS here
// (infini_train/src/kernels/cuda/common/gemm.cu:45-75).
//
// Signalling inside the pair (no cluster multicast anywhere):
//   * TMA loads of BOTH CTAs complete on the leader's `full` barrier (cta_group::2 form of the load);
//   * the leader's MMA warp commits to its own `empty` barrier and, with a second commit, to the
//     peer's, which frees that stage in both CTAs;
//   * accumulator-full is committed to both CTAs' barriers the same way; accumulator-empty is
//     counted on the leader's barrier (4 local + 4 remote warp arrivals).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "gemm_epilogue.cuh"
#include "kernels.h"

namespace itb {

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_outer);

namespace pair {

constexpr int BMC = 128;        // rows of A per CTA (pair: 256)
constexpr int BNC = 128;        // columns of B per CTA (pair: 256)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 5;
constexpr int kThreads = 192;
constexpr int kABytes = BMC * BK * 2;
constexpr int kBBytes = BNC * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;                 // 32 KB
constexpr int kSlotBytes = 32 * 128;                           // 32 rows x 64 bf16, 128-byte swizzle
constexpr int kWarpStaging = 4 * kSlotBytes;                   // two sets of (C, C2 / operand) slots
constexpr int kStagingOffset = kStages * kStageBytes;
constexpr int kBarOffset = kStagingOffset + 4 * kWarpStaging;
constexpr int kSmemTotal = kBarOffset + (2 * kStages + 4 + 4) * 8 + 16;
constexpr uint32_t kTmemCols = 512;                            // two 256-column accumulators

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_c2,
                      const __grid_constant__ CUtensorMap tma_e, const GemmDev p) {
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
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        int tm, tn, kb0, kb1;
        decode_tile(t, tm, tn, kb0, kb1);
        const int row0 = tm * 256 + cta * BMC;     // this CTA's rows of A
        const int col0 = tn * 256 + cta * BNC;     // this CTA's columns of B
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
    if (leader) {
      constexpr uint32_t idesc = make_idesc_bf16_f32(256, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++local) {
        int tm, tn, kb0, kb1;
        decode_tile(t, tm, tn, kb0, kb1);
        const int acc = local & 1;
        if (kb1 <= kb0) continue;
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1) || *abort_flag) {
          if (lane == 0) atomicCAS(p.err, 0, 112);
          *abort_flag = 1;
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase) || *abort_flag) {
            if (lane == 0) atomicCAS(p.err, 0, 113);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t sa = smem_u32(smem + stage * kStageBytes);
            const uint32_t sb = sa + kABytes;
            const uint64_t adesc0 = A_MN ? make_smem_desc_sw128(sa, 64 * BK * 2, 1024)
                                         : make_smem_desc_sw128(sa, 16, 1024);
            const uint64_t bdesc0 = B_MN ? make_smem_desc_sw128(sb, 64 * BK * 2, 1024)
                                         : make_smem_desc_sw128(sb, 16, 1024);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adesc = adesc0 + (A_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              const uint64_t bdesc = bdesc0 + (B_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
              umma_f16_ss_pair(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            // free this stage in both CTAs
            const uint32_t eb = smem_u32(&empty_bar[stage]);
            umma_commit_pair(eb);
            umma_commit_pair(mapa_u32(eb, 1));
            if (kb == kb1 - 1) {
              const uint32_t fb = smem_u32(&tmem_full[acc]);
              umma_commit_pair(fb);
              umma_commit_pair(mapa_u32(fb, 1));
            }
          }
          __syncwarp();
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
    for (int t = pair_id; t < total_tiles; t += num_pairs, ++local) {
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
          uint8_t* s0 = wstage + (group & 1) * (2 * kSlotBytes);
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
          if (lane == 0 && ok && row0 < p.M) {
            tma_store_2d(&tma_c, s0, col0, row0);
            if (dual) tma_store_2d(&tma_c2, s1, col0, row0);
            tma_store_commit();
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
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tc2,
                  const CUtensorMap& te, const GemmDev& p, int pairs, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  constexpr int smem = kSmemTotal + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  kern<<<2 * pairs, kThreads, smem, stream>>>(ta, tb, tc, tc2, te, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pair
}  // namespace itb

extern "C" int itb_gemm_bf16_pair(const ItbGemmArgs* a, cudaStream_t stream) {
  using namespace itb;
  using namespace itb::pair;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) || (a->lda % 8) ||
      (a->ldb % 8))
    return -2;
  CUtensorMap ta, tb;
  int rc;
  if (!a->a_mn_major)
    rc = make_tmap_bf16_2d(&ta, a->A, a->K, a->M, a->lda, 64, BMC);
  else
    rc = make_tmap_bf16_2d(&ta, a->A, a->M, a->K, a->lda, 64, 64);
  if (rc) return rc;
  if (!a->b_mn_major)
    rc = make_tmap_bf16_2d(&tb, a->B, a->K, a->N, a->ldb, 64, BNC);
  else
    rc = make_tmap_bf16_2d(&tb, a->B, a->N, a->K, a->ldb, 64, 64);
  if (rc) return rc;
  GemmDev p;
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.k_blocks = (a->K + BK - 1) / BK;
  p.tiles_m = (a->M + 255) / 256;
  p.tiles_n = (a->N + 255) / 256;
  p.C = a->C;
  p.ldc = a->ldc;
  p.C2 = a->C2;
  p.bias = a->bias;
  p.residual = a->residual;
  p.ldr = a->ldr;
  p.aux = static_cast<const __nv_bfloat16*>(a->aux);
  p.ld_aux = a->ld_aux;
  p.flags = a->flags;
  p.err = a->err;
  // bf16 outputs go through shared memory and TMA stores when every matrix the epilogue touches
  // can be described by a tensor map
  CUtensorMap tc = ta, tc2 = ta, te = ta;
  p.staged = 0;
  if (!(a->flags & kGemmOutF32)) {
    auto ok16 = [](const void* q, long long ld) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0 && ld % 8 == 0; };
    bool ok = ok16(a->C, a->ldc);
    if (a->flags & kGemmGeluDual) ok = ok && ok16(a->C2, a->ldc);
    if (a->flags & kGemmResidual) ok = ok && ok16(a->residual, a->ldr);
    if (a->flags & kGemmDGelu) ok = ok && ok16(a->aux, a->ld_aux);
    if (ok) {
      rc = make_tmap_bf16_2d(&tc, a->C, a->N, a->M, a->ldc, 64, 32);
      if (!rc && (a->flags & kGemmGeluDual)) rc = make_tmap_bf16_2d(&tc2, a->C2, a->N, a->M, a->ldc, 64, 32);
      if (!rc && (a->flags & kGemmResidual)) rc = make_tmap_bf16_2d(&te, a->residual, a->N, a->M, a->ldr, 64, 32);
      if (!rc && (a->flags & kGemmDGelu)) rc = make_tmap_bf16_2d(&te, a->aux, a->N, a->M, a->ld_aux, 64, 32);
      if (rc) return rc;
      p.staged = 1;
    }
  }
  if ((a->flags & kGemmOutF32) && !(a->flags & (kGemmResidual | kGemmGeluDual | kGemmDGelu)) &&
      (reinterpret_cast<uintptr_t>(a->C) & 15) == 0 && a->ldc % 4 == 0) {
    rc = make_tmap_f32_2d(&tc, a->C, a->N, a->M, a->ldc, 32);
    if (rc) return rc;
    p.staged = 2;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int max_pairs = sms / 2;
  int split = 1;
  if (a->flags & kGemmAtomic) {
    const int tiles = p.tiles_m * p.tiles_n;
    if (a->split_k > 0) {
      split = a->split_k;
    } else {
      // Fewest pair-waves x (k-blocks per split + a fixed per-tile cost of pipeline fill, epilogue
      // tail and the extra pass of add traffic), over every split that leaves >= 4 k-blocks.
      const int max_split = p.k_blocks / 4 > 0 ? p.k_blocks / 4 : 1;
      long best = -1;
      for (int s = 1; s <= max_split && s <= 64; ++s) {
        const int per = (p.k_blocks + s - 1) / s;
        const int eff = (p.k_blocks + per - 1) / per;
        const long waves = (static_cast<long>(tiles) * eff + max_pairs - 1) / max_pairs;
        const long cost = waves * (per + 6);
        if (best < 0 || cost < best) best = cost, split = eff;
      }
    }
    const int per = (p.k_blocks + split - 1) / split;
    split = (p.k_blocks + per - 1) / per;
  }
  p.split_k = split;
  const int total = p.tiles_m * p.tiles_n * split;
  const int pairs = total < max_pairs ? total : max_pairs;
  const bool amn = a->a_mn_major, bmn = a->b_mn_major;
  if (!amn && !bmn) return launch<false, false>(ta, tb, tc, tc2, te, p, pairs, stream);
  if (!amn && bmn) return launch<false, true>(ta, tb, tc, tc2, te, p, pairs, stream);
  if (amn && bmn) return launch<true, true>(ta, tb, tc, tc2, te, p, pairs, stream);
  return launch<true, false>(ta, tb, tc, tc2, te, p, pairs, stream);
}
