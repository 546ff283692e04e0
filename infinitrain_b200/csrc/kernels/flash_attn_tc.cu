// Flash attention forward and backward on the 5th-generation tensor cores (tcgen05, accumulators
// in TMEM, operands staged by TMA), causal or full, grouped-query heads, head size 64 or 128.
//
// Backward: one CTA owns 128 keys of one KV head and walks over the 128-row query tiles (and the query heads
// of the group) that attend to them.  Per tile, with n = key row, m = query row, d = head column:
//
//   S^T[n,m]  = K[n,:] . Q[m,:]            tcgen05.mma  K (K-major)  x Q (K-major)   -> TMEM cols 0..127
//   dP^T[n,m] = V[n,:] . dO[m,:]           tcgen05.mma  V            x dO            -> TMEM cols 128..255
//   P^T = exp2(S^T c - lse[m]),  dS^T = P^T (dP^T - delta[m])      256 threads, half a key row each;
//                                          written as bf16 to shared memory in the swizzled operand layout
//   dV[n,d] += P^T[n,m]  dO[m,d]           tcgen05.mma  P^T (K-major)  x dO (MN-major) -> TMEM cols 256..
//   dK[n,d] += dS^T[n,m] Q[m,d]            tcgen05.mma  dS^T (K-major) x Q  (MN-major) -> TMEM cols 256+D..
//   dQ[m,d]  = dS[m,n]   K[n,d]            tcgen05.mma  dS^T read MN-major x K (MN-major) -> TMEM, then added
//                                          to the fp32 dQ buffer with vector reductions
//
// Warp roles: warp 0 issues the TMA loads, warp 1 the MMAs, warps 2-9 do the softmax recomputation
// and the TMEM read-outs (two warps per TMEM lane quarter, each taking half of the columns).  With
// head size 64 dQ has TMEM columns of its own, so S^T / dP^T of the next tile are computed while the
// softmax warps still read dQ out; with head size 128 dQ overwrites the spent S^T.  Every wait is
// bounded; a wait that gives up records a code in the status word and the CTA drains without
// touching the tensor pipe again.
//
// The reference composes attention from batched cuBLAS matmuls, a mask and a 3-pass softmax and
// lets autograd differentiate them (infini_train/src/nn/modules/transformer/causal_self_attention.cc:86-130).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <float.h>
#include <math.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "kernels.h"

namespace itb {

int make_tmap_bf16_3d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t d1, uint64_t d2,
                      uint64_t ld1, uint64_t ld2, uint32_t box_inner, uint32_t box_d1);

int make_tmap_f32_3d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t d1, uint64_t d2,
                     uint64_t ld1, uint64_t ld2, uint32_t box_d1);

namespace fatc {

constexpr int kThreads = 320;     // TMA warp, MMA warp, 8 softmax / read-out warps
constexpr int kSoftmaxThreads = 256;
constexpr int kAtom = 128 * 128;   // bytes of one [128 rows][64 x bf16] swizzled block
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void softmax_warps_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 u;
  __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) b2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  return u;
}

template <int D>
struct BwdCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr int kTile = kAtoms * kAtom;          // one [128][D] bf16 tile
  static constexpr int kQStages = D == 64 ? 2 : 1;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTile;
  static constexpr int kOffQ = 2 * kTile;
  static constexpr int kOffdO = kOffQ + kQStages * kTile;
  static constexpr int kOffP = kOffdO + kQStages * kTile;    // [2 m-chunks][128 n][64 m]
  static constexpr int kOffdS = kOffP + 2 * kAtom;
  static constexpr int kOffStat = kOffdS + 2 * kAtom;        // lse*log2e [2][128], delta [2][128]
  static constexpr int kOffBar = kOffStat + 4 * 128 * 4;
  static constexpr int kSmem = kOffBar + 12 * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                    const __grid_constant__ CUtensorMap tdq, const ItbAttnArgs a, int* err) {
  using Cfg = BwdCfg<D>;
  constexpr int S = Cfg::kQStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* s_lse = reinterpret_cast<float*>(smem + Cfg::kOffStat);
  float* s_delta = s_lse + 2 * 128;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  uint64_t* q_full = kv_full + 1;
  uint64_t* q_empty = q_full + 2;
  uint64_t* s_full = q_empty + 2;
  uint64_t* p_full = s_full + 1;
  uint64_t* dq_full = p_full + 1;
  uint64_t* dq_drained = dq_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(dq_drained + 1);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The (query head of the group, query tile) pairs that meet this CTA's 128 keys are dealt out to
  // `nparts` CTAs in turn (a.bwd_parts > 1 when the plain grid would leave most SMs idle: few key
  // tiles, one KV head per rank under tensor parallelism); each then adds its dK / dV into fp32
  // accumulators instead of writing them.
  const int nparts = a.bwd_parts > 1 ? a.bwd_parts : 1;
  const int nb = blockIdx.x, hk = blockIdx.y / nparts, part = blockIdx.y % nparts, b = blockIdx.z;
  const int G = a.H / a.KV;
  const int n0 = nb * 128;
  const int n_qblocks = (a.T + 127) / 128;
  const int mb_first = a.causal ? nb : 0;
  const int per_head = n_qblocks - mb_first;
  const int total_iters = per_head * G;
  const int iters = total_iters > part ? (total_iters - part + nparts - 1) / nparts : 0;
  auto tile_of = [&](int it, int& h, int& mb) {
    const int g = part + it * nparts;
    h = hk * G + g / per_head;
    mb = mb_first + g % per_head;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, kSoftmaxThreads);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, kSoftmaxThreads / 32);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_S = tmem_base, tm_dP = tmem_base + 128, tm_dV = tmem_base + 256, tm_dK = tmem_base + 256 + D;
  constexpr bool kAlias = D > 64;     // no TMEM columns left for dQ: it goes over the spent S^T
  const uint32_t tm_dQ = kAlias ? tmem_base : tmem_base + 256 + 2 * D;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      tma_prefetch_desc(&tdo);
      mbar_expect_tx(kv_full, 2 * Cfg::kTile);
#pragma unroll
      for (int at = 0; at < Cfg::kAtoms; ++at) {
        tma_load_3d(smem + Cfg::kOffK + at * kAtom, &tk, kv_full, hk * D + at * 64, n0, b);
        tma_load_3d(smem + Cfg::kOffV + at * kAtom, &tv, kv_full, hk * D + at * 64, n0, b);
      }
      for (int it = 0; it < iters; ++it) {
        const int st = it % S;
        const uint32_t ph = (it / S) & 1;
        if (!mbar_wait(&q_empty[st], ph ^ 1) || *abort_flag) {
          atomicCAS(err, 0, 201);
          *abort_flag = 1;
          break;
        }
        int h, mb;
        tile_of(it, h, mb);
        mbar_expect_tx(&q_full[st], 2 * Cfg::kTile);
#pragma unroll
        for (int at = 0; at < Cfg::kAtoms; ++at) {
          tma_load_3d(smem + Cfg::kOffQ + st * Cfg::kTile + at * kAtom, &tq, &q_full[st], h * D + at * 64, mb * 128, b);
          tma_load_3d(smem + Cfg::kOffdO + st * Cfg::kTile + at * kAtom, &tdo, &q_full[st], h * D + at * 64, mb * 128,
                      b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t id_s = make_idesc_bf16_f32(128, 128, false, false);
    constexpr uint32_t id_kv = make_idesc_bf16_f32(128, D, false, true);
    constexpr uint32_t id_q = make_idesc_bf16_f32(128, D, true, true);
    const uint32_t aK = smem_u32(smem + Cfg::kOffK), aV = smem_u32(smem + Cfg::kOffV);
    const uint32_t aP = smem_u32(smem + Cfg::kOffP), adS = smem_u32(smem + Cfg::kOffdS);
    // Shared-memory descriptors are built once; a k-step only adds its byte offset (>> 4) to them.
    const uint64_t dK_k = make_smem_desc_sw128(aK, 16, 1024), dV_k = make_smem_desc_sw128(aV, 16, 1024);
    const uint64_t dP_k = make_smem_desc_sw128(aP, 16, 1024), ddS_k = make_smem_desc_sw128(adS, 16, 1024);
    const uint64_t ddS_m = make_smem_desc_sw128(adS, kAtom, 1024), dK_m = make_smem_desc_sw128(aK, kAtom, 1024);
    const uint32_t aQ0 = smem_u32(smem + Cfg::kOffQ), adO0 = smem_u32(smem + Cfg::kOffdO);
    const uint64_t dQ_k0 = make_smem_desc_sw128(aQ0, 16, 1024), ddO_k0 = make_smem_desc_sw128(adO0, 16, 1024);
    const uint64_t dQ_m0 = make_smem_desc_sw128(aQ0, kAtom, 1024), ddO_m0 = make_smem_desc_sw128(adO0, kAtom, 1024);
    constexpr uint64_t kStageStep = (S > 1 ? Cfg::kTile : 0) >> 4;
    bool ok = mbar_wait(kv_full, 0);
    if (!ok && lane == 0) atomicCAS(err, 0, 202);
    auto issue_scores = [&](int it) {     // S^T and dP^T of tile `it`
      const int st = it % S;
      if (!mbar_wait(&q_full[st], (it / S) & 1) || *abort_flag) return false;
      // with aliasing, dQ of the previous tile sits over S^T until the softmax warps have read it out
      if (kAlias && it > 0 && (!mbar_wait(dq_drained, (it - 1) & 1) || *abort_flag)) return false;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint64_t dQ_k = dQ_k0 + st * kStageStep, ddO_k = ddO_k0 + st * kStageStep;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = ((kk >> 2) * kAtom + (kk & 3) * 32) >> 4;
          umma_f16_ss(tm_S, dK_k + off, dQ_k + off, id_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = ((kk >> 2) * kAtom + (kk & 3) * 32) >> 4;
          umma_f16_ss(tm_dP, dV_k + off, ddO_k + off, id_s, kk > 0);
        }
        umma_commit(s_full);
      }
      __syncwarp();
      return true;
    };
    if (ok && iters > 0 && !issue_scores(0)) {
      if (lane == 0) atomicCAS(err, 0, 203);
      ok = false;
    }
    for (int it = 0; it < iters && ok; ++it) {
      const int st = it % S;
      ok = mbar_wait(p_full, it & 1) && !*abort_flag;
      // its own dQ columns are rewritten below: the previous tile's dQ must have been read out
      if (ok && !kAlias && it > 0) ok = mbar_wait(dq_drained, (it - 1) & 1) && !*abort_flag;
      if (!ok) {
        if (lane == 0) atomicCAS(err, 0, 204);
        break;
      }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint64_t dQ_m = dQ_m0 + st * kStageStep, ddO_m = ddO_m0 + st * kStageStep;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {       // contraction over the 128 query rows of the tile
          const uint64_t koff = ((kk >> 2) * kAtom + (kk & 3) * 32) >> 4;   // K-major operand: P^T / dS^T
          const uint64_t moff = (kk * 2048) >> 4;                            // MN-major operand: 16 rows down
          umma_f16_ss(tm_dV, dP_k + koff, ddO_m + moff, id_kv, (it > 0 || kk > 0));
          umma_f16_ss(tm_dK, ddS_k + koff, dQ_m + moff, id_kv, (it > 0 || kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {       // contraction over the 128 keys
          const uint64_t moff = (kk * 2048) >> 4;
          umma_f16_ss(tm_dQ, ddS_m + moff, dK_m + moff, id_q, kk > 0);
        }
        umma_commit(&q_empty[st]);
        umma_commit(dq_full);
      }
      __syncwarp();
      if (it + 1 < iters && !issue_scores(it + 1)) {
        if (lane == 0) atomicCAS(err, 0, 203);
        ok = false;
      }
    }
    if (!ok) *abort_flag = 1;
  } else {
    // ------------------------------------------------------------------ softmax / read-out warps
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;           // which half of the columns this warp takes
    const int row = qd * 32 + lane;             // key row (softmax) and query row (dQ read-out)
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    const int tid = (warp - 2) * 32 + lane;     // 0..255, for the per-tile statistics
    const float sl2 = a.scale * kLog2e;
    uint8_t* sP = smem + Cfg::kOffP;
    uint8_t* sdS = smem + Cfg::kOffdS;
    bool ok = true;
    // lse * log2(e) (threads 0..127) or delta (threads 128..255) of query row tid & 127 of tile `it`;
    // rows beyond the sequence get probability 0 (lse = +inf) and delta 0
    auto load_stat = [&](int it) -> float {
      int h, mb;
      tile_of(it, h, mb);
      const int qrow = mb * 128 + (tid & 127);
      const long long so = (static_cast<long long>(b) * a.H + h) * a.T + qrow;
      if (tid < 128) return qrow < a.T ? __ldg(a.lse + so) * kLog2e : INFINITY;
      return qrow < a.T ? __ldg(a.delta + so) : 0.f;
    };
    float stat_next = iters > 0 ? load_stat(0) : 0.f;
    for (int it = 0; it < iters; ++it) {
      int h, mb;
      tile_of(it, h, mb);
      const int sb = it & 1;
      // this tile's statistics were fetched while the previous tile was being processed
      if (tid < 128)
        s_lse[sb * 128 + tid] = stat_next;
      else
        s_delta[sb * 128 + tid - 128] = stat_next;
      if (it + 1 < iters) stat_next = load_stat(it + 1);
      softmax_warps_sync();
      if (ok) {
        ok = mbar_wait(s_full, it & 1) && !*abort_flag;
        if (!ok) {
          atomicCAS(err, 0, 205);
          *abort_flag = 1;
        }
      }
      if (ok) {
        tc_fence_after_sync();
        const bool key_ok = n0 + row < a.T;
        // the mask matters on the diagonal tile and for the keys beyond the sequence only
        const bool diag = a.causal && mb == nb;
        const bool need_mask = diag || (n0 + 128 > a.T);
        const float* lse = s_lse + sb * 128;
        const float* dl = s_delta + sb * 128;
#pragma unroll 1
        for (int cg = 2 * half; cg < 2 * half + 2; ++cg) {
          uint32_t rs[32], rp[32];
          tmem_ld_32x32(tm_S + lane_addr + cg * 32, rs);
          tmem_ld_32x32(tm_dP + lane_addr + cg * 32, rp);
          tmem_ld_wait();
          float pv[32], dv[32];
#pragma unroll
          for (int j4 = 0; j4 < 32; j4 += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(lse + cg * 32 + j4);
            const float4 d4 = *reinterpret_cast<const float4*>(dl + cg * 32 + j4);
            const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = j4 + e, m = cg * 32 + j;
              float p = ex2(fmaf(__uint_as_float(rs[j]), sl2, -lv[e]));
              if (need_mask && (!key_ok || (diag && row > m))) p = 0.f;
              pv[j] = p;
              dv[j] = p * (__uint_as_float(rp[j]) - dd[e]);
            }
          }
          uint8_t* rowP = sP + (cg >> 1) * kAtom + row * 128;
          uint8_t* rowS = sdS + (cg >> 1) * kAtom + row * 128;
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            const int pos = (((cg & 1) << 2) + c8) ^ (row & 7);
            *reinterpret_cast<uint4*>(rowP + pos * 16) = pack8(&pv[c8 * 8]);
            *reinterpret_cast<uint4*>(rowS + pos * 16) = pack8(&dv[c8 * 8]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(p_full);
        ok = mbar_wait(dq_full, it & 1) && !*abort_flag;
        if (!ok) {
          atomicCAS(err, 0, 206);
          *abort_flag = 1;
        }
      }
      if (ok) {
        // dQ of the tile: TMEM -> fp32 staging over the spent P^T / dS^T buffers (32 columns per
        // 16 KB block, 128-byte swizzle) -> one bulk add-reduction per block into the fp32 dQ buffer
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tm_dQ + lane_addr + c * 32, r);
          tmem_ld_wait();
          uint8_t* dst = smem + Cfg::kOffP + c * kAtom + row * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(dst + ((j ^ (row & 7)) << 4)) =
                make_float4(__uint_as_float(r[4 * j]) * a.scale, __uint_as_float(r[4 * j + 1]) * a.scale,
                            __uint_as_float(r[4 * j + 2]) * a.scale, __uint_as_float(r[4 * j + 3]) * a.scale);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_drained);
      }
      softmax_warps_sync();     // every row of the staging blocks is written
      if (ok && tid == 0) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c)
          tma_reduce_add_3d(&tdq, smem + Cfg::kOffP + c * kAtom, h * D + c * 32, mb * 128, b);
        tma_store_commit();
        // the staging blocks are P^T / dS^T again after the barrier at the top of the next tile
        tma_store_wait_read<0>();
      }
    }
    if (tid == 0) tma_store_wait<0>();
    if (ok && iters > 0 && nparts > 1) {
      // this CTA's share of dK (scaled) and dV: added to the fp32 accumulators [2][B, T, KV, D]
      const int krow = n0 + row;
      const long long plane = static_cast<long long>(a.B) * a.T * a.KV * D;
      float* dka = a.dkv_accum + ((static_cast<long long>(b) * a.T + krow) * a.KV + hk) * D;
      float* dva = dka + plane;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t rk[32], rv[32];
        tmem_ld_32x32(tm_dK + lane_addr + c * 32, rk);
        tmem_ld_32x32(tm_dV + lane_addr + c * 32, rv);
        tmem_ld_wait();
        if (krow < a.T) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dka + c * 32 + j),
                         "f"(__uint_as_float(rk[j]) * a.scale), "f"(__uint_as_float(rk[j + 1]) * a.scale),
                         "f"(__uint_as_float(rk[j + 2]) * a.scale), "f"(__uint_as_float(rk[j + 3]) * a.scale)
                         : "memory");
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dva + c * 32 + j),
                         "f"(__uint_as_float(rv[j])), "f"(__uint_as_float(rv[j + 1])), "f"(__uint_as_float(rv[j + 2])),
                         "f"(__uint_as_float(rv[j + 3]))
                         : "memory");
          }
        }
      }
    } else if (ok && nparts == 1) {
      // dK (scaled) and dV of this CTA's 128 keys; the last dq_full covered the MMAs that wrote them
      const int krow = n0 + row;
      __nv_bfloat16* dkg = static_cast<__nv_bfloat16*>(a.dk) + b * a.k_batch_stride +
                           static_cast<long long>(krow) * a.k_row_stride + hk * D;
      __nv_bfloat16* dvg = static_cast<__nv_bfloat16*>(a.dv) + b * a.v_batch_stride +
                           static_cast<long long>(krow) * a.v_row_stride + hk * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t rk[32], rv[32];
        tmem_ld_32x32(tm_dK + lane_addr + c * 32, rk);
        tmem_ld_32x32(tm_dV + lane_addr + c * 32, rv);
        tmem_ld_wait();
        if (krow < a.T) {
          float fk[32], fv[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            fk[j] = __uint_as_float(rk[j]) * a.scale;
            fv[j] = __uint_as_float(rv[j]);
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            *reinterpret_cast<uint4*>(dkg + c * 32 + j) = pack8(&fk[j]);
            *reinterpret_cast<uint4*>(dvg + c * 32 + j) = pack8(&fv[j]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------ forward
// One CTA owns 128 query rows of one head and walks over the 128-key tiles up to the diagonal:
//   S[m,n] = Q[m,:] . K[n,:]     tcgen05.mma  Q (K-major) x K (K-major)          -> TMEM cols 0..127
//   online softmax: one thread per query row reads its row of S from TMEM twice (maximum, then
//   exponentials), so nothing crosses threads; P is written as bf16 in the swizzled operand layout
//   O_j[m,d] = P[m,n] V[n,d]     tcgen05.mma  P (K-major) x V (MN-major)         -> TMEM cols 128..
//   o = o * exp2(m_old - m_new) + O_j   in registers
// 192 threads (TMA warp, MMA warp, 4 softmax warps) and 80 KB of shared memory at head size 64, so
// two CTAs share an SM and one's tensor-core and TMA latencies hide behind the other's softmax.
template <int D>
struct FwdCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr int kTile = kAtoms * kAtom;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kTile;
  static constexpr int kOffV = 2 * kTile;
  static constexpr int kOffP = 3 * kTile;                 // [2 n-chunks][128 m][64 n]
  static constexpr int kOffBar = kOffP + 2 * kAtom;
  static constexpr int kSmem = kOffBar + 12 * 8 + 16;
  static constexpr int kTmemCols = 256;
};
constexpr int kFwdThreads = 192;

template <int D>
__global__ void __launch_bounds__(kFwdThreads, D == 64 ? 2 : 1)
flash_fwd_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const ItbAttnArgs a, int* err) {
  using Cfg = FwdCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + 1;
  uint64_t* v_full = k_empty + 1;
  uint64_t* v_empty = v_full + 1;
  uint64_t* s_full = v_empty + 1;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = p_full + 1;
  uint64_t* o_drained = o_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_drained + 1);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavier (later) query tiles first, so that the tail of the grid is made of short CTAs
  const int mb = a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.H / a.KV);
  const int m0 = mb * 128;
  int n_blocks = (a.T + 127) / 128;
  if (a.causal) n_blocks = min(n_blocks, mb + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(o_drained, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_S = tmem_base, tm_O = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      mbar_expect_tx(q_full, Cfg::kTile);
#pragma unroll
      for (int at = 0; at < Cfg::kAtoms; ++at)
        tma_load_3d(smem + Cfg::kOffQ + at * kAtom, &tq, q_full, h * D + at * 64, m0, b);
      for (int j = 0; j < n_blocks; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_empty, ph ^ 1) || *abort_flag) {
          atomicCAS(err, 0, 211);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(k_full, Cfg::kTile);
#pragma unroll
        for (int at = 0; at < Cfg::kAtoms; ++at)
          tma_load_3d(smem + Cfg::kOffK + at * kAtom, &tk, k_full, hk * D + at * 64, j * 128, b);
        if (!mbar_wait(v_empty, ph ^ 1) || *abort_flag) {
          atomicCAS(err, 0, 212);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(v_full, Cfg::kTile);
#pragma unroll
        for (int at = 0; at < Cfg::kAtoms; ++at)
          tma_load_3d(smem + Cfg::kOffV + at * kAtom, &tv, v_full, hk * D + at * 64, j * 128, b);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t id_s = make_idesc_bf16_f32(128, 128, false, false);
    constexpr uint32_t id_o = make_idesc_bf16_f32(128, D, false, true);
    const uint32_t aQ = smem_u32(smem + Cfg::kOffQ), aK = smem_u32(smem + Cfg::kOffK);
    const uint32_t aV = smem_u32(smem + Cfg::kOffV), aP = smem_u32(smem + Cfg::kOffP);
    auto issue_scores = [&](int j) {
      if (!mbar_wait(k_full, j & 1) || *abort_flag) return false;
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kAtom + (kk & 3) * 32;
          umma_f16_ss(tm_S, make_smem_desc_sw128(aQ + off, 16, 1024), make_smem_desc_sw128(aK + off, 16, 1024), id_s,
                      kk > 0);
        }
        umma_commit(k_empty);
        umma_commit(s_full);
      }
      __syncwarp();
      return true;
    };
    bool ok = mbar_wait(q_full, 0);
    if (ok && n_blocks > 0) ok = issue_scores(0);
    if (!ok && lane == 0) atomicCAS(err, 0, 213);
    for (int j = 0; j < n_blocks && ok; ++j) {
      ok = mbar_wait(p_full, j & 1) && !*abort_flag;
      if (ok && j > 0) ok = mbar_wait(o_drained, (j - 1) & 1) && !*abort_flag;
      if (ok) ok = mbar_wait(v_full, j & 1) && !*abort_flag;
      if (!ok) {
        if (lane == 0) atomicCAS(err, 0, 214);
        break;
      }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {       // contraction over the 128 keys of the tile
          const uint32_t koff = (kk >> 2) * kAtom + (kk & 3) * 32;
          umma_f16_ss(tm_O, make_smem_desc_sw128(aP + koff, 16, 1024), make_smem_desc_sw128(aV + kk * 2048, kAtom, 1024),
                      id_o, kk > 0);
        }
        umma_commit(v_empty);
        umma_commit(o_full);
      }
      __syncwarp();
      if (j + 1 < n_blocks && !issue_scores(j + 1)) {
        if (lane == 0) atomicCAS(err, 0, 213);
        ok = false;
      }
    }
    if (!ok) *abort_flag = 1;
  } else {
    const int qd = warp & 3;
    const int row = qd * 32 + lane;                 // query row of the tile
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    const float sl2 = a.scale * kLog2e;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;           // running maximum (scaled, log2 domain) and sum
    uint8_t* rowP = smem + Cfg::kOffP + row * 128;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      ok = mbar_wait(s_full, j & 1) && !*abort_flag;
      if (!ok) {
        atomicCAS(err, 0, 215);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      // only the diagonal tile and a ragged last tile need the mask
      const bool masked = (a.causal && j == mb) || ((j + 1) * 128 > a.T);
      const int n_lim = masked ? min(a.causal && j == mb ? row + 1 : 128, a.T - j * 128) : 128;   // keys [0, n_lim) visible
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tm_S + lane_addr + c * 32, r);
        tmem_ld_wait();
        if (!masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < n_lim) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      mx *= sl2;      // sl2 > 0: scaling commutes with the maximum
      const float m_new = fmaxf(m_run, mx);
      // a row with no visible key so far keeps -inf: use 0 as the base so that exp2 yields 0, not NaN
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float corr = ex2(m_run - base);
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tm_S + lane_addr + c * 32, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p = ex2(fmaf(__uint_as_float(r[i]), sl2, -base));
          if (masked && c * 32 + i >= n_lim) p = 0.f;
          pv[i] = p;
          sum += p;
        }
        uint8_t* dst = rowP + (c >> 1) * kAtom;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8)
          *reinterpret_cast<uint4*>(dst + (((((c & 1) << 2) + c8) ^ (row & 7)) << 4)) = pack8(&pv[c8 * 8]);
      }
      l_run = l_run * corr + sum;
      m_run = m_new;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
      ok = mbar_wait(o_full, j & 1) && !*abort_flag;
      if (!ok) {
        atomicCAS(err, 0, 216);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tm_O + lane_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], corr, __uint_as_float(r[i]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_drained);
    }
    const int qrow = m0 + row;
    if (ok && qrow < a.T) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.o) + b * a.o_batch_stride +
                          static_cast<long long>(qrow) * a.o_row_stride + h * D;
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        float t[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t[e] = o[i + e] * inv;
        *reinterpret_cast<uint4*>(op + i) = pack8(t);
      }
      a.lse[(static_cast<long long>(b) * a.H + h) * a.T + qrow] =
          l_run > 0.f ? m_run * 0.6931471805599453f + logf(l_run) : -FLT_MAX;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int D>
static int fwd_launch(const ItbAttnArgs* a, int* err, cudaStream_t s) {
  using Cfg = FwdCfg<D>;
  constexpr int smem = Cfg::kSmem + 1024;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_bf16_3d(&tq, a->q, static_cast<uint64_t>(a->H) * D, a->T, a->B, a->q_row_stride,
                             a->q_batch_stride, 64, 128);
  if (!rc) rc = make_tmap_bf16_3d(&tk, a->k, static_cast<uint64_t>(a->KV) * D, a->T, a->B, a->k_row_stride,
                                  a->k_batch_stride, 64, 128);
  if (!rc) rc = make_tmap_bf16_3d(&tv, a->v, static_cast<uint64_t>(a->KV) * D, a->T, a->B, a->v_row_stride,
                                  a->v_batch_stride, 64, 128);
  if (rc) return rc;
  dim3 grid((a->T + 127) / 128, a->H, a->B);
  flash_fwd_tc_kernel<D><<<grid, kFwdThreads, smem, s>>>(tq, tk, tv, *a, err);
  return static_cast<int>(cudaGetLastError());
}

__global__ void attn_delta_tc_kernel(const ItbAttnArgs a, int D) {
  // delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; D / 8 threads per (b,t,h), 16 bytes each
  const int tpr = D >> 3;                                        // threads per row: 8 or 16
  const long long gid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long w = gid / tpr;
  const int part = static_cast<int>(gid % tpr);
  const long long total = static_cast<long long>(a.B) * a.T * a.H;
  float acc = 0.f;
  int h = 0, t = 0, b = 0;
  if (w < total) {
    h = static_cast<int>(w % a.H);
    const long long bt = w / a.H;
    t = static_cast<int>(bt % a.T);
    b = static_cast<int>(bt / a.T);
    const long long off = b * a.o_batch_stride + static_cast<long long>(t) * a.o_row_stride + h * D + part * 8;
    const uint4 x = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.o) + off);
    const uint4 y = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.dout) + off);
    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162* yb = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 xf = __bfloat1622float2(xb[e]), yf = __bfloat1622float2(yb[e]);
      acc += xf.x * yf.x + xf.y * yf.y;
    }
  }
  for (int s = tpr >> 1; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (w < total && part == 0) a.delta[(static_cast<long long>(b) * a.H + h) * a.T + t] = acc;
}

__global__ void attn_dq_convert_tc_kernel(const ItbAttnArgs a, int D) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;  // 4 elements each
  const int dv = D / 4;
  const long long total = static_cast<long long>(a.B) * a.T * a.H * dv;
  if (i >= total) return;
  const int c = static_cast<int>(i % dv) * 4;
  long long r = i / dv;
  const int h = static_cast<int>(r % a.H);
  r /= a.H;
  const int t = static_cast<int>(r % a.T), b = static_cast<int>(r / a.T);
  const float4 v = *reinterpret_cast<const float4*>(a.dq_accum + i * 4);
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.dq) + b * a.q_batch_stride +
                       static_cast<long long>(t) * a.q_row_stride + h * D + c;
  uint2 u;
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = u;
}

// dk, dv (bf16, strided) = the fp32 accumulators [2][B, T, KV, D]
__global__ void attn_dkv_convert_tc_kernel(const ItbAttnArgs a, int D) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;  // 4 elements each
  const int dv = D / 4;
  const long long plane4 = static_cast<long long>(a.B) * a.T * a.KV * dv;
  if (i >= 2 * plane4) return;
  const bool is_v = i >= plane4;
  long long r = is_v ? i - plane4 : i;
  const int c = static_cast<int>(r % dv) * 4;
  r /= dv;
  const int h = static_cast<int>(r % a.KV);
  r /= a.KV;
  const int t = static_cast<int>(r % a.T), b = static_cast<int>(r / a.T);
  const float4 v = *reinterpret_cast<const float4*>(a.dkv_accum + i * 4);
  __nv_bfloat16* dst = is_v ? static_cast<__nv_bfloat16*>(a.dv) + b * a.v_batch_stride + static_cast<long long>(t) * a.v_row_stride
                            : static_cast<__nv_bfloat16*>(a.dk) + b * a.k_batch_stride + static_cast<long long>(t) * a.k_row_stride;
  dst += h * D + c;
  uint2 u;
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = u;
}

template <int D>
static int bwd_launch(const ItbAttnArgs* a_in, int* err, cudaStream_t s) {
  ItbAttnArgs args = *a_in;
  args.bwd_parts = args.dkv_accum ? itb_flash_attn_bwd_parts(args.B, args.T, args.H, args.KV, args.causal) : 1;
  const ItbAttnArgs* a = &args;
  using Cfg = BwdCfg<D>;
  constexpr int smem = Cfg::kSmem + 1024;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  CUtensorMap tq, tk, tv, tdo, tdq;
  int rc = make_tmap_f32_3d(&tdq, a->dq_accum, static_cast<uint64_t>(a->H) * D, a->T, a->B,
                            static_cast<uint64_t>(a->H) * D, static_cast<uint64_t>(a->T) * a->H * D, 128);
  if (!rc) rc = make_tmap_bf16_3d(&tq, a->q, static_cast<uint64_t>(a->H) * D, a->T, a->B, a->q_row_stride,
                             a->q_batch_stride, 64, 128);
  if (!rc) rc = make_tmap_bf16_3d(&tk, a->k, static_cast<uint64_t>(a->KV) * D, a->T, a->B, a->k_row_stride,
                                  a->k_batch_stride, 64, 128);
  if (!rc) rc = make_tmap_bf16_3d(&tv, a->v, static_cast<uint64_t>(a->KV) * D, a->T, a->B, a->v_row_stride,
                                  a->v_batch_stride, 64, 128);
  if (!rc) rc = make_tmap_bf16_3d(&tdo, a->dout, static_cast<uint64_t>(a->H) * D, a->T, a->B, a->o_row_stride,
                                  a->o_batch_stride, 64, 128);
  if (rc) return rc;
  const long long nrow = static_cast<long long>(a->B) * a->T * a->H;
  cudaError_t e = cudaMemsetAsync(a->dq_accum, 0, nrow * D * sizeof(float), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  attn_delta_tc_kernel<<<static_cast<int>((nrow * (D / 8) + 255) / 256), 256, 0, s>>>(*a, D);
  const int parts = a->bwd_parts > 1 ? a->bwd_parts : 1;
  const long long kv_vecs = 2LL * a->B * a->T * a->KV * (D / 4);
  if (parts > 1) {
    e = cudaMemsetAsync(a->dkv_accum, 0, kv_vecs * 4 * sizeof(float), s);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid((a->T + 127) / 128, a->KV * parts, a->B);
  flash_bwd_tc_kernel<D><<<grid, kThreads, smem, s>>>(tq, tk, tv, tdo, tdq, *a, err);
  const long long nvec = nrow * (D / 4);
  attn_dq_convert_tc_kernel<<<static_cast<int>((nvec + 255) / 256), 256, 0, s>>>(*a, D);
  if (parts > 1) attn_dkv_convert_tc_kernel<<<static_cast<int>((kv_vecs + 255) / 256), 256, 0, s>>>(*a, D);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fatc
}  // namespace itb

extern "C" int itb_flash_attn_bwd_parts(int B, int T, int H, int KV, int causal) {
  (void)causal;
  const long long ctas = static_cast<long long>((T + 127) / 128) * KV * B;
  const int sms = 148;
  if (ctas <= 0 || ctas * 2 > sms) return 1;                 // at least half a wave as it is
  const int most = ((T + 127) / 128) * (H / KV);             // tiles of the busiest CTA
  int parts = static_cast<int>(sms / ctas);
  if (parts > most) parts = most;
  if (parts > 16) parts = 16;
  return parts < 1 ? 1 : parts;
}

extern "C" int itb_flash_attn_bwd_tc(const ItbAttnArgs* a, int* err, cudaStream_t s) {
  if (a->B <= 0 || a->T <= 0) return 0;
  if (a->H % a->KV) return -3;
  if ((a->q_row_stride | a->k_row_stride | a->v_row_stride | a->o_row_stride | a->q_batch_stride |
       a->k_batch_stride | a->v_batch_stride | a->o_batch_stride) & 7)
    return -2;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->o) | reinterpret_cast<uintptr_t>(a->dq) | reinterpret_cast<uintptr_t>(a->dk) |
       reinterpret_cast<uintptr_t>(a->dv) | reinterpret_cast<uintptr_t>(a->dout)) & 15)
    return -2;
  if (a->D == 64) return itb::fatc::bwd_launch<64>(a, err, s);
  if (a->D == 128) return itb::fatc::bwd_launch<128>(a, err, s);
  return -4;
}

extern "C" int itb_flash_attn_fwd_tc(const ItbAttnArgs* a, int* err, cudaStream_t s) {
  if (a->B <= 0 || a->T <= 0) return 0;
  if (a->H % a->KV) return -3;
  if ((a->q_row_stride | a->k_row_stride | a->v_row_stride | a->o_row_stride | a->q_batch_stride |
       a->k_batch_stride | a->v_batch_stride | a->o_batch_stride) & 7)
    return -2;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->o)) & 15)
    return -2;
  if (a->D == 64) return itb::fatc::fwd_launch<64>(a, err, s);
  if (a->D == 128) return itb::fatc::fwd_launch<128>(a, err, s);
  return -4;
}
