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

#include "gemm_pair_body.cuh"

namespace itb {

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_outer);

namespace pair {

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tc2,
                  const CUtensorMap& te, const GemmDev& p, int pairs, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, false>;
  constexpr int smem = kSmemTotal + 1024;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  kern<<<2 * pairs, kThreads, smem, stream>>>(ta, tb, tc, tc2, te, p, TpDev{});
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
