// Tensor-parallel GEMMs fused with their collective over NVLink / NVSwitch: one launch of the
// CTA-pair tcgen05 GEMM (kernels/gemm_pair_body.cuh, kTp hooks) per rank does
//
//   * all-gather + GEMM (column-parallel linear under sequence parallelism): the epilogue warps,
//     idle while the first accumulator fills, push this rank's activation shard into every rank's
//     gathered buffer (`multimem.st` through the switch, or one store per peer) and count their
//     arrival on every rank; the TMA producer starts with the tiles of the local shard and waits for
//     a peer's counter only when it reaches that peer's rows, so the transfer hides behind the math;
//   * GEMM + reduce-scatter (row-parallel linear): each output tile leaves the epilogue as bf16
//     rows stored straight into the owner rank's slab for this source, the owner's rows last; when
//     a rank has run out of tiles it waits for the slabs of every source and sums them in fp32
//     with bias and residual;
//   * GEMM + all-reduce (tensor parallelism without sequence parallelism): the scattering GEMM whose
//     closing phase writes the summed rows to every rank (`multimem.st` or peer stores);
//   * the same push in front of a scattering GEMM, for the backward pass of a column-parallel
//     linear: dX = reduce-scatter(dY W) while X is re-gathered for the weight gradient that follows
//     (itb_tp_wait holds that GEMM back until the shards have arrived).
//
// The reference does these as separate NCCL all-gather / reduce-scatter calls around cuBLAS
// (infini_train/src/nn/parallel/tensor_parallel.cc:173-232, 270-370).
//
// Waits are bounded: a rank that gives up records a code in the status word and skips its work.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../kernels/gemm_pair_body.cuh"
#include "comm.h"

namespace itb {

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

namespace pair {

template <bool A_MN, bool B_MN>
static int launch_tp(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tc2,
                     const CUtensorMap& te, const GemmDev& p, const TpDev& tp, int pairs, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, true>;
  constexpr int smem = kSmemTotal + 1024;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  kern<<<2 * pairs, kThreads, smem, stream>>>(ta, tb, tc, tc2, te, p, tp);
  return static_cast<int>(cudaGetLastError());
}

__global__ void tp_wait_kernel(const int* arrive, const int* total, int world, int* err) {
  if (*static_cast<volatile int*>(err) != 0) return;
  if (threadIdx.x < world) {
    if (!tp_wait_ge(arrive + threadIdx.x, *total)) atomicCAS(err, 0, 124);
  }
}

}  // namespace pair
}  // namespace itb

static int tp_pairs(int M, int N) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = ((M + 255) / 256) * ((N + 255) / 256);
  const int max_pairs = sms / 2;
  return total < max_pairs ? total : max_pairs;
}

extern "C" int itb_tp_gemm_ctas(int M, int N) { return 2 * tp_pairs(M, N); }

extern "C" int itb_tp_gemm(const void* gemm, const ItbTpArgs* t, cudaStream_t stream) {
  const ItbGemmArgs* a = static_cast<const ItbGemmArgs*>(gemm);
  using namespace itb;
  using namespace itb::pair;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return -1;
  if (t->world < 2 || t->world > kTpMaxRanks || t->rank < 0 || t->rank >= t->world) return -3;
  if (t->Tl * t->world != t->T || t->batch * t->T != a->M || (t->Tl % 256)) return -4;
  if (a->flags & (kGemmOutF32 | kGemmAtomic | kGemmAccum)) return -5;
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) || (a->lda % 8) ||
      (a->ldb % 8))
    return -2;
  const bool scatter = t->mode & kTpScatter;
  if (scatter && ((a->N % 8) || (a->flags & (kGemmBias | kGemmResidual | kGemmGeluDual | kGemmDGelu)))) return -6;
  if ((t->mode & kTpPush) && (t->push_cols % 8)) return -7;

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
  p.split_k = 1;
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
  p.staged = 1;

  CUtensorMap tc = ta, tc2 = ta, te = ta;
  if (!scatter) {
    auto ok16 = [](const void* q, long long ld) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0 && ld % 8 == 0; };
    bool ok = ok16(a->C, a->ldc);
    if (a->flags & kGemmGeluDual) ok = ok && ok16(a->C2, a->ldc);
    if (a->flags & kGemmResidual) ok = ok && ok16(a->residual, a->ldr);
    if (a->flags & kGemmDGelu) ok = ok && ok16(a->aux, a->ld_aux);
    if (!ok) return -8;
    rc = make_tmap_bf16_2d(&tc, a->C, a->N, a->M, a->ldc, 64, 32);
    if (!rc && (a->flags & kGemmGeluDual)) rc = make_tmap_bf16_2d(&tc2, a->C2, a->N, a->M, a->ldc, 64, 32);
    if (!rc && (a->flags & kGemmResidual)) rc = make_tmap_bf16_2d(&te, a->residual, a->N, a->M, a->ldr, 64, 32);
    if (!rc && (a->flags & kGemmDGelu)) rc = make_tmap_bf16_2d(&te, a->aux, a->N, a->M, a->ld_aux, 64, 32);
    if (rc) return rc;
  }

  TpDev d;
  d.mode = t->mode;
  d.rank = t->rank;
  d.world = t->world;
  d.T = t->T;
  d.Tl = t->Tl;
  d.batch = t->batch;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    d.started[r] = static_cast<int*>(t->started.p[r]);
    d.gather[r] = static_cast<uint4*>(t->gather.p[r]);
    d.push_arrive[r] = static_cast<int*>(t->push_arrive.p[r]);
    d.slab[r] = static_cast<__nv_bfloat16*>(t->slab.p[r]);
    d.rs_arrive[r] = static_cast<int*>(t->rs_arrive.p[r]);
    d.ar_out[r] = static_cast<__nv_bfloat16*>(t->ar_out.p[r]);
    d.ar_arrive[r] = static_cast<int*>(t->ar_arrive.p[r]);
  }
  d.ar_mc = static_cast<uint4*>(t->ar_mc);
  d.ar_total = t->ar_total;
  d.ar_lag = t->ar_lag;
  if ((t->mode & kTpBroadcast) && (!scatter || !d.ar_total || !d.ar_out[0])) return -10;
  d.launch_ctr = t->launch_ctr;
  d.cta_done = t->cta_done;
  d.err = a->err;
  d.push_src = static_cast<const uint4*>(t->push_src);
  d.push_row_vecs = t->push_cols / 8;
  d.gather_mc = static_cast<uint4*>(t->gather_mc);
  d.push_total = t->push_total;
  d.push_lag = t->push_lag;
  d.gate_arrive = t->gate_arrive;
  d.gate_total = t->gate_total;
  d.gate_includes_this_launch = t->gate_includes_this_launch;
  d.rs_total = t->rs_total;
  d.rs_lag = t->rs_lag;
  d.rs_out = t->rs_out;
  d.rs_ld_out = t->rs_ld_out;
  d.rs_out_f32 = t->rs_out_f32;
  d.rs_bias = t->rs_bias;
  d.rs_residual = static_cast<const __nv_bfloat16*>(t->rs_residual);
  d.rs_ld_res = t->rs_ld_res;
  if (scatter && !(t->mode & kTpBroadcast) && ((reinterpret_cast<uintptr_t>(d.rs_out) & 15) || (d.rs_ld_out % 8) ||
                  (d.rs_residual && ((reinterpret_cast<uintptr_t>(d.rs_residual) & 15) || (d.rs_ld_res % 8)))))
    return -9;

  const int pairs = tp_pairs(a->M, a->N);
  const bool amn = a->a_mn_major, bmn = a->b_mn_major;
  if (!amn && !bmn) return launch_tp<false, false>(ta, tb, tc, tc2, te, p, d, pairs, stream);
  if (!amn && bmn) return launch_tp<false, true>(ta, tb, tc, tc2, te, p, d, pairs, stream);
  if (amn && bmn) return launch_tp<true, true>(ta, tb, tc, tc2, te, p, d, pairs, stream);
  return launch_tp<true, false>(ta, tb, tc, tc2, te, p, d, pairs, stream);
}

extern "C" int itb_tp_wait(const int* arrive, const int* total, int world, int* err, cudaStream_t stream) {
  itb::pair::tp_wait_kernel<<<1, 32, 0, stream>>>(arrive, total, world, err);
  return static_cast<int>(cudaGetLastError());
}
