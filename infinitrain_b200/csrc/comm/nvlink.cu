// Collectives written as CUDA kernels that move data over NVLink / NVSwitch themselves, fused with
// the arithmetic that surrounds them.  Every rank launches the same kernel on its own GPU; the
// buffers live in symmetric memory (same allocation on every rank, peer-mapped, plus an NVLS
// multicast mapping when the switch offers one).
//
//   * all-reduce(avg) of a gradient bucket in place                      (DDP reducer, ZeRO-0)
//   * reduce-scatter + scale + AdamW on the owner shard + broadcast of the updated fp32 weights and
//     their bf16 shadow to every rank                                     (ZeRO-1/2 optimizer step)
//
// The reference issues ncclAllReduce / ncclReduceScatter / ncclAllGather from the host on a side
// stream and runs Adam as separate per-tensor launches (infini_train/src/nn/parallel/
// process_group.cc:128-195, ddp/param_and_grad_buffer.cc:237-378, src/optimizer.cc:53-71).
//
// Two data paths, chosen per launch: `multimem` (multimem.ld_reduce sums the value of every rank
// inside the switch, multimem.st writes to every rank at once) and plain peer pointers (each rank
// reads its slice from every peer and stores the result to every peer).
//
// Ranks synchronise through flag words in symmetric memory: block b of rank r writes the launch's
// epoch into slot [b][r] of every peer and waits until its own slots [b][*] have reached that
// epoch.  Epochs only grow, so no flag is ever reset.  Every wait is bounded: when it gives up the
// block records an error code in the status word and skips its work; the host checks the word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.h"

namespace itb {

constexpr int kCommThreads = 512;
#ifndef ITB_AR_UNROLL
#define ITB_AR_UNROLL 8
#endif
#ifndef ITB_ZERO_UNROLL
#define ITB_ZERO_UNROLL 2
#endif
constexpr int kArUnroll = ITB_AR_UNROLL;       // 16-byte reductions in flight per thread (all-reduce)
constexpr int kZeroUnroll = ITB_ZERO_UNROLL;   // 32-byte chunks in flight per thread (ZeRO step)
// ~2^24 polls with a short sleep: of the order of a few seconds of skew tolerated between ranks.
constexpr unsigned kSpinLimit = 1u << 24;

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-wide barrier across ranks on channel `ch`.  Returns false when a peer did not arrive.
__device__ __forceinline__ bool rank_barrier(const ItbPeerPtrs& flags, int rank, int world, int ch,
                                             int epoch, int* err, int code) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();  // also orders this block's earlier memory traffic before the signal below
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(static_cast<int*>(flags.p[peer]) + ch * kItbMaxRanks + rank, epoch);
    const int* mine = static_cast<const int*>(flags.p[rank]) + ch * kItbMaxRanks + peer;
    bool ok = false;
    for (unsigned i = 0; i < kSpinLimit; ++i) {
      if (ld_acquire_sys(mine) - epoch >= 0) {
        ok = true;
        break;
      }
      if (i > 32) __nanosleep(100);
    }
    if (!ok) {
      atomicCAS(err, 0, code);
      ok_flag = 0;
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

__device__ __forceinline__ float4 mm_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_f32x4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void mm_st_bf16x8(__nv_bfloat16* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

template <bool kMC>
__device__ __forceinline__ float4 reduce4(const ItbPeerPtrs& bufs, const float* mc, long long i,
                                          int world) {
  if (kMC) return mm_ld_reduce_f32x4(mc + i);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
  for (int r = 0; r < world; ++r) {
    const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(bufs.p[r]) + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  return acc;
}
template <bool kMC>
__device__ __forceinline__ void bcast4(const ItbPeerPtrs& bufs, float* mc, long long i, int world,
                                       float4 v) {
  if (kMC) {
    mm_st_f32x4(mc + i, v);
  } else {
#pragma unroll 1
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<float4*>(static_cast<float*>(bufs.p[r]) + i) = v;
  }
}

// ------------------------------------------------------------------ all-reduce (average)
// In place on elements [off, off + n) of a symmetric fp32 buffer; n and off multiples of 4.
template <bool kMC>
__global__ void __launch_bounds__(kCommThreads)
allreduce_scale_kernel(ItbPeerPtrs bufs, float* mc, ItbPeerPtrs flags, long long off, long long n,
                       int rank, int world, int ch0, int epoch, float scale, int* err,
                       int* __restrict__ epoch_ctr) {
  // an earlier launch gave up on a peer: the flags are no longer in step, do not wait again
  if (*static_cast<volatile int*>(err) != 0) return;
  const int ch = ch0 + blockIdx.x;
  // Device-side epoch (one counter per channel, private to this GPU): lets a captured CUDA graph
  // replay the launch; every rank's counter advances in lockstep because every rank replays the
  // same launches.
  if (epoch_ctr) epoch = epoch_ctr[ch] + 1;
  if (!rank_barrier(flags, rank, world, ch, epoch, err, 201)) return;
  // slice of this rank, in units of 4 elements
  const long long nv = n / 4;
  const long long per = (nv + world - 1) / world;
  const long long v0 = min(nv, per * rank), v1 = min(nv, v0 + per);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // A reduction through the switch (or a round of peer loads) takes microseconds to come back:
  // every thread keeps kArUnroll of them in flight before it touches the first result.
  for (long long v = v0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < v1;
       v += stride * kArUnroll) {
    float4 s[kArUnroll];
#pragma unroll
    for (int u = 0; u < kArUnroll; ++u) {
      const long long vu = v + u * stride;
      if (vu < v1) s[u] = reduce4<kMC>(bufs, mc, off + vu * 4, world);
    }
#pragma unroll
    for (int u = 0; u < kArUnroll; ++u) {
      const long long vu = v + u * stride;
      if (vu < v1) {
        s[u].x *= scale; s[u].y *= scale; s[u].z *= scale; s[u].w *= scale;
        bcast4<kMC>(bufs, mc, off + vu * 4, world, s[u]);
      }
    }
  }
  rank_barrier(flags, rank, world, ch, epoch + 1, err, 202);
  if (epoch_ctr && threadIdx.x == 0) epoch_ctr[ch] = epoch + 1;
}

// ------------------------------------------------------------------ reduce-scatter + AdamW + broadcast
// Bucket = elements [off, off + n) of the symmetric gradient / parameter / shadow buffers; rank r
// owns [off + r n / world, off + (r+1) n / world).  m and v hold the owner shard only.
template <bool kMC>
__global__ void __launch_bounds__(kCommThreads)
rs_adamw_bcast_kernel(ItbPeerPtrs grads, const float* mc_grads, ItbPeerPtrs params, float* mc_params,
                      ItbPeerPtrs shadows, __nv_bfloat16* mc_shadows, float* __restrict__ m,
                      float* __restrict__ v, ItbPeerPtrs flags, long long off, long long n, int rank,
                      int world, int ch0, int epoch, ItbAdamHyper h, int* err,
                      int* __restrict__ epoch_ctr, const float* __restrict__ dev_hyper) {
  if (*static_cast<volatile int*>(err) != 0) return;
  const int ch = ch0 + blockIdx.x;
  if (epoch_ctr) epoch = epoch_ctr[ch] + 1;
  if (dev_hyper) {   // [lr, 1/bc1, 1/bc2] refreshed by the host before every graph replay
    h.lr = dev_hyper[0];
    h.inv_bc1 = dev_hyper[1];
    h.inv_bc2 = dev_hyper[2];
  }
  if (!rank_barrier(flags, rank, world, ch, epoch, err, 203)) return;
  const long long shard = n / world;           // multiple of 8 by construction of the buckets
  const long long s0 = off + shard * rank;
  const long long nv = shard / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const float* my_params = static_cast<const float*>(params.p[rank]);
  // kZeroUnroll chunks of 8 elements per thread and pass: the gradient reductions and the local
  // loads of all of them are issued before the arithmetic of the first
  for (long long k0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; k0 < nv;
       k0 += stride * kZeroUnroll) {
    float g[kZeroUnroll][8], p[kZeroUnroll][8], mm[kZeroUnroll][8], vv[kZeroUnroll][8];
#pragma unroll
    for (int u = 0; u < kZeroUnroll; ++u) {
      const long long k = k0 + u * stride;
      if (k < nv) {
        const long long i = s0 + k * 8;   // index in the flat buffers
        const long long j = k * 8;        // index in the shard-local state
        *reinterpret_cast<float4*>(g[u]) = reduce4<kMC>(grads, mc_grads, i, world);
        *reinterpret_cast<float4*>(g[u] + 4) = reduce4<kMC>(grads, mc_grads, i + 4, world);
        *reinterpret_cast<float4*>(p[u]) = *reinterpret_cast<const float4*>(my_params + i);
        *reinterpret_cast<float4*>(p[u] + 4) = *reinterpret_cast<const float4*>(my_params + i + 4);
        *reinterpret_cast<float4*>(mm[u]) = *reinterpret_cast<const float4*>(m + j);
        *reinterpret_cast<float4*>(mm[u] + 4) = *reinterpret_cast<const float4*>(m + j + 4);
        *reinterpret_cast<float4*>(vv[u]) = *reinterpret_cast<const float4*>(v + j);
        *reinterpret_cast<float4*>(vv[u] + 4) = *reinterpret_cast<const float4*>(v + j + 4);
      }
    }
#pragma unroll
    for (int u = 0; u < kZeroUnroll; ++u) {
      const long long k = k0 + u * stride;
      if (k >= nv) continue;
      const long long i = s0 + k * 8;
      const long long j = k * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float ge = g[u][e] * h.grad_scale;
        mm[u][e] = h.beta1 * mm[u][e] + (1.f - h.beta1) * ge;
        vv[u][e] = h.beta2 * vv[u][e] + (1.f - h.beta2) * ge * ge;
        const float mhat = mm[u][e] * h.inv_bc1, vhat = vv[u][e] * h.inv_bc2;
        p[u][e] -= h.lr * (mhat / (sqrtf(vhat) + h.eps) + h.weight_decay * p[u][e]);
      }
      *reinterpret_cast<float4*>(m + j) = *reinterpret_cast<float4*>(mm[u]);
      *reinterpret_cast<float4*>(m + j + 4) = *reinterpret_cast<float4*>(mm[u] + 4);
      *reinterpret_cast<float4*>(v + j) = *reinterpret_cast<float4*>(vv[u]);
      *reinterpret_cast<float4*>(v + j + 4) = *reinterpret_cast<float4*>(vv[u] + 4);
      bcast4<kMC>(params, mc_params, i, world, *reinterpret_cast<float4*>(p[u]));
      bcast4<kMC>(params, mc_params, i + 4, world, *reinterpret_cast<float4*>(p[u] + 4));
      uint4 sh;
      __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&sh);
#pragma unroll
      for (int e = 0; e < 4; ++e) hb[e] = __floats2bfloat162_rn(p[u][2 * e], p[u][2 * e + 1]);
      if (kMC) {
        mm_st_bf16x8(mc_shadows + i, sh);
      } else {
#pragma unroll 1
        for (int r = 0; r < world; ++r)
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(shadows.p[r]) + i) = sh;
      }
    }
  }
  rank_barrier(flags, rank, world, ch, epoch + 1, err, 204);
  if (epoch_ctr && threadIdx.x == 0) epoch_ctr[ch] = epoch + 1;
}

// ------------------------------------------------------------------ vocab-parallel cross-entropy merge
// Every rank holds, per token row, the log-sum-exp of its vocabulary shard and (if it owns the
// target column) the target logit.  Block b handles a slice of the rows: it stores its (lse, target)
// pairs into slot [rank] of every rank's symmetric buffer, meets the same block of the other ranks
// at a flag barrier, merges the `world` pairs of each of its rows into the global log-sum-exp and
// the row loss, and meets them again so that nobody overwrites pairs that are still being read.
// Replaces the reference's three all-reduces (max, sum-exp, predicted logit) and ~20 elementwise
// launches (infini_train/src/nn/parallel/tensor_parallel.cc:436-541) by this one launch after the
// local pass over the logits.
__global__ void __launch_bounds__(kCommThreads)
ce_merge_kernel(ItbPeerPtrs bufs, ItbPeerPtrs flags, const float* __restrict__ lse_local,
                const float* __restrict__ row_loss, const long long* __restrict__ t_local, int vocab_valid,
                float* __restrict__ lse_out, float* __restrict__ loss_out, int rows, int rows_cap, int rank,
                int world, int ch0, int* err, int* __restrict__ epoch_ctr) {
  if (*static_cast<volatile int*>(err) != 0) return;
  const int ch = ch0 + blockIdx.x;
  const int epoch = epoch_ctr[ch] + 1;
  const int chunk = (rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * chunk, r1 = min(rows, r0 + chunk);
  for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
    const long long t = t_local[r];
    const float l = lse_local[r];
    const float2 v = make_float2(l, (t >= 0 && t < vocab_valid) ? l - row_loss[r] : 0.f);
    for (int p = 0; p < world; ++p)
      static_cast<float2*>(bufs.p[(rank + p) % world])[static_cast<long long>(rank) * rows_cap + r] = v;
  }
  if (!rank_barrier(flags, rank, world, ch, epoch, err, 301)) return;
  const float2* mine = static_cast<const float2*>(bufs.p[rank]);
  for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
    float m = -INFINITY, tg = 0.f;
    for (int w = 0; w < world; ++w) {
      const float2 v = __ldcg(mine + static_cast<long long>(w) * rows_cap + r);
      m = fmaxf(m, v.x);
      tg += v.y;
    }
    float s = 0.f;
    for (int w = 0; w < world; ++w) s += __expf(__ldcg(mine + static_cast<long long>(w) * rows_cap + r).x - m);
    const float lse = m + __logf(s);
    lse_out[r] = lse;
    loss_out[r] = lse - tg;
  }
  rank_barrier(flags, rank, world, ch, epoch + 1, err, 302);
  if (threadIdx.x == 0) epoch_ctr[ch] = epoch + 1;
}

}  // namespace itb

using namespace itb;

extern "C" int itb_nvl_ce_merge(const ItbPeerPtrs* bufs, const ItbPeerPtrs* flags, const float* lse_local,
                                const float* row_loss, const long long* t_local, int vocab_valid,
                                float* lse_out, float* loss_out, int rows, int rows_cap, int rank, int world,
                                int ch0, int* err, int* epoch_ctr, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (world < 1 || world > kItbMaxRanks || rows > rows_cap || !epoch_ctr) return -4;
  int blocks = (rows + kCommThreads - 1) / kCommThreads;
  if (blocks > kItbMaxCommBlocks) blocks = kItbMaxCommBlocks;
  ce_merge_kernel<<<blocks, kCommThreads, 0, s>>>(*bufs, *flags, lse_local, row_loss, t_local, vocab_valid, lse_out,
                                                  loss_out, rows, rows_cap, rank, world, ch0, err, epoch_ctr);
  return static_cast<int>(cudaGetLastError());
}

// The bounded wait of the flag protocols on its own: one thread polls `flag` until it has reached
// `target` or `limit` polls have passed; on a time-out it records `code` in the status word and
// returns.  Lets the host-visible error path be exercised on a single GPU with a flag that nothing
// sets, without any peer and without hanging anything.
__global__ void wait_flag_kernel(const int* flag, int target, unsigned limit, int code, int* err) {
  bool ok = false;
  for (unsigned i = 0; i < limit; ++i) {
    if (ld_acquire_sys(flag) - target >= 0) {
      ok = true;
      break;
    }
    if (i > 32) __nanosleep(100);
  }
  if (!ok) atomicCAS(err, 0, code);
}

extern "C" int itb_wait_flag(const int* flag, int target, unsigned limit, int code, int* err,
                             cudaStream_t stream) {
  wait_flag_kernel<<<1, 1, 0, stream>>>(flag, target, limit, code, err);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_comm_blocks(long long n_elements_per_rank) {
  long long b = (n_elements_per_rank / 4 + kCommThreads - 1) / kCommThreads;
  if (b < 1) b = 1;
  if (b > kItbMaxCommBlocks) b = kItbMaxCommBlocks;
  return static_cast<int>(b);
}

extern "C" int itb_nvl_allreduce_scale(const ItbPeerPtrs* bufs, void* mc, const ItbPeerPtrs* flags,
                                       long long off, long long n, int rank, int world, int ch0,
                                       int epoch, float scale, int* err, int* epoch_ctr,
                                       cudaStream_t s) {
  if (n <= 0) return 0;
  if ((off | n) & 3) return -3;
  if (world < 1 || world > kItbMaxRanks) return -4;
  const int blocks = itb_comm_blocks((n + world - 1) / world);
  if (mc)
    allreduce_scale_kernel<true><<<blocks, kCommThreads, 0, s>>>(
        *bufs, static_cast<float*>(mc), *flags, off, n, rank, world, ch0, epoch, scale, err, epoch_ctr);
  else
    allreduce_scale_kernel<false><<<blocks, kCommThreads, 0, s>>>(
        *bufs, nullptr, *flags, off, n, rank, world, ch0, epoch, scale, err, epoch_ctr);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_nvl_rs_adamw_bcast(const ItbPeerPtrs* grads, const void* mc_grads,
                                      const ItbPeerPtrs* params, void* mc_params,
                                      const ItbPeerPtrs* shadows, void* mc_shadows, float* m, float* v,
                                      const ItbPeerPtrs* flags, long long off, long long n, int rank,
                                      int world, int ch0, int epoch, const ItbAdamHyper* h, int* err,
                                      int* epoch_ctr, const float* dev_hyper, cudaStream_t s) {
  if (n <= 0) return 0;
  if (world < 1 || world > kItbMaxRanks) return -4;
  if (n % (8LL * world) || (off & 7)) return -3;
  const bool mc = mc_grads && mc_params && mc_shadows;
  const int blocks = itb_comm_blocks(n / world / 2);
  if (mc)
    rs_adamw_bcast_kernel<true><<<blocks, kCommThreads, 0, s>>>(
        *grads, static_cast<const float*>(mc_grads), *params, static_cast<float*>(mc_params),
        *shadows, static_cast<__nv_bfloat16*>(mc_shadows), m, v, *flags, off, n, rank, world, ch0,
        epoch, *h, err, epoch_ctr, dev_hyper);
  else
    rs_adamw_bcast_kernel<false><<<blocks, kCommThreads, 0, s>>>(
        *grads, nullptr, *params, nullptr, *shadows, nullptr, m, v, *flags, off, n, rank, world, ch0,
        epoch, *h, err, epoch_ctr, dev_hyper);
  return static_cast<int>(cudaGetLastError());
}
