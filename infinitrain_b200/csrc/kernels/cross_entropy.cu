// Softmax cross-entropy over [rows, V] logits, forward (per-row loss, log-sum-exp, on-device mean)
// and backward (dlogits written over the logits buffer).
//
// Reference behaviour covered: infini_train/src/kernels/cuda/cross_entropy.cu:23-220 (three passes
// per row, per-row losses copied to the host and averaged there).  Here one block handles one row
// with an online max/sum (a single pass over the row), the mean is accumulated on the device, and
// the backward pass rewrites the logits in place so that no second [rows, V] buffer exists.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "kernels.h"

namespace itb {

constexpr int kCeThreads = 256;

template <typename T>
__device__ __forceinline__ void ce_load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void ce_load8<float>(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void ce_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ void ce_store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void ce_store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void ce_store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// Merge two (max, sum of exp relative to max) pairs.
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  float mn = fmaxf(m, m2);
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

// Per-row (max, sum-exp) over columns [0, V) of `row`; result valid in every thread.
template <typename T>
__device__ __forceinline__ void row_max_sum(const T* row, int V, float& m_out, float& s_out) {
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32];
  float m = -FLT_MAX, s = 0.f;
  const int nvec = V / 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(row) & (sizeof(T) * 8 - 1)) == 0;
  if (aligned) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float v[8];
      ce_load8<T>(row + i * 8, v);
      float lm = v[0];
#pragma unroll
      for (int e = 1; e < 8; ++e) lm = fmaxf(lm, v[e]);
      float mn = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += __expf(v[e] - mn);
      s = s * __expf(m - mn) + acc;
      m = mn;
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
      float x = static_cast<float>(row[i]);
      online_merge(m, s, x, 1.f);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float x = static_cast<float>(row[i]);
      online_merge(m, s, x, 1.f);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  m = sm[0];
  s = ss[0];
#pragma unroll
  for (int w = 1; w < kCeThreads / 32; ++w) online_merge(m, s, sm[w], ss[w]);
  __syncthreads();
  m_out = m;
  s_out = s;
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ target,
              float* __restrict__ row_loss, float* __restrict__ lse_out,
              float* __restrict__ loss_mean, int rows, int V) {
  const int r = blockIdx.x;
  const T* row = logits + static_cast<long long>(r) * ld;
  float m, s;
  row_max_sum<T>(row, V, m, s);
  if (threadIdx.x == 0) {
    const float lse = m + __logf(s);
    const long long t = target[r];
    float loss = 0.f;
    if (t >= 0 && t < V) loss = lse - static_cast<float>(row[t]);
    if (row_loss) row_loss[r] = loss;
    lse_out[r] = lse;
    if (loss_mean) atomicAdd(loss_mean, loss / rows);
  }
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_bwd_kernel(T* __restrict__ logits, long long ld, const long long* __restrict__ target,
              const float* __restrict__ lse, const float* __restrict__ grad_out, int rows, int V,
              int ignore_oob) {
  const int r = blockIdx.x;
  T* row = logits + static_cast<long long>(r) * ld;
  const long long t = target[r];
  const bool valid = t >= 0 && t < V;
  // ignore_oob: a row whose target is out of range contributes nothing (ignored label).
  // Otherwise (vocabulary-parallel shard) the row still receives the softmax term; only the
  // one-hot term is absent because another shard owns the target column.
  const float g = (valid || !ignore_oob) ? (grad_out ? *grad_out : 1.f) / rows : 0.f;
  const float l = lse[r];
  const int ldi = static_cast<int>(ld);
  const int nvec = V / 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(row) & (sizeof(T) * 8 - 1)) == 0;
  if (aligned) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float v[8];
      ce_load8<T>(row + i * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float p = __expf(v[e] - l);
        v[e] = (p - ((i * 8 + e) == t ? 1.f : 0.f)) * g;
      }
      ce_store8<T>(row + i * 8, v);
    }
    for (int i = nvec * 8 + threadIdx.x; i < ldi; i += blockDim.x) {
      float o = 0.f;
      if (i < V) o = (__expf(static_cast<float>(row[i]) - l) - (i == t ? 1.f : 0.f)) * g;
      row[i] = static_cast<T>(o);
    }
  } else {
    for (int i = threadIdx.x; i < ldi; i += blockDim.x) {
      float o = 0.f;
      if (i < V) o = (__expf(static_cast<float>(row[i]) - l) - (i == t ? 1.f : 0.f)) * g;
      row[i] = static_cast<T>(o);
    }
  }
}

}  // namespace itb

using namespace itb;

extern "C" int itb_ce_fwd(const void* logits, int dtype, long long ld, const long long* target,
                          float* row_loss, float* lse, float* loss_mean, int rows, int V,
                          cudaStream_t s) {
  if (rows <= 0) return 0;
  if (dtype == kItbBF16)
    ce_fwd_kernel<__nv_bfloat16><<<rows, kCeThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, target, row_loss, lse, loss_mean, rows, V);
  else
    ce_fwd_kernel<float><<<rows, kCeThreads, 0, s>>>(static_cast<const float*>(logits), ld, target,
                                                     row_loss, lse, loss_mean, rows, V);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_ce_bwd(void* logits, int dtype, long long ld, const long long* target,
                          const float* lse, const float* grad_out, int rows, int V, int ignore_oob,
                          cudaStream_t s) {
  if (rows <= 0) return 0;
  if (dtype == kItbBF16)
    ce_bwd_kernel<__nv_bfloat16><<<rows, kCeThreads, 0, s>>>(static_cast<__nv_bfloat16*>(logits), ld,
                                                             target, lse, grad_out, rows, V, ignore_oob);
  else
    ce_bwd_kernel<float><<<rows, kCeThreads, 0, s>>>(static_cast<float*>(logits), ld, target, lse,
                                                     grad_out, rows, V, ignore_oob);
  return static_cast<int>(cudaGetLastError());
}
