// Fused optimizer updates over a flat buffer: Adam / AdamW and SGD with fp32 master weights, fp32
// or bf16 gradients, and an optional bf16 shadow copy of the weights written in the same pass (the
// copy the GEMMs read, so no separate cast kernel runs per forward).
//
// Reference behaviour covered: infini_train/src/kernels/cuda/accumulate_grad.cu:14-86 (one launch
// per parameter tensor, state in the parameter dtype, no weight decay).  Here the whole parameter
// set (or one ZeRO shard of it) is a single launch; weight_decay = 0 reproduces the reference's
// update rule  p -= lr * (m / bc1) / (sqrt(v / bc2) + eps).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace itb {

template <typename TG>
__device__ __forceinline__ float4 load_g4(const TG* g, long long i);
template <>
__device__ __forceinline__ float4 load_g4<float>(const float* g, long long i) {
  return *reinterpret_cast<const float4*>(g + i);
}
template <>
__device__ __forceinline__ float4 load_g4<__nv_bfloat16>(const __nv_bfloat16* g, long long i) {
  uint2 u = *reinterpret_cast<const uint2*>(g + i);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ float adam_one(float& p, float g, float& m, float& v, float lr, float b1,
                                          float b2, float eps, float wd, float inv_bc1,
                                          float inv_bc2) {
  m = b1 * m + (1.f - b1) * g;
  v = b2 * v + (1.f - b2) * g * g;
  const float mhat = m * inv_bc1;
  const float vhat = v * inv_bc2;
  p -= lr * (mhat / (sqrtf(vhat) + eps) + wd * p);
  return p;
}

template <typename TG>
__global__ void adamw_kernel(float* __restrict__ p, const TG* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n,
                             float lr, float b1, float b2, float eps, float wd, float inv_bc1,
                             float inv_bc2, float gscale, const float* __restrict__ dev_hyper) {
  // Hyper-parameters that change from step to step may live in device memory ([lr, 1/bc1, 1/bc2])
  // so that a captured CUDA graph can be replayed with new values.
  if (dev_hyper) {
    lr = dev_hyper[0];
    inv_bc1 = dev_hyper[1];
    inv_bc2 = dev_hyper[2];
  }
  const long long nvec = n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (long long i = tid; i < nvec; i += stride) {
    const long long o = i * 4;
    float4 pv = *reinterpret_cast<float4*>(p + o);
    float4 gv = load_g4<TG>(g, o);
    float4 mv = *reinterpret_cast<float4*>(m + o);
    float4 vv = *reinterpret_cast<float4*>(v + o);
    adam_one(pv.x, gv.x * gscale, mv.x, vv.x, lr, b1, b2, eps, wd, inv_bc1, inv_bc2);
    adam_one(pv.y, gv.y * gscale, mv.y, vv.y, lr, b1, b2, eps, wd, inv_bc1, inv_bc2);
    adam_one(pv.z, gv.z * gscale, mv.z, vv.z, lr, b1, b2, eps, wd, inv_bc1, inv_bc2);
    adam_one(pv.w, gv.w * gscale, mv.w, vv.w, lr, b1, b2, eps, wd, inv_bc1, inv_bc2);
    *reinterpret_cast<float4*>(p + o) = pv;
    *reinterpret_cast<float4*>(m + o) = mv;
    *reinterpret_cast<float4*>(v + o) = vv;
    if (shadow) {
      uint2 u;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
      h[0] = __floats2bfloat162_rn(pv.x, pv.y);
      h[1] = __floats2bfloat162_rn(pv.z, pv.w);
      *reinterpret_cast<uint2*>(shadow + o) = u;
    }
  }
  for (long long i = nvec * 4 + tid; i < n; i += stride) {
    float pv = p[i], mv = m[i], vv = v[i];
    float gv = static_cast<float>(g[i]) * gscale;
    adam_one(pv, gv, mv, vv, lr, b1, b2, eps, wd, inv_bc1, inv_bc2);
    p[i] = pv;
    m[i] = mv;
    v[i] = vv;
    if (shadow) shadow[i] = __float2bfloat16(pv);
  }
}

template <typename TG>
__global__ void sgd_kernel(float* __restrict__ p, const TG* __restrict__ g,
                           __nv_bfloat16* __restrict__ shadow, long long n, float lr, float gscale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += stride) {
    float pv = p[i] - lr * gscale * static_cast<float>(g[i]);
    p[i] = pv;
    if (shadow) shadow[i] = __float2bfloat16(pv);
  }
}

static inline int opt_grid(long long n) {
  long long b = (n / 4 + 255) / 256;
  const long long cap = 148LL * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace itb

using namespace itb;

extern "C" int itb_adamw(float* p, const void* g, int g_dtype, float* m, float* v,
                         void* shadow_bf16, long long n, float lr, float b1, float b2, float eps,
                         float wd, float bc1, float bc2, float grad_scale, const float* dev_hyper,
                         cudaStream_t s) {
  if (n <= 0) return 0;
  // Vector path needs 16-byte aligned fp32 buffers (8-byte for bf16 gradients / shadow).
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -2;
  if (g_dtype == kItbF32 && (reinterpret_cast<uintptr_t>(g) & 15)) return -2;
  if (g_dtype == kItbBF16 && (reinterpret_cast<uintptr_t>(g) & 7)) return -2;
  if (shadow_bf16 && (reinterpret_cast<uintptr_t>(shadow_bf16) & 7)) return -2;
  const int grid = opt_grid(n);
  if (g_dtype == kItbBF16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        p, static_cast<const __nv_bfloat16*>(g), m, v, static_cast<__nv_bfloat16*>(shadow_bf16), n,
        lr, b1, b2, eps, wd, 1.f / bc1, 1.f / bc2, grad_scale, dev_hyper);
  else
    adamw_kernel<float><<<grid, 256, 0, s>>>(p, static_cast<const float*>(g), m, v,
                                             static_cast<__nv_bfloat16*>(shadow_bf16), n, lr, b1,
                                             b2, eps, wd, 1.f / bc1, 1.f / bc2, grad_scale, dev_hyper);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_sgd(float* p, const void* g, int g_dtype, void* shadow_bf16, long long n,
                       float lr, float grad_scale, cudaStream_t s) {
  if (n <= 0) return 0;
  const int grid = opt_grid(n * 4);
  if (g_dtype == kItbBF16)
    sgd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p, static_cast<const __nv_bfloat16*>(g),
                                                   static_cast<__nv_bfloat16*>(shadow_bf16), n, lr,
                                                   grad_scale);
  else
    sgd_kernel<float><<<grid, 256, 0, s>>>(p, static_cast<const float*>(g),
                                           static_cast<__nv_bfloat16*>(shadow_bf16), n, lr,
                                           grad_scale);
  return static_cast<int>(cudaGetLastError());
}

// Device-resident Adam step state: hyper = [lr, 1/bc1, 1/bc2, t].  One thread advances t and
// recomputes the bias corrections, so that a whole training step (including this launch) can be
// captured once in a CUDA graph and replayed: nothing step-dependent comes from the host.
__global__ void adam_advance_kernel(float* __restrict__ hyper, float b1, float b2) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const double t = static_cast<double>(hyper[3]) + 1.0;
    hyper[3] = static_cast<float>(t);
    hyper[1] = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(b1), t)));
    hyper[2] = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(b2), t)));
  }
}

extern "C" int itb_adam_advance(float* hyper, float b1, float b2, cudaStream_t s) {
  adam_advance_kernel<<<1, 32, 0, s>>>(hyper, b1, b2);
  return static_cast<int>(cudaGetLastError());
}
