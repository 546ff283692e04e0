// LayerNorm and RMSNorm, forward and backward, for rows of a [rows, C] matrix (bf16 or fp32 in and
// out, statistics and parameter gradients in fp32).
//
// Reference behaviour covered: infini_train/src/kernels/cuda/layernorm.cu:15-199 (one block per
// token, atomics into dW/db from every token) and the seven-launch composed RMSNorm of
// infini_train/src/nn/modules/normalization.cc:35-45.  Here: one warp per row with 16-byte loads,
// the row kept in registers between the statistics pass and the output pass, a two-pass variance
// (E[(x-mean)^2]), and parameter gradients reduced in two stages without atomics: every block
// writes one fp32 partial row, a second kernel sums the partial rows.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace itb {

constexpr int kNormWarps = 4;           // rows per block in flight
constexpr int kNormThreads = kNormWarps * 32;
constexpr int kMaxPartialRows = 592;    // 4 blocks per SM on 148 SMs

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Load / store 8 consecutive elements (C is required to be a multiple of 8).
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
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
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// Rows up to kMaxVec*256 elements wide stay in registers (kMaxVec chunks of 8 per lane); the part
// of a wider row beyond that is re-read from global memory.  kMaxVec is a template parameter so
// that narrow rows (GPT-2: 768) do not pay the register cost of wide ones.

template <typename TX, typename TY, bool kRms, int kMaxVec>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ gamma,
                const float* __restrict__ beta, TY* __restrict__ y, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int rows, int C, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C / 8;
  for (int row = blockIdx.x * kNormWarps + warp; row < rows; row += gridDim.x * kNormWarps) {
    const TX* xr = x + static_cast<long long>(row) * C;
    TY* yr = y + static_cast<long long>(row) * C;
    float cache[kMaxVec][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) {
        load8<TX>(xr + vi * 8, cache[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += kRms ? cache[i][e] * cache[i][e] : cache[i][e];
      }
    }
    for (int vi = lane + kMaxVec * 32; vi < nvec; vi += 32) {
      float t[8];
      load8<TX>(xr + vi * 8, t);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += kRms ? t[e] * t[e] : t[e];
    }
    sum = warp_sum(sum);
    float mean = 0.f, rstd;
    if (kRms) {
      rstd = rsqrtf(sum / C + eps);
    } else {
      mean = sum / C;
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        int vi = lane + i * 32;
        if (vi < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float d = cache[i][e] - mean;
            var += d * d;
          }
        }
      }
      for (int vi = lane + kMaxVec * 32; vi < nvec; vi += 32) {
        float t[8];
        load8<TX>(xr + vi * 8, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float d = t[e] - mean;
          var += d * d;
        }
      }
      var = warp_sum(var);
      rstd = rsqrtf(var / C + eps);
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    auto emit = [&](int vi, float (&xv)[8]) {
      float g[8], o[8];
      load8<float>(gamma + vi * 8, g);
      if (!kRms && beta) {
        float b[8];
        load8<float>(beta + vi * 8, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (xv[e] - mean) * rstd * g[e] + b[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (xv[e] - mean) * rstd * g[e];
      }
      store8<TY>(yr + vi * 8, o);
    };
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) emit(vi, cache[i]);
    }
    for (int vi = lane + kMaxVec * 32; vi < nvec; vi += 32) {
      float t[8];
      load8<TX>(xr + vi * 8, t);
      emit(vi, t);
    }
  }
}

// Backward.  With xhat = (x - mean) * rstd and g = dy * gamma:
//   LayerNorm: dx = rstd * (g - mean_C(g) - xhat * mean_C(g * xhat))
//   RMSNorm:   dx = rstd * (g - xhat * mean_C(g * xhat))                    (mean = 0)
// dgamma += dy * xhat, dbeta += dy, accumulated per block in shared memory (fp32 atomics on shared
// memory only), then written as one partial row per block.
template <typename TDY, typename TX, typename TDX, bool kRms, int kMaxVec>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x,
                const float* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, TDX* __restrict__ dx,
                float* __restrict__ partial, int rows, int C) {
  extern __shared__ float sh[];  // [2*C]: dgamma | dbeta (dbeta unused for RMSNorm)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C / 8;
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) sh[i] = 0.f;
  __syncthreads();
  // Per-lane register accumulators for the first kMaxVec chunks: summed over this warp's rows,
  // flushed to shared memory once at the end.
  float acc_g[kMaxVec][8], acc_b[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc_g[i][e] = acc_b[i][e] = 0.f;

  for (int row = blockIdx.x * kNormWarps + warp; row < rows; row += gridDim.x * kNormWarps) {
    const TDY* dyr = dy + static_cast<long long>(row) * C;
    const TX* xr = x + static_cast<long long>(row) * C;
    TDX* dxr = dx + static_cast<long long>(row) * C;
    const float mean = kRms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) {
        float d[8], xv[8], g[8];
        load8<TDY>(dyr + vi * 8, d);
        load8<TX>(xr + vi * 8, xv);
        load8<float>(gamma + vi * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float xhat = (xv[e] - mean) * rstd;
          float gg = d[e] * g[e];
          s1 += gg;
          s2 += gg * xhat;
          acc_g[i][e] += d[e] * xhat;
          acc_b[i][e] += d[e];
        }
      }
    }
    for (int vi = lane + kMaxVec * 32; vi < nvec; vi += 32) {
      float d[8], xv[8], g[8];
      load8<TDY>(dyr + vi * 8, d);
      load8<TX>(xr + vi * 8, xv);
      load8<float>(gamma + vi * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float xhat = (xv[e] - mean) * rstd;
        float gg = d[e] * g[e];
        s1 += gg;
        s2 += gg * xhat;
        atomicAdd(&sh[vi * 8 + e], d[e] * xhat);
        if (!kRms) atomicAdd(&sh[C + vi * 8 + e], d[e]);
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
    if (kRms) s1 = 0.f;
    // Second pass re-reads the row (it is in L1 / L2 from the first pass) instead of holding it in
    // registers: the kernel is bound by loads in flight, so occupancy matters more than the re-read.
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int vi = lane + i * 32;
      if (vi < nvec) {
        float d[8], xv[8], g[8], o[8];
        load8<TDY>(dyr + vi * 8, d);
        load8<TX>(xr + vi * 8, xv);
        load8<float>(gamma + vi * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float xhat = (xv[e] - mean) * rstd;
          o[e] = rstd * (d[e] * g[e] - s1 - xhat * s2);
        }
        store8<TDX>(dxr + vi * 8, o);
      }
    }
    for (int vi = lane + kMaxVec * 32; vi < nvec; vi += 32) {
      float d[8], xv[8], g[8], o[8];
      load8<TDY>(dyr + vi * 8, d);
      load8<TX>(xr + vi * 8, xv);
      load8<float>(gamma + vi * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float xhat = (xv[e] - mean) * rstd;
        o[e] = rstd * (d[e] * g[e] - s1 - xhat * s2);
      }
      store8<TDX>(dxr + vi * 8, o);
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    int vi = lane + i * 32;
    if (vi < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        atomicAdd(&sh[vi * 8 + e], acc_g[i][e]);
        if (!kRms) atomicAdd(&sh[C + vi * 8 + e], acc_b[i][e]);
      }
    }
  }
  __syncthreads();
  float* prow = partial + static_cast<long long>(blockIdx.x) * 2 * C;
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) prow[i] = sh[i];
}

// out[c] (+)= sum_r partial[r, c]: a block of 32 columns x 8 row lanes; the row lanes are combined
// in shared memory.
__global__ void __launch_bounds__(256)
partial_reduce_kernel(const float* __restrict__ partial, int prow_stride, int nrows,
                      float* __restrict__ out_a, float* __restrict__ out_b, int C, int accumulate) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < 2 * C)
    for (int r = ry; r < nrows; r += 8) s += partial[static_cast<long long>(r) * prow_stride + c];
  sh[ry][cx] = s;
  __syncthreads();
  if (ry != 0 || c >= 2 * C) return;
  float t = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) t += sh[r][cx];
  float* out = c < C ? out_a : out_b;
  if (!out) return;
  const int oc = c < C ? c : c - C;
  out[oc] = accumulate ? out[oc] + t : t;
}

static int norm_grid(int rows) {
  int blocks = (rows + kNormWarps - 1) / kNormWarps;
  return blocks < kMaxPartialRows ? blocks : kMaxPartialRows;
}

template <bool kRms>
static int norm_fwd_dispatch(const void* x, int xd, const float* gamma, const float* beta, void* y,
                             int yd, float* mean, float* rstd, int rows, int C, float eps,
                             cudaStream_t s) {
  if (C % 8) return -3;
  int grid = (rows + kNormWarps - 1) / kNormWarps;
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) return 0;
#define LAUNCH(TX, TY)                                                                           \
  do {                                                                                           \
    if (C <= 1024)                                                                               \
      norm_fwd_kernel<TX, TY, kRms, 4><<<grid, kNormThreads, 0, s>>>(                            \
          static_cast<const TX*>(x), gamma, beta, static_cast<TY*>(y), mean, rstd, rows, C, eps); \
    else                                                                                         \
      norm_fwd_kernel<TX, TY, kRms, 8><<<grid, kNormThreads, 0, s>>>(                            \
          static_cast<const TX*>(x), gamma, beta, static_cast<TY*>(y), mean, rstd, rows, C, eps); \
  } while (0)
  if (xd == kItbBF16 && yd == kItbBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (xd == kItbF32 && yd == kItbBF16) LAUNCH(float, __nv_bfloat16);
  else if (xd == kItbF32 && yd == kItbF32) LAUNCH(float, float);
  else if (xd == kItbBF16 && yd == kItbF32) LAUNCH(__nv_bfloat16, float);
  else return -4;
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

template <bool kRms>
static int norm_bwd_dispatch(const void* dy, int dyd, const void* x, int xd, const float* gamma,
                             const float* mean, const float* rstd, void* dx, int dxd,
                             float* dgamma, float* dbeta, float* partial, int rows, int C,
                             int accumulate, cudaStream_t s) {
  if (C % 8) return -3;
  if (rows < 1) return 0;
  const int grid = norm_grid(rows);
  const int smem = 2 * C * sizeof(float);
  if (smem > 48 * 1024) return -5;
#define LAUNCH(TDY, TX, TDX)                                                                     \
  do {                                                                                           \
    if (C <= 768)                                                                                \
      norm_bwd_kernel<TDY, TX, TDX, kRms, 3><<<grid, kNormThreads, smem, s>>>(                   \
          static_cast<const TDY*>(dy), static_cast<const TX*>(x), gamma, mean, rstd,             \
          static_cast<TDX*>(dx), partial, rows, C);                                              \
    else if (C <= 1024)                                                                          \
      norm_bwd_kernel<TDY, TX, TDX, kRms, 4><<<grid, kNormThreads, smem, s>>>(                   \
          static_cast<const TDY*>(dy), static_cast<const TX*>(x), gamma, mean, rstd,             \
          static_cast<TDX*>(dx), partial, rows, C);                                              \
    else                                                                                         \
      norm_bwd_kernel<TDY, TX, TDX, kRms, 8><<<grid, kNormThreads, smem, s>>>(                   \
          static_cast<const TDY*>(dy), static_cast<const TX*>(x), gamma, mean, rstd,             \
          static_cast<TDX*>(dx), partial, rows, C);                                              \
  } while (0)
  if (dyd == kItbBF16 && xd == kItbBF16 && dxd == kItbBF16)
    LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (dyd == kItbBF16 && xd == kItbF32 && dxd == kItbF32) LAUNCH(__nv_bfloat16, float, float);
  else if (dyd == kItbF32 && xd == kItbF32 && dxd == kItbF32) LAUNCH(float, float, float);
  else if (dyd == kItbBF16 && xd == kItbBF16 && dxd == kItbF32)
    LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
  else if (dyd == kItbF32 && xd == kItbBF16 && dxd == kItbBF16)
    LAUNCH(float, __nv_bfloat16, __nv_bfloat16);
  else return -4;
#undef LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  partial_reduce_kernel<<<(2 * C + 31) / 32, 256, 0, s>>>(partial, 2 * C, grid, dgamma, dbeta, C,
                                                           accumulate);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace itb

extern "C" int itb_norm_partial_rows(int rows) { return itb::norm_grid(rows); }

extern "C" int itb_layernorm_fwd(const void* x, int x_dtype, const float* gamma, const float* beta,
                                 void* y, int y_dtype, float* mean, float* rstd, int rows, int C,
                                 float eps, cudaStream_t stream) {
  return itb::norm_fwd_dispatch<false>(x, x_dtype, gamma, beta, y, y_dtype, mean, rstd, rows, C,
                                       eps, stream);
}
extern "C" int itb_layernorm_bwd(const void* dy, int dy_dtype, const void* x, int x_dtype,
                                 const float* gamma, const float* mean, const float* rstd, void* dx,
                                 int dx_dtype, float* dgamma, float* dbeta, float* partial,
                                 int rows, int C, int accumulate, cudaStream_t stream) {
  return itb::norm_bwd_dispatch<false>(dy, dy_dtype, x, x_dtype, gamma, mean, rstd, dx, dx_dtype,
                                       dgamma, dbeta, partial, rows, C, accumulate, stream);
}
extern "C" int itb_rmsnorm_fwd(const void* x, int x_dtype, const float* gamma, void* y, int y_dtype,
                               float* rstd, int rows, int C, float eps, cudaStream_t stream) {
  return itb::norm_fwd_dispatch<true>(x, x_dtype, gamma, nullptr, y, y_dtype, nullptr, rstd, rows,
                                      C, eps, stream);
}
extern "C" int itb_rmsnorm_bwd(const void* dy, int dy_dtype, const void* x, int x_dtype,
                               const float* gamma, const float* rstd, void* dx, int dx_dtype,
                               float* dgamma, float* partial, int rows, int C, int accumulate,
                               cudaStream_t stream) {
  return itb::norm_bwd_dispatch<true>(dy, dy_dtype, x, x_dtype, gamma, nullptr, rstd, dx, dx_dtype,
                                      dgamma, nullptr, partial, rows, C, accumulate, stream);
}
