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
#ifndef ITB_NORM_FWD_BLOCKS_PER_SM
#define ITB_NORM_FWD_BLOCKS_PER_SM 8
#endif
constexpr int kNormFwdBlocksPerSm = ITB_NORM_FWD_BLOCKS_PER_SM;
// warp-per-row backward: two sets of packed row chunks (current and prefetched) beside the per-lane
// parameter-gradient accumulators need more than 168 registers
#ifndef ITB_NORM_BWD_BLOCKS_PER_SM
#define ITB_NORM_BWD_BLOCKS_PER_SM 2
#endif
constexpr int kNormBwdBlocksPerSm = ITB_NORM_BWD_BLOCKS_PER_SM;

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

// Eight consecutive elements as they come out of one or two 16-byte loads, kept packed in registers
// (a bf16 chunk costs 4 registers instead of 8) and unpacked where they are used.
template <typename T>
struct Raw8;
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <>
struct Raw8<__nv_bfloat16> {
  uint4 u;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

// Rows up to kMaxVec*256 elements wide stay (packed) in registers (kMaxVec chunks of 8 per lane); the
// part of a wider row beyond that is re-read from global memory.  kMaxVec is a template parameter so
// that narrow rows (GPT-2: 768) do not pay the register cost of wide ones.  The grid is one resident
// wave; a warp walks its rows with the loads of the NEXT row issued before the current row's
// arithmetic, so a row's memory latency hides behind its predecessor's reductions and stores.

template <typename TX, typename TY, bool kRms, int kMaxVec>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ gamma,
                const float* __restrict__ beta, TY* __restrict__ y, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int rows, int C, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C / 8;
  const int step = static_cast<int>(gridDim.x) * kNormWarps;
  Raw8<TX> cur[kMaxVec], nxt[kMaxVec];
  auto fetch = [&](int r, Raw8<TX> (&buf)[kMaxVec]) {
    const TX* xr = x + static_cast<long long>(r) * C;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) buf[i].load(xr + vi * 8);
    }
  };
  int row = blockIdx.x * kNormWarps + warp;
  if (row < rows) fetch(row, cur);
  for (; row < rows; row += step) {
    if (row + step < rows) fetch(row + step, nxt);
    const TX* xr = x + static_cast<long long>(row) * C;
    TY* yr = y + static_cast<long long>(row) * C;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      if (lane + i * 32 < nvec) {
        float v[8];
        cur[i].unpack(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += kRms ? v[e] * v[e] : v[e];
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
        if (lane + i * 32 < nvec) {
          float v[8];
          cur[i].unpack(v);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float d = v[e] - mean;
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
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float v[8];
        cur[i].unpack(v);
        emit(vi, v);
      }
    }
    for (int vi = lane + kMaxVec * 32; vi < nvec; vi += 32) {
      float t[8];
      load8<TX>(xr + vi * 8, t);
      emit(vi, t);
    }
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) cur[i] = nxt[i];
  }
}

// Backward.  With xhat = (x - mean) * rstd and g = dy * gamma:
//   LayerNorm: dx = rstd * (g - mean_C(g) - xhat * mean_C(g * xhat))
//   RMSNorm:   dx = rstd * (g - xhat * mean_C(g * xhat))                    (mean = 0)
// One pass over the row: dy and x stay (packed) in registers between the statistics and the output.
// kRes: the norm sits on a residual stream, out = dx + dres where dres is the gradient that reaches
// the stream past the norm (the skip connection); its column sums come out as a third partial row
// (they are the bias gradient of the projection that wrote into the stream).
//
// kWide = false: one warp per row (rows up to 1024 wide), kChunks chunks of 8 per lane.
// kWide = true:  the whole block works on one row at a time (rows up to kChunks * 1024 wide); the two
//                row statistics cross the warps through a double-buffered shared-memory slot, one
//                __syncthreads per row.
// dgamma += dy * xhat, dbeta += dy and the dres sums live in per-lane registers over all rows a block
// handles and leave as ONE partial row of 3 C per block, without atomics: in the warp-per-row layout
// the warps add their registers to a shared-memory row in turns; in the wide layout every thread owns
// its columns.
template <typename TDY, typename TX, typename TDX, bool kRms, int kChunks, bool kRes, bool kWide>
__global__ void __launch_bounds__(kNormThreads, kWide ? 4 : kNormBwdBlocksPerSm)
norm_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x,
                const float* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const TDX* __restrict__ dres,
                TDX* __restrict__ dx, float* __restrict__ partial, int rows, int C) {
  extern __shared__ float sh[];  // warp-per-row: [3*C] combine row; wide: [2][kNormWarps][2] statistics
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C / 8;
  // chunk i of this thread covers elements [8 * vi(i), 8 * vi(i) + 8) of a row
  auto vi_of = [&](int i) { return kWide ? static_cast<int>(threadIdx.x) + i * kNormThreads : lane + i * 32; };
  float gam[kChunks][8];
  float acc_g[kChunks][8], acc_b[kRms ? 1 : kChunks][8], acc_r[kRes ? kChunks : 1][8];
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    const int vi = vi_of(i);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      gam[i][e] = vi < nvec ? gamma[vi * 8 + e] : 0.f;
      acc_g[i][e] = 0.f;
      if (!kRms) acc_b[i][e] = 0.f;
      if (kRes) acc_r[i][e] = 0.f;
    }
  }
  const int row_step = kWide ? static_cast<int>(gridDim.x) : static_cast<int>(gridDim.x) * kNormWarps;
  int parity = 0;
  // The loads of the NEXT row are issued before the current row's arithmetic (kPrefetch: the
  // warp-per-row layout, where the register budget allows a second set of packed chunks).
  constexpr bool kPrefetch = !kWide;
  Raw8<TDY> rd[kChunks], nd[kPrefetch ? kChunks : 1];
  Raw8<TX> rx[kChunks], nx[kPrefetch ? kChunks : 1];
  Raw8<TDX> rres[kRes ? kChunks : 1], nres[(kRes && kPrefetch) ? kChunks : 1];
  auto fetch = [&](int r, Raw8<TDY>* bd, Raw8<TX>* bx, Raw8<TDX>* br) {
    const TDY* dyr = dy + static_cast<long long>(r) * C;
    const TX* xr = x + static_cast<long long>(r) * C;
    const TDX* rr = kRes ? dres + static_cast<long long>(r) * C : nullptr;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      const int vi = vi_of(i);
      if (vi < nvec) {
        bd[i].load(dyr + vi * 8);
        bx[i].load(xr + vi * 8);
        if (kRes) br[i].load(rr + vi * 8);
      }
    }
  };
  int row = kWide ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) * kNormWarps + warp;
  float mean_n = 0.f, rstd_n = 0.f;
  if (kPrefetch && row < rows) {
    fetch(row, rd, rx, rres);
    mean_n = kRms ? 0.f : mean_in[row];
    rstd_n = rstd_in[row];
  }
  for (; row < rows; row += row_step) {
    TDX* dxr = dx + static_cast<long long>(row) * C;
    float mean, rstd;
    if (kPrefetch) {
      mean = mean_n, rstd = rstd_n;
      if (row + row_step < rows) {
        fetch(row + row_step, nd, nx, nres);
        mean_n = kRms ? 0.f : mean_in[row + row_step];
        rstd_n = rstd_in[row + row_step];
      }
    } else {
      // every load of the row is issued before anything waits on one
      fetch(row, rd, rx, rres);
      mean = kRms ? 0.f : mean_in[row];
      rstd = rstd_in[row];
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      if (vi_of(i) < nvec) {
        float d[8], xv[8];
        rd[i].unpack(d);
        rx[i].unpack(xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhat = (xv[e] - mean) * rstd;
          const float gg = d[e] * gam[i][e];
          s1 += gg;
          s2 += gg * xhat;
          acc_g[i][e] += d[e] * xhat;
          if (!kRms) acc_b[i][e] += d[e];
        }
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (kWide) {
      float* slot = sh + parity * (2 * kNormWarps);
      if (lane == 0) {
        slot[2 * warp] = s1;
        slot[2 * warp + 1] = s2;
      }
      __syncthreads();
      s1 = s2 = 0.f;
#pragma unroll
      for (int w = 0; w < kNormWarps; ++w) {
        s1 += slot[2 * w];
        s2 += slot[2 * w + 1];
      }
      parity ^= 1;
    }
    s1 = kRms ? 0.f : s1 / C;
    s2 /= C;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      const int vi = vi_of(i);
      if (vi < nvec) {
        float d[8], xv[8], o[8];
        rd[i].unpack(d);
        rx[i].unpack(xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhat = (xv[e] - mean) * rstd;
          o[e] = rstd * (d[e] * gam[i][e] - s1 - xhat * s2);
        }
        if (kRes) {
          float r[8];
          rres[i].unpack(r);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            o[e] += r[e];
            acc_r[i][e] += r[e];
          }
        }
        store8<TDX>(dxr + vi * 8, o);
      }
    }
    if (kPrefetch) {
#pragma unroll
      for (int i = 0; i < kChunks; ++i) {
        rd[i] = nd[i];
        rx[i] = nx[i];
        if (kRes) rres[i] = nres[i];
      }
    }
  }
  float* prow = partial + static_cast<long long>(blockIdx.x) * 3 * C;
  if (kWide) {
    // every thread owns its columns: straight to the block's partial row
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      const int vi = vi_of(i);
      if (vi < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          prow[vi * 8 + e] = acc_g[i][e];
          prow[C + vi * 8 + e] = kRms ? 0.f : acc_b[i][e];
          prow[2 * C + vi * 8 + e] = kRes ? acc_r[i][e] : 0.f;
        }
      }
    }
    return;
  }
  // warp-per-row: the warps add their registers to the shared row one after the other
  for (int w = 0; w < kNormWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < kChunks; ++i) {
        const int vi = vi_of(i);
        if (vi < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int c = vi * 8 + e;
            sh[c] = (w ? sh[c] : 0.f) + acc_g[i][e];
            sh[C + c] = kRms ? 0.f : (w ? sh[C + c] : 0.f) + acc_b[i][e];
            sh[2 * C + c] = kRes ? (w ? sh[2 * C + c] : 0.f) + acc_r[i][e] : 0.f;
          }
        }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < 3 * C; i += blockDim.x) prow[i] = sh[i];
}

// out[c] (+)= sum_r partial[r, c] for the three column groups of a partial row (dgamma | dbeta | dres
// sums): a block of 32 columns x 32 row lanes; the row lanes are combined in shared memory.  A null
// output skips its group; `accumulate` bit k adds to output k instead of overwriting it.
constexpr int kReduceLanes = 32;   // row lanes of partial_reduce_kernel (block = 32 columns x 32 lanes)
__global__ void __launch_bounds__(32 * kReduceLanes)
partial_reduce_kernel(const float* __restrict__ partial, int prow_stride, int nrows,
                      float* __restrict__ out_a, float* __restrict__ out_b, float* __restrict__ out_c, int C,
                      int accumulate) {
  __shared__ float sh[kReduceLanes][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  const int which = c < C ? 0 : (c < 2 * C ? 1 : 2);
  float* out = which == 0 ? out_a : (which == 1 ? out_b : out_c);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < 3 * C && out) {
    const float* p = partial + c;
    int r = ry;
    // four independent loads in flight per thread
    for (; r + 3 * kReduceLanes < nrows; r += 4 * kReduceLanes) {
      s0 += p[static_cast<long long>(r) * prow_stride];
      s1 += p[static_cast<long long>(r + kReduceLanes) * prow_stride];
      s2 += p[static_cast<long long>(r + 2 * kReduceLanes) * prow_stride];
      s3 += p[static_cast<long long>(r + 3 * kReduceLanes) * prow_stride];
    }
    for (; r < nrows; r += kReduceLanes) s0 += p[static_cast<long long>(r) * prow_stride];
  }
  sh[ry][cx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (ry != 0 || c >= 3 * C || !out) return;
  float t = 0.f;
#pragma unroll
  for (int r = 0; r < kReduceLanes; ++r) t += sh[r][cx];
  const int oc = c - which * C;
  out[oc] = ((accumulate >> which) & 1) ? out[oc] + t : t;
}

// Upper bound of the backward grid for `rows` rows in either layout: what callers size `partial` with.
static int norm_grid(int rows) { return rows < kMaxPartialRows ? (rows < 1 ? 1 : rows) : kMaxPartialRows; }
static int norm_bwd_grid(int rows, bool wide, int blocks_per_sm) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int want = wide ? rows : (rows + kNormWarps - 1) / kNormWarps;
  int cap = sms * blocks_per_sm;
  if (cap > kMaxPartialRows) cap = kMaxPartialRows;
  return want < cap ? want : cap;
}

template <bool kRms>
static int norm_fwd_dispatch(const void* x, int xd, const float* gamma, const float* beta, void* y,
                             int yd, float* mean, float* rstd, int rows, int C, float eps,
                             cudaStream_t s) {
  if (C % 8) return -3;
  const int want = (rows + kNormWarps - 1) / kNormWarps;
  if (want < 1) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // one wave of resident blocks: what the kernel's register use lets an SM hold, at most kNormFwdBlocksPerSm
#define LAUNCH_V(TX, TY, V)                                                                      \
  do {                                                                                           \
    static int per_sm = 0;                                                                       \
    if (per_sm == 0) {                                                                           \
      int n = 0;                                                                                 \
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, norm_fwd_kernel<TX, TY, kRms, V>, kNormThreads, 0); \
      per_sm = n < 1 ? 1 : (n > kNormFwdBlocksPerSm ? kNormFwdBlocksPerSm : n);                  \
    }                                                                                            \
    const int grid = want < sms * per_sm ? want : sms * per_sm;                                  \
    norm_fwd_kernel<TX, TY, kRms, V><<<grid, kNormThreads, 0, s>>>(                              \
        static_cast<const TX*>(x), gamma, beta, static_cast<TY*>(y), mean, rstd, rows, C, eps);  \
  } while (0)
#define LAUNCH(TX, TY)              \
  do {                              \
    if (C <= 1024) LAUNCH_V(TX, TY, 4); \
    else LAUNCH_V(TX, TY, 8);       \
  } while (0)
  if (xd == kItbBF16 && yd == kItbBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (xd == kItbF32 && yd == kItbBF16) LAUNCH(float, __nv_bfloat16);
  else if (xd == kItbF32 && yd == kItbF32) LAUNCH(float, float);
  else if (xd == kItbBF16 && yd == kItbF32) LAUNCH(__nv_bfloat16, float);
  else return -4;
#undef LAUNCH
#undef LAUNCH_V
  return static_cast<int>(cudaGetLastError());
}

template <bool kRms>
static int norm_bwd_dispatch(const void* dy, int dyd, const void* x, int xd, const float* gamma,
                             const float* mean, const float* rstd, const void* dres, void* dx, int dxd,
                             float* dgamma, float* dbeta, float* dres_sum, float* partial, int rows, int C,
                             int accumulate, cudaStream_t s) {
  if (C % 8 || C > 6144) return -3;
  if (rows < 1) return 0;
  const bool wide = C > 1024;
  const int grid = norm_bwd_grid(rows, wide, wide ? 4 : kNormBwdBlocksPerSm);
  const int smem = wide ? 2 * kNormWarps * 2 * static_cast<int>(sizeof(float)) : 3 * C * static_cast<int>(sizeof(float));
#define LAUNCH_K(TDY, TX, TDX, CH, RES, WIDE)                                                     \
  norm_bwd_kernel<TDY, TX, TDX, kRms, CH, RES, WIDE><<<grid, kNormThreads, smem, s>>>(            \
      static_cast<const TDY*>(dy), static_cast<const TX*>(x), gamma, mean, rstd,                  \
      static_cast<const TDX*>(dres), static_cast<TDX*>(dx), partial, rows, C)
#define LAUNCH_R(TDY, TX, TDX, RES)                                  \
  do {                                                               \
    if (C <= 768) LAUNCH_K(TDY, TX, TDX, 3, RES, false);             \
    else if (C <= 1024) LAUNCH_K(TDY, TX, TDX, 4, RES, false);       \
    else if (C <= 2048) LAUNCH_K(TDY, TX, TDX, 2, RES, true);        \
    else if (C <= 4096) LAUNCH_K(TDY, TX, TDX, 4, RES, true);        \
    else LAUNCH_K(TDY, TX, TDX, 6, RES, true);                       \
  } while (0)
#define LAUNCH(TDY, TX, TDX)                  \
  do {                                        \
    if (dres) LAUNCH_R(TDY, TX, TDX, true);   \
    else LAUNCH_R(TDY, TX, TDX, false);       \
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
#undef LAUNCH_R
#undef LAUNCH_K
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  partial_reduce_kernel<<<(3 * C + 31) / 32, 32 * kReduceLanes, 0, s>>>(partial, 3 * C, grid, dgamma, dbeta,
                                                           dres ? dres_sum : nullptr, C, accumulate);
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
  return itb::norm_bwd_dispatch<false>(dy, dy_dtype, x, x_dtype, gamma, mean, rstd, nullptr, dx, dx_dtype,
                                       dgamma, dbeta, nullptr, partial, rows, C, accumulate ? 3 : 0, stream);
}
// The same with the residual stream's gradient folded in: dx = norm backward + dres, and (when
// dres_sum is not null) dres_sum[c] (+)= sum over rows of dres.  `accumulate` is a bit mask: bit 0
// dgamma, bit 1 dbeta, bit 2 dres_sum are added to instead of overwritten.  partial: [rows of
// itb_norm_partial_rows(rows), 3 C] fp32.
extern "C" int itb_layernorm_bwd_res(const void* dy, int dy_dtype, const void* x, int x_dtype,
                                     const float* gamma, const float* mean, const float* rstd,
                                     const void* dres, void* dx, int dx_dtype, float* dgamma, float* dbeta,
                                     float* dres_sum, float* partial, int rows, int C, int accumulate,
                                     cudaStream_t stream) {
  return itb::norm_bwd_dispatch<false>(dy, dy_dtype, x, x_dtype, gamma, mean, rstd, dres, dx, dx_dtype,
                                       dgamma, dbeta, dres_sum, partial, rows, C, accumulate, stream);
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
  return itb::norm_bwd_dispatch<true>(dy, dy_dtype, x, x_dtype, gamma, nullptr, rstd, nullptr, dx, dx_dtype,
                                      dgamma, nullptr, nullptr, partial, rows, C, accumulate ? 1 : 0, stream);
}
extern "C" int itb_rmsnorm_bwd_res(const void* dy, int dy_dtype, const void* x, int x_dtype,
                                   const float* gamma, const float* rstd, const void* dres, void* dx,
                                   int dx_dtype, float* dgamma, float* dres_sum, float* partial, int rows,
                                   int C, int accumulate, cudaStream_t stream) {
  return itb::norm_bwd_dispatch<true>(dy, dy_dtype, x, x_dtype, gamma, nullptr, rstd, dres, dx, dx_dtype,
                                      dgamma, nullptr, dres_sum, partial, rows, C, accumulate, stream);
}
