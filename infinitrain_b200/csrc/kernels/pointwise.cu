// Bandwidth-bound pointwise kernels: tanh-GELU, SiLU-gated product (SwiGLU), rotary embedding,
// token/position embedding, dtype cast and column sums (bias gradients).
//
// In the reference these are chains of generic elementwise launches, each materialising its output
// (infini_train/src/nn/modules/activations.cc:15-23, transformer/causal_self_attention.cc:133-167,
// src/kernels/cuda/embedding.cu:13-116, cast.cu:16-51, linear.cu:138-156).  Here each is one pass
// with 16-byte accesses, sized as a grid-stride loop over 148 SMs.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace itb {

constexpr int kPwThreads = 256;
static inline int pw_grid(long long work_items) {
  long long b = (work_items + kPwThreads - 1) / kPwThreads;
  const long long cap = 148LL * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

template <typename T>
struct Vec8;
template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

__device__ __forceinline__ float gelu_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float dgelu_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float x2 = x * x, t = tanhf(k0 * (x + k1 * x * x2));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x2);
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------ GELU
template <typename T, bool kBwd>
__global__ void gelu_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ out,
                            long long n) {
  const long long nvec = n / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += stride) {
    float xv[8], o[8];
    Vec8<T>::load(x + i * 8, xv);
    if (kBwd) {
      float d[8];
      Vec8<T>::load(dy + i * 8, d);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = d[e] * dgelu_f(xv[e]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = gelu_f(xv[e]);
    }
    Vec8<T>::store(out + i * 8, o);
  }
  // tail
  for (long long i = nvec * 8 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += stride) {
    float xv = static_cast<float>(x[i]);
    float o = kBwd ? static_cast<float>(dy[i]) * dgelu_f(xv) : gelu_f(xv);
    out[i] = static_cast<T>(o);
  }
}

// ------------------------------------------------------------------ SwiGLU: out = a * silu(b)
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, long long ld_in,
                                  T* __restrict__ out, long long ld_out, int rows, int F) {
  const int fv = F / 8;
  const long long total = static_cast<long long>(rows) * fv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += stride) {
    const long long r = i / fv;
    const int c = static_cast<int>(i - r * fv) * 8;
    float av[8], bv[8], o[8];
    Vec8<T>::load(a + r * ld_in + c, av);
    Vec8<T>::load(b + r * ld_in + c, bv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = av[e] * bv[e] * sigmoid_f(bv[e]);
    Vec8<T>::store(out + r * ld_out + c, o);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dout, long long ld_dout,
                                  const T* __restrict__ a, const T* __restrict__ b, long long ld_in,
                                  T* __restrict__ da, T* __restrict__ db, long long ld_dab, int rows,
                                  int F) {
  const int fv = F / 8;
  const long long total = static_cast<long long>(rows) * fv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += stride) {
    const long long r = i / fv;
    const int c = static_cast<int>(i - r * fv) * 8;
    float av[8], bv[8], d[8], oa[8], ob[8];
    Vec8<T>::load(a + r * ld_in + c, av);
    Vec8<T>::load(b + r * ld_in + c, bv);
    Vec8<T>::load(dout + r * ld_dout + c, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float s = sigmoid_f(bv[e]);
      float silu = bv[e] * s;
      oa[e] = d[e] * silu;
      ob[e] = d[e] * av[e] * (s + silu * (1.f - s));
    }
    Vec8<T>::store(da + r * ld_dab + c, oa);
    Vec8<T>::store(db + r * ld_dab + c, ob);
  }
}

// ------------------------------------------------------------------ RoPE (interleaved pairs)
// One thread rotates 4 pairs (8 elements) of one head of one token.
template <typename T>
__global__ void rope_kernel(T* __restrict__ qkv, const float* __restrict__ freqs, int B, int T_,
                            int n_heads, int D, long long row_stride, int pos0, int inverse) {
  const int dv = D / 8;
  const long long total = static_cast<long long>(B) * T_ * n_heads * dv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += stride) {
    const int c = static_cast<int>(i % dv);
    long long r = i / dv;
    const int h = static_cast<int>(r % n_heads);
    r /= n_heads;
    const int t = static_cast<int>(r % T_);
    T* p = qkv + r * row_stride + static_cast<long long>(h) * D + c * 8;
    const float* f = freqs + (static_cast<long long>(pos0 + t) * (D / 2) + c * 4) * 2;
    float v[8], o[8], cs[8];
    Vec8<T>::load(p, v);
    Vec8<float>::load(f, cs);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float co = cs[2 * e], si = inverse ? -cs[2 * e + 1] : cs[2 * e + 1];
      o[2 * e] = v[2 * e] * co - v[2 * e + 1] * si;
      o[2 * e + 1] = v[2 * e] * si + v[2 * e + 1] * co;
    }
    Vec8<T>::store(p, o);
  }
}

// ------------------------------------------------------------------ embedding
template <typename TT, typename TO>
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx, const TT* __restrict__ wte,
                                     const TT* __restrict__ wpe, TO* __restrict__ out, int B, int T_,
                                     int C, int pos0, int vocab_start, int vocab_end) {
  const int cv = C / 8;
  const long long total = static_cast<long long>(B) * T_ * cv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += stride) {
    const int c = static_cast<int>(i % cv) * 8;
    const long long bt = i / cv;
    const int t = static_cast<int>(bt % T_);
    const long long id = idx[bt];
    float v[8];
    if (id >= vocab_start && id < vocab_end) {
      Vec8<TT>::load(wte + (id - vocab_start) * C + c, v);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;  // token owned by another vocabulary shard
    }
    if (wpe) {
      float p[8];
      Vec8<TT>::load(wpe + static_cast<long long>(pos0 + t) * C + c, p);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += p[e];
    }
    Vec8<TO>::store(out + bt * C + c, v);
  }
}

// Token-table gradient: one warp per token, lanes stride over the row with fp32 atomics (different
// tokens that share an id collide; the order of the sums is not fixed).
template <typename TD>
__global__ void embedding_bwd_wte_kernel(const long long* __restrict__ idx,
                                         const TD* __restrict__ dout, float* __restrict__ dwte,
                                         long long n_tokens, int C, int vocab_start, int vocab_end) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long tok = warp0; tok < n_tokens; tok += nwarps) {
    const long long id = idx[tok];
    if (id < vocab_start || id >= vocab_end) continue;
    const TD* src = dout + tok * C;
    float* dst = dwte + (id - vocab_start) * C;
    for (int c = lane * 8; c < C; c += 256) {
      float v[8];
      Vec8<TD>::load(src + c, v);
#pragma unroll
      for (int e = 0; e < 8; e += 4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c + e), "f"(v[e]),
                     "f"(v[e + 1]), "f"(v[e + 2]), "f"(v[e + 3])
                     : "memory");
    }
  }
}
// Position-table gradient: dwpe[pos0 + t, c] += sum_b dout[b, t, c]; no atomics.
template <typename TD>
__global__ void embedding_bwd_wpe_kernel(const TD* __restrict__ dout, float* __restrict__ dwpe,
                                         int B, int T_, int C, int pos0) {
  const int cv = C / 8;
  const long long total = static_cast<long long>(T_) * cv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += stride) {
    const int c = static_cast<int>(i % cv) * 8;
    const int t = static_cast<int>(i / cv);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < B; ++b) {
      float v[8];
      Vec8<TD>::load(dout + (static_cast<long long>(b) * T_ + t) * C + c, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    float* dst = dwpe + static_cast<long long>(pos0 + t) * C + c;
    float cur[8];
    Vec8<float>::load(dst, cur);
#pragma unroll
    for (int e = 0; e < 8; ++e) cur[e] += acc[e];
    Vec8<float>::store(dst, cur);
  }
}

// ------------------------------------------------------------------ cast
template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
  const long long nvec = n / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 31) == 0;
  if (aligned) {
    for (long long i = tid; i < nvec; i += stride) {
      float v[8];
      Vec8<TS>::load(src + i * 8, v);
      Vec8<TD>::store(dst + i * 8, v);
    }
    for (long long i = nvec * 8 + tid; i < n; i += stride)
      dst[i] = static_cast<TD>(static_cast<float>(src[i]));
  } else {
    for (long long i = tid; i < n; i += stride) dst[i] = static_cast<TD>(static_cast<float>(src[i]));
  }
}

// ------------------------------------------------------------------ column sum (bias gradient)
// Stage 1: a block of 32 x 8 threads covers 256 columns (32 groups of 8) and kColsumRowsPerBlock
// rows; thread (cx, ry) sums rows ry, ry + 8, ... of its 8 columns (a warp reads 512 contiguous
// bytes of one row), the 8 row lanes are combined in shared memory and the block writes one
// partial row.  Stage 2 sums the partial rows.
constexpr int kColsumRowsPerBlock = 128;
template <typename T>
__global__ void __launch_bounds__(256)
colsum_stage1_kernel(const T* __restrict__ x, long long ld, float* __restrict__ partial, int rows,
                     int N) {
  __shared__ float sh[8][32][9];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int cg = blockIdx.x * 32 + cx;  // column group of 8
  const bool col_ok = cg * 8 < N;
  const int r0 = blockIdx.y * kColsumRowsPerBlock;
  const int r1 = min(rows, r0 + kColsumRowsPerBlock);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col_ok) {
    for (int r = r0 + ry; r < r1; r += 8) {
      float v[8];
      Vec8<T>::load(x + static_cast<long long>(r) * ld + cg * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) sh[ry][cx][e] = acc[e];
  __syncthreads();
  // 256 threads -> 256 columns of this block
  const int c = threadIdx.x;           // column within the block
  const int gcx = c >> 3, ge = c & 7;
  const int col = blockIdx.x * 256 + c;
  if (col < N) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) s += sh[r][gcx][ge];
    partial[static_cast<long long>(blockIdx.y) * N + col] = s;
  }
}
// out[c] (+)= sum_r partial[r, c]: 32 columns x 8 row lanes per block.
__global__ void __launch_bounds__(256)
colsum_stage2_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out, int N,
                     int accumulate) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < N)
    for (int r = ry; r < nparts; r += 8) s += partial[static_cast<long long>(r) * N + c];
  sh[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < N) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += sh[r][cx];
    out[c] = accumulate ? out[c] + t : t;
  }
}

}  // namespace itb

using namespace itb;

extern "C" int itb_gelu_fwd(const void* x, void* y, int dtype, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 31) return -2;
  if (dtype == kItbBF16)
    gelu_kernel<__nv_bfloat16, false><<<pw_grid(n / 8 + 1), kPwThreads, 0, s>>>(
        nullptr, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n);
  else
    gelu_kernel<float, false><<<pw_grid(n / 8 + 1), kPwThreads, 0, s>>>(
        nullptr, static_cast<const float*>(x), static_cast<float*>(y), n);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int itb_gelu_bwd(const void* dy, const void* x, void* dx, int dtype, long long n,
                            cudaStream_t s) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
       reinterpret_cast<uintptr_t>(dx)) & 31)
    return -2;
  if (dtype == kItbBF16)
    gelu_kernel<__nv_bfloat16, true><<<pw_grid(n / 8 + 1), kPwThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
        static_cast<__nv_bfloat16*>(dx), n);
  else
    gelu_kernel<float, true><<<pw_grid(n / 8 + 1), kPwThreads, 0, s>>>(
        static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<float*>(dx), n);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_swiglu_fwd(const void* a, const void* b, long long ld_in, void* out,
                              long long ld_out, int dtype, int rows, int F, cudaStream_t s) {
  if (rows <= 0 || F <= 0) return 0;
  if (F % 8 || ld_in % 8 || ld_out % 8) return -3;
  const long long work = static_cast<long long>(rows) * (F / 8);
  if (dtype == kItbBF16)
    swiglu_fwd_kernel<__nv_bfloat16><<<pw_grid(work), kPwThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), ld_in,
        static_cast<__nv_bfloat16*>(out), ld_out, rows, F);
  else
    swiglu_fwd_kernel<float><<<pw_grid(work), kPwThreads, 0, s>>>(
        static_cast<const float*>(a), static_cast<const float*>(b), ld_in, static_cast<float*>(out),
        ld_out, rows, F);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int itb_swiglu_bwd(const void* dout, long long ld_dout, const void* a, const void* b,
                              long long ld_in, void* da, void* db, long long ld_dab, int dtype,
                              int rows, int F, cudaStream_t s) {
  if (rows <= 0 || F <= 0) return 0;
  if (F % 8 || ld_in % 8 || ld_dout % 8 || ld_dab % 8) return -3;
  const long long work = static_cast<long long>(rows) * (F / 8);
  if (dtype == kItbBF16)
    swiglu_bwd_kernel<__nv_bfloat16><<<pw_grid(work), kPwThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dout), ld_dout, static_cast<const __nv_bfloat16*>(a),
        static_cast<const __nv_bfloat16*>(b), ld_in, static_cast<__nv_bfloat16*>(da),
        static_cast<__nv_bfloat16*>(db), ld_dab, rows, F);
  else
    swiglu_bwd_kernel<float><<<pw_grid(work), kPwThreads, 0, s>>>(
        static_cast<const float*>(dout), ld_dout, static_cast<const float*>(a),
        static_cast<const float*>(b), ld_in, static_cast<float*>(da), static_cast<float*>(db),
        ld_dab, rows, F);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_rope_inplace(void* qkv, int dtype, const float* freqs, int B, int T, int n_heads,
                                int D, long long row_stride, int pos0, int inverse,
                                cudaStream_t s) {
  if (B <= 0 || T <= 0 || n_heads <= 0) return 0;
  if (D % 8 || row_stride % 8) return -3;
  const long long work = static_cast<long long>(B) * T * n_heads * (D / 8);
  if (dtype == kItbBF16)
    rope_kernel<__nv_bfloat16><<<pw_grid(work), kPwThreads, 0, s>>>(
        static_cast<__nv_bfloat16*>(qkv), freqs, B, T, n_heads, D, row_stride, pos0, inverse);
  else
    rope_kernel<float><<<pw_grid(work), kPwThreads, 0, s>>>(static_cast<float*>(qkv), freqs, B, T,
                                                            n_heads, D, row_stride, pos0, inverse);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_embedding_fwd(const long long* idx, const void* wte, const void* wpe,
                                 int table_dtype, void* out, int out_dtype, int B, int T, int C,
                                 int pos0, int vocab_start, int vocab_end, cudaStream_t s) {
  if (B <= 0 || T <= 0) return 0;
  if (C % 8) return -3;
  const long long work = static_cast<long long>(B) * T * (C / 8);
#define LAUNCH(TT, TO)                                                                         \
  embedding_fwd_kernel<TT, TO><<<pw_grid(work), kPwThreads, 0, s>>>(                           \
      idx, static_cast<const TT*>(wte), static_cast<const TT*>(wpe), static_cast<TO*>(out), B, T, \
      C, pos0, vocab_start, vocab_end)
  if (table_dtype == kItbF32 && out_dtype == kItbBF16) LAUNCH(float, __nv_bfloat16);
  else if (table_dtype == kItbF32 && out_dtype == kItbF32) LAUNCH(float, float);
  else if (table_dtype == kItbBF16 && out_dtype == kItbBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == kItbBF16 && out_dtype == kItbF32) LAUNCH(__nv_bfloat16, float);
  else return -4;
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_embedding_bwd(const long long* idx, const void* dout, int dout_dtype,
                                 float* dwte, float* dwpe, int B, int T, int C, int pos0,
                                 int vocab_start, int vocab_end, cudaStream_t s) {
  if (B <= 0 || T <= 0) return 0;
  if (C % 8) return -3;
  const long long ntok = static_cast<long long>(B) * T;
  if (dwte) {
    const int grid = pw_grid(ntok * 32);
    if (dout_dtype == kItbBF16)
      embedding_bwd_wte_kernel<__nv_bfloat16><<<grid, kPwThreads, 0, s>>>(
          idx, static_cast<const __nv_bfloat16*>(dout), dwte, ntok, C, vocab_start, vocab_end);
    else
      embedding_bwd_wte_kernel<float><<<grid, kPwThreads, 0, s>>>(
          idx, static_cast<const float*>(dout), dwte, ntok, C, vocab_start, vocab_end);
  }
  if (dwpe) {
    const long long work = static_cast<long long>(T) * (C / 8);
    if (dout_dtype == kItbBF16)
      embedding_bwd_wpe_kernel<__nv_bfloat16><<<pw_grid(work), kPwThreads, 0, s>>>(
          static_cast<const __nv_bfloat16*>(dout), dwpe, B, T, C, pos0);
    else
      embedding_bwd_wpe_kernel<float><<<pw_grid(work), kPwThreads, 0, s>>>(
          static_cast<const float*>(dout), dwpe, B, T, C, pos0);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_cast(const void* src, int sd, void* dst, int dd, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  const int grid = pw_grid(n / 8 + 1);
#define LAUNCH(TS, TD) \
  cast_kernel<TS, TD><<<grid, kPwThreads, 0, s>>>(static_cast<const TS*>(src), static_cast<TD*>(dst), n)
  if (sd == kItbF32 && dd == kItbBF16) LAUNCH(float, __nv_bfloat16);
  else if (sd == kItbBF16 && dd == kItbF32) LAUNCH(__nv_bfloat16, float);
  else if (sd == kItbF32 && dd == kItbF32) LAUNCH(float, float);
  else if (sd == kItbBF16 && dd == kItbBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return -4;
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

extern "C" int itb_colsum_partial_rows(int rows) {
  return (rows + kColsumRowsPerBlock - 1) / kColsumRowsPerBlock;
}
extern "C" int itb_colsum(const void* x, int dtype, long long ld, float* out, float* partial,
                          int rows, int N, int accumulate, cudaStream_t s) {
  if (rows <= 0 || N <= 0) return 0;
  if (N % 8 || ld % 8 || ld < N || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  const int nparts = itb_colsum_partial_rows(rows);
  if (nparts > 65535) return -3;      // grid.y limit
  dim3 grid((N + 255) / 256, nparts);
  if (dtype == kItbBF16)
    colsum_stage1_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                             ld, partial, rows, N);
  else
    colsum_stage1_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), ld, partial, rows,
                                                     N);
  colsum_stage2_kernel<<<(N + 31) / 32, 256, 0, s>>>(partial, nparts, out, N, accumulate);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ column sum without allocation
// Same two kernels as itb_colsum, with the stage-1 partial sums in a fixed device array instead of a
// caller-provided buffer (see no_alloc.h for who needs this and for the rules).
#include "no_alloc.h"

static __device__ __align__(256) float g_colsum_static_scratch[kItbColsumStaticMaxPartials];

namespace {
constexpr int kMaxDevices = 64;
// Device address of g_colsum_static_scratch per device ordinal.  In host code the array's name is
// only a handle for the runtime, not a device pointer: the address must be looked up.
float* g_scratch_addr[kMaxDevices] = {nullptr};

int colsum_static_scratch(float** out_ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -6;
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_colsum_static_scratch);  // for the CURRENT device
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out_ptr = g_scratch_addr[dev];
  return 0;
}
}  // namespace

extern "C" int itb_colsum_static(const void* x, int dtype, long long ld, float* out, int rows, int N,
                                 int accumulate, cudaStream_t s) {
  if (rows <= 0 || N <= 0) return 0;
  // 16-byte vector loads of x: aligned base, row stride and width in multiples of 8 elements
  if (N % 8 || ld % 8 || ld < N || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  if (dtype != kItbBF16 && dtype != kItbF32) return -4;
  const int nparts = itb_colsum_partial_rows(rows);
  if (nparts > 65535) return -3;      // grid.y limit (more than 8.3 M rows)
  if (static_cast<long long>(nparts) * N > kItbColsumStaticMaxPartials) return kItbErrScratchTooSmall;
  float* partial = nullptr;
  if (int rc = colsum_static_scratch(&partial)) return rc;
  dim3 grid((N + 255) / 256, nparts);
  if (dtype == kItbBF16)
    colsum_stage1_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                             ld, partial, rows, N);
  else
    colsum_stage1_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), ld, partial, rows,
                                                     N);
  colsum_stage2_kernel<<<(N + 31) / 32, 256, 0, s>>>(partial, nparts, out, N, accumulate);
  return static_cast<int>(cudaGetLastError());
}
