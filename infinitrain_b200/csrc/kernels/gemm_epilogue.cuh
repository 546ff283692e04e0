// Shared pieces of the tcgen05 GEMM kernels: the device-side argument block and the epilogue that
// turns 32 fp32 accumulator columns of one output row into the stored result (bias, GELU dual
// store, GELU derivative, residual add, fp32 / bf16 output, atomic split-K accumulation).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace itb {

struct GemmDev {
  int M, N, K;
  int k_blocks;        // ceil(K / BK)
  int split_k;         // >= 1
  int tiles_m, tiles_n;
  void* C;             // bf16 or fp32, row-major, leading dimension ldc
  long long ldc;
  void* C2;            // second bf16 output: gelu(h) when kGemmGeluDual
  const float* bias;   // [N] fp32
  const void* residual;  // same dtype as C, leading dimension ldr
  long long ldr;
  const __nv_bfloat16* aux;  // [M, N] bf16 pre-activation for kGemmDGelu
  long long ld_aux;
  int flags;
  int* err;            // device word: 0 ok, else a code of the wait that gave up
  int staged;          // 1: bf16 outputs leave through shared memory and TMA stores; 2: fp32 outputs
                       // leave through shared memory and TMA stores / add-reductions (both need
                       // 16-byte aligned bases and row pitches); 0: direct stores from registers
};

// One MUFU instruction; relative error about 2^-11, below bf16 resolution.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanh_fast(u));
}
__device__ __forceinline__ float dgelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float x2 = x * x;
  float u = k0 * (x + k1 * x * x2);
  float t = tanh_fast(u);
  float du = k0 * (1.f + 3.f * k1 * x2);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

// v: 32 consecutive accumulator columns [col0, col0 + 32) of output row `row`.
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmDev& p, int row, bool row_ok, int col0,
                                                    float (&v)[32]) {
  const bool out_f32 = p.flags & kGemmOutF32;
          const bool full = (col0 + 32 <= p.N);
          if (p.flags & kGemmBias) {
  #pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += __ldg(p.bias + col0 + j);
          }
          if (row_ok) {
            if (p.flags & kGemmDGelu) {
              const __nv_bfloat16* h = p.aux + static_cast<long long>(row) * p.ld_aux + col0;
              if (full && ((reinterpret_cast<uintptr_t>(h) & 15) == 0)) {
  #pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 u = *reinterpret_cast<const uint4*>(h + j);
                  const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&u);
  #pragma unroll
                  for (int e = 0; e < 8; ++e) v[j + e] *= dgelu_tanh(__bfloat162float(hb[e]));
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) v[j] *= dgelu_tanh(__bfloat162float(h[j]));
              }
            }
            if (p.flags & kGemmGeluDual) {
              // C receives the pre-activation, C2 the activation (both bf16).
              __nv_bfloat16* c1 = static_cast<__nv_bfloat16*>(p.C) +
                                  static_cast<long long>(row) * p.ldc + col0;
              __nv_bfloat16* c2 = static_cast<__nv_bfloat16*>(p.C2) +
                                  static_cast<long long>(row) * p.ldc + col0;
              if (full && ((reinterpret_cast<uintptr_t>(c1) & 15) == 0) &&
                  ((reinterpret_cast<uintptr_t>(c2) & 15) == 0)) {
  #pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 u1, u2;
                  __nv_bfloat16* b1 = reinterpret_cast<__nv_bfloat16*>(&u1);
                  __nv_bfloat16* b2 = reinterpret_cast<__nv_bfloat16*>(&u2);
  #pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    b1[e] = __float2bfloat16(v[j + e]);
                    // The activation is computed from the rounded pre-activation so that the
                    // backward pass, which only sees the stored bf16 value, is consistent.
                    b2[e] = __float2bfloat16(gelu_tanh(__bfloat162float(b1[e])));
                  }
                  *reinterpret_cast<uint4*>(c1 + j) = u1;
                  *reinterpret_cast<uint4*>(c2 + j) = u2;
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) {
                    __nv_bfloat16 hb = __float2bfloat16(v[j]);
                    c1[j] = hb;
                    c2[j] = __float2bfloat16(gelu_tanh(__bfloat162float(hb)));
                  }
              }
            } else if (out_f32) {
              float* cp = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
              if (p.flags & kGemmResidual) {
                const float* rp =
                    static_cast<const float*>(p.residual) + static_cast<long long>(row) * p.ldr + col0;
                for (int j = 0; j < 32; ++j)
                  if (full || col0 + j < p.N) v[j] += rp[j];
              }
              const bool vec = full && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
              if (p.flags & kGemmAtomic) {
                if (vec) {
  #pragma unroll
                  for (int j = 0; j < 32; j += 4)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + j),
                                 "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3])
                                 : "memory");
                } else {
                  for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.N) atomicAdd(cp + j, v[j]);
                }
              } else if (p.flags & kGemmAccum) {
                for (int j = 0; j < 32; ++j)
                  if (full || col0 + j < p.N) cp[j] += v[j];
              } else if (vec) {
  #pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(cp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) cp[j] = v[j];
              }
            } else {
              __nv_bfloat16* cp =
                  static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
              const bool vec = full && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
              if (p.flags & kGemmResidual) {
                const __nv_bfloat16* rp = static_cast<const __nv_bfloat16*>(p.residual) +
                                          static_cast<long long>(row) * p.ldr + col0;
                if (vec && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
  #pragma unroll
                  for (int j = 0; j < 32; j += 8) {
                    uint4 u = *reinterpret_cast<const uint4*>(rp + j);
                    const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&u);
  #pragma unroll
                    for (int e = 0; e < 8; ++e) v[j + e] += __bfloat162float(rb[e]);
                  }
                } else {
                  for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
                }
              }
              if (vec) {
  #pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 u;
                  __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&u);
  #pragma unroll
                  for (int e = 0; e < 4; ++e)
                    b2[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                  *reinterpret_cast<uint4*>(cp + j) = u;
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) cp[j] = __float2bfloat16(v[j]);
              }
            }
          }
}

// ---- staged bf16 epilogue: a warp owns 32 output rows and moves 64 columns at a time through a
// 32 x 128-byte shared-memory slot laid out with the 128-byte swizzle of the TMA tensor maps
// (16-byte chunk j of row r sits at chunk position j ^ (r & 7)), so the global write is one bulk
// tensor store per slot instead of 32-way row-strided vector stores.

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 u;
  __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) b2[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  return u;
}

// Writes columns [32*half, 32*half + 32) of this lane's row into the slot.
__device__ __forceinline__ void stage_put32(uint8_t* slot, int lane, int half, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int pos = (half * 4 + j) ^ (lane & 7);
    *reinterpret_cast<uint4*>(slot + lane * 128 + pos * 16) = pack8_bf16(&v[8 * j]);
  }
}

// fp32 flavour: the slot holds 32 rows x 32 columns.
__device__ __forceinline__ void stage_put32_f32(uint8_t* slot, int lane, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int pos = j ^ (lane & 7);
    *reinterpret_cast<float4*>(slot + lane * 128 + pos * 16) =
        make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
}

// Same, plus gelu(rounded value) into slot2 (the activation is computed from the rounded
// pre-activation so that the backward pass, which only sees the stored bf16 value, is consistent).
__device__ __forceinline__ void stage_put32_gelu(uint8_t* slot, uint8_t* slot2, int lane, int half,
                                                 const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int pos = (half * 4 + j) ^ (lane & 7);
    uint4 u1 = pack8_bf16(&v[8 * j]);
    const __nv_bfloat16* b1 = reinterpret_cast<const __nv_bfloat16*>(&u1);
    float g[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = gelu_tanh(__bfloat162float(b1[e]));
    *reinterpret_cast<uint4*>(slot + lane * 128 + pos * 16) = u1;
    *reinterpret_cast<uint4*>(slot2 + lane * 128 + pos * 16) = pack8_bf16(g);
  }
}

// Reads columns [32*half, 32*half + 32) of this lane's row of a bf16 operand tile (residual or
// GELU pre-activation) that a TMA load placed in the slot and folds it into v.
template <bool kDGelu>
__device__ __forceinline__ void stage_fold32(const uint8_t* slot, int lane, int half, float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int pos = (half * 4 + j) ^ (lane & 7);
    const uint4 u = *reinterpret_cast<const uint4*>(slot + lane * 128 + pos * 16);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if constexpr (kDGelu)
        v[8 * j + e] *= dgelu_tanh(__bfloat162float(b[e]));
      else
        v[8 * j + e] += __bfloat162float(b[e]);
    }
  }
}

__device__ __forceinline__ void add_bias32(const GemmDev& p, int col0, float (&v)[32]) {
  if (col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + j));
      v[j] += b.x, v[j + 1] += b.y, v[j + 2] += b.z, v[j + 3] += b.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) v[j] += __ldg(p.bias + col0 + j);
  }
}

}  // namespace itb
