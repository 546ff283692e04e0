// Causal flash attention with grouped-query heads, forward and backward, bf16 in / fp32 softmax
// statistics.  The T x T score matrix is never materialised and K/V heads are never repeated.
//
// The reference builds attention from Matmul + MulScalar + MaskedFill + Softmax + Matmul with
// RepeatInterleave for GQA and keeps three [B, H, T, T] tensors for backward
// (infini_train/src/nn/modules/transformer/causal_self_attention.cc:86-130, 169-257; "flash" is a
// dead flag at :232-233).  This file is the tiled online-softmax formulation: 64-query x 64-key
// tiles, cp.async double buffering, tensor-core products through warp-level mma (m16n8k16, bf16,
// fp32 accumulate).  q/k/v are addressed through explicit row/batch strides so they can alias
// column blocks of the packed QKV projection output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "kernels.h"

namespace itb {

constexpr int kBlkM = 64;  // query rows per tile
constexpr int kBlkN = 64;  // key rows per tile
constexpr int kAttnThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t s_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const int sz = pred ? 16 : 0;  // src-size 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s_u32(smem)), "l"(gmem),
               "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s_u32(p)));
}
// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Shared-memory tile of 64 rows x W bf16 with the 16-byte chunks of a row XOR-swizzled by the row
// index so that ldmatrix reads are bank-conflict free.
template <int W>
__device__ __forceinline__ int sw_off(int row, int chunk) {
  return row * W + ((chunk ^ (row & 7)) << 3);
}

// Loads rows [r0, r0+64) x W columns of a strided global matrix into a swizzled tile; rows >= rows
// are zero-filled.
template <int W>
__device__ __forceinline__ void load_tile(__nv_bfloat16* tile, const __nv_bfloat16* g,
                                          long long row_stride, int r0, int rows) {
  constexpr int kChunks = W / 8;
#pragma unroll
  for (int i = 0; i < (64 * kChunks) / kAttnThreads; ++i) {
    const int idx = threadIdx.x + i * kAttnThreads;
    const int r = idx / kChunks, c = idx % kChunks;
    const bool ok = (r0 + r) < rows;
    const __nv_bfloat16* src = g + (ok ? (static_cast<long long>(r0 + r) * row_stride + c * 8) : 0);
    cp_async16(tile + sw_off<W>(r, c), src, ok);
  }
}

// A operand (16 rows x 16 k) of a row-major tile at (row0, k0).
template <int W>
__device__ __forceinline__ void lda(uint32_t (&r)[4], const __nv_bfloat16* tile, int row0, int k0) {
  const int lane = threadIdx.x & 31;
  ldsm_x4(r, tile + sw_off<W>(row0 + (lane & 15), (k0 >> 3) + (lane >> 4)));
}
// B operand for two adjacent 8-wide n-blocks from a tile stored [n][k]: r0,r1 -> n-block 0 (k lo,
// k hi), r2,r3 -> n-block 1.
template <int W>
__device__ __forceinline__ void ldb_nk(uint32_t (&r)[4], const __nv_bfloat16* tile, int n0, int k0) {
  const int lane = threadIdx.x & 31;
  ldsm_x4(r, tile + sw_off<W>(n0 + (lane & 7) + ((lane >> 4) << 3), (k0 >> 3) + ((lane >> 3) & 1)));
}
// B operand for two adjacent n-blocks from a tile stored [k][n] (transposing load).
template <int W>
__device__ __forceinline__ void ldb_kn(uint32_t (&r)[4], const __nv_bfloat16* tile, int k0, int n0) {
  const int lane = threadIdx.x & 31;
  ldsm_x4_t(r, tile + sw_off<W>(k0 + (lane & 7) + (((lane >> 3) & 1) << 3), (n0 >> 3) + (lane >> 4)));
}
// A operand (16 rows m x 16 k) from a tile stored [k][m] (transposing load).
template <int W>
__device__ __forceinline__ void lda_km(uint32_t (&r)[4], const __nv_bfloat16* tile, int k0, int m0) {
  const int lane = threadIdx.x & 31;
  const int q = lane >> 3;
  ldsm_x4_t(r, tile + sw_off<W>(k0 + (lane & 7) + ((q >> 1) << 3), (m0 >> 3) + (q & 1)));
}

// ===================================================================== forward
template <int D>
__global__ void __launch_bounds__(kAttnThreads)
flash_fwd_kernel(const ItbAttnArgs a) {
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  __nv_bfloat16* sK = sQ + 64 * D;      // 2 buffers
  __nv_bfloat16* sV = sK + 2 * 64 * D;  // 2 buffers

  // Heavier (later) query tiles first so that the tail of the grid is made of short CTAs.
  const int mb = a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.H / a.KV);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int m0 = mb * kBlkM;

  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q) + b * a.q_batch_stride + h * D;
  const __nv_bfloat16* k = static_cast<const __nv_bfloat16*>(a.k) + b * a.k_batch_stride + hk * D;
  const __nv_bfloat16* v = static_cast<const __nv_bfloat16*>(a.v) + b * a.v_batch_stride + hk * D;

  int n_blocks = (a.T + kBlkN - 1) / kBlkN;
  if (a.causal) n_blocks = min(n_blocks, mb + 1);

  load_tile<D>(sQ, q, a.q_row_stride, m0, a.T);
  load_tile<D>(sK, k, a.k_row_stride, 0, a.T);
  load_tile<D>(sV, v, a.v_row_stride, 0, a.T);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float row_m[2] = {-FLT_MAX, -FLT_MAX}, row_l[2] = {0.f, 0.f};
  const float sl2 = a.scale * kLog2e;

  for (int j = 0; j < n_blocks; ++j) {
    cp_async_wait_all();
    __syncthreads();
    if (j + 1 < n_blocks) {
      load_tile<D>(sK + ((j + 1) & 1) * 64 * D, k, a.k_row_stride, (j + 1) * kBlkN, a.T);
      load_tile<D>(sV + ((j + 1) & 1) * 64 * D, v, a.v_row_stride, (j + 1) * kBlkN, a.T);
      cp_async_commit();
    }
    if (j == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) lda<D>(qf[kk], sQ, warp * 16, kk * 16);
    }
    const __nv_bfloat16* tK = sK + (j & 1) * 64 * D;
    const __nv_bfloat16* tV = sV + (j & 1) * 64 * D;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int nb2 = 0; nb2 < 4; ++nb2) {
        uint32_t bf[4];
        ldb_nk<D>(bf, tK, nb2 * 16, kk * 16);
        mma_bf16(s[2 * nb2], qf[kk], bf[0], bf[1]);
        mma_bf16(s[2 * nb2 + 1], qf[kk], bf[2], bf[3]);
      }
    }
    // Mask: keys beyond the sequence, and keys after the query on the diagonal tile.
    const bool need_mask = (a.causal && j == mb) || ((j + 1) * kBlkN > a.T);
    if (need_mask) {
#pragma unroll
      for (int nb = 0; nb < 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = j * kBlkN + nb * 8 + t4 * 2 + (e & 1);
          const int row = m0 + warp * 16 + g + ((e >> 1) << 3);
          if (col >= a.T || (a.causal && col > row)) s[nb][e] = -FLT_MAX;
        }
    }
    // Online softmax for the two rows this thread owns (g and g + 8).
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = s[0][2 * r];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) mx = fmaxf(mx, fmaxf(s[nb][2 * r], s[nb][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(row_m[r], mx);
      // A fully masked row keeps m_new = -FLT_MAX: use 0 as the exponent base so exp2 yields 0.
      const float base = (m_new == -FLT_MAX) ? 0.f : m_new * sl2;
      const float corr = exp2f(row_m[r] * sl2 - base);
      float sum = 0.f;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        float p0 = exp2f(s[nb][2 * r] * sl2 - base);
        float p1 = exp2f(s[nb][2 * r + 1] * sl2 - base);
        s[nb][2 * r] = p0;
        s[nb][2 * r + 1] = p1;
        sum += p0 + p1;
      }
      row_l[r] = row_l[r] * corr + sum;
      row_m[r] = m_new;
#pragma unroll
      for (int db = 0; db < D / 8; ++db) {
        o[db][2 * r] *= corr;
        o[db][2 * r + 1] *= corr;
      }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int db2 = 0; db2 < D / 16; ++db2) {
        uint32_t bf[4];
        ldb_kn<D>(bf, tV, kk * 16, db2 * 16);
        mma_bf16(o[2 * db2], pa, bf[0], bf[1]);
        mma_bf16(o[2 * db2 + 1], pa, bf[2], bf[3]);
      }
    }
  }

  // Finalise: row sums are partial per quad lane.
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.o) + b * a.o_batch_stride + h * D;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = row_l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = m0 + warp * 16 + g + r * 8;
    if (row < a.T) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = op + static_cast<long long>(row) * a.o_row_stride;
#pragma unroll
      for (int db = 0; db < D / 8; ++db) {
        *reinterpret_cast<uint32_t*>(orow + db * 8 + t4 * 2) =
            pack_bf16(o[db][2 * r] * inv, o[db][2 * r + 1] * inv);
      }
      if (t4 == 0)
        a.lse[(static_cast<long long>(b) * a.H + h) * a.T + row] =
            (l > 0.f) ? row_m[r] * a.scale + logf(l) : -FLT_MAX;
    }
  }
}

// ===================================================================== backward
// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per (b,t,h).
template <int D>
__global__ void attn_delta_kernel(const ItbAttnArgs a) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(a.B) * a.T * a.H;
  if (w >= total) return;
  const int h = static_cast<int>(w % a.H);
  const long long bt = w / a.H;
  const int t = static_cast<int>(bt % a.T);
  const int b = static_cast<int>(bt / a.T);
  const long long off = b * a.o_batch_stride + static_cast<long long>(t) * a.o_row_stride + h * D;
  const __nv_bfloat16* o = static_cast<const __nv_bfloat16*>(a.o) + off;
  const __nv_bfloat16* d = static_cast<const __nv_bfloat16*>(a.dout) + off;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + c));
    float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d + c));
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) a.delta[(static_cast<long long>(b) * a.H + h) * a.T + t] = acc;
}

// dq (bf16, strided) = dq_accum (fp32, [B,T,H,D] contiguous)
template <int D>
__global__ void attn_dq_convert_kernel(const ItbAttnArgs a) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;  // 4 elements
  const long long total = static_cast<long long>(a.B) * a.T * a.H * (D / 4);
  if (i >= total) return;
  const int c = static_cast<int>(i % (D / 4)) * 4;
  long long r = i / (D / 4);
  const int h = static_cast<int>(r % a.H);
  r /= a.H;
  const int t = static_cast<int>(r % a.T);
  const int b = static_cast<int>(r / a.T);
  const float4 v = *reinterpret_cast<const float4*>(a.dq_accum + i * 4);
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.dq) + b * a.q_batch_stride +
                       static_cast<long long>(t) * a.q_row_stride + h * D + c;
  uint2 u;
  u.x = pack_bf16(v.x, v.y);
  u.y = pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = u;
}

// One CTA owns a 64-row key/value tile of one KV head and walks over the query tiles (and the
// query heads of the group) that attend to it.  Warp w owns key rows [16w, 16w+16): it keeps
// dK/dV for them in registers; dQ contributions go to an fp32 buffer with atomics because every
// key tile contributes to every later query tile.
template <int D>
__global__ void __launch_bounds__(kAttnThreads)
flash_bwd_kernel(const ItbAttnArgs a) {
  extern __shared__ __align__(128) uint8_t smem_attn[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_attn);
  __nv_bfloat16* sV = sK + 64 * D;
  __nv_bfloat16* sQ = sV + 64 * D;        // 2 buffers
  __nv_bfloat16* sdO = sQ + 2 * 64 * D;   // 2 buffers
  __nv_bfloat16* sdS = sdO + 2 * 64 * D;  // [64 n][64 m]
  float* sLse = reinterpret_cast<float*>(sdS + 64 * 64);  // 2 x 64
  float* sDelta = sLse + 2 * 64;                          // 2 x 64

  const int nb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = a.H / a.KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int n0 = nb * kBlkN;
  const int n_qblocks = (a.T + kBlkM - 1) / kBlkM;
  const int mb_first = a.causal ? nb : 0;
  const int per_head = n_qblocks - mb_first;
  const int iters = per_head * G;
  const float sl2 = a.scale * kLog2e;

  const __nv_bfloat16* kg = static_cast<const __nv_bfloat16*>(a.k) + b * a.k_batch_stride + hk * D;
  const __nv_bfloat16* vg = static_cast<const __nv_bfloat16*>(a.v) + b * a.v_batch_stride + hk * D;

  auto issue = [&](int it) {
    const int gi = it / per_head, mb = mb_first + it % per_head;
    const int h = hk * G + gi;
    const int buf = it & 1;
    const __nv_bfloat16* qg = static_cast<const __nv_bfloat16*>(a.q) + b * a.q_batch_stride + h * D;
    const __nv_bfloat16* dog =
        static_cast<const __nv_bfloat16*>(a.dout) + b * a.o_batch_stride + h * D;
    load_tile<D>(sQ + buf * 64 * D, qg, a.q_row_stride, mb * kBlkM, a.T);
    load_tile<D>(sdO + buf * 64 * D, dog, a.o_row_stride, mb * kBlkM, a.T);
    if (threadIdx.x < 64) {
      const int row = mb * kBlkM + threadIdx.x;
      const long long so = (static_cast<long long>(b) * a.H + h) * a.T + row;
      // Rows beyond the sequence get lse = +inf (probability 0) and delta = 0.
      sLse[buf * 64 + threadIdx.x] = row < a.T ? a.lse[so] * kLog2e : INFINITY;
      sDelta[buf * 64 + threadIdx.x] = row < a.T ? a.delta[so] : 0.f;
    }
  };

  load_tile<D>(sK, kg, a.k_row_stride, n0, a.T);
  load_tile<D>(sV, vg, a.v_row_stride, n0, a.T);
  if (iters > 0) issue(0);
  cp_async_commit();

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[i][e] = dv[i][e] = 0.f;

  for (int it = 0; it < iters; ++it) {
    cp_async_wait_all();
    __syncthreads();  // tiles of `it` visible; everyone is done with the buffers of it-1
    if (it + 1 < iters) {
      issue(it + 1);
      cp_async_commit();
    }
    const int gi = it / per_head, mb = mb_first + it % per_head;
    const int h = hk * G + gi;
    const int buf = it & 1;
    const __nv_bfloat16* tQ = sQ + buf * 64 * D;
    const __nv_bfloat16* tdO = sdO + buf * 64 * D;
    const float* lse = sLse + buf * 64;
    const float* delta = sDelta + buf * 64;

    // St[n, m] = K[n,:] . Q[m,:]   and   dPt[n, m] = V[n,:] . dO[m,:]
    float st[8][4], dpt[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) st[i][e] = dpt[i][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t ka[4], va[4];
      lda<D>(ka, sK, warp * 16, kk * 16);
      lda<D>(va, sV, warp * 16, kk * 16);
#pragma unroll
      for (int mb2 = 0; mb2 < 4; ++mb2) {
        uint32_t bq[4], bd[4];
        ldb_nk<D>(bq, tQ, mb2 * 16, kk * 16);
        ldb_nk<D>(bd, tdO, mb2 * 16, kk * 16);
        mma_bf16(st[2 * mb2], ka, bq[0], bq[1]);
        mma_bf16(st[2 * mb2 + 1], ka, bq[2], bq[3]);
        mma_bf16(dpt[2 * mb2], va, bd[0], bd[1]);
        mma_bf16(dpt[2 * mb2 + 1], va, bd[2], bd[3]);
      }
    }
    // Pt = exp(St * scale - lse[m]); dSt = Pt * (dPt - delta[m]).  Element e of block i sits at
    // key row n = 16*warp + g + 8*(e>>1), query column m = 8*i + 2*t4 + (e&1).
    const bool diag = a.causal && (mb == nb);
    uint32_t pa[4][4], dsa[4][4];  // A fragments (16 n x 16 m) for the four m k-steps
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float pv[4], dsv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ml = i * 8 + t4 * 2 + (e & 1);
        const int nl = warp * 16 + g + ((e >> 1) << 3);
        float p = exp2f(st[i][e] * sl2 - lse[ml]);
        const bool masked = (n0 + nl >= a.T) || (diag && nl > ml);
        p = masked ? 0.f : p;
        pv[e] = p;
        dsv[e] = p * (dpt[i][e] - delta[ml]);
      }
      pa[i >> 1][(i & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
      pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
      dsa[i >> 1][(i & 1) * 2 + 0] = pack_bf16(dsv[0], dsv[1]);
      dsa[i >> 1][(i & 1) * 2 + 1] = pack_bf16(dsv[2], dsv[3]);
      // dSt to shared memory, layout [n][m], for the dQ product of the other warps.
      *reinterpret_cast<uint32_t*>(sdS + sw_off<64>(warp * 16 + g, i) + t4 * 2) =
          pack_bf16(dsv[0], dsv[1]);
      *reinterpret_cast<uint32_t*>(sdS + sw_off<64>(warp * 16 + g + 8, i) + t4 * 2) =
          pack_bf16(dsv[2], dsv[3]);
    }
    // dV[n, d] += Pt[n, m] dO[m, d];  dK[n, d] += dSt[n, m] Q[m, d]
#pragma unroll
    for (int mk = 0; mk < 4; ++mk) {
#pragma unroll
      for (int db2 = 0; db2 < D / 16; ++db2) {
        uint32_t bd[4], bq[4];
        ldb_kn<D>(bd, tdO, mk * 16, db2 * 16);
        ldb_kn<D>(bq, tQ, mk * 16, db2 * 16);
        mma_bf16(dv[2 * db2], pa[mk], bd[0], bd[1]);
        mma_bf16(dv[2 * db2 + 1], pa[mk], bd[2], bd[3]);
        mma_bf16(dk[2 * db2], dsa[mk], bq[0], bq[1]);
        mma_bf16(dk[2 * db2 + 1], dsa[mk], bq[2], bq[3]);
      }
    }
    __syncthreads();  // dSt of all four warps is in shared memory
    // dQ[m, d] += scale * sum_n dS[m, n] K[n, d]; warp w takes query rows [16w, 16w+16).
    float* dqg = a.dq_accum +
                 ((static_cast<long long>(b) * a.T + mb * kBlkM) * a.H + h) * D;
#pragma unroll
    for (int dh = 0; dh < D / 64; ++dh) {
      float dq[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) dq[i][e] = 0.f;
#pragma unroll
      for (int kn = 0; kn < 4; ++kn) {
        uint32_t af[4];
        lda_km<64>(af, sdS, kn * 16, warp * 16);
#pragma unroll
        for (int db2 = 0; db2 < 4; ++db2) {
          uint32_t bk[4];
          ldb_kn<D>(bk, sK, kn * 16, dh * 64 + db2 * 16);
          mma_bf16(dq[2 * db2], af, bk[0], bk[1]);
          mma_bf16(dq[2 * db2 + 1], af, bk[2], bk[3]);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int ml = warp * 16 + g + r * 8;
          if (mb * kBlkM + ml < a.T) {
            float* p = dqg + static_cast<long long>(ml) * a.H * D + dh * 64 + i * 8 + t4 * 2;
            asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p),
                         "f"(dq[i][2 * r] * a.scale), "f"(dq[i][2 * r + 1] * a.scale)
                         : "memory");
          }
        }
    }
  }

  // Write dK (scaled) and dV for this warp's 16 key rows.
  __nv_bfloat16* dkg = static_cast<__nv_bfloat16*>(a.dk) + b * a.k_batch_stride + hk * D;
  __nv_bfloat16* dvg = static_cast<__nv_bfloat16*>(a.dv) + b * a.v_batch_stride + hk * D;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = n0 + warp * 16 + g + r * 8;
    if (row < a.T) {
#pragma unroll
      for (int db = 0; db < D / 8; ++db) {
        *reinterpret_cast<uint32_t*>(dkg + static_cast<long long>(row) * a.k_row_stride + db * 8 +
                                     t4 * 2) =
            pack_bf16(dk[db][2 * r] * a.scale, dk[db][2 * r + 1] * a.scale);
        *reinterpret_cast<uint32_t*>(dvg + static_cast<long long>(row) * a.v_row_stride + db * 8 +
                                     t4 * 2) = pack_bf16(dv[db][2 * r], dv[db][2 * r + 1]);
      }
    }
  }
}

template <int D>
static int attn_fwd_launch(const ItbAttnArgs* a, cudaStream_t s) {
  constexpr int smem = 5 * 64 * D * 2;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid((a->T + kBlkM - 1) / kBlkM, a->H, a->B);
  flash_fwd_kernel<D><<<grid, kAttnThreads, smem, s>>>(*a);
  return static_cast<int>(cudaGetLastError());
}

template <int D>
static int attn_bwd_launch(const ItbAttnArgs* a, cudaStream_t s) {
  constexpr int smem = 6 * 64 * D * 2 + 64 * 64 * 2 + 4 * 64 * 4;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const long long nrow = static_cast<long long>(a->B) * a->T * a->H;
  cudaError_t e = cudaMemsetAsync(a->dq_accum, 0, nrow * D * sizeof(float), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  attn_delta_kernel<D><<<static_cast<int>((nrow * 32 + 255) / 256), 256, 0, s>>>(*a);
  dim3 grid((a->T + kBlkN - 1) / kBlkN, a->KV, a->B);
  flash_bwd_kernel<D><<<grid, kAttnThreads, smem, s>>>(*a);
  const long long nvec = nrow * (D / 4);
  attn_dq_convert_kernel<D><<<static_cast<int>((nvec + 255) / 256), 256, 0, s>>>(*a);
  return static_cast<int>(cudaGetLastError());
}

static int attn_check(const ItbAttnArgs* a) {
  if (a->H % a->KV) return -3;
  if ((a->q_row_stride | a->k_row_stride | a->v_row_stride | a->o_row_stride | a->q_batch_stride |
       a->k_batch_stride | a->v_batch_stride | a->o_batch_stride) & 7)
    return -2;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) |
       reinterpret_cast<uintptr_t>(a->v) | reinterpret_cast<uintptr_t>(a->o)) & 15)
    return -2;
  return 0;
}

}  // namespace itb

extern "C" int itb_flash_attn_fwd(const ItbAttnArgs* a, cudaStream_t s) {
  if (a->B <= 0 || a->T <= 0) return 0;
  if (int rc = itb::attn_check(a)) return rc;
  if (a->D == 64) return itb::attn_fwd_launch<64>(a, s);
  if (a->D == 128) return itb::attn_fwd_launch<128>(a, s);
  return -4;
}

extern "C" int itb_flash_attn_bwd(const ItbAttnArgs* a, cudaStream_t s) {
  if (a->B <= 0 || a->T <= 0) return 0;
  if (int rc = itb::attn_check(a)) return rc;
  if ((reinterpret_cast<uintptr_t>(a->dq) | reinterpret_cast<uintptr_t>(a->dk) |
       reinterpret_cast<uintptr_t>(a->dv) | reinterpret_cast<uintptr_t>(a->dout)) & 15)
    return -2;
  if (a->D == 64) return itb::attn_bwd_launch<64>(a, s);
  if (a->D == 128) return itb::attn_bwd_launch<128>(a, s);
  return -4;
}
