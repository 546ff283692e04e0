// bf16 GEMM on the 5th-generation tensor cores (sm_100a): C[M,N] = A[M,K] * B[N,K]^T with fp32
// accumulation in TMEM, operands staged in shared memory by TMA (128-byte swizzle, no cluster
// multicast), tcgen05.mma issued by one elected thread, tcgen05.ld in the epilogue warps.
//
// It replaces the reference's cuBLAS calls plus the separate bias / activation / cast / add kernels
// (reference: infini_train/src/kernels/cuda/common/gemm.cu:45-75, linear.cu:30-324,
// matmul.cu:16-216): bias add, residual add, tanh-GELU (forward: pre-activation and activation are
// both stored; backward: multiply by gelu'(h)), fp32 output and split-K accumulation for weight
// gradients all live in the epilogue.
//
// Operand layouts.  "K-major" = the contraction dimension is contiguous in memory; "MN-major" =
// the M (or N) dimension is contiguous.  The three products of a Linear layer map to
//   forward   y  = x W^T        A = x  [M,K] K-major,  B = W [N,K] K-major
//   dgrad     dx = dy W         A = dy [M,N] K-major,  B = W [N,K] read as MN-major (contraction N)
//   wgrad     dW = dy^T x       A = dy [M,N] MN-major, B = x [M,K] MN-major (contraction M)
//
// Kernel shape: persistent, one CTA per SM, 192 threads = 1 TMA warp + 1 MMA warp + 4 epilogue
// warps; tile 128 x BN x 64 with a 4-deep shared-memory ring and two TMEM accumulators so that
// the epilogue of tile i overlaps the main loop of tile i+1.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <mutex>
#include <unordered_map>

#include "../common/ptx.cuh"
#include "gemm_epilogue.cuh"
#include "kernels.h"

namespace itb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  // full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], tmem holder, abort flag
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 16;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                         const __grid_constant__ CUtensorMap tma_b, const GemmDev p) {
  using L = SmemLayout<BN>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // The dynamic shared window is only guaranteed 16-byte aligned: round up to 1024 (swizzle atom).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_holder + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512: a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  const int total_tiles = p.tiles_m * p.tiles_n * p.split_k;
  const int kb_per_split = (p.k_blocks + p.split_k - 1) / p.split_k;
  constexpr int kGroupM = 16;

  auto decode_tile = [&](int t, int& tm, int& tn, int& kb0, int& kb1) {
    int ks = t % p.split_k;
    int t2 = t / p.split_k;
    int width = kGroupM * p.tiles_n;
    int group = t2 / width;
    int first_m = group * kGroupM;
    int gsz = min(p.tiles_m - first_m, kGroupM);
    int in_group = t2 - group * width;
    tm = first_m + in_group % gsz;
    tn = in_group / gsz;
    kb0 = ks * kb_per_split;
    kb1 = min(p.k_blocks, kb0 + kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tm, tn, kb0, kb1;
        decode_tile(t, tm, tn, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1) || *abort_flag) {
            atomicCAS(p.err, 0, 101);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(sa + i * (64 * BK * 2), &tma_a, &full_bar[stage], tm * BM + i * 64,
                          kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sb + i * (64 * BK * 2), &tma_b, &full_bar[stage], tn * BN + i * 64,
                          kb * BK);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // Loads still in flight land in this CTA's shared memory; the MMA warp consumes every stage
      // that was issued before it leaves its loop, so nothing is outstanding at exit on the normal
      // path.  On the abort path wait (bounded) for the stages that were issued.
      if (!ok) {
        for (int s = 0; s < kStages; ++s) mbar_wait(&full_bar[s], phase);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16_f32(BM, BN, A_MN, B_MN);
    // One thread runs the loop: wait for a stage, issue its MMAs, release it with a commit.  The
    // operands arrive through the async proxy, so the k-loop needs no tcgen05 fence; the fence after a
    // thread synchronisation belongs where the epilogue warps hand an accumulator back.
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase0 = 0, acc_phase1 = 0;
    int local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok && lane == 0; t += gridDim.x, ++local) {
      int tm, tn, kb0, kb1;
      decode_tile(t, tm, tn, kb0, kb1);
      const int acc = local & 1;
      if (kb1 <= kb0) continue;  // empty K-split: mirrors the epilogue's skip
      // Wait until the epilogue has drained this accumulator (first use passes immediately).
      const uint32_t ap = acc ? acc_phase1 : acc_phase0;
      if (!mbar_wait(&tmem_empty[acc], ap ^ 1) || *abort_flag) {
        atomicCAS(p.err, 0, 102);
        *abort_flag = 1;
        break;
      }
      if (acc) acc_phase1 ^= 1; else acc_phase0 ^= 1;
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + acc * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) {
          atomicCAS(p.err, 0, 103);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
        const uint32_t sb = sa + L::kABytes;
        const uint64_t adesc0 = A_MN ? make_smem_desc_sw128(sa, 64 * BK * 2, 1024)
                                     : make_smem_desc_sw128(sa, 16, 1024);
        const uint64_t bdesc0 = B_MN ? make_smem_desc_sw128(sb, 64 * BK * 2, 1024)
                                     : make_smem_desc_sw128(sb, 16, 1024);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // K-major: 16 elements = 32 bytes along the swizzled row.
          // MN-major: 16 k-rows = 2 groups of 8 rows x 128 bytes = 2048 bytes.
          const uint64_t adesc = adesc0 + (A_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
          const uint64_t bdesc = bdesc0 + (B_MN ? (k * 2048) >> 4 : (k * 32) >> 4);
          umma_f16_ss(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
        if (kb == kb1 - 1) umma_commit(&tmem_full[acc]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
      int tm, tn, kb0, kb1;
      decode_tile(t, tm, tn, kb0, kb1);
      const int acc = local & 1;
      if (kb1 <= kb0) {
        // Empty K-split (can only happen when split_k does not divide the k-blocks): the MMA warp
        // committed nothing, so there is nothing to wait for or to add.
        continue;
      }
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc]) || *abort_flag) {
        if (lane == 0) atomicCAS(p.err, 0, 104);
        *abort_flag = 1;
        break;
      }
      acc_phase[acc] ^= 1;
      tc_fence_after_sync();
      const int row = tm * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        const int col0 = tn * BN + c;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr0 + c, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        gemm_epilogue_chunk(p, row, row_ok, col0, v);
      }
      // All of this thread's TMEM reads have completed (wait::ld above): hand the accumulator back.
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Driver-API calls need a context bound to the calling thread.  A thread that has only been handed
// work (an autograd worker whose first CUDA operation is one of these GEMMs, on device 0 where no
// cudaSetDevice was needed) has none yet; one runtime call binds the primary context.
static void ensure_context_on_this_thread() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

static EncodeTiledFn get_encode_fn() {
  ensure_context_on_this_thread();
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows `ld` elements apart.
int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 3-D bf16 tensor map [d2][d1][inner] with element strides ld1 (between d1 rows) and ld2 (between d2
// slabs); boxes are box_inner x box_d1 x 1, 128-byte swizzle.
int make_tmap_bf16_3d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t d1, uint64_t d2,
                      uint64_t ld1, uint64_t ld2, uint32_t box_inner, uint32_t box_d1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {inner, d1, d2};
  cuuint64_t strides[2] = {ld1 * 2, ld2 * 2};
  cuuint32_t box[3] = {box_inner, box_d1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 3-D fp32 tensor map [d2][d1][inner], boxes of 32 columns (128 bytes) x box_d1 x 1, 128-byte swizzle.
int make_tmap_f32_3d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t d1, uint64_t d2,
                     uint64_t ld1, uint64_t ld2, uint32_t box_d1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {inner, d1, d2};
  cuuint64_t strides[2] = {ld1 * 4, ld2 * 4};
  cuuint32_t box[3] = {32, box_d1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// fp32 matrix, box of 32 columns (128 bytes) x box_outer rows, 128-byte swizzle.
int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {32, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmDev& p, int grid,
                  cudaStream_t stream) {
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN>;
  constexpr int smem = SmemLayout<BN>::kTotal + 1024;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  kern<<<grid, kGemmThreads, smem, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace itb

extern "C" int itb_gemm_bf16(const ItbGemmArgs* a, cudaStream_t stream) {
  using namespace itb;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  // TMA needs 16-byte aligned bases and row strides.
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) ||
      (a->lda % 8) || (a->ldb % 8))
    return -2;
  CUtensorMap ta, tb;
  int rc;
  if (!a->a_mn_major)
    rc = make_tmap_bf16_2d(&ta, a->A, a->K, a->M, a->lda, 64, BM);
  else
    rc = make_tmap_bf16_2d(&ta, a->A, a->M, a->K, a->lda, 64, 64);
  if (rc) return rc;
  const int BN = 256;
  if (!a->b_mn_major)
    rc = make_tmap_bf16_2d(&tb, a->B, a->K, a->N, a->ldb, 64, BN);
  else
    rc = make_tmap_bf16_2d(&tb, a->B, a->N, a->K, a->ldb, 64, 64);
  if (rc) return rc;

  GemmDev p;
  p.staged = 0;
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.k_blocks = (a->K + BK - 1) / BK;
  p.tiles_m = (a->M + BM - 1) / BM;
  p.tiles_n = (a->N + BN - 1) / BN;
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
  int split = 1;
  if (a->flags & kGemmAtomic) {
    // Split the contraction so that a small output (a weight gradient) still fills the machine;
    // every split adds its partial product with vector atomics into the fp32 output.
    const int tiles = p.tiles_m * p.tiles_n;
    const int sms = num_sms();
    split = a->split_k > 0 ? a->split_k : (2 * sms + tiles - 1) / tiles;
    const int max_split = p.k_blocks / 4 > 0 ? p.k_blocks / 4 : 1;
    if (split > max_split) split = max_split;
    if (split < 1) split = 1;
    // Make every split non-empty.
    const int per = (p.k_blocks + split - 1) / split;
    split = (p.k_blocks + per - 1) / per;
  }
  p.split_k = split;
  const int total = p.tiles_m * p.tiles_n * split;
  const int grid = total < num_sms() ? total : num_sms();
  const bool amn = a->a_mn_major, bmn = a->b_mn_major;
  if (!amn && !bmn) return launch<256, false, false>(ta, tb, p, grid, stream);
  if (!amn && bmn) return launch<256, false, true>(ta, tb, p, grid, stream);
  if (amn && bmn) return launch<256, true, true>(ta, tb, p, grid, stream);
  return launch<256, true, false>(ta, tb, p, grid, stream);
}
