// C launch interface of the single-GPU sm_100a kernels.  Everything takes raw device pointers and
// a stream, returns 0 on success (a CUDA error code or a negative argument error otherwise) and
// allocates nothing: callers own inputs, outputs and scratch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// dtype codes used across the interface
enum { kItbF32 = 0, kItbBF16 = 1 };

// ------------------------------------------------------------------ GEMM (tcgen05)
enum {
  kGemmOutF32 = 1,     // C is fp32 (default bf16)
  kGemmAtomic = 2,     // C += A*B with vector atomics, contraction split across CTAs (needs OutF32)
  kGemmAccum = 4,      // C += A*B, no split (needs OutF32)
  kGemmBias = 8,       // + bias[n]
  kGemmResidual = 16,  // + residual[m,n] (same dtype as C)
  kGemmGeluDual = 32,  // C = h (bf16), C2 = gelu_tanh(h) (bf16)
  kGemmDGelu = 64,     // C = (A*B) * gelu_tanh'(aux[m,n])
  // Timing probes of the CTA-pair pipeline (results are meaningless): the same launch with the
  // operand loads left out (the MMA warp finds every stage "full" at once: issue rate + shared-memory
  // reads of the tensor core alone) or with the MMAs left out (TMA fill rate of the ring alone).
  kGemmProbeNoLoad = 1 << 20,
  kGemmProbeNoMma = 1 << 21,
};

typedef struct {
  int M, N, K;            // C is M x N, contraction length K
  const void* A;          // bf16.  K-major: [M, K] rows lda apart.  MN-major: [K, M] rows lda apart.
  long long lda;
  int a_mn_major;
  const void* B;          // bf16.  K-major: [N, K] rows ldb apart.  MN-major: [K, N] rows ldb apart.
  long long ldb;
  int b_mn_major;
  void* C;
  long long ldc;
  void* C2;
  const float* bias;
  const void* residual;
  long long ldr;
  const void* aux;
  long long ld_aux;
  int flags;
  int split_k;            // 0 = choose
  int* err;               // device status word (must be zero before the launch)
} ItbGemmArgs;

int itb_gemm_bf16(const ItbGemmArgs* args, cudaStream_t stream);
// Same contract, computed by CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles per pair).
int itb_gemm_bf16_pair(const ItbGemmArgs* args, cudaStream_t stream);

// ------------------------------------------------------------------ normalisation
// y = (x - mean) * rstd * gamma + beta over the last dimension C of [rows, C].
int itb_layernorm_fwd(const void* x, int x_dtype, const float* gamma, const float* beta, void* y,
                      int y_dtype, float* mean, float* rstd, int rows, int C, float eps,
                      cudaStream_t stream);
// dx = LN'(dy); dgamma/dbeta are reduced in two stages through `partial` (fp32,
// [itb_norm_partial_rows(rows), 3*C]) and ADDED to dgamma/dbeta when accumulate != 0.
int itb_norm_partial_rows(int rows);
int itb_layernorm_bwd(const void* dy, int dy_dtype, const void* x, int x_dtype, const float* gamma,
                      const float* mean, const float* rstd, void* dx, int dx_dtype, float* dgamma,
                      float* dbeta, float* partial, int rows, int C, int accumulate,
                      cudaStream_t stream);
// The norm on a residual stream: dx = LN'(dy) + dres, where dres (dtype of dx) is the gradient that
// reaches the stream past the norm; when dres_sum is not null, dres_sum[c] (+)= sum over rows of
// dres (the bias gradient of the projection that wrote into the stream).  `accumulate` is a bit mask:
// bit 0 dgamma, bit 1 dbeta, bit 2 dres_sum are added to instead of overwritten.
int itb_layernorm_bwd_res(const void* dy, int dy_dtype, const void* x, int x_dtype, const float* gamma,
                          const float* mean, const float* rstd, const void* dres, void* dx, int dx_dtype,
                          float* dgamma, float* dbeta, float* dres_sum, float* partial, int rows, int C,
                          int accumulate, cudaStream_t stream);
// y = x * rsqrt(mean(x^2) + eps) * gamma
int itb_rmsnorm_fwd(const void* x, int x_dtype, const float* gamma, void* y, int y_dtype,
                    float* rstd, int rows, int C, float eps, cudaStream_t stream);
int itb_rmsnorm_bwd(const void* dy, int dy_dtype, const void* x, int x_dtype, const float* gamma,
                    const float* rstd, void* dx, int dx_dtype, float* dgamma, float* partial,
                    int rows, int C, int accumulate, cudaStream_t stream);
int itb_rmsnorm_bwd_res(const void* dy, int dy_dtype, const void* x, int x_dtype, const float* gamma,
                        const float* rstd, const void* dres, void* dx, int dx_dtype, float* dgamma,
                        float* dres_sum, float* partial, int rows, int C, int accumulate,
                        cudaStream_t stream);

// ------------------------------------------------------------------ activations
// tanh-GELU and SiLU-gated product on bf16 or fp32 tensors of n elements.
int itb_gelu_fwd(const void* x, void* y, int dtype, long long n, cudaStream_t stream);
int itb_gelu_bwd(const void* dy, const void* x, void* dx, int dtype, long long n,
                 cudaStream_t stream);
// out[r, f] = a[r, f] * silu(b[r, f]); a and b may be column blocks of one [rows, ld] matrix.
int itb_swiglu_fwd(const void* a, const void* b, long long ld_in, void* out, long long ld_out,
                   int dtype, int rows, int F, cudaStream_t stream);
int itb_swiglu_bwd(const void* dout, long long ld_dout, const void* a, const void* b,
                   long long ld_in, void* da, void* db, long long ld_dab, int dtype, int rows,
                   int F, cudaStream_t stream);

// ------------------------------------------------------------------ rotary embedding
// In-place rotation of interleaved (even, odd) pairs of q and k heads inside a packed
// [B, T, (H + 2*KV) * D] bf16 buffer.  freqs is [T_max, D/2, 2] fp32 (cos, sin); position of row t
// is pos0 + t.  inverse != 0 applies the transpose rotation (backward).
int itb_rope_inplace(void* qkv, int dtype, const float* freqs, int B, int T, int n_rot_heads,
                     int D, long long row_stride, int pos0, int inverse, cudaStream_t stream);

// ------------------------------------------------------------------ embedding
// out[b,t,:] = wte[idx[b,t],:] (+ wpe[pos0 + t,:]); tables fp32 or bf16, output bf16 or fp32.
int itb_embedding_fwd(const long long* idx, const void* wte, const void* wpe, int table_dtype,
                      void* out, int out_dtype, int B, int T, int C, int pos0, int vocab_start,
                      int vocab_end, cudaStream_t stream);
// dwte[idx,:] += dout (fp32 atomics, one warp per token), dwpe[t,:] += sum_b dout[b,t,:].
int itb_embedding_bwd(const long long* idx, const void* dout, int dout_dtype, float* dwte,
                      float* dwpe, int B, int T, int C, int pos0, int vocab_start, int vocab_end,
                      cudaStream_t stream);

// ------------------------------------------------------------------ softmax cross-entropy
// Per-row loss and log-sum-exp over logits [rows, V] (row stride ld >= V); the mean over rows is
// accumulated on the device into *loss_mean (must be zeroed by the caller).  Rows whose target
// is < 0 are ignored (loss 0) but still counted in the mean's denominator `rows`.
int itb_ce_fwd(const void* logits, int dtype, long long ld, const long long* target, float* row_loss,
               float* lse, float* loss_mean, int rows, int V, cudaStream_t stream);
// dlogits = (softmax - onehot) * (*grad_out) / rows, written over the logits buffer (columns
// V..ld-1 are zeroed).  softmax = exp(logit - lse[row]), so a vocabulary shard passes the GLOBAL
// log-sum-exp.  ignore_oob != 0: rows whose target is outside [0, V) get a zero gradient;
// ignore_oob == 0: they get the softmax term without the one-hot (the target lives on another shard).
int itb_ce_bwd(void* logits, int dtype, long long ld, const long long* target, const float* lse,
               const float* grad_out, int rows, int V, int ignore_oob, cudaStream_t stream);

// ------------------------------------------------------------------ optimizer
// One launch over a flat buffer: Adam / AdamW with fp32 master weights and optional bf16 shadow.
//   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p -= lr * (m/bc1 / (sqrt(v/bc2) + eps) + wd * p)
// grad_scale multiplies g first (1/dp, 1/accum).  g is fp32 or bf16.  dev_hyper (optional, device
// memory, [lr, 1/bc1, 1/bc2]) overrides lr / bc1 / bc2 at run time: a captured CUDA graph keeps the
// pointer and the host refreshes the three floats before every replay.
int itb_adamw(float* p, const void* g, int g_dtype, float* m, float* v, void* shadow_bf16,
              long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
              float grad_scale, const float* dev_hyper, cudaStream_t stream);
int itb_sgd(float* p, const void* g, int g_dtype, void* shadow_bf16, long long n, float lr,
            float grad_scale, cudaStream_t stream);
// hyper = [lr, 1/bc1, 1/bc2, t] in device memory: t += 1 and the bias corrections are recomputed
// on the device (graph-replayable step counter).
int itb_adam_advance(float* hyper, float b1, float b2, cudaStream_t stream);

// ------------------------------------------------------------------ utilities
int itb_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
             cudaStream_t stream);
// out[n] (+)= sum_m x[m, n]; x bf16 or fp32 [rows, N]; two-stage through `partial`
// (fp32 [itb_colsum_partial_rows(rows), N]).
int itb_colsum_partial_rows(int rows);
int itb_colsum(const void* x, int dtype, long long ld, float* out, float* partial, int rows, int N,
               int accumulate, cudaStream_t stream);

// ------------------------------------------------------------------ flash attention
// q [B, T, H, D], k/v [B, T, KV, D] bf16 with explicit row (token) and batch strides in elements
// (so they can alias a packed qkv buffer); o [B, T, H, D] contiguous; lse [B, H, T] fp32.
typedef struct {
  const void *q, *k, *v;
  void* o;
  float* lse;
  long long q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  long long q_batch_stride, k_batch_stride, v_batch_stride, o_batch_stride;
  int B, T, H, KV, D;
  float scale;
  int causal;
  // backward only
  const void* dout;       // [B, T, H, D], row/batch strides = o's
  void *dq, *dk, *dv;     // same strides as q, k, v
  float* delta;           // scratch [B, H, T] fp32
  float* dq_accum;        // scratch [B, T, H, D] fp32 (zeroed by the call)
  // tensor-core backward only, optional: scratch [2][B, T, KV, D] fp32 (zeroed by the call).  When it is
  // there and the grid of one CTA per (key tile, KV head, batch) would fill less than half of the
  // SMs, itb_flash_attn_bwd_parts() CTAs share each key tile and sum their dK / dV here.
  float* dkv_accum;
  int bwd_parts;          // set by the launcher
} ItbAttnArgs;
// How many CTAs the tensor-core backward puts on one (key tile, KV head, batch); 1 = the scratch
// buffer `dkv_accum` is not needed.
int itb_flash_attn_bwd_parts(int B, int T, int H, int KV, int causal);

int itb_flash_attn_fwd(const ItbAttnArgs* args, cudaStream_t stream);
int itb_flash_attn_bwd(const ItbAttnArgs* args, cudaStream_t stream);
// Same contract on the tcgen05 tensor cores (128 x 128 tiles, accumulators in TMEM, TMA operands).
// `err` is a device status word (zero before the launch) that receives a code when a wait gives up.
int itb_flash_attn_bwd_tc(const ItbAttnArgs* args, int* err, cudaStream_t stream);
int itb_flash_attn_fwd_tc(const ItbAttnArgs* args, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
