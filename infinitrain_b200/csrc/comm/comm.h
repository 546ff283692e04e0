// C launch interface of the multi-GPU (NVLink / NVSwitch) kernels.  Buffers are symmetric-memory
// allocations: `ItbPeerPtrs::p[r]` is rank r's copy of the buffer mapped into this process and the
// optional multicast pointer addresses all copies at once (NVLS).  Nothing here allocates.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { kItbMaxRanks = 8, kItbMaxCommBlocks = 32 };

typedef struct {
  void* p[kItbMaxRanks];
} ItbPeerPtrs;

typedef struct {
  float lr, beta1, beta2, eps, weight_decay, inv_bc1, inv_bc2, grad_scale;
} ItbAdamHyper;

// Number of thread blocks (= flag channels) a launch over `n_elements_per_rank` elements uses.
int itb_comm_blocks(long long n_elements_per_rank);

// In-place all-reduce of fp32 elements [off, off+n) followed by a multiplication with `scale`
// (1/world for an average).  `flags` are the symmetric flag words ([channels][kItbMaxRanks] int32
// per rank); channels ch0 .. ch0 + itb_comm_blocks(...) - 1 are used; `epoch` must grow by 2 between
// launches that use the same channels.  mc == NULL selects the peer-pointer path.  epoch_ctr
// (optional, device memory of THIS GPU, one int per channel) replaces `epoch` by a counter the
// kernel reads and advances itself, so that the launch can be replayed from a CUDA graph.
int itb_nvl_allreduce_scale(const ItbPeerPtrs* bufs, void* mc, const ItbPeerPtrs* flags,
                            long long off, long long n, int rank, int world, int ch0, int epoch,
                            float scale, int* err, int* epoch_ctr, cudaStream_t stream);

// Bucket [off, off+n) of the flat gradient / parameter / bf16-shadow buffers: reduce every rank's
// gradients for this rank's 1/world shard, scale, AdamW on the shard (m, v: shard-local fp32 state),
// then write the updated fp32 weights and their bf16 copy into EVERY rank's buffers.
int itb_nvl_rs_adamw_bcast(const ItbPeerPtrs* grads, const void* mc_grads, const ItbPeerPtrs* params,
                           void* mc_params, const ItbPeerPtrs* shadows, void* mc_shadows, float* m,
                           float* v, const ItbPeerPtrs* flags, long long off, long long n, int rank,
                           int world, int ch0, int epoch, const ItbAdamHyper* hyper, int* err,
                           int* epoch_ctr, const float* dev_hyper, cudaStream_t stream);

// Vocab-parallel cross-entropy: merges every rank's per-row (log-sum-exp of its vocabulary shard,
// target logit if owned) into the global log-sum-exp and the row loss inside one kernel that
// exchanges the pairs through `bufs` (symmetric, float2 [world][rows_cap] per rank) and meets the
// other ranks at flag barriers.  row_loss is the local pass's lse_local - target logit (owner rows).
// Uses channels ch0 .. ch0 + kItbMaxCommBlocks - 1; epochs come from epoch_ctr (device memory).
int itb_nvl_ce_merge(const ItbPeerPtrs* bufs, const ItbPeerPtrs* flags, const float* lse_local,
                     const float* row_loss, const long long* t_local, int vocab_valid, float* lse_out,
                     float* loss_out, int rows, int rows_cap, int rank, int world, int ch0, int* err,
                     int* epoch_ctr, cudaStream_t stream);

// One thread polls `*flag` until it is >= target or `limit` polls have passed; a time-out writes
// `code` into `*err` and the kernel returns (the bounded wait of the flag protocols, on its own).
int itb_wait_flag(const int* flag, int target, unsigned limit, int code, int* err, cudaStream_t stream);

// ---- tensor-parallel GEMMs fused with all-gather / reduce-scatter (tp_gemm.cu)
// Activations are [batch * T, cols] with row = b * T + t; under sequence parallelism rank s holds
// t in [s * Tl, (s + 1) * Tl), Tl = T / world (a multiple of 256).  All pointer tables are
// symmetric-memory addresses of the same buffer on every rank; counters marked "this GPU" are
// ordinary device memory that the kernels advance themselves (replayable from a CUDA graph).
enum { kItbTpPush = 1, kItbTpGateA = 2, kItbTpScatter = 4, kItbTpBroadcast = 8 };

typedef struct {
  int mode;                   // kItbTpPush | kItbTpGateA | kItbTpScatter
  int rank, world;
  int T, Tl, batch;
  ItbPeerPtrs started;        // int32[world] on each rank: 1 + index of the latest launch rank r began
  int* launch_ctr;            // this GPU
  unsigned* cta_done;         // this GPU, zero between launches
  // push of the local shard [batch * Tl, push_cols] bf16 into every rank's gathered [batch * T, push_cols]
  const void* push_src;
  int push_cols;
  ItbPeerPtrs gather;
  void* gather_mc;            // multicast address of the gathered buffer or NULL
  ItbPeerPtrs push_arrive;    // int32[world] on each rank
  int* push_total;            // this GPU: arrivals per source the pushes so far add up to
  int push_lag;               // launches since the gathered buffer was last used (large = never)
  // loads of A (the gathered buffer) wait for the shard they read
  const int* gate_arrive;     // this rank's arrival counters of that buffer
  const int* gate_total;      // this GPU: that buffer's push_total
  int gate_includes_this_launch;
  // reduce-scatter of the output rows: slab [world][batch * Tl, N] bf16 on each rank
  ItbPeerPtrs slab;
  ItbPeerPtrs rs_arrive;      // int32[world] on each rank
  int* rs_total;              // this GPU
  int rs_lag;
  void* rs_out;               // [batch * Tl, N] bf16 or fp32
  long long rs_ld_out;
  int rs_out_f32;
  const float* rs_bias;       // optional, added once after the sum
  const void* rs_residual;    // optional bf16 [batch * Tl, N]
  long long rs_ld_res;
  // kItbTpBroadcast (together with kItbTpScatter): the summed rows are written to every rank's full
  // [batch * T, N] bf16 buffer instead of rs_out -- a GEMM + all-reduce.  A consumer waits for
  // `*ar_total` arrivals of every rank on ar_arrive (itb_tp_wait) before it reads the buffer.
  ItbPeerPtrs ar_out;
  void* ar_mc;
  ItbPeerPtrs ar_arrive;      // int32[world] on each rank
  int* ar_total;              // this GPU
  int ar_lag;
} ItbTpArgs;

// `gemm` is an ItbGemmArgs (kernels/kernels.h); bf16 output only.  With kItbTpScatter the GEMM's own
// C / bias / residual are unused.  Returns 0, a CUDA error, or a negative argument error.
int itb_tp_gemm(const void* gemm, const ItbTpArgs* tp, cudaStream_t stream);
// Thread blocks the launch for an M x N output uses.
int itb_tp_gemm_ctas(int M, int N);
// Holds the stream until `*total` arrivals of every rank have been counted.
int itb_tp_wait(const int* arrive, const int* total, int world, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
