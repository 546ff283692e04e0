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

#ifdef __cplusplus
}
#endif
