"""Options of DistributedDataParallel (reference:
infini_train/include/nn/parallel/ddp/distributed_data_parallel_config.h:12-66)."""
from __future__ import annotations

from dataclasses import dataclass

kFirstBucketCapMB = 1
kNormalBucketCapMB = 25


@dataclass
class DistributedDataParallelConfig:
    # Reducer (ZeRO-0): size-capped buckets, first bucket smaller so communication starts early.
    first_bucket_cap_mb: int = kFirstBucketCapMB
    normal_bucket_cap_mb: int = kNormalBucketCapMB
    gradient_as_bucket_view: bool = True
    gradient_bucketing_enabled: bool = True
    # Distributed optimizer (ZeRO >= 1)
    overlap_grad_reduce: bool = True
    zero_stage: int = 0
    overlap_param_gather: bool = True
    average_in_collective: bool = True
    check_for_nan_in_grad: bool = False
    check_for_large_grads: bool = False
    num_distributed_optimizer_instances: int = 1
    bucket_size_in_elements: int = 1_000_000
    pad_buckets_for_high_nccl_busbw: bool = False
    # Use the NVLink kernels of parallel.symm (NVLS multimem reduce + fused AdamW) instead of NCCL
    # for the bucket collectives when the group lives on one NVSwitch domain.
    use_fused_nvlink_kernels: bool = False
