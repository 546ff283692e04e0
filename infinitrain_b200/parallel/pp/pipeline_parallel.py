"""Pipeline parallelism: stage, schedule executor and the ``PipelineParallel`` module.

Reference: infini_train/src/nn/parallel/pp/{pipeline_parallel,pipeline_stage,pipeline_schedule}.cc.
``TrainStep`` splits the batch into micro-batches, zeroes gradients, walks the task list (1F1B /
interleaved by default, GPipe selectable) and steps the optimizer; it returns the summed
``loss / n`` on the last stage and 0 elsewhere.

Transfers are organised by STEP of the task table, not by task: after the tasks of step b every stage
runs one exchange that holds its sends of what step b produced and its receives of what the
neighbours produced in step b, all in one batched point-to-point call.  Two neighbours that owe each
other a tensor in the same step (an activation one way, a gradient the other: the steady state of
1F1B) therefore cannot block one another, and an exchange of step b depends only on exchanges of
earlier steps, whatever the transport buffers.  A tensor that arrives before its consumer's step
waits in a dictionary.  With data parallelism each chunk is a DistributedDataParallel module and
gradient synchronisation is armed only for the last micro-batch.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import List, Optional, Sequence

import torch

from ...autocast import AutocastGuard
from ...datatype import DataType, to_torch_dtype
from ...nn.layers import Sequential
from ...nn.module import Module, kPPChunkNamePrefix, kPPFirstStageName, kPPLastStageName
from .. import global_env as genv
from ..process_group import ProcessGroup, pp_group
from .schedule import GenerateGPipeSchedule, GenerateInterleaved1F1BSchedule, PrintScheduleTable, Task
from .stage_info import GetStageInfo, StageInfo


class PipelineStage:
    def __init__(self, stage_index: int, num_stages: int, recv_shape: Sequence[Sequence[int]], device,
                 chunks: List[torch.nn.Module]):
        self.stage_index_, self.num_stages_ = stage_index, num_stages
        self.recv_shape_ = [tuple(s) for s in recv_shape]
        self.device_ = device
        self.chunks_ = chunks
        self.prev_rank_ = stage_index - 1 if stage_index > 0 else -1
        self.next_rank_ = stage_index + 1 if stage_index < num_stages - 1 else -1

    def ForwardOneChunk(self, inputs, local_chunk_idx: int = 0):
        return self.chunks_[local_chunk_idx](*inputs)

    def IsFirstStage(self): return self.stage_index_ == 0
    def IsLastStage(self): return self.stage_index_ == self.num_stages_ - 1
    def stage_index(self): return self.stage_index_
    def num_stages(self): return self.num_stages_
    def prev_rank(self): return self.prev_rank_
    def next_rank(self): return self.next_rank_
    def recv_shape(self): return self.recv_shape_
    def device(self): return self.device_
    def mutable_chunks(self): return self.chunks_


class PipelineSchedule:
    def __init__(self, stage: PipelineStage, num_stages: int, num_micro_batches: int, pg: Optional[ProcessGroup] = None,
                 schedule: str = "1f1b", vpp_size: Optional[int] = None, boundary_dtype: Optional[torch.dtype] = None):
        self.stage = stage
        self.num_stages = num_stages
        self.n = num_micro_batches
        self.pg = pg or pp_group()
        self.kind = schedule
        self.vpp = vpp_size if vpp_size is not None else genv.GetVirtualPipelineParallelSize()
        self.boundary_dtype = boundary_dtype
        self._printed = False
        self._messages = None

    # ------------------------------------------------------------------ task list
    def tasks(self) -> List[Task]:
        gen = GenerateGPipeSchedule if self.kind == "gpipe" else GenerateInterleaved1F1BSchedule
        return gen(self.n, self.num_stages, self.vpp)

    # ------------------------------------------------------------------ transfers
    def messages(self, schedule: List[Task]):
        """What every step produces for another chunk: step -> [(key, src stage, dst stage)] in task
        order, with key = (is activation, micro-batch, consumer's global chunk)."""
        S = self.num_stages
        when = {(t.is_forward, t.microbatch_id, t.global_chunk_id): t.step for t in schedule}
        out = {}
        for t in schedule:
            if t.is_forward and not t.is_last_chunk:
                key = (True, t.microbatch_id, t.global_chunk_id + 1)
            elif not t.is_forward and not t.is_first_chunk:
                key = (False, t.microbatch_id, t.global_chunk_id - 1)
            else:
                continue
            assert when[key] > t.step, "schedule consumes a tensor before the step after its production"
            out.setdefault(t.step, []).append((key, t.stage_id, key[2] % S))
        return out

    def _exchange(self, msgs, outbox, inbox, in_flight, dtype):
        me = self.stage.stage_index()
        ops, received = [], []
        for key, src, dst in msgs:
            if src == me and dst == me:
                inbox[key] = (outbox[key], None)
            elif src == me:
                ops.append((True, outbox[key], dst))
            elif dst == me:
                buf = torch.empty(self.stage.recv_shape()[0], dtype=dtype, device=self.stage.device())
                ops.append((False, buf, src))
                received.append((key, buf))
        if not ops:
            return
        work = self.pg.BatchSendRecv(ops, async_op=True)
        for key, buf in received:
            inbox[key] = (buf, work)
        sent = [t for is_send, t, _ in ops if is_send]
        if sent:
            in_flight.append((work, sent))   # the payloads live until the step's end

    @staticmethod
    def _take(inbox, key):
        buf, work = inbox.pop(key)
        if work is not None:
            work.WaitNonBlocking()
        return buf

    # ------------------------------------------------------------------ execution
    def StepMicroBatches(self, microbatch_inputs, microbatch_targets, loss_fn, dtype) -> float:
        stage, S = self.stage, self.num_stages
        sidx = stage.stage_index()
        schedule = self.tasks()
        if not self._printed and sidx == 0 and genv.MyRank() == 0:
            self._printed = True
            self.schedule_table = PrintScheduleTable(schedule, self.n, S, self.vpp)
        if self._messages is None:
            self._messages = self.messages(schedule)
        dev = stage.device()
        tdtype = to_torch_dtype(dtype) if not isinstance(dtype, torch.dtype) else dtype
        use_autocast = tdtype != torch.float32
        bdtype = self.boundary_dtype or (tdtype if (use_autocast and torch.device(dev).type == "cuda") else torch.float32)
        saved = {}          # (local chunk, mb) -> (input tensor or None, output tensor)
        inbox, in_flight = {}, []
        total_loss = torch.zeros((), device=dev)
        last_bwd = {}       # local chunk -> index of its last backward task (arms DDP sync)
        for i, t in enumerate(schedule):
            if t.stage_id == sidx and not t.is_forward:
                last_bwd[t.local_chunk_idx] = i
        steps = (max(t.step for t in schedule) + 1) if schedule else 0
        by_step = {}
        for i, t in enumerate(schedule):
            if t.stage_id == sidx:
                by_step.setdefault(t.step, []).append((i, t))
        for step in range(steps):
            outbox = {}
            for i, t in by_step.get(step, ()):
                mb, lc = t.microbatch_id, t.local_chunk_idx
                chunk = stage.chunks_[lc]
                if t.is_forward:
                    if t.is_first_chunk:
                        x_in, inputs = None, (microbatch_inputs[mb],)
                    else:
                        x_in = self._take(inbox, (True, mb, t.global_chunk_id)).requires_grad_(True)
                        inputs = (x_in,)
                    with AutocastGuard(dtype=tdtype, enabled=use_autocast):
                        out = stage.ForwardOneChunk(inputs, lc)
                    saved[(lc, mb)] = (x_in, out)
                    if not t.is_last_chunk:
                        outbox[(True, mb, t.global_chunk_id + 1)] = out.detach().to(bdtype).contiguous()
                else:
                    x_in, out = saved.pop((lc, mb))
                    sync_ctx = nullcontext()
                    if hasattr(chunk, "no_sync"):
                        if i != last_bwd[lc]:
                            sync_ctx = chunk.no_sync()
                        elif getattr(chunk, "reducer", None) is not None:
                            chunk.reducer.PrepareForBackward()   # arm the bucket counters for this pass only
                    with sync_ctx:
                        if t.is_last_chunk:
                            with AutocastGuard(dtype=tdtype, enabled=use_autocast):
                                loss = loss_fn(out, microbatch_targets[mb].to(out.device)) / self.n
                            total_loss += loss.detach().float()
                            loss.backward()
                        else:
                            g = self._take(inbox, (False, mb, t.global_chunk_id))
                            out.backward(g.to(out.dtype))
                    if not t.is_first_chunk:
                        outbox[(False, mb, t.global_chunk_id - 1)] = x_in.grad.to(bdtype).contiguous()
            self._exchange(self._messages.get(step, ()), outbox, inbox, in_flight, bdtype)
        for w, _ in in_flight:
            if w is not None:
                w.WaitNonBlocking()
        assert not inbox and not saved, "pipeline step ended with undelivered tensors"
        return float(total_loss.item())

    def Step(self, input, target, optimizer, loss_fn, dtype) -> float:
        mbs = tgs = [None] * self.n
        if self.stage.IsFirstStage():
            mbs = list(input.chunk(self.n, dim=0))
        if self.stage.IsLastStage():
            tgs = list(target.chunk(self.n, dim=0))
        optimizer.ZeroGrad()
        loss = self.StepMicroBatches(mbs, tgs, loss_fn, dtype)
        # under sequence parallelism the replicated parameters of this stage (norm weights, position
        # table, row-parallel biases) hold the gradient of their sequence slice only
        from ..tensor_parallel import AllReduceSequenceParallelGrads

        for chunk in self.stage.mutable_chunks():
            AllReduceSequenceParallelGrads(chunk)
        optimizer.Step()
        return loss


class PipelineParallel(Module):
    kType = "PipelineParallel"
    kModuleName = "module"

    def __init__(self, module: Module, num_stages: int, num_micro_batches: int, recv_shape, pp_rank: int, device,
                 chunk_size: int = 1, schedule: str = "1f1b", pg: Optional[ProcessGroup] = None,
                 boundary_dtype: Optional[torch.dtype] = None):
        super().__init__(self.kType)
        self.add_module(self.kModuleName, module)
        self.num_stages_, self.rank_ = num_stages, pp_rank
        chunks: List[torch.nn.Module] = []
        for cid in range(chunk_size):
            parts = []
            if cid == 0 and pp_rank == 0:
                parts.append(module.mutable_module(kPPFirstStageName))
            parts.append(module.mutable_module(kPPChunkNamePrefix + str(cid)))
            if cid == chunk_size - 1 and pp_rank == num_stages - 1:
                parts.append(module.mutable_module(kPPLastStageName))
            chunks.append(Sequential(*parts))
        if recv_shape and not isinstance(recv_shape[0], (list, tuple)):
            recv_shape = [recv_shape]
        self.pipeline_stage_ = PipelineStage(pp_rank, num_stages, recv_shape, device, chunks)
        self.schedule_ = PipelineSchedule(self.pipeline_stage_, num_stages, num_micro_batches, pg, schedule,
                                          chunk_size, boundary_dtype)

    def mutable_chunks(self):
        return self.pipeline_stage_.mutable_chunks()

    def TrainStep(self, inputs, targets, optimizer, loss_fn, dtype=DataType.kFLOAT32) -> float:
        x = inputs[0] if isinstance(inputs, (list, tuple)) else inputs
        y = targets[0] if isinstance(targets, (list, tuple)) else targets
        return self.schedule_.Step(x if self.rank_ == 0 else None, y, optimizer, loss_fn, dtype)

    def Parameters(self):
        return list(self._modules[self.kModuleName].parameters())

    def Forward(self, *a, **k):
        raise RuntimeError("PipelineParallel runs through TrainStep")

    GetStageInfo = staticmethod(GetStageInfo)
