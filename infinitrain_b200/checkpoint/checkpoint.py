"""Checkpoints: binary state-dict files, trainer state, save / resume / pruning.

Reference: infini_train/src/checkpoint/checkpoint.cc:112-215, checkpoint_manager.cc:21-120.
A checkpoint directory holds ``model.ckpt``, ``optimizer.ckpt`` (optional) and
``trainer_state.json``; with more than one rank every rank saves its own shard under
``rank_%06d``.  State-dict files use the reference's layout (magic 0x54504B43, version 1) and are
written by the native runtime through a temporary file + rename.  ``trainer_state.json`` is valid JSON
here (the reference omits a comma); the reader accepts both.  Resume validates the model shape and
the (ddp, tp, sp, pp) topology; ``allow_dp_resize`` lets the data-parallel size differ (ZeRO optimizer
state is re-sharded), under the same tensor / pipeline layout.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import time
from collections import OrderedDict
from dataclasses import asdict, dataclass
from typing import Dict, Optional

import torch

from .. import _ext
from ..parallel import global_env as genv


@dataclass
class TrainerState:
    global_step: int = 0
    consumed_batches: int = 0
    last_lr: float = 0.0
    n_layer: int = 0
    n_head: int = 0
    n_kv_head: int = 0
    n_embd: int = 0
    vocab_size: int = 0
    ddp_size: int = 1
    tp_size: int = 1
    sp_size: int = 1
    pp_size: int = 1


def _native():
    C = _ext.load(required=False)
    if C is None:
        raise RuntimeError("checkpoint IO needs the native runtime (infinitrain_b200._C)")
    return C


class Checkpoint:
    @staticmethod
    def SaveStateDict(path: str, state_dict: Dict[str, torch.Tensor]) -> None:
        names = list(state_dict.keys())
        _native().save_state_dict(path, names, [state_dict[k].detach() for k in names])

    @staticmethod
    def LoadStateDict(path: str) -> "OrderedDict[str, torch.Tensor]":
        return OrderedDict(_native().load_state_dict(path))

    @staticmethod
    def SaveTrainerState(path: str, state: TrainerState) -> None:
        order = ["n_layer", "n_head", "n_kv_head", "n_embd", "vocab_size", "global_step", "consumed_batches", "last_lr",
                 "ddp_size", "tp_size", "sp_size", "pp_size"]
        d = asdict(state)
        # written last of a checkpoint's files and through a temporary file + rename: a trainer_state.json
        # that exists is whole, and marks its directory as a complete checkpoint of its rank
        with open(path + ".tmp", "w") as f:
            f.write("{\n" + ",\n".join(f'  "{k}": {d[k]}' for k in order) + "\n}\n")
        os.replace(path + ".tmp", path)

    @staticmethod
    def LoadTrainerState(path: str) -> TrainerState:
        text = open(path).read()
        st = TrainerState()
        for k, v in asdict(st).items():
            m = re.search(r'"%s"\s*:\s*(-?[0-9.eE+-]+)' % re.escape(k), text)   # tolerant field scan
            if m:
                setattr(st, k, type(v)(float(m.group(1))) if isinstance(v, int) else float(m.group(1)))
        return st

    @staticmethod
    def Save(checkpoint_dir: str, model, optimizer, state: TrainerState, save_optimizer_state: bool = True,
             reference_buffers: bool = False) -> None:
        os.makedirs(checkpoint_dir, exist_ok=True)
        sd = model.StateDict() if hasattr(model, "StateDict") else model.state_dict()
        if reference_buffers:
            sd = Checkpoint.WithReferenceBuffers(sd, model)
        Checkpoint.SaveStateDict(os.path.join(checkpoint_dir, "model.ckpt"), sd)
        if save_optimizer_state and optimizer is not None:
            osd = optimizer.StateDict()
            if osd:
                Checkpoint.SaveStateDict(os.path.join(checkpoint_dir, "optimizer.ckpt"), osd)
        Checkpoint.SaveTrainerState(os.path.join(checkpoint_dir, "trainer_state.json"), state)

    @staticmethod
    def WithReferenceBuffers(sd, model):
        """Adds what the reference's strict loader expects beyond the parameters: the causal-mask buffer
        ``transformer.h.<i>.attn.bias`` (``[1, 1, block, block]`` lower-triangular ones) that its GPT-2
        attention registers (src/nn/modules/transformer/causal_self_attention.cc:46-50).  This framework
        has no such buffer (the attention kernels mask in place) and ignores it on load."""
        cfg = getattr(model, "config", None)
        if cfg is None or int(getattr(cfg, "attention_type", 0)) != 0:
            return sd
        out = OrderedDict(sd)
        layers = sorted({k.split(".")[2] for k in sd if k.startswith("transformer.h.") and k.split(".")[2].isdigit()}, key=int)
        mask = torch.tril(torch.ones(cfg.block_size, cfg.block_size)).view(1, 1, cfg.block_size, cfg.block_size)
        for i in layers:
            out[f"transformer.h.{i}.attn.bias"] = mask
        return out

    @staticmethod
    def Load(checkpoint_dir: str, model, optimizer, load_optimizer_state: bool = True) -> TrainerState:
        sd = Checkpoint.LoadStateDict(os.path.join(checkpoint_dir, "model.ckpt"))
        model.LoadStateDict(sd)
        if load_optimizer_state and optimizer is not None:
            opt_path = os.path.join(checkpoint_dir, "optimizer.ckpt")
            if os.path.exists(opt_path):
                optimizer.LoadStateDict(Checkpoint.LoadStateDict(opt_path))
            elif optimizer.StateDict():
                raise FileNotFoundError(f"Optimizer checkpoint not found at: {opt_path}")
        return Checkpoint.LoadTrainerState(os.path.join(checkpoint_dir, "trainer_state.json"))


def _rank_dir(root: str, rank: int, world: int) -> str:
    return os.path.join(root, f"rank_{rank:06d}") if world > 1 else root


def SaveCheckpoint(checkpoint_root_dir: str, global_step: int, model, optimizer, model_config, consumed_batches: int = 0,
                   last_lr: float = 0.0, save_optimizer_state: bool = True, max_checkpoint_keep: int = 0,
                   rank: Optional[int] = None, reference_buffers: bool = False) -> str:
    """Writes ``<root>/checkpoint_step_%06d[/rank_%06d]`` and prunes old step directories (rank 0,
    lexicographic order of the zero-padded names, keep the newest ``max_checkpoint_keep``)."""
    rank = genv.MyRank() if rank is None else rank
    world = genv.GetWorldSize()
    t0 = time.time()
    step_dir = os.path.join(checkpoint_root_dir, f"checkpoint_step_{global_step:06d}")
    state = TrainerState(global_step, consumed_batches, last_lr, model_config.n_layer, model_config.n_head,
                         model_config.n_kv_head, model_config.n_embd, model_config.vocab_size,
                         genv.GetDataParallelSize(), genv.GetTensorParallelSize(), genv.GetSequenceParallelSize(),
                         genv.GetPipelineParallelSize())
    Checkpoint.Save(_rank_dir(step_dir, rank, world), model, optimizer, state, save_optimizer_state, reference_buffers)
    if rank == 0 and max_checkpoint_keep > 0 and os.path.isdir(checkpoint_root_dir):
        ckpts = sorted(d for d in os.listdir(checkpoint_root_dir)       # numbered step directories only
                       if re.fullmatch(r"checkpoint_step_\d+", d) and os.path.isdir(os.path.join(checkpoint_root_dir, d)))
        while len(ckpts) > max_checkpoint_keep:
            shutil.rmtree(os.path.join(checkpoint_root_dir, ckpts.pop(0)), ignore_errors=True)
    return step_dir


def NewestCompleteCheckpoint(checkpoint_root_dir: str, rank: Optional[int] = None) -> int:
    """The newest step under ``<root>`` whose checkpoint is complete for this rank: its ``trainer_state.json``,
    the file a rank writes last, is there, parses and names that step.  0 when there is none.  Ranks of one job
    agree on a step by taking the minimum of what each of them finds (a job that its launcher restarted after
    a failure resumes from there)."""
    rank = genv.MyRank() if rank is None else rank
    world = genv.GetWorldSize()
    if not os.path.isdir(checkpoint_root_dir):
        return 0
    steps = sorted((int(m.group(1)), d) for d in os.listdir(checkpoint_root_dir)
                   for m in [re.fullmatch(r"checkpoint_step_(\d+)", d)] if m)
    for step, d in reversed(steps):
        try:
            st = Checkpoint.LoadTrainerState(os.path.join(_rank_dir(os.path.join(checkpoint_root_dir, d), rank, world),
                                                          "trainer_state.json"))
        except (OSError, ValueError, KeyError):
            continue
        if st.global_step == step:
            return step
    return 0


def _resume_on_other_dp_size(resume_root: str, old_ranks, model, optimizer, load_optimizer_state: bool):
    """A data-parallel group saved by the ``len(old_ranks)`` ranks listed (the ranks that share this
    rank's tensor / pipeline coordinates), resumed by a different number: the weights are replicated
    over the group (the first rank's file will do); ZeRO optimizer state is re-sharded from all the old
    ranks' files (:mod:`reshard`), replicated optimizer state is taken from the first."""
    from .reshard import reshard_zero_optimizer_state

    first = os.path.join(resume_root, old_ranks[0])
    model.LoadStateDict(Checkpoint.LoadStateDict(os.path.join(first, "model.ckpt")))
    if load_optimizer_state and optimizer is not None and optimizer.StateDict():
        paths = [os.path.join(resume_root, r, "optimizer.ckpt") for r in old_ranks]
        missing = [p for p in paths if not os.path.exists(p)]
        if missing:
            raise FileNotFoundError(f"Optimizer checkpoint not found at: {missing[0]}")
        buffers = getattr(optimizer, "buffers", None)
        if buffers:
            if len(buffers) != 1:
                raise ValueError("re-sharding optimizer state supports one flat buffer per rank")
            buf = buffers[0]
            old_states = [Checkpoint.LoadStateDict(p) for p in paths]
            new_state = reshard_zero_optimizer_state(
                old_states, [p.numel() for p in buf.params], buf.dp_size, buf.dp_rank,
                bucket_size_in_elements=buf.config.bucket_size_in_elements,
                pad_for_busbw=buf.config.pad_buckets_for_high_nccl_busbw)
            optimizer.LoadStateDict(new_state)
        else:
            optimizer.LoadStateDict(Checkpoint.LoadStateDict(paths[0]))
    return Checkpoint.LoadTrainerState(os.path.join(first, "trainer_state.json"))


@dataclass
class ResumeFromCheckpointResult:
    global_step: int = 0
    consumed_batches: int = 0
    last_lr: float = 0.0


def ResumeFromCheckpoint(resume_root: str, model, optimizer, model_config, load_optimizer_state: bool = True,
                         rank: Optional[int] = None, allow_dp_resize: bool = False) -> ResumeFromCheckpointResult:
    res = ResumeFromCheckpointResult()
    if not resume_root:
        return res
    rank = genv.MyRank() if rank is None else rank
    d = resume_root
    rd = os.path.join(resume_root, f"rank_{rank:06d}")
    old_ranks = sorted(x for x in os.listdir(resume_root) if x.startswith("rank_")) if os.path.isdir(resume_root) else []
    tp, pp = genv.GetTensorParallelSize(), genv.GetPipelineParallelSize()
    if allow_dp_resize and old_ranks and len(old_ranks) != genv.GetWorldSize() and len(old_ranks) % (tp * pp) == 0:
        # another data-parallel size under the same tensor / pipeline layout: the ranks that held this rank's
        # (tp, pp) coordinates in the old job, by their data-parallel rank (TP fastest, then DP, then PP)
        old_dp = len(old_ranks) // (tp * pp)
        _, tp_rank, pp_rank = genv.GetCoordOf(rank)
        mine = [f"rank_{tp_rank + tp * (d + old_dp * pp_rank):06d}" for d in range(old_dp)]
        absent = [m for m in mine if m not in old_ranks]
        if absent:
            raise FileNotFoundError(f"{resume_root} has no {absent[0]}: was it written with TP={tp}, PP={pp}?")
        head = Checkpoint.LoadTrainerState(os.path.join(resume_root, mine[0], "trainer_state.json"))
        for k, cur in (("tp_size", tp), ("sp_size", genv.GetSequenceParallelSize()), ("pp_size", pp)):
            if getattr(head, k) != cur:
                raise ValueError(f"{k.upper()} mismatch: checkpoint has {getattr(head, k)}, but current run has {cur} "
                                 "(only the data-parallel size may change)")
        st = _resume_on_other_dp_size(resume_root, mine, model, optimizer, load_optimizer_state)
        for k in ("n_layer", "n_head", "n_kv_head", "n_embd", "vocab_size"):
            if getattr(st, k) != getattr(model_config, k):
                raise ValueError(f"{k} mismatch: ckpt={getattr(st, k)}, config={getattr(model_config, k)}")
        # a rank consumes 1/dp of the batches: keep the position in the token stream
        res.global_step, res.last_lr = st.global_step, st.last_lr
        res.consumed_batches = max(st.consumed_batches, 0) * old_dp // max(genv.GetDataParallelSize(), 1)
        return res
    if genv.GetWorldSize() > 1 and os.path.isdir(rd):
        d = rd
    # model shape and topology are checked BEFORE any tensor is loaded (reference: checkpoint_manager.cc:45-63);
    # a checkpoint of several ranks keeps its files in rank directories
    state_file = os.path.join(d, "trainer_state.json")
    if not os.path.exists(state_file) and old_ranks:
        state_file = os.path.join(resume_root, old_ranks[0], "trainer_state.json")
    if not os.path.exists(state_file):
        raise FileNotFoundError(f"no trainer_state.json under {resume_root}")
    st = Checkpoint.LoadTrainerState(state_file)
    for k in ("n_layer", "n_head", "n_kv_head", "n_embd", "vocab_size"):
        if getattr(st, k) != getattr(model_config, k):
            raise ValueError(f"{k} mismatch: ckpt={getattr(st, k)}, config={getattr(model_config, k)}")
    topo = {"ddp_size": genv.GetDataParallelSize(), "tp_size": genv.GetTensorParallelSize(),
            "sp_size": genv.GetSequenceParallelSize(), "pp_size": genv.GetPipelineParallelSize()}
    for k, cur in topo.items():
        if getattr(st, k) != cur and not (k == "ddp_size" and allow_dp_resize and not load_optimizer_state):
            raise ValueError(f"{k.upper()} mismatch: checkpoint has {getattr(st, k)}, but current run has {cur}")
    st = Checkpoint.Load(d, model, optimizer, load_optimizer_state)
    res.global_step, res.consumed_batches, res.last_lr = st.global_step, max(st.consumed_batches, 0), st.last_lr
    return res
