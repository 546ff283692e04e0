"""Shared training driver of the GPT-2 and LLaMA-3 examples.

Flags, defaults and control flow follow the reference trainers (example/gpt2/main.cc:47-100,
128-530; example/llama3/main.cc): process groups from the 3-axis layout, model from an llm.c file
or random init, LoRA, pipeline / DDP / ZeRO wrapping, gradient accumulation, per-step loss
all-reduce, the step log line, optional sampling and checkpointing.  Differences: one process per
GPU (``--nthread_per_process`` is accepted and ignored), AdamW / SGD selectable for both families,
synthetic token data when no ``--input_bin`` is given.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def epochs(loader):
    """The loader's batches, epoch after epoch: a run longer than its token file starts the file over
    (the reference's loop is undefined past the end of its data)."""
    while True:
        n = 0
        for batch in loader:
            n += 1
            yield batch
        if n == 0:
            raise ValueError("the token file holds less than one batch for this rank")


def build_parser(family: str) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=f"{family} training (infinitrain_b200)")
    a = p.add_argument
    a("--input_bin", default="")
    a("--input_val_bin", default="")
    a("--tokenizer_bin", default="")
    a("--llmc_filepath", default="")
    a("--model", default="gpt2" if family == "gpt2" else "llama3-1b")
    a("--batch_size", type=int, default=4)
    a("--sequence_length", type=int, default=64)
    a("--total_batch_size", type=int, default=256)
    a("--num_iteration", type=int, default=10)
    a("--freq_generate_txt", type=int, default=0)
    a("--text_length", type=int, default=64)
    a("--learning_rate", type=float, default=1e-4)
    a("--weight_decay", type=float, default=0.0)
    a("--optimizer", default="sgd" if family == "gpt2" else "adam", choices=["sgd", "adam", "adamw"])
    a("--zero_stage", type=int, default=0)
    a("--val_loss_every", type=int, default=0,
      help="every N steps (and after the last one) log the mean loss over --val_max_batches batches of --input_val_bin")
    a("--val_max_batches", type=int, default=20)
    a("--sample_every", type=int, default=0)
    a("--overfit_single_batch", action="store_true")
    a("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a("--nthread_per_process", type=int, default=1)
    a("--tensor_parallel", type=int, default=1)
    a("--sequence_parallel", action="store_true")
    a("--pipeline_parallel", type=int, default=1)
    a("--virtual_pipeline_parallel", type=int, default=1)
    a("--pipeline_schedule", default="1f1b", choices=["1f1b", "gpipe"])
    a("--dtype", default="float32")
    a("--save_interval", type=int, default=0)
    a("--load", default="")
    a("--save", default="")
    a("--max_checkpoint_keep", type=int, default=0)
    a("--save_optimizer_state", action="store_true")
    a("--save_reference_buffers", action="store_true",
      help="also write the causal-mask buffers the reference's strict checkpoint loader expects (GPT-2)")
    a("--precision_check", default="")
    a("--lora_rank", type=int, default=0)
    a("--lora_alpha", type=float, default=16.0)
    a("--lora_target_modules", default="c_attn,c_proj")
    a("--lora_save_path", default="")
    a("--lora_load_path", default="")
    a("--lora_merge_check", action="store_true",
      help="after training, fold the adapters into the base weights, compare the loss of one batch before and "
           "after, and unfold them again (not with pipeline parallelism)")
    a("--fused_nvlink", type=int, default=1)
    a("--profile", action="store_true")
    a("--untie_weights", action="store_true",
      help="GPT-2: keep wte and lm_head as two parameters (both start from the file's wte).  The reference's CUDA "
           "build trains them untied -- its Module::To re-creates the parameters -- so GPU parity runs need this")
    a("--residual_dtype", default="bfloat16", choices=["bfloat16", "float32"],
      help="dtype of the residual stream under bf16 autocast (float32 = the reference's arithmetic)")
    a("--seed", type=int, default=42)
    a("--n_layer", type=int, default=0, help="override the layer count (smoke tests)")
    a("--n_embd", type=int, default=0, help="override the hidden size (smoke tests)")
    a("--n_head", type=int, default=0)
    a("--n_kv_head", type=int, default=0)
    a("--vocab_size", type=int, default=0)
    a("--metrics_jsonl", default="", help="append one JSON record per step to this file (last rank)")
    a("--elastic_resume", action="store_true",
      help="allow --load to resume a checkpoint on a different number of data-parallel ranks, under the same "
           "tensor / pipeline layout (ZeRO optimizer state is re-sharded)")
    a("--heartbeat_timeout", type=float, default=0.0,
      help="seconds without a peer's step heartbeat before the run stops with exit code 75 (0 = off); "
           "ITB_FAULT=<rank>:<step>:<raise|exit|stall|mute> injects a host-side fault before that step (steps "
           "count from 1, as in the log lines)")
    return p


def main(family: str, argv=None) -> int:
    args = build_parser(family).parse_args(argv)
    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.checkpoint import ResumeFromCheckpoint, SaveCheckpoint
    from infinitrain_b200.data import DeviceFeeder, DistributedDataLoader, TinyShakespeareDataset, Tokenizer, write_token_file
    from infinitrain_b200.datatype import DataType, parse_dtype, to_torch_dtype
    from infinitrain_b200.device import Device, DeviceGuardImpl
    from infinitrain_b200.models import gpt2_config, llama3_config, llmc
    from infinitrain_b200.nn import CrossEntropyLoss, lora
    from infinitrain_b200.nn.transformer import TransformerModel
    from infinitrain_b200.optim import SGD, Adam
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.ddp.config import DistributedDataParallelConfig
    from infinitrain_b200.parallel.ddp.distributed_data_parallel import DistributedDataParallel
    from infinitrain_b200.parallel.ddp.distributed_optimizer import DistributedOptimizer
    from infinitrain_b200.parallel.pp.pipeline_parallel import PipelineParallel
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory, ReduceOpType
    from infinitrain_b200.parallel.tensor_parallel import AllReduceSequenceParallelGrads, VocabParallelCrossEntropyLoss
    from infinitrain_b200.utils.logging import LOG, format_step_line
    from infinitrain_b200.utils.precision_checker import (PrecisionCheckConfig, PrecisionCheckEnv, PrecisionChecker,
                                                          PrecisionCheckLevel)
    from infinitrain_b200.utils.profiler import Profiler

    genv.InitAllEnv(args.nthread_per_process, args.tensor_parallel, args.sequence_parallel, args.pipeline_parallel,
                    args.virtual_pipeline_parallel)
    rank, world = genv.MyRank(), genv.GetWorldSize()
    use_cuda = args.device == "cuda" and torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(genv.GetLocalProcRank())
    dev = torch.device("cuda", genv.GetLocalProcRank()) if use_cuda else torch.device("cpu")
    device = Device.from_torch(dev)
    ProcessGroupFactory.Instance().Init(device=dev)
    heartbeat = injector = None
    if args.heartbeat_timeout > 0 and world > 1:
        import datetime

        import torch.distributed as dist

        from infinitrain_b200.utils.fault_tolerance import FaultInjector, Heartbeat

        # the heartbeats travel over their own TCP store (CPU side channel), next to the rendezvous port
        hb_port = int(os.environ.get("MASTER_PORT", "29500")) + 7
        store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), hb_port, world, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=60))
        heartbeat = Heartbeat(store, rank, world, timeout_s=args.heartbeat_timeout,
                              poll_s=min(0.5, args.heartbeat_timeout / 4)).start()
    if os.environ.get("ITB_FAULT"):
        from infinitrain_b200.utils.fault_tolerance import FaultInjector

        injector = FaultInjector(rank, heartbeat=heartbeat)     # host-side fault injection, with or without heartbeats
    pc = PrecisionCheckConfig.Parse(args.precision_check)
    PrecisionCheckEnv.Instance().Init(pc, rank)
    if rank == 0:
        LOG("INFO", genv.ProcessGroupOverview())
    dp, tp, pp = genv.GetDataParallelSize(), genv.GetTensorParallelSize(), genv.GetPipelineParallelSize()
    sp = genv.GetSequenceParallelSize()
    dp_rank, pp_rank = genv.GetDataParallelRank(), genv.GetPipelineParallelRank()
    B, T = args.batch_size, args.sequence_length
    tokens_per_fwdbwd = B * T * dp
    if args.total_batch_size % tokens_per_fwdbwd:
        raise SystemExit(f"total_batch_size must be a multiple of batch*seq*dp = {tokens_per_fwdbwd}")
    grad_accum = args.total_batch_size // tokens_per_fwdbwd
    if args.sequence_parallel and tp > 1 and T % tp:
        raise SystemExit(f"sequence_length ({T}) must be divisible by the tensor-parallel size ({tp}) under sequence parallelism")
    dtype = parse_dtype(args.dtype)
    torch.manual_seed(args.seed)

    # ---- model
    over_common = {"residual_dtype": torch.float32 if args.residual_dtype == "float32" else torch.bfloat16}
    if args.untie_weights:
        over_common["tie_weights"] = False
    if args.llmc_filepath:
        model = (llmc.GPT2FromLLMC if family == "gpt2" else llmc.LLaMA3FromLLMC)(args.llmc_filepath, **over_common)
    else:
        over = {k: getattr(args, k) for k in ("n_layer", "n_embd", "n_head", "n_kv_head") if getattr(args, k)}
        over.update(over_common)
        if args.vocab_size:
            over.update(vocab_size=args.vocab_size, original_vocab_size=args.vocab_size)
        cfg = gpt2_config(args.model, **over) if family == "gpt2" else llama3_config(args.model, **over)
        model = TransformerModel(cfg)
    cfg = model.config
    model.to(dev)
    PrecisionChecker.BuildNameMap(model)
    if args.lora_rank > 0:
        # every adapter draws its A from a generator keyed by its whole-model path: the start does not depend on
        # the layout that builds the model
        lcfg = lora.LoRAConfig(rank=args.lora_rank, alpha=args.lora_alpha,
                               target_modules=lora.ParseLoRATargetModules(args.lora_target_modules),
                               seed=(args.seed ^ 0x4C6F5241) | 1)
        model = lora.GetLoRAModel(model, lcfg)
        if args.lora_load_path:
            lora.LoadFullLoRAWeights(model, args.lora_load_path)    # whole-model file, sharded on load
        if rank == 0:
            lora.PrintLoRASummary(model, lambda s: LOG("INFO", s))
    trainable = [p for p in model.parameters() if p.requires_grad]

    # ---- parallel wrapping
    ddp_cfg = DistributedDataParallelConfig(zero_stage=args.zero_stage, use_fused_nvlink_kernels=bool(args.fused_nvlink))
    pipeline = None
    ddp_chunks = []
    if pp > 1:
        pipeline = PipelineParallel(model, pp, grad_accum, [B, T // sp, cfg.n_embd], pp_rank, dev,
                                    args.virtual_pipeline_parallel, schedule=args.pipeline_schedule)
        if dp > 1:
            chunks = pipeline.mutable_chunks()
            for i in range(len(chunks)):
                chunks[i] = DistributedDataParallel(chunks[i], config=ddp_cfg)
                ddp_chunks.append(chunks[i])
    elif dp > 1:
        model = DistributedDataParallel(model, config=ddp_cfg)
        ddp_chunks.append(model)

    # ---- optimizer
    if args.optimizer == "sgd":
        creator = SGD.Create(args.learning_rate)
    else:
        creator = Adam.Create(args.learning_rate, weight_decay=args.weight_decay if args.optimizer == "adamw" else 0.0)
    if args.zero_stage >= 1 and ddp_chunks:
        optimizer = DistributedOptimizer(creator, trainable, ddp_chunks)
    else:
        optimizer = creator(trainable)
    loss_fn = VocabParallelCrossEntropyLoss(cfg.original_vocab_size) if tp > 1 else CrossEntropyLoss()

    # ---- data
    if args.input_bin:
        data_path = args.input_bin
    else:
        data_path = f"/tmp/itb_synth_{family}_{os.getpid()}_{rank}.bin"
        g = torch.Generator().manual_seed(1234)
        n_tok = max(B * T * (grad_accum * dp * (args.num_iteration + 2) + 4), 4 * T)
        write_token_file(data_path, torch.randint(0, cfg.original_vocab_size, (n_tok,), generator=g).numpy(),
                         llama3=(family != "gpt2"))
    loader_batch = B * grad_accum if pp > 1 else B
    train_ds = TinyShakespeareDataset(data_path, T)
    loader = DistributedDataLoader(train_ds, loader_batch, dp_rank, dp)
    tokenizer = Tokenizer(args.tokenizer_bin) if args.tokenizer_bin else None
    val_loader = None
    if args.input_val_bin and args.val_loss_every > 0:
        val_loader = DistributedDataLoader(TinyShakespeareDataset(args.input_val_bin, T), B, dp_rank, dp)

    # ---- resume
    start_step = 0
    # batches reach the device through the feeder: asynchronous copies out of the loader's pinned ring,
    # ordered against the ring's slot reuse (several micro-batches may be in flight before a host sync)
    it = DeviceFeeder(epochs(loader), dev)
    # A job that its launcher started again after a failure (ITB_RESTART_COUNT > 0, infini_run --max_restarts) goes
    # on from the newest checkpoint under --save that every rank finds complete, unless --load says otherwise.
    restart_count = int(os.environ.get("ITB_RESTART_COUNT", "0") or 0)
    if not args.load and restart_count > 0 and args.save:
        from infinitrain_b200.checkpoint import NewestCompleteCheckpoint
        import torch.distributed as dist

        newest = torch.tensor([NewestCompleteCheckpoint(args.save)], dtype=torch.int64, device=dev)
        if dist.is_initialized() and world > 1:
            dist.all_reduce(newest, op=dist.ReduceOp.MIN)
        if int(newest.item()) > 0:
            args.load = os.path.join(args.save, f"checkpoint_step_{int(newest.item()):06d}")
        if rank == 0:
            LOG("INFO", f"restart {restart_count}: " + (f"resuming from {args.load}" if args.load else
                                                         "no complete checkpoint yet, starting over"))
    if args.load:
        res = ResumeFromCheckpoint(args.load, model, optimizer, cfg, load_optimizer_state=args.save_optimizer_state,
                                   allow_dp_resize=args.elastic_resume)
        start_step = res.global_step
        it.skip(res.consumed_batches)
    consumed = start_step * (1 if pp > 1 else grad_accum)
    profiler = Profiler.Instance()
    if args.profile:
        profiler.Enable()
    impl = DeviceGuardImpl
    cached = None
    last_rank = world - 1

    metrics = None
    for step in range(start_step, args.num_iteration):
        if injector is not None and heartbeat is None:
            injector.maybe_fire(step + 1)        # a faulty rank leaves here, with nothing of its own in flight
        if heartbeat is not None:
            from infinitrain_b200.utils.fault_tolerance import RankFailure

            try:
                if injector is not None:
                    injector.maybe_fire(step + 1)   # (steps count from 1, as in the log lines and in the C++ trainer)
                heartbeat.step(step)
                heartbeat.wait_peers(step)       # every peer is alive before this step's first collective
            except RankFailure as e:
                LOG("ERROR", f"peer failure detected at step {step + 1}: {e}; stopping before the next collective "
                             f"(resume from the last checkpoint)")
                heartbeat.stop()
                sys.stdout.flush()
                sys.stderr.flush()
                os._exit(75)
        PrecisionChecker.ResetCounters()
        impl.ResetMemPoolHighWatermarks(device)
        profiler.SetTag(f"Step_{step}")
        t0 = time.perf_counter()
        if use_cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        lossf = 0.0
        if pipeline is not None:
            if cached is None or not args.overfit_single_batch:
                x, y = next(it)
                cached = (x, y)
                consumed += 1
            x, y = cached
            lossf = pipeline.TrainStep([x], [y], optimizer, loss_fn, dtype)
        else:
            optimizer.ZeroGrad()
            loss_acc = torch.zeros((), device=dev)
            for micro in range(grad_accum):
                if cached is None or not args.overfit_single_batch:
                    x, y = next(it)
                    cached = (x, y)
                    consumed += 1
                x, y = cached
                last = micro == grad_accum - 1
                ctxs = [c.no_sync() for c in ddp_chunks] if (not last and ddp_chunks) else []
                for c in ctxs:
                    c.__enter__()
                with AutocastGuard(dtype=dtype, enabled=to_torch_dtype(dtype) != torch.float32):
                    loss = loss_fn(model(x), y) / grad_accum
                loss_acc += loss.detach().float()
                loss.backward()
                for c in ctxs:
                    c.__exit__(None, None, None)
            AllReduceSequenceParallelGrads(model)
            for c in ddp_chunks:
                c.FinishGradSync()
            optimizer.Step()
            lossf = float(loss_acc.item())
        if dp > 1:
            lt = torch.tensor([lossf], device=dev)
            ProcessGroupFactory.Instance().dp_group().AllReduce(lt, ReduceOpType.kAvg)
            lossf = float(lt.item())
        if use_cuda:
            ev1.record()
            torch.cuda.synchronize()
            # the step's one sync point: a bounded device-side wait that gave up (a fused NVLink
            # collective that lost a peer) has skipped its reduction -- stop like the heartbeat path does
            from infinitrain_b200.utils.fault_tolerance import KernelTimeout, check_device_status

            try:
                check_device_status(sync=True)
            except KernelTimeout as e:
                LOG("ERROR", f"step {step + 1}: {e}; stopping (resume from the last checkpoint)")
                if heartbeat is not None:
                    heartbeat.request_abort(str(e))
                    heartbeat.stop()
                sys.stdout.flush()
                sys.stderr.flush()
                os._exit(75)
        dur_ms = (time.perf_counter() - t0) * 1e3
        tps = args.total_batch_size / (dur_ms / 1e3)
        if rank == last_rank:
            used, reserved = impl.GetMemPoolPeakMB(device)
            LOG("ERROR", format_step_line(step + 1, args.num_iteration, lossf, args.learning_rate, dur_ms, tps, used,
                                          reserved, dp, tp, sp, pp))
            dev_ms = ev0.elapsed_time(ev1) if use_cuda else None
            if use_cuda:
                LOG("INFO", f"step {step + 1} device-timed {dev_ms:.2f} ms")
            if args.metrics_jsonl:
                if metrics is None:
                    from infinitrain_b200.utils.logging import MetricsSink

                    metrics = MetricsSink(args.metrics_jsonl)
                metrics.write(step=step + 1, loss=lossf, lr=args.learning_rate, host_ms=dur_ms, device_ms=dev_ms,
                              tokens_per_s=tps, peak_used_mb=used, peak_reserved_mb=reserved, dp=dp, tp=tp, sp=sp, pp=pp)
        if (val_loader is not None and pp == 1
                and ((step + 1) % args.val_loss_every == 0 or step + 1 == args.num_iteration)):
            # validation loss (a TODO in the reference's loop, example/gpt2/main.cc:401-404): no gradients, the
            # first batches of this rank's share of the file, averaged over the data-parallel group
            with torch.no_grad():
                total, n = torch.zeros((), device=dev), 0
                for vx, vy in val_loader:
                    with AutocastGuard(dtype=dtype, enabled=to_torch_dtype(dtype) != torch.float32):
                        total += loss_fn(model(vx.to(dev)), vy.to(dev)).float()
                    n += 1
                    if n >= args.val_max_batches:
                        break
                total /= max(n, 1)
                if dp > 1:
                    ProcessGroupFactory.Instance().dp_group().AllReduce(total, ReduceOpType.kAvg)
            if rank == last_rank:
                LOG("ERROR", f"step {step + 1:4d}/{args.num_iteration} | val loss {total.item():.6f} ({n} batches)")
        if tokenizer is not None and args.freq_generate_txt and (step + 1) % args.freq_generate_txt == 0 and pp == 1:
            tokenizer.GenerateText(model, B, T, args.text_length, dev)
        if args.save and args.save_interval and (step + 1) % args.save_interval == 0:
            SaveCheckpoint(args.save, step + 1, model, optimizer, cfg, consumed, args.learning_rate,
                           args.save_optimizer_state, args.max_checkpoint_keep,
                           reference_buffers=args.save_reference_buffers)
    if args.lora_rank > 0 and args.lora_merge_check and pp == 1 and cached is not None:
        # merged and unmerged adapters must give the same function (reference: tests/lora/test_lora.cc:108-147)
        def _eval_loss():
            with torch.no_grad(), AutocastGuard(dtype=dtype, enabled=to_torch_dtype(dtype) != torch.float32):
                return float(loss_fn(model(cached[0]), cached[1]).float())

        before = _eval_loss()
        lora.MergeLoRAWeights(model)
        merged = _eval_loss()
        lora.UnmergeLoRAWeights(model)
        after = _eval_loss()
        ok = abs(before - merged) <= 1e-3 * max(1.0, abs(before)) and abs(before - after) <= 1e-3 * max(1.0, abs(before))
        if rank == last_rank:
            LOG("ERROR", f"lora merge check: loss {before:.6f} unmerged, {merged:.6f} merged, {after:.6f} unmerged again: "
                         f"{'ok' if ok else 'MISMATCH'}")
        if not ok:
            return 3
    if args.lora_rank > 0 and args.lora_save_path:
        # one whole-model file gathered from every tensor- and pipeline-parallel rank (a collective)
        lora.SaveFullLoRAWeights(model, args.lora_save_path)
    if args.profile:
        profiler.Report(f"{family}.report.rank{rank}")
        profiler.PrintRecords(f"{family}.records.log.rank{rank}")
        profiler.Disable()
    if not args.input_bin:
        try:
            os.remove(data_path)
        except OSError:
            pass
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0
