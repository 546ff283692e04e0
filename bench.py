"""Headline benchmark: GPT-2 124M training throughput (tokens/s), bf16 autocast with fp32
accumulation, AdamW, micro-batch 16 x 1024 tokens per GPU, DDP with gradient bucketing + ZeRO-2 when
more than one GPU is used (weak scaling: per-GPU work is fixed).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events around the K steps, max over
ranks, inputs resident on the device); ``e2e`` repeats the measurement through the public training
API with, every step, the host->device copy of that step's tokens from pinned memory and a
device->host read of the loss.  Data are synthetic uniform token ids; weights are random-init.

The headline metric has a second half, LLaMA-3 8B with tensor parallelism over all GPUs of the node
plus sequence parallelism and the vocabulary-parallel loss (1 x 2048 tokens per step): on 8 GPUs
the same line carries it as ``secondary`` (same keys), measured right after the GPT-2 run by one
fresh process per rank.  ``--secondary on|off`` forces or suppresses it.

Other configurations: ``--model llama3-8b --tp 8`` (that secondary on its own), ``--model llama3-1b
--tp 2 --pp 2 --vpp 2`` (hybrid data x tensor+sequence x pipeline parallelism, 8 micro-batches of one
sequence) and ``--model llama3-8b --lora-rank 16 --zero 1 --batch 2`` (LoRA fine-tune, ZeRO-1 over the
adapter state); the last two run through the example trainer's command line.

``--impl reference`` runs the unmodified reference's stock trainers (built by
``baseline/build_reference.py``) on the same shapes and prints the same line, ``secondary`` included.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput number

HERE = os.path.dirname(os.path.abspath(__file__))
GPT2_METRIC = "tokens/sec GPT-2 124M training (bf16 autocast, AdamW, DDP + ZeRO-2 for N>1), max over ranks"


def _parallelism(world, tp, pp, vpp, zero, lora):
    dp = world // max(tp * pp, 1)
    parts = []
    if dp > 1:
        parts.append(f"dp{dp}+zero{zero}")
    if tp > 1:
        parts.append(f"tp{tp}+sp")
    if pp > 1:
        parts.append(f"pp{pp}" + (f"xvpp{vpp}" if vpp > 1 else ""))
    s = " x ".join(parts) or "single"
    return s + (f", lora r{lora}" if lora else "")


def _metric(model, world, tp, pp, vpp, zero, lora):
    if model == "gpt2" and tp == 1 and pp == 1 and not lora:
        return GPT2_METRIC
    return (f"tokens/sec {model} training (bf16 autocast, AdamW, {_parallelism(world, tp, pp, vpp, zero, lora)}), "
            "max over ranks")


# ------------------------------------------------------------------------------------------- reference arm
def _write_llama3_weight_file(path, cfg):
    """Random-init llm.c LLaMA-3 weight file of ``cfg``'s shape, streamed (an 8B file is 32 GB of
    fp32): matrices repeat one 64 Mi block of N(0, 0.02) values, norm weights are ones."""
    import struct

    import numpy as np

    from infinitrain_b200.models import llmc

    header = bytearray(1024)
    struct.pack_into("<8i", header, 0, llmc.kLlama3Magic, llmc.kLlama3Fp32Version, cfg.block_size, cfg.vocab_size,
                     cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.n_embd)
    struct.pack_into("<f", header, 32, float(cfg.ffn_dim_multiplier or 0.0))
    struct.pack_into("<i", header, 36, cfg.multiple_of)
    struct.pack_into("<f", header, 40, float(cfg.norm_eps))
    struct.pack_into("<f", header, 44, float(cfg.rope_theta))
    struct.pack_into("<4i", header, 48, int(cfg.use_scaled_rope), cfg.max_gen_batch_size, 3, 1)
    block = (np.random.default_rng(42).standard_normal(64 << 20, dtype=np.float32) * 0.02).tobytes()
    with open(path, "wb") as f:
        f.write(bytes(header))
        for kind, shape in llmc._llama3_layout(cfg):
            left = 4 * int(np.prod(shape))
            if kind.startswith("ln_"):
                f.write(np.ones(left // 4, dtype=np.float32).tobytes())
                continue
            while left > 0:
                f.write(block[:left])
                left -= min(left, len(block))


class _WeightFile:
    """The llm.c weight file of a LLaMA-3 shape, written by a background thread (so that it can be
    produced while another measurement runs); ``path()`` waits for it."""

    def __init__(self, model_name, layers):
        import shutil

        import numpy as np

        from infinitrain_b200.models import llama3_config, llmc

        self.cfg = llama3_config(model_name, **({"n_layer": layers} if layers else {}))
        self.nbytes = 1024 + 4 * sum(int(np.prod(sh)) for _, sh in llmc._llama3_layout(self.cfg))
        root = next((d for d in ("/dev/shm", "/tmp")
                     if os.path.isdir(d) and shutil.disk_usage(d).free > self.nbytes + (4 << 30)), None)
        self.file = os.path.join(root, f"itb_ref_llama3_{os.getpid()}.bin") if root else None
        self.error = None
        self._thread = None
        if self.file is not None:
            self._thread = threading.Thread(target=self._write, daemon=True)
            self._thread.start()

    def _write(self):
        try:
            _write_llama3_weight_file(self.file, self.cfg)
        except Exception as e:  # noqa: BLE001
            self.error = f"{type(e).__name__}: {e}"

    def path(self):
        if self._thread is not None:
            self._thread.join()
        return self.file

    def remove(self):
        if self._thread is not None:
            self._thread.join()
        if self.file:
            try:
                os.remove(self.file)
            except OSError:
                pass


def _reference_measure(args, model, tp, pp, vpp, lora, zero, batch, seq, weights=None, time_limit=1500):
    """One run of the UNMODIFIED reference (``baseline/_ref``) through its stock ``example/gpt2`` or
    ``example/llama3`` trainer; returns the JSON record (or ``{"impl": "reference", "unavailable": ...}``).
    The reference is one process with one thread per GPU; its step time is its own host clock around
    each step (which ends with the loss read-back); its optimizers are the ones its examples
    hard-code (SGD for GPT-2, Adam for LLaMA-3).  The stock LLaMA-3 trainer builds only the 1B shape
    from scratch, so other shapes reach it as a random-init llm.c weight file."""
    import re

    def unavailable(why):
        return {"impl": "reference", "unavailable": why}

    llama = model.startswith("llama3")
    on_cpu = os.environ.get("ITB_REFERENCE_DEVICE", "cuda") == "cpu"       # plumbing checks without a GPU
    exe = os.path.join(HERE, "baseline", "_ref", "bin", ("llama3" if llama else "gpt2") + ("_cpu" if on_cpu else ""))
    n = args.gpus
    if (not llama and (model != "gpt2" or tp != 1 or pp != 1 or lora)) or n % max(tp * pp, 1):
        return unavailable("this model / parallelism is not wired to the reference's stock trainers")
    # the reference checkout: ITB_REFERENCE_SRC, else a directory named "reference" beside this repository
    ref_src = os.environ.get("ITB_REFERENCE_SRC") or os.path.join(os.path.dirname(HERE), "reference")
    if not os.path.exists(exe) and os.path.isdir(os.path.join(ref_src, "infini_train")):
        try:     # one-off offline build (nvcc, no GPU needed); see baseline/build_reference.py
            subprocess.run([sys.executable, os.path.join(HERE, "baseline", "build_reference.py"), "--src", ref_src]
                           + (["--cpu-only"] if on_cpu else []), capture_output=True, text=True, timeout=1800)
        except Exception:  # noqa: BLE001
            pass
    if not os.path.exists(exe):
        return unavailable(f"baseline/_ref/bin/{os.path.basename(exe)} is not built: pip cannot install the reference "
                           "checkout (no setup.py / pyproject.toml); build it with python baseline/build_reference.py "
                           "--src <checkout>")
    if not on_cpu:
        import ctypes

        try:
            ctypes.CDLL("libcuda.so.1")
        except OSError:
            return unavailable("no CUDA driver on this machine (libcuda.so.1 does not load); the reference's CUDA "
                               "build needs a GPU")
    import numpy as np

    B, T = batch, seq
    dp = n // max(tp * pp, 1)
    n_micro = args.micro_batches if pp > 1 else 1
    iters = args.warmup + args.steps
    scratch = []
    tok_path = f"/tmp/itb_ref_tokens_{os.getpid()}_{model}.bin"
    scratch.append(tok_path)
    n_tok = B * T * dp * n_micro * (iters + 2) + 1
    rng = np.random.default_rng(1234)
    header = np.zeros(256, dtype=np.int32)                 # llm.c token file: 1024-byte header, uint16 / uint32 ids
    header[0], header[1], header[2] = (20240801, 7, n_tok) if llama else (20240520, 1, n_tok)
    with open(tok_path, "wb") as f:
        f.write(header.tobytes())
        if llama:
            f.write(rng.integers(0, 128256, size=n_tok, dtype=np.uint32).tobytes())
        else:
            f.write(rng.integers(0, 50257, size=n_tok, dtype=np.uint16).tobytes())
    dtype = "float32" if on_cpu else "bfloat16"
    cmd = [exe, "--input_bin", tok_path, "--batch_size", str(B), "--sequence_length", str(T),
           "--total_batch_size", str(B * T * dp * n_micro), "--num_iteration", str(iters), "--dtype", dtype,
           "--learning_rate", "1e-4", "--freq_generate_txt", "1000000", "--overfit_single_batch=false"]
    cmd += ["--device", "cpu"] if on_cpu else ["--nthread_per_process", str(n)]
    own_weights = None
    if llama:
        from infinitrain_b200.models import llama3_config

        mcfg = llama3_config(model, **({"n_layer": args.layers} if args.layers else {}))
        cmd += ["--model", "llama3"]
        if model != "llama3-1b" or args.layers:
            if weights is None:
                weights = own_weights = _WeightFile(model, args.layers)
            w_path = weights.path()
            if w_path is None or weights.error:
                return unavailable(weights.error or f"no scratch space for the {weights.nbytes >> 30} GiB llm.c weight "
                                   "file the reference's stock LLaMA-3 trainer needs for this shape")
            cmd += ["--llmc_filepath", w_path]
        if tp > 1:
            cmd += ["--tensor_parallel", str(tp), "--sequence_parallel"]
        if pp > 1:
            cmd += ["--pipeline_parallel", str(pp), "--virtual_pipeline_parallel", str(vpp)]
        if lora:
            cmd += ["--lora_rank", str(lora), "--lora_alpha", str(2 * lora), "--lora_target_modules", "c_attn,attn.c_proj"]
        model_desc = (f"LLaMA-3 {model} shape through the reference's example/llama3"
                      + ("" if model == "llama3-1b" and not args.layers else " and a random-init llm.c file")
                      + f" ({mcfg.n_layer}L, {mcfg.n_embd} wide, {mcfg.n_head}q/{mcfg.n_kv_head}kv heads, "
                      f"vocab {mcfg.vocab_size})")
        opt_desc = "Adam lr 1e-4 (hard-coded in the reference's example/llama3/main.cc)"
    else:
        # "d12" is the stock trainer's from-scratch GPT-2 124M shape (12 layers, 12 heads, 768 wide); its
        # "gpt2" name is only defined together with an llm.c weight file
        cmd += ["--model", "d12"]
        model_desc = "GPT-2 124M (reference example/gpt2, --model d12: 12L, 12H, 768, vocab 50257, ctx 1024)"
        opt_desc = "SGD lr 1e-4 (hard-coded in the reference's example/gpt2/main.cc)"
    if dp > 1:
        cmd += ["--zero_stage", str(zero)]
    env = dict(os.environ)
    # the launcher's rendezvous variables mean nothing to the reference, and its OMP_NUM_THREADS=1 would
    # throttle the reference's host-side loops
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "LOCAL_WORLD_SIZE", "GROUP_RANK",
              "OMP_NUM_THREADS"):
        env.pop(k, None)
    sampler = ClockSampler(0)
    sampler.start()
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=time_limit, env=env,
                           cwd=os.path.join(HERE, "baseline", "_ref"))
    except subprocess.TimeoutExpired:
        sampler.stop()
        return unavailable(f"the reference trainer did not finish within {time_limit} s")
    finally:
        for path in scratch:
            try:
                os.remove(path)
            except OSError:
                pass
        if own_weights is not None:
            own_weights.remove()
    clocks = sampler.stop()
    pat = re.compile(r"step\s+(\d+)/\d+\s+\|\s+train loss\s+([-0-9.eE+naif]+).*?\(\s*([0-9.]+)\s*ms\s*\|\s*([0-9.]+)\s*tok/s")
    steps = {}
    for line in (r.stdout + "\n" + r.stderr).splitlines():
        m = pat.search(line)
        if m:
            steps[int(m.group(1))] = (float(m.group(2)), float(m.group(3)))
    timed = [steps[i][1] for i in range(args.warmup + 1, iters + 1) if i in steps]
    if r.returncode != 0 or len(timed) != args.steps:
        tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or [""]
        return unavailable(f"the reference trainer exited with code {r.returncode} after {len(steps)} of {iters} "
                           f"steps: {tail[0][:200]}")
    ms = sum(timed)
    tokens_per_step = B * T * dp * n_micro
    value = tokens_per_step * args.steps / (ms / 1e3)
    return {
        "impl": "reference", "metric": _metric(model, n, tp, pp, vpp, zero, lora),
        "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak" if tp * pp <= 1 else "strong",
        "vs_baseline": None, "dtype": "fp32 (CPU plumbing check)" if on_cpu else "bf16",
        "data": "synthetic uniform token ids (llm.c token file), random-init weights",
        "config": {"model": model_desc, "global_batch": B * dp * n_micro, "micro_batch_per_gpu": B, "seq_len": T,
                   "parallelism": _parallelism(n, tp, pp, vpp, zero, lora) + (" (threads of one process)" if n > 1 else ""),
                   "optimizer": opt_desc,
                   "timing": "the reference's own host clock around each step; a step ends with the loss read-back",
                   "l2": "inputs larger than L2"},
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms / args.steps,
                "h2d_bytes_per_step": 2 * B * T * n_micro * 8, "d2h_bytes_per_step": 4 * n_micro,
                "note": "the reference's loop copies each batch from host memory and reads the loss back every step, so "
                        "its only timing is end to end"},
        "gpu_launches": None, "final_loss": steps[iters][0],
    }


def reference_arm(args):
    """``--impl reference``: rank 0 drives the reference (a single multi-threaded process) and prints
    the line; with the secondary on, the LLaMA-3 8B weight file is written while GPT-2 runs."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    llama = args.model.startswith("llama3")
    B, T = args.batch or (1 if llama else 16), args.seq or (2048 if llama else 1024)
    weights, sec_err = None, ""
    t_start = time.time()
    if _secondary_wanted(args):
        try:
            weights = _WeightFile("llama3-8b", args.layers)
        except Exception as e:  # noqa: BLE001
            sec_err = f"{type(e).__name__}: {e}"
    out = _reference_measure(args, args.model, args.tp, args.pp, args.vpp, args.lora_rank, args.zero, B, T)
    if _secondary_wanted(args):
        if weights is None:
            out["secondary"] = {"impl": "reference", "unavailable": sec_err}
        else:
            left = max(120, int(args.reference_secondary_budget - (time.time() - t_start)))
            try:
                out["secondary"] = _reference_measure(args, "llama3-8b", args.gpus, 1, 1, 0, args.zero, 1, 2048,
                                                      weights=weights, time_limit=left)
            except Exception as e:  # noqa: BLE001  (the first measurement is printed whatever happens to the second)
                out["secondary"] = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}
            finally:
                weights.remove()
    print(json.dumps(out), flush=True)
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc = None
        self.path = f"/tmp/itb_clocks_{os.getpid()}_{id(self)}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "200"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        try:
            os.remove(self.path)
        except OSError:
            pass
        return out


# ------------------------------------------------------------------------------------------- this framework
def _secondary_wanted(args) -> bool:
    """The LLaMA-3 8B tensor-parallel half of the headline metric rides on the default GPT-2 run of a
    full node (8 GPUs); ``--secondary on`` forces it at any N > 1, ``off`` suppresses it."""
    plain_gpt2 = args.model == "gpt2" and args.tp == 1 and args.pp == 1 and not args.lora_rank
    if not plain_gpt2 or args.secondary == "off" or args.gpus < 2:
        return False
    return args.secondary == "on" or args.gpus == 8


def _run_secondary(args, rank, script=None, sp=subprocess):
    """LLaMA-3 8B, tensor parallel over all ranks + sequence parallelism, as one fresh process per
    rank (this process has released its process group; a crash or a hang in the second measurement
    cannot take the first one with it).  Two attempts share the time budget: the step captured in a
    CUDA graph, then, if any rank's process failed or ran out of time, the eager step.  The ranks'
    parent processes have no communicator left, so they agree on the outcome of an attempt through
    one small file per rank in the temporary directory.  Returns rank 0's record."""
    import tempfile

    world = args.gpus
    base_port = int(os.environ.get("MASTER_PORT", "29511"))
    key = os.path.join(tempfile.gettempdir(), f"itb_secondary_{os.getppid()}_{base_port}")
    log_dir = os.environ.get("ITB_TEST_ARTIFACTS") or tempfile.gettempdir()
    attempts = [("cuda graph", ["--graph", "1"]), ("eager", ["--graph", "0"])]
    per_attempt = max(60, args.secondary_budget // len(attempts))
    reasons = []
    for k, (name, flags) in enumerate(attempts):
        # the children rendezvous among themselves: rank 0's child serves the store on a port of its
        # own, so nothing may tell them that a launcher's agent already hosts one (torchrun does, through
        # TORCHELASTIC_USE_AGENT_STORE: every rank would then connect as a client to a server that does not exist)
        env = {k_: v for k_, v in os.environ.items() if not k_.startswith("TORCHELASTIC_")}
        env["MASTER_PORT"] = str(base_port + 13 + 7 * k)
        env["ITB_PG_TIMEOUT_S"] = str(max(60, per_attempt - 30))   # a rank that never joins ends the others' rendezvous in time
        cmd = [sys.executable, script or os.path.abspath(__file__), "--gpus", str(world), "--steps", str(args.steps), "--warmup",
               str(args.warmup), "--model", "llama3-8b", "--tp", str(world), "--secondary", "off", *flags]
        if args.layers:
            cmd += ["--layers", str(args.layers)]
        log = os.path.join(log_dir, f"bench_secondary_attempt{k}_rank{rank}.log")
        record, why = None, ""
        with open(log, "w") as lf:
            proc = sp.Popen(cmd, stdout=sp.PIPE, stderr=lf, text=True, env=env)
            try:
                stdout, _ = proc.communicate(timeout=per_attempt)
            except sp.TimeoutExpired:
                proc.kill()
                stdout, _ = proc.communicate()
                why = f"did not finish within {per_attempt} s"
        if not why and proc.returncode != 0:
            why = f"exited with code {proc.returncode}"
        if not why and rank == 0:
            for line in reversed((stdout or "").strip().splitlines()):
                if line.startswith("{"):
                    try:
                        record = json.loads(line)
                    except ValueError:
                        pass
                    break
            if record is None:
                why = "printed no record"
        if why:
            try:
                tail = [ln for ln in open(log).read().strip().splitlines() if ln.strip()][-1:]
            except OSError:
                tail = []
            why = f"{name}: {why}" + (f" ({tail[0][:200]})" if tail else "")
        # every parent learns whether every rank's process succeeded
        with open(f"{key}_a{k}_r{rank}", "w") as f:
            f.write(why or "ok")
        deadline = time.time() + 60
        states = []
        while time.time() < deadline:
            states = []
            for r in range(world):
                try:
                    states.append(open(f"{key}_a{k}_r{r}").read())
                except OSError:
                    break
            if len(states) == world and all(states):
                break
            time.sleep(0.2)
        failed = [st for st in states if st != "ok"] if len(states) == world else ["a rank's parent process did not report"]
        if not failed:
            if rank == 0:
                record["attempt"] = name
                if reasons:
                    record["earlier_attempts"] = reasons
            return record
        reasons.append(failed[0])
    return {"unavailable": "the LLaMA-3 8B tensor-parallel run failed: " + "; ".join(reasons)} if rank == 0 else None


def _via_trainer(args):
    """Pipeline-parallel and LoRA configurations run through the example trainer's command line
    (``examples/llama3/main.py``, i.e. the call a user makes), in this process; the record is built
    from the per-step metrics file the trainer's last rank writes.  A step's time is the trainer's
    host clock around the whole step: data loading, host-to-device copies, forward / backward /
    optimizer over every micro-batch, the loss read-back and a device synchronisation."""
    import torch  # noqa: F401

    sys.path.insert(0, HERE)
    from examples.common import trainer
    from infinitrain_b200.ops import functional as ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    llama = args.model.startswith("llama3")
    B, T = args.batch or 1, args.seq or (2048 if llama else 1024)
    tp, pp, vpp = args.tp, args.pp, args.vpp
    dp = world // (tp * pp)
    n_micro = args.micro_batches if pp > 1 else 1
    iters = args.warmup + args.steps
    mfile = f"/tmp/itb_bench_metrics_{os.environ.get('MASTER_PORT', '0')}_{args.model}.jsonl"
    if rank == 0 and os.path.exists(mfile):
        os.remove(mfile)
    argv = ["--model", args.model, "--batch_size", str(B), "--sequence_length", str(T), "--total_batch_size",
            str(B * T * dp * n_micro), "--num_iteration", str(iters), "--dtype", "bfloat16", "--optimizer", "adamw",
            "--weight_decay", "0.1", "--learning_rate", "1e-4", "--tensor_parallel", str(tp), "--pipeline_parallel",
            str(pp), "--virtual_pipeline_parallel", str(vpp), "--zero_stage", str(args.zero if dp > 1 else 0),
            "--metrics_jsonl", mfile]
    if tp > 1:
        argv += ["--sequence_parallel"]
    if args.layers:
        argv += ["--n_layer", str(args.layers)]
    if args.lora_rank:
        argv += ["--lora_rank", str(args.lora_rank), "--lora_alpha", str(2 * args.lora_rank), "--lora_target_modules",
                 "c_attn,attn.c_proj", "--lora_merge_check"]
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    n0 = ops.launch_count()
    rc = trainer.main("llama3" if llama else "gpt2", argv)
    launches = ops.launch_count() - n0
    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        return 0
    recs = [json.loads(l) for l in open(mfile)] if os.path.exists(mfile) else []
    timed = [r for r in recs if r["step"] > args.warmup]
    if rc != 0 or len(timed) != args.steps:
        print(json.dumps({"unavailable": f"the example trainer returned {rc} with {len(recs)} of {iters} step records"}))
        return 0
    host_ms = sum(r["host_ms"] for r in timed)
    dev_ms = sum(r["device_ms"] or r["host_ms"] for r in timed)
    tokens = B * T * dp * n_micro * args.steps
    print(json.dumps({
        "metric": _metric(args.model, world, tp, pp, vpp, args.zero, args.lora_rank),
        "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong" if tp * pp > 1 else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids (llm.c token file), random-init weights",
        "config": {"model": args.model, "global_batch": B * dp * n_micro, "micro_batch_per_gpu": B, "seq_len": T,
                   "micro_batches_per_step": n_micro, "parallelism": _parallelism(world, tp, pp, vpp, args.zero, args.lora_rank),
                   "optimizer": "AdamW lr 1e-4 wd 0.1", "through": "examples/llama3/main.py (example trainer CLI)",
                   "timing": "value: CUDA events around each step on the last rank (ranks synchronise every step); "
                             "e2e: the trainer's host clock around each step",
                   "l2": "inputs larger than L2"},
        "clocks": clocks,
        "e2e": {"value": tokens / (host_ms / 1e3), "unit": "tokens/s", "ms_per_step": host_ms / args.steps,
                "h2d_bytes_per_step": 2 * B * T * n_micro * 8, "d2h_bytes_per_step": 4 * n_micro},
        "gpu_launches": int(launches * args.steps / iters), "final_loss": timed[-1]["loss"],
    }), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="micro-batch per GPU (16 for gpt2, 1 for llama3-*)")
    ap.add_argument("--seq", type=int, default=None, help="sequence length (1024 for gpt2, 2048 for llama3-*)")
    ap.add_argument("--zero", type=int, default=2)
    ap.add_argument("--model", default="gpt2", help="gpt2 | llama3-1b | llama3-3b | llama3-8b")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (sequence parallelism on when > 1)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline-parallel stages (runs through the example trainer)")
    ap.add_argument("--vpp", type=int, default=1, help="virtual pipeline chunks per stage")
    ap.add_argument("--micro-batches", type=int, default=8, help="micro-batches per step under pipeline parallelism")
    ap.add_argument("--lora-rank", type=int, default=0, help="LoRA fine-tune of the q/k/v/o projections (alpha = 2 r)")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the model's own)")
    ap.add_argument("--kernel-table", default="", help="after the measurement, trace 2 more steps with torch.profiler "
                    "on rank 0 and write the per-kernel device-time table to this file (analysis aid, not a metric)")
    ap.add_argument("--residual", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--graph", type=int, default=None,
                    help="capture the whole training step in a CUDA graph (default: 1)")
    ap.add_argument("--secondary", default="auto", choices=["auto", "on", "off"],
                    help="also measure LLaMA-3 8B tensor-parallel over all GPUs (auto: on 8 GPUs)")
    ap.add_argument("--secondary-budget", type=int, default=420, help="seconds the secondary measurement may take")
    ap.add_argument("--reference-secondary-budget", type=int, default=780,
                    help="seconds both measurements of --impl reference may take together")
    ap.add_argument("--extra", default="auto", choices=["auto", "on", "off"],
                    help="on one GPU, also time the fp32-residual-stream variant (the reference's precision)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.pp > 1 or args.lora_rank:
        return _via_trainer(args)

    import torch

    if os.environ.get("ITB_BENCH_WATCHDOG_S"):
        # debugging aid: print every thread's stack and exit if the run takes longer than this
        import faulthandler

        faulthandler.dump_traceback_later(int(os.environ["ITB_BENCH_WATCHDOG_S"]), exit=True)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    from infinitrain_b200 import _ext
    from infinitrain_b200.autocast import AutocastGuard
    from infinitrain_b200.datatype import DataType
    from infinitrain_b200.device import DeviceType
    from infinitrain_b200.models import GPT2, LLaMA3
    from infinitrain_b200.nn import CrossEntropyLoss
    from infinitrain_b200.ops import functional as ops
    from infinitrain_b200.optim import Adam
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory

    C = _ext.load(required=True)
    tp = args.tp
    if args.graph is None:
        args.graph = 1
    if world % tp:
        raise SystemExit(f"--tp {tp} does not divide the world size {world}")
    dp = world // tp
    genv.InitAllEnv(world_size=world, rank=rank, tensor_parallel_size=tp, sequence_parallel_enabled=tp > 1)
    ProcessGroupFactory.Instance().Init(device=dev)

    llama = args.model.startswith("llama3")
    B = args.batch or (1 if llama else 16)
    T = args.seq or (2048 if llama else 1024)
    over = {"n_layer": args.layers} if args.layers else {}

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def build(residual):
        """Model, optimizer and the training step (the public API a user calls)."""
        torch.manual_seed(42)
        res_dtype = torch.bfloat16 if residual == "bf16" else torch.float32
        with torch.device(dev):
            model = (LLaMA3(args.model, residual_dtype=res_dtype, **over) if llama
                     else GPT2(args.model, residual_dtype=res_dtype, **over))
        model = model.to(dev)
        mcfg = model.config
        sp_sync = None
        if tp > 1:
            from infinitrain_b200.parallel.tensor_parallel import (AllReduceSequenceParallelGrads,
                                                                   VocabParallelCrossEntropyLoss)

            loss_fn = VocabParallelCrossEntropyLoss(mcfg.original_vocab_size)
            sp_sync = AllReduceSequenceParallelGrads
        else:
            loss_fn = CrossEntropyLoss()
        creator = Adam.Create(1e-4, 0.9, 0.95, 1e-8, weight_decay=0.1)
        if dp == 1:
            opt = creator(model.Parameters())
        else:
            from infinitrain_b200.parallel.ddp.config import DistributedDataParallelConfig
            from infinitrain_b200.parallel.ddp.distributed_data_parallel import DistributedDataParallel
            from infinitrain_b200.parallel.ddp.distributed_optimizer import DistributedOptimizer

            cfg = DistributedDataParallelConfig(zero_stage=args.zero, use_fused_nvlink_kernels=True)
            model = DistributedDataParallel(model, config=cfg)
            opt = DistributedOptimizer(creator, model.Parameters(), model) if args.zero >= 1 else creator(model.Parameters())

        def train_step(x, y):
            opt.ZeroGrad()
            with AutocastGuard(DeviceType.kCUDA, DataType.kBFLOAT16):
                loss = loss_fn(model(x), y)
            loss.backward()
            if sp_sync is not None:
                sp_sync(model)
            opt.Step()
            return loss

        return model, mcfg, opt, train_step

    model, mcfg, opt, eager_step = build(args.residual)
    parallelism = _parallelism(world, tp, 1, 1, args.zero, 0)
    V = mcfg.original_vocab_size
    # ranks of one tensor-parallel group read the same tokens
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank // tp)
    n_host = 8
    host_x = [torch.randint(0, V, (B, T), generator=gen).pin_memory() for _ in range(n_host)]
    host_y = [torch.randint(0, V, (B, T), generator=gen).pin_memory() for _ in range(n_host)]
    dev_x = [t.to(dev) for t in host_x]
    dev_y = [t.to(dev) for t in host_y]

    def graphed(step_fn):
        if not args.graph:
            return step_fn
        from infinitrain_b200.utils.cuda_graph import GraphedTrainStep

        # Capture one complete step (zero-grad, forward, backward with the bucket kernels, optimizer)
        # and replay it: the host only copies the next tokens into the static input buffers.
        return GraphedTrainStep(step_fn, (dev_x[0], dev_y[0]), warmup=3)

    def timed_steps(step_fn):
        """K steps between two events, inputs resident on the device."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            loss = step_fn(dev_x[i % n_host], dev_y[i % n_host])
        e1.record()
        barrier()
        return e0.elapsed_time(e1), loss

    train_step = graphed(eager_step)
    for i in range(args.warmup):
        train_step(dev_x[i % n_host], dev_y[i % n_host])
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- device-timed region: K steps, inputs already on the device
    launches0 = ops.launch_count()
    dev_ms, _ = timed_steps(train_step)
    launches = ops.launch_count() - launches0

    # ---- end-to-end region: pinned H2D of the step's tokens + D2H of the loss, every step
    xb = torch.empty((B, T), dtype=torch.int64, device=dev)
    yb = torch.empty((B, T), dtype=torch.int64, device=dev)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from infinitrain_b200.utils.cuda_graph import LaggedScalar

    # every step: its tokens from pinned host memory (a graphed step copies them straight into its
    # static input buffers) and its loss to the host; the loss of step i is looked at after step
    # i + 1 has been queued, so the read-back does not drain the device
    reader = LaggedScalar()
    e2.record()
    last = 0.0
    for i in range(args.steps):
        if args.graph:
            loss_t = train_step(host_x[i % n_host], host_y[i % n_host])
        else:
            xb.copy_(host_x[i % n_host], non_blocking=True)
            yb.copy_(host_y[i % n_host], non_blocking=True)
            loss_t = train_step(xb, yb)
        reader.push(loss_t)
        if i >= 1:
            last = reader.pop()
    for last in reader.drain():
        pass
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3)
    clocks = sampler.stop() if rank == 0 else None

    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile

        barrier()
        if rank == 0:
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for i in range(2):
                    train_step(dev_x[i % n_host], dev_y[i % n_host])
                torch.cuda.synchronize()
            with open(args.kernel_table, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=70))
        else:
            for i in range(2):
                train_step(dev_x[i % n_host], dev_y[i % n_host])
            torch.cuda.synchronize()
        barrier()
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    status = C.kernel_status()
    tp_paths = None
    if tp > 1:
        from infinitrain_b200.parallel import symm

        tp_paths = dict(symm.tp_path_counts)

    # ---- the reference keeps its residual stream in fp32: time that variant too (one GPU)
    extra = None
    if world == 1 and not llama and args.residual == "bf16" and args.extra != "off":
        train_step = eager_step = model = opt = None
        torch.cuda.empty_cache()
        model, _, opt, eager32 = build("fp32")
        step32 = graphed(eager32)
        for i in range(args.warmup):
            step32(dev_x[i % n_host], dev_y[i % n_host])
        ms32, loss32 = timed_steps(step32)
        extra = {"residual_stream_fp32": {"value": B * T * args.steps / (ms32 / 1e3), "unit": "tokens/s",
                                          "ms_per_step": ms32 / args.steps, "final_loss": float(loss32.item()),
                                          "note": "same step with the residual stream kept in fp32, as the reference does; "
                                                  "device-timed, inputs resident"}}
        step32 = eager32 = None

    out = None
    if rank == 0:
        tokens = B * T * dp * args.steps
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (e2e_ms / 1e3)
        out = {
            "metric": _metric(args.model, world, tp, 1, 1, args.zero, 0),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            # data parallelism fixes the work per GPU; one tensor-parallel group splits a fixed batch
            "scaling": "weak" if tp <= 1 else "strong",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": ("GPT-2 124M (12L, 12H, 768, vocab 50257, ctx 1024, tied embeddings)" if not llama else
                                 f"{args.model} ({mcfg.n_layer}L, {mcfg.n_embd} wide, "
                                 f"{mcfg.n_head}q/{mcfg.n_kv_head}kv heads, vocab {V})"),
                       "global_batch": B * dp, "micro_batch_per_gpu": B, "seq_len": T,
                       "parallelism": parallelism, "optimizer": "AdamW lr 1e-4 wd 0.1",
                       "residual_stream": args.residual, "cuda_graph": bool(args.graph),
                       "l2": "inputs larger than L2: the working set of a step (activations, fp32 weights, gradients "
                             "and moments) is gigabytes against 126 MB of L2, so no explicit flush is needed"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 2 * B * T * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "final_loss": last, "kernel_status": status,
        }
        if tp_paths is not None:
            out["config"]["tp_linear_paths"] = tp_paths
        if dp > 1 and args.zero == 2:
            # what "zero2" means on the fused NVLink path: sharded optimizer state and updates, full gradient buffer
            out["config"]["zero2_memory"] = ("fused NVLink kernels: optimizer state and the weight update are sharded over the "
                                             "data-parallel ranks, the fp32 gradient buffer stays whole on every rank (peers read "
                                             "it in place): ZeRO-1 memory")
        if extra is not None:
            out["extra"] = extra

    # ---- teardown: the captured step holds work of this communicator, so the graph goes first
    import gc

    train_step = eager_step = model = opt = None
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    if world > 1:
        barrier()
    if not _secondary_wanted(args):
        if rank == 0:
            print(json.dumps(out), flush=True)
        if world > 1:
            _destroy_process_group(torch)
        return 0

    # ---- the second half of the headline metric, in fresh processes (this one lets go of the GPUs first)
    _destroy_process_group(torch, exit_on_timeout=False)
    try:
        sec = _run_secondary(args, rank)
    except Exception as e:  # noqa: BLE001  (the first measurement is printed whatever happens to the second)
        sec = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0:
        out["secondary"] = sec
        print(json.dumps(out), flush=True)
    return 0


def _destroy_process_group(torch, limit_s: float = 60.0, exit_on_timeout: bool = True):
    """``destroy_process_group`` with a bound: the result is already measured (and, without a
    secondary, printed), so a communicator that does not shut down within the limit must not turn a
    finished run into a hung one."""
    done = threading.Event()

    def run():
        try:
            torch.distributed.destroy_process_group()
        finally:
            done.set()

    t = threading.Thread(target=run, daemon=True)
    t.start()
    if not done.wait(limit_s) and exit_on_timeout:
        sys.stdout.flush()
        sys.stderr.write("bench.py: destroy_process_group did not return in time; leaving without it\n")
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    sys.exit(main())
