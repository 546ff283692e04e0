"""Spawn N CPU ranks (gloo) that run one function; failures in any rank fail the test."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fn, args, tp, sp, pp, vpp, errq):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world)
        os.environ["LOCAL_RANK"] = str(rank)
        torch.set_num_threads(1)
        from infinitrain_b200.parallel import global_env as genv
        from infinitrain_b200.parallel.process_group import ProcessGroupFactory

        genv.InitAllEnv(1, tp, sp, pp, vpp, world_size=world, rank=rank)
        ProcessGroupFactory.Reset()
        ProcessGroupFactory.Instance().Init(backend="gloo", timeout_s=120)
        fn(rank, world, *args)
        import torch.distributed as dist

        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world, args=(), tp=1, sp=False, pp=1, vpp=1, timeout=240):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, tp, sp, pp, vpp, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errs.append((-1, "rank timed out"))
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    assert not errs and not bad, "\n".join(f"[rank {r}]\n{t}" for r, t in errs) or f"exit codes {bad}"
