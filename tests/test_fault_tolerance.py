"""Failure detection on the host: heartbeats, watchdog, coordinated abort, injected faults among
CPU ranks, corrupted checkpoints.  Nothing here touches a GPU."""
import os
import socket
import time

import pytest
import torch
import torch.multiprocessing as mp

from infinitrain_b200.utils.fault_tolerance import (DictStore, FaultInjector, Heartbeat, KernelTimeout, RankFailure,
                                                    check_kernel_status, corrupt_file)


def test_watchdog_reports_a_stale_peer():
    store = DictStore()
    seen = []
    a = Heartbeat(store, 0, 2, timeout_s=0.3, poll_s=0.05, on_failure=seen.append).start()
    b = Heartbeat(store, 1, 2, timeout_s=0.3, poll_s=0.05)
    for step in range(3):
        a.step(step)
        b.beat(step)
        time.sleep(0.05)
    assert a.failure is None
    # rank 1 goes quiet; rank 0 keeps stepping until its watchdog notices
    deadline = time.time() + 5
    with pytest.raises(RankFailure):
        step = 3
        while time.time() < deadline:
            a.step(step)
            step += 1
            time.sleep(0.05)
    a.stop()
    assert seen and seen[0].kind == "stale_heartbeat" and seen[0].rank == 1 and seen[0].step == 2


def test_abort_request_reaches_every_rank():
    store = DictStore()
    hbs = [Heartbeat(store, r, 3, timeout_s=30, poll_s=0.05).start() for r in range(3)]
    hbs[2].request_abort("loss is NaN")
    time.sleep(0.4)
    for r in (0, 1):
        assert hbs[r].failure is not None and hbs[r].failure.kind == "peer_abort" and hbs[r].failure.rank == 2
        with pytest.raises(RankFailure):
            hbs[r].step(1)
    assert hbs[2].failure is None          # the requester is not told about its own request
    for h in hbs:
        h.stop()


def test_injector_kinds():
    store = DictStore()
    hb = Heartbeat(store, 1, 2, timeout_s=30)
    inj = FaultInjector(1, "1:2:raise")
    inj.maybe_fire(1)
    with pytest.raises(RuntimeError):
        inj.maybe_fire(2)
    inj.maybe_fire(2)                      # fires once
    FaultInjector(0, "1:2:raise").maybe_fire(2)     # another rank: nothing happens
    mute = FaultInjector(1, "1:0:mute", heartbeat=hb)
    hb.beat(0)
    first = store.get("itb/hb/1")
    mute.maybe_fire(0)
    hb.beat(5)
    assert store.get("itb/hb/1") == first  # heartbeats stopped although the rank is still running
    t0 = time.time()
    FaultInjector(1, "1:0:stall:0.2").maybe_fire(0)
    assert time.time() - t0 >= 0.2


def test_kernel_status_word_becomes_an_exception():
    check_kernel_status(lambda: 0)
    with pytest.raises(KernelTimeout) as e:
        check_kernel_status(lambda: 121, "all-gather GEMM")
    assert "121" in str(e.value)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, store_port, pg_port, outdir, fault):
    import datetime

    import torch.distributed as dist

    torch.set_num_threads(1)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{pg_port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, timeout_s=1.0, poll_s=0.1).start()
    inj = FaultInjector(rank, fault, heartbeat=hb)
    x = torch.ones(4)
    result = "finished"
    try:
        for step in range(6):
            inj.maybe_fire(step)           # a faulty rank leaves here: nothing of its own is in flight
            hb.step(step)
            hb.wait_peers(step, timeout_s=2.0)      # every rank is known to be alive before the collective
            dist.all_reduce(x)
    except RankFailure as e:
        result = f"RankFailure at step {step}: {e}"
    with open(os.path.join(outdir, f"rank{rank}.txt"), "w") as f:
        f.write(result)
    hb.stop()
    os._exit(0)                            # no collective shutdown: a peer may be gone


@pytest.mark.parametrize("fault", ["1:3:exit", "2:2:raise"])
def test_cpu_ranks_detect_a_lost_peer_without_hanging(tmp_path, fault):
    world = 3
    ctx = mp.get_context("spawn")
    sp, pp = _free_port(), _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, sp, pp, str(tmp_path), fault)) for r in range(world)]
    t0 = time.time()
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(not p.is_alive() for p in procs), "a rank hung"
    assert time.time() - t0 < 50
    bad_rank, bad_step = int(fault.split(":")[0]), int(fault.split(":")[1])
    for r in range(world):
        if r == bad_rank:
            continue
        text = (tmp_path / f"rank{r}.txt").read_text()
        assert text.startswith(f"RankFailure at step {bad_step}"), text
    assert procs[bad_rank].exitcode != 0


def test_corrupted_checkpoint_is_rejected(tmp_path):
    from infinitrain_b200.checkpoint.checkpoint import Checkpoint

    path = str(tmp_path / "model.ckpt")
    Checkpoint.SaveStateDict(path, {"w": torch.arange(12, dtype=torch.float32).view(3, 4)})
    assert torch.equal(Checkpoint.LoadStateDict(path)["w"], torch.arange(12, dtype=torch.float32).view(3, 4))
    corrupt_file(path, 0, 4)               # the magic number
    with pytest.raises(Exception):
        Checkpoint.LoadStateDict(path)


def test_file_rendezvous(tmp_path):
    """Ranks with no MASTER_ADDR meet through a file on a shared filesystem (the reference's scheme)."""
    import subprocess
    import sys

    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rdzv_worker.py")
    path = str(tmp_path / "rendezvous.bin")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", path], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "rank 0 ok" in outs[0] and "rank 1 ok" in outs[1]
