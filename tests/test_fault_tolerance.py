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


def test_corrupt_record_fields_give_clear_errors_before_any_allocation(tmp_path):
    """A damaged dimension or byte-count field must be refused by the record's own consistency checks
    (not by an attempt to allocate what the field says), and a file cut short must say so."""
    import struct

    from infinitrain_b200.checkpoint.checkpoint import Checkpoint

    path = str(tmp_path / "model.ckpt")
    Checkpoint.SaveStateDict(path, {"w": torch.arange(12, dtype=torch.float32).view(3, 4)})
    good = open(path, "rb").read()
    # header 12 B, then: name_len u32 @12, "w" @16, dtype @17, ndim u32 @18, dims i64 @22 and @30, bytes u64 @38, data @46
    assert struct.unpack_from("<q", good, 22)[0] == 3 and struct.unpack_from("<Q", good, 38)[0] == 48

    def damaged(offset, fmt, value):
        b = bytearray(good)
        struct.pack_into(fmt, b, offset, value)
        with open(path, "wb") as f:
            f.write(bytes(b))

    damaged(22, "<q", 1 << 40)                     # a dimension that would ask for terabytes
    with pytest.raises(Exception, match="bytes mismatch|overflow"):
        Checkpoint.LoadStateDict(path)
    damaged(22, "<q", -3)
    with pytest.raises(Exception, match="negative dimension"):
        Checkpoint.LoadStateDict(path)
    damaged(38, "<Q", 1 << 50)                     # byte count that disagrees with the dimensions
    with pytest.raises(Exception, match="bytes mismatch"):
        Checkpoint.LoadStateDict(path)
    with open(path, "wb") as f:                    # consistent record, data cut short
        f.write(good[:-16])
    with pytest.raises(Exception, match="Truncated"):
        Checkpoint.LoadStateDict(path)
    with open(path, "wb") as f:
        f.write(good)
    assert torch.equal(Checkpoint.LoadStateDict(path)["w"], torch.arange(12, dtype=torch.float32).view(3, 4))


def test_a_timed_out_fused_collective_stops_training_on_the_host():
    """The status word of an NVLink context is read at the step's sync point (synchronously) and at the
    fused optimizer step / graph replay (pinned mirror, no sync); a non-zero word raises ``KernelTimeout``.
    The context here is a stand-in: no GPU, no peer, nothing waits."""
    from infinitrain_b200.parallel import symm
    from infinitrain_b200.utils.fault_tolerance import check_device_status

    class _PG:
        name = "DP0"

    ctx = symm.NvlinkContext.__new__(symm.NvlinkContext)
    ctx.pg = _PG()
    ctx.err = torch.zeros(4, dtype=torch.int32)
    ctx.err_host = torch.zeros(4, dtype=torch.int32)
    symm.NvlinkContext._by_group["test:cpu"] = ctx
    try:
        check_device_status(sync=True)             # all clear
        ctx.check()
        ctx.err[0] = 203                           # what rs_adamw_bcast_kernel records when a peer never arrives
        ctx.check()                                # the mirror has not been refreshed yet
        with pytest.raises(KernelTimeout, match="203"):
            check_device_status(sync=True)
        ctx.poll_status()
        with pytest.raises(KernelTimeout, match="not reduced"):
            ctx.check(sync=False)
        with pytest.raises(KernelTimeout):
            check_device_status(sync=False)
    finally:
        del symm.NvlinkContext._by_group["test:cpu"]


def test_injector_refuses_to_kill_a_cuda_rank_with_multicast_on(monkeypatch):
    """``exit`` faults are for CPU ranks, or for GPU runs with NVLS off in NCCL and in this framework:
    a rank that dies while its memory is bound to an NVLink multicast object faults its peers."""
    import infinitrain_b200.utils.fault_tolerance as ft

    assert ft.FaultInjector.exit_allowed()         # this process has no CUDA context
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "is_initialized", lambda: True)
    monkeypatch.delenv("ITB_NVLS", raising=False)
    monkeypatch.delenv("NCCL_NVLS_ENABLE", raising=False)
    assert not ft.FaultInjector.exit_allowed()
    inj = ft.FaultInjector(0, "0:2:exit:17")
    with pytest.raises(RuntimeError, match="refused"):
        inj.maybe_fire(2)
    monkeypatch.setenv("ITB_NVLS", "0")
    assert not ft.FaultInjector.exit_allowed()     # NCCL's own multicast is still on
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    assert ft.FaultInjector.exit_allowed()


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


def test_work_reports_the_communicators_asynchronous_error():
    """CheckCclStatus asks the operation and then its communicator (reference: work.cc:118-132 over
    ncclCommGetAsyncError); the NCCL call is faked here: a backend whose get_error() turns to
    COMM_ERROR after the collective was issued."""
    from infinitrain_b200.parallel.process_group import CclStatus, ProcessGroup, Work

    class FakeBackend:
        code = 0

        def get_error(self):
            return self.code

    class FakePg:
        def __init__(self):
            self.b = FakeBackend()

        def _get_backend(self, device):
            return self.b

    class Group(ProcessGroup):
        backend = "nccl"

    class Handle:
        done = False

        def is_completed(self):
            return self.done

        def exception(self):
            return None

        def wait(self):
            self.done = True

    g = Group("DP0", [0, 1], FakePg())
    assert g.AsyncError() == 0
    w = Work(Handle(), group=g)
    assert w.CheckCclStatus() == CclStatus.kInProgress and not w.IsSuccess()
    g.pg.b.code = 2   # the watchdog saw the communicator fail
    assert g.AsyncError() == 2
    assert w.CheckCclStatus() == CclStatus.kError
    assert "DP0" in str(w.exception()) and not w.IsSuccess()
    # an operation whose own handle carries the error
    h = Handle()
    h.exception = lambda: RuntimeError("remote rank gone")
    w2 = Work(h, group=Group("TP0", [0, 1], FakePg()))
    assert w2.CheckCclStatus() == CclStatus.kError and "remote rank gone" in str(w2.exception())
