"""Failure detection on the host: step heartbeats, a watchdog thread, coordinated abort and
host-side fault injection.

The reference has none of this: a lost peer leaves every other rank inside a collective for ever
(only ``Work::WaitBlocking(timeout)`` and the NCCL async-error query exist, work.cc:37-73,
nccl_impl.cc:63-69).  Here

* every rank publishes ``(step, wall time)`` to a key-value store on a CPU side channel (a
  ``torch.distributed.TCPStore``; any object with ``set`` / ``get`` works) after each step;
* a daemon thread per rank reads the peers' heartbeats and, when one is older than ``timeout_s`` or a
  peer has posted an abort reason, calls ``on_failure(FailureReport)`` -- by default it posts the
  abort reason for everybody else, aborts the process groups it was given (``ncclCommAbort`` through
  ``ProcessGroup.abort`` when the backend has it) and raises ``RankFailure`` in the training thread
  at its next ``Heartbeat.step()``;
* the device-side protocols never wait without a bound: a kernel that gives up writes a code into a
  status word and returns, and ``check_kernel_status`` turns a non-zero word into ``KernelTimeout``
  on the host, so the CUDA context stays usable;
* faults are injected on the host only (``FaultInjector``): a rank can be told through
  ``ITB_FAULT`` to raise, exit, stall or stop sending heartbeats at a given step, and a checkpoint
  file can be corrupted for the loader's error path.  Nothing here makes a GPU fault, trap or hang.
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional


class RankFailure(RuntimeError):
    """A peer stopped sending heartbeats or asked for an abort."""


class KernelTimeout(RuntimeError):
    """A bounded wait inside a kernel ran out; the status word holds the code of the wait."""


@dataclass
class FailureReport:
    kind: str                  # "stale_heartbeat" | "peer_abort" | "self"
    rank: int                  # the rank the report is about
    detail: str = ""
    step: int = -1
    detected_at: float = field(default_factory=time.time)


class DictStore:
    """In-process stand-in for a TCPStore (tests of one process, or threads as ranks)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            if key not in self._d:
                raise KeyError(key)
            return self._d[key]

    def check(self, keys: List[str]) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


def _store_get(store, key: str) -> Optional[bytes]:
    """Non-blocking read: TCPStore.get blocks until the key exists, so ask ``check`` first."""
    try:
        if hasattr(store, "check") and not store.check([key]):
            return None
        return store.get(key)
    except Exception:  # noqa: BLE001
        return None


class Heartbeat:
    """Step heartbeats of one rank plus the watchdog that reads everybody else's."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 60.0, poll_s: float = 0.5,
                 on_failure: Optional[Callable[[FailureReport], None]] = None, process_groups: Iterable = (),
                 prefix: str = "itb/hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.timeout_s, self.poll_s, self.prefix = timeout_s, poll_s, prefix
        self.process_groups = list(process_groups)
        self.on_failure = on_failure or self._default_on_failure
        self.failure: Optional[FailureReport] = None
        self._stop = threading.Event()
        self._muted = False              # fault injection: keep running, stop beating
        self._thread: Optional[threading.Thread] = None
        self._step = -1
        self._started = time.time()

    # ------------------------------------------------------------------ publishing
    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self._step = step
        if not self._muted:
            self.store.set(self._key(self.rank), f"{step}:{time.time():.6f}")

    def step(self, step: int) -> None:
        """Call once per training step: publishes the heartbeat and raises ``RankFailure`` in the
        calling (training) thread when the watchdog has seen a failure."""
        if self.failure is not None:
            raise RankFailure(f"rank {self.failure.rank}: {self.failure.kind} {self.failure.detail}".strip())
        self.beat(step)

    def wait_peers(self, step: int, timeout_s: Optional[float] = None) -> None:
        """Blocks until every peer has published a heartbeat of ``step`` or later; raises
        ``RankFailure`` when one has not within ``timeout_s`` (default: the watchdog's).  Called before
        the first collective of a step, it turns "a peer is gone" into an exception on the host
        instead of a collective that never returns."""
        deadline = time.time() + (self.timeout_s if timeout_s is None else timeout_s)
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            if self.failure is not None:
                raise RankFailure(f"rank {self.failure.rank}: {self.failure.kind} {self.failure.detail}".strip())
            raw = _store_get(self.store, f"{self.prefix}/abort")
            if raw is not None and int(raw.decode().partition(":")[0]) != self.rank:
                who, _, why = raw.decode().partition(":")
                self.failure = FailureReport("peer_abort", int(who), why, step)
                continue
            still = []
            for r in pending:
                raw = _store_get(self.store, self._key(r))
                if raw is None or int(raw.decode().partition(":")[0]) < step:
                    still.append(r)
            pending = still
            if pending:
                if time.time() > deadline:
                    self.failure = FailureReport("stale_heartbeat", pending[0],
                                                 f"did not reach step {step} within the time limit", step)
                    try:
                        self.request_abort(f"rank {pending[0]} did not reach step {step}")
                    except Exception:  # noqa: BLE001
                        pass
                    continue
                time.sleep(min(0.01, self.poll_s))

    def request_abort(self, reason: str) -> None:
        """Tells every rank to stop (they see it at their next watchdog poll)."""
        self.store.set(f"{self.prefix}/abort", f"{self.rank}:{reason}")

    # ------------------------------------------------------------------ watching
    def start(self) -> "Heartbeat":
        self.beat(self._step)
        self._thread = threading.Thread(target=self._watch, name=f"itb-watchdog-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5 * self.poll_s + 1)

    def scan(self, now: Optional[float] = None) -> Optional[FailureReport]:
        """One pass over the store (the watchdog thread calls this; tests may call it directly)."""
        now = time.time() if now is None else now
        raw = _store_get(self.store, f"{self.prefix}/abort")
        if raw is not None:
            who, _, why = raw.decode().partition(":")
            if int(who) != self.rank:
                return FailureReport("peer_abort", int(who), why, self._step)
        for r in range(self.world):
            if r == self.rank:
                continue
            raw = _store_get(self.store, self._key(r))
            if raw is None:
                # never seen: stale only once the grace period since our own start has passed
                if now - self._started > self.timeout_s:
                    return FailureReport("stale_heartbeat", r, "no heartbeat was ever published", self._step)
                continue
            step_s, _, t_s = raw.decode().partition(":")
            if now - float(t_s) > self.timeout_s:
                return FailureReport("stale_heartbeat", r, f"last heartbeat at step {step_s}, "
                                     f"{now - float(t_s):.1f} s ago", int(step_s))
        return None

    def _watch(self) -> None:
        while not self._stop.wait(self.poll_s):
            rep = self.scan()
            if rep is not None:
                self.failure = rep
                try:
                    self.on_failure(rep)
                finally:
                    return

    def _default_on_failure(self, rep: FailureReport) -> None:
        if rep.kind != "peer_abort":
            try:
                self.request_abort(f"{rep.kind} of rank {rep.rank}")
            except Exception:  # noqa: BLE001
                pass
        for pg in self.process_groups:
            abort = getattr(pg, "abort", None)
            if abort is not None:
                try:
                    abort()
                except Exception:  # noqa: BLE001
                    pass


def check_kernel_status(status_fn: Callable[[], int], what: str = "kernel") -> None:
    """Raises ``KernelTimeout`` when a device status word is non-zero.  ``status_fn`` reads the word
    (``_C.kernel_status`` for the single-GPU kernels, ``NvlinkContext.status`` for the NVLink ones)."""
    code = int(status_fn())
    if code != 0:
        raise KernelTimeout(f"{what}: a bounded device-side wait gave up (code {code})")


def check_device_status(sync: bool = True) -> None:
    """One call for a training loop's per-step sync point: raises ``KernelTimeout`` when a bounded
    wait of the single-GPU kernels or of any fused NVLink collective of this process has given up.
    ``sync=True`` reads the words with synchronous copies (use it where the loop has just
    synchronised anyway, e.g. after reading the loss); ``sync=False`` only looks at the pinned host
    mirrors that ``NvlinkContext.poll_status`` refreshes.  Does nothing on CPU ranks."""
    import sys

    symm = sys.modules.get("infinitrain_b200.parallel.symm")
    if symm is not None:
        symm.NvlinkContext.check_all(sync)
    if sync:
        from .. import _ext

        C = _ext.load(required=False)
        import torch

        if C is not None and torch.cuda.is_available() and torch.cuda.is_initialized():
            check_kernel_status(C.kernel_status, "single-GPU kernel")


# --------------------------------------------------------------------------- fault injection (host only)
class FaultInjector:
    """``ITB_FAULT="<rank>:<step>:<kind>[:<arg>]"`` with kind one of

    * ``raise``  -- the rank raises ``RuntimeError`` at that step;
    * ``exit``   -- the rank leaves the process with ``os._exit(arg or 17)`` between two steps;
    * ``stall``  -- the rank sleeps ``arg`` seconds (a straggler);
    * ``mute``   -- the rank keeps training but stops publishing heartbeats.

    ``maybe_fire(step)`` is called by the training loop before it launches anything for the step,
    so no kernel or collective of the faulty rank is in flight when it goes away.  The trainers pass the
    step number as it appears in their log lines (from 1).  A fault read from the environment belongs to
    a job's first attempt: under ``ITB_RESTART_COUNT > 0`` (a job its launcher started again) it is ignored."""

    def __init__(self, rank: int, spec: Optional[str] = None, heartbeat: Optional[Heartbeat] = None):
        self.rank, self.heartbeat = rank, heartbeat
        self.target_rank = self.step = None
        self.kind, self.arg = "", ""
        if spec is None:
            # a fault from the environment belongs to a job's first attempt: the attempt that the launcher starts
            # after it (ITB_RESTART_COUNT > 0) must be able to get past the step
            spec = os.environ.get("ITB_FAULT", "") if int(os.environ.get("ITB_RESTART_COUNT", "0") or 0) == 0 else ""
        if spec:
            parts = spec.split(":")
            self.target_rank, self.step, self.kind = int(parts[0]), int(parts[1]), parts[2]
            self.arg = parts[3] if len(parts) > 3 else ""
        self.fired = False

    @staticmethod
    def exit_allowed() -> bool:
        """A process may be killed by the injector when it has no CUDA context, or when neither NCCL
        nor this framework's kernels use NVLS multicast (``NCCL_NVLS_ENABLE=0`` and ``ITB_NVLS=0``)."""
        import sys

        torch = sys.modules.get("torch")
        on_cuda = torch is not None and torch.cuda.is_available() and torch.cuda.is_initialized()
        if not on_cuda:
            return True
        return os.environ.get("ITB_NVLS", "1") == "0" and os.environ.get("NCCL_NVLS_ENABLE", "") == "0"

    def maybe_fire(self, step: int) -> None:
        if self.fired or self.kind == "" or self.rank != self.target_rank or step != self.step:
            return
        self.fired = True
        if self.kind == "raise":
            raise RuntimeError(f"injected fault on rank {self.rank} at step {step}")
        if self.kind == "exit":
            if not self.exit_allowed():
                raise RuntimeError(
                    "ITB_FAULT ...:exit refused: this process holds CUDA memory that may be bound to an NVLink "
                    "multicast object, and a rank that dies like that faults its peers' GPUs; rerun on CPU ranks, or "
                    "with ITB_NVLS=0 and NCCL_NVLS_ENABLE=0")
            os._exit(int(self.arg or 17))
        if self.kind == "stall":
            time.sleep(float(self.arg or 1.0))
        elif self.kind == "mute":
            if self.heartbeat is not None:
                self.heartbeat._muted = True
        else:
            raise ValueError(f"unknown fault kind {self.kind!r}")


def corrupt_file(path: str, offset: int = 0, nbytes: int = 8) -> None:
    """Flips ``nbytes`` bytes of a file in place (checkpoint-corruption tests)."""
    with open(path, "r+b") as f:
        f.seek(offset)
        data = bytearray(f.read(nbytes))
        for i in range(len(data)):
            data[i] ^= 0xFF
        f.seek(offset)
        f.write(bytes(data))
