"""Devices, the RAII device guard and stream / event helpers.

Reference: infini_train/include/device.h:11-47, infini_train/include/core/runtime/device_guard.h:59-233,
infini_train/src/core/runtime/cuda/cuda_guard_impl.cc.  The reference registers one guard
implementation per backend behind a virtual API; here there is a single accelerator backend (CUDA
on sm_100a) so the guard is a thin layer over ``torch.cuda``: the PyTorch caching allocator replaces
``cudaMallocAsync``, one compute stream per device plus named high-priority side streams replace the
per-group communication streams.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, Optional

import torch


class DeviceType(enum.IntEnum):
    kCPU = 0
    kCUDA = 1


@dataclass(frozen=True)
class Device:
    type: DeviceType = DeviceType.kCPU
    index: int = 0

    @staticmethod
    def CPU() -> "Device":
        return Device(DeviceType.kCPU, 0)

    @staticmethod
    def CUDA(index: int = 0) -> "Device":
        return Device(DeviceType.kCUDA, index)

    @staticmethod
    def from_torch(d) -> "Device":
        d = torch.device(d)
        return Device(DeviceType.kCUDA if d.type == "cuda" else DeviceType.kCPU, d.index or 0)

    def IsCPU(self) -> bool:
        return self.type == DeviceType.kCPU

    def IsCUDA(self) -> bool:
        return self.type == DeviceType.kCUDA

    def torch_device(self) -> torch.device:
        return torch.device("cuda", self.index) if self.IsCUDA() else torch.device("cpu")

    def Rank(self):
        """(process rank, local rank) coordinates of the rank that drives this device."""
        from .parallel import global_env
        from .parallel.rank import Rank

        return Rank(global_env.GetGlobalProcRank(), self.index, global_env.GetWorldSize(), 1)

    def ToString(self) -> str:
        return f"Device({'CUDA' if self.IsCUDA() else 'CPU'}, {self.index})"

    __str__ = ToString


class DeviceGuard:
    """Makes ``device`` current for the ``with`` body and restores the previous one after."""

    def __init__(self, device: Device):
        self.device = device
        self._ctx = None

    def __enter__(self):
        if self.device.IsCUDA() and torch.cuda.is_available():
            self._ctx = torch.cuda.device(self.device.index)
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
        return False


class DeviceGuardImpl:
    """Runtime services of one backend: streams, events, synchronisation, memory statistics."""

    _side_streams: Dict[tuple, "torch.cuda.Stream"] = {}

    @staticmethod
    def DeviceCount() -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    @staticmethod
    def GetStream(device: Device):
        return torch.cuda.current_stream(device.index) if device.IsCUDA() else None

    @classmethod
    def GetSideStream(cls, device: Device, name: str = "comm", high_priority: bool = True):
        """A named non-blocking stream per device, created on first use (high priority by default,
        like the reference's communication streams)."""
        if not device.IsCUDA():
            return None
        key = (device.index, name)
        if key not in cls._side_streams:
            cls._side_streams[key] = torch.cuda.Stream(device=device.index, priority=-1 if high_priority else 0)
        return cls._side_streams[key]

    @staticmethod
    def CreateStream(device: Device):
        return torch.cuda.Stream(device=device.index) if device.IsCUDA() else None

    @staticmethod
    def CreateStreamWithPriority(device: Device, priority: int):
        """``priority`` as the CUDA runtime counts: 0 = default, negative = higher."""
        return torch.cuda.Stream(device=device.index, priority=priority) if device.IsCUDA() else None

    @staticmethod
    def GetStreamPriorityRange():
        """(lowest, highest) priority a stream can be created with; the highest is the most negative."""
        if not torch.cuda.is_available():
            return 0, 0
        low, high = torch.cuda.Stream.priority_range()
        return low, high

    @staticmethod
    def CreateEvent(timing: bool = False):
        return torch.cuda.Event(enable_timing=timing)

    # Events: on a CPU device every call is a no-op that reports success (work has completed when the
    # call that issued it returns), so code written against this interface also runs in CPU tests.
    @staticmethod
    def EventRecord(event, stream=None) -> None:
        if event is not None:
            event.record(stream) if stream is not None else event.record()

    @staticmethod
    def StreamWaitEvent(stream, event) -> None:
        if stream is not None and event is not None:
            stream.wait_event(event)

    @staticmethod
    def EventSynchronize(event) -> bool:
        if event is not None:
            event.synchronize()
        return True

    @staticmethod
    def EventQuery(event) -> bool:
        return True if event is None else bool(event.query())

    @staticmethod
    def EventElapsedTime(start, stop) -> float:
        """Milliseconds between two recorded timing events (0 on a CPU device)."""
        return 0.0 if start is None or stop is None else float(start.elapsed_time(stop))

    @staticmethod
    def SynchronizeStream(stream) -> None:
        if stream is not None:
            stream.synchronize()

    @staticmethod
    def Malloc(device: Device, nbytes: int, stream=None) -> int:
        """A raw block out of the caching allocator the tensors use (so it shows in the same statistics);
        returns its address.  With ``stream`` the block may be reused by later work of that stream as soon
        as it is freed (the reference's MallocAsync)."""
        if not device.IsCUDA():
            raise RuntimeError("raw device memory exists on CUDA devices only")
        return int(torch.cuda.caching_allocator_alloc(nbytes, device.index, stream))

    MallocAsync = Malloc

    @staticmethod
    def Free(ptr: int) -> None:
        if ptr:
            torch.cuda.caching_allocator_delete(ptr)

    @staticmethod
    def SynchronizeDevice(device: Device) -> None:
        if device.IsCUDA():
            torch.cuda.synchronize(device.index)

    @staticmethod
    def ResetMemPoolHighWatermarks(device: Device) -> None:
        if device.IsCUDA():
            torch.cuda.reset_peak_memory_stats(device.index)

    @staticmethod
    def GetMemPoolPeakMB(device: Device):
        """(peak used MB, peak reserved MB) since the last reset."""
        if not device.IsCUDA():
            return 0.0, 0.0
        return (torch.cuda.max_memory_allocated(device.index) / (1 << 20),
                torch.cuda.max_memory_reserved(device.index) / (1 << 20))


def GetDeviceGuardImpl(device_type: DeviceType = DeviceType.kCUDA) -> type:
    return DeviceGuardImpl
