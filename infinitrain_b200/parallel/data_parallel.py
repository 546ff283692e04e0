"""Legacy single-process DataParallel ("parameter server" style).

Reference: infini_train/src/nn/parallel/data_parallel.cc:22-100 with the communication autograd
functions of infini_train/src/autograd/comm.cc:13-124: the input batch is scattered over the devices,
the module is replicated each forward, replicas run in threads, outputs are gathered on the output
device; backward flows through the scatter / gather / broadcast nodes so that parameter gradients
end up reduce-added on the source module.  Kept for API parity — the examples use
DistributedDataParallel, one process per GPU.
"""
from __future__ import annotations

import threading
from typing import List, Optional, Sequence

import torch

from ..nn.module import Module
from . import functional as PF


class _Broadcast(torch.autograd.Function):
    """Copies tensors to every device; backward reduce-adds the per-device gradients."""

    @staticmethod
    def forward(ctx, devices, *tensors):
        ctx.n, ctx.src = len(tensors), [t.device for t in tensors]
        out = []
        for d in devices:
            out += [t.detach().to(d) for t in tensors]
        return tuple(out)

    @staticmethod
    def backward(ctx, *grads):
        n = ctx.n
        res = []
        for i in range(n):
            acc = None
            for k in range(i, len(grads), n):
                if grads[k] is not None:
                    g = grads[k].to(ctx.src[i])
                    acc = g if acc is None else acc + g
            res.append(acc)
        return (None, *res)


class DataParallel(Module):
    kType = "DataParallel"
    kModuleName = "module"

    def __init__(self, module: torch.nn.Module, dim: int = 0, devices: Optional[Sequence[torch.device]] = None):
        super().__init__(self.kType)
        self.add_module(self.kModuleName, module)
        self.dim = dim
        if devices is None:
            n = torch.cuda.device_count() if torch.cuda.is_available() else 0
            devices = [torch.device("cuda", i) for i in range(n)] or [torch.device("cpu")]
        self.devices = list(devices)
        self.output_device = self.devices[0]

    def Forward(self, *inputs):
        module = self._modules[self.kModuleName]
        if len(self.devices) == 1:
            return module(*[x.to(self.devices[0]) for x in inputs])
        scattered = [PF.Scatter(x, self.devices, self.dim) for x in inputs]
        params = list(module.parameters())
        copies = _Broadcast.apply(self.devices, *params)
        outputs: List[Optional[torch.Tensor]] = [None] * len(self.devices)
        errors: List[Optional[BaseException]] = [None] * len(self.devices)

        def run(i, dev):
            try:
                rep_params = copies[i * len(params):(i + 1) * len(params)]
                names = [n for n, _ in module.named_parameters()]
                out = torch.func.functional_call(module, dict(zip(names, rep_params)), tuple(s[i] for s in scattered))
                outputs[i] = out
            except BaseException as e:  # noqa: BLE001
                errors[i] = e

        threads = [threading.Thread(target=run, args=(i, d)) for i, d in enumerate(self.devices)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for e in errors:
            if e is not None:
                raise e
        return PF.Gather(outputs, self.output_device, self.dim)
