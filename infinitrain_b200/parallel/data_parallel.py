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
        self._replicas: Optional[List[torch.nn.Module]] = None

    def _replica_shells(self, module: torch.nn.Module) -> List[torch.nn.Module]:
        """One module object per device.  The replicas' own parameter tensors are never used: every
        forward runs them on the freshly broadcast copies of the source module's parameters (the
        reference replicates the module each forward, data_parallel.cc:61-100).  Separate objects are
        needed because the replicas run in threads, and substituting parameters into ONE module from
        several threads at once would leave it holding a replica's tensors."""
        if self._replicas is None:
            import copy

            self._replicas = [module] + [copy.deepcopy(module).to(d) for d in self.devices[1:]]
        return self._replicas

    def Forward(self, *inputs):
        module = self._modules[self.kModuleName]
        if len(self.devices) == 1:
            return module(*[x.to(self.devices[0]) for x in inputs])
        scattered = [PF.Scatter(x, self.devices, self.dim) for x in inputs]
        names = [n for n, _ in module.named_parameters()]
        params = [p for _, p in module.named_parameters()]
        copies = _Broadcast.apply(self.devices, *params)
        buffers = list(module.named_buffers())
        replicas = self._replica_shells(module)
        outputs: List[Optional[torch.Tensor]] = [None] * len(self.devices)
        errors: List[Optional[BaseException]] = [None] * len(self.devices)

        def run(i, dev):
            try:
                if scattered and scattered[0][i:i + 1] == []:
                    return            # fewer chunks than devices (batch smaller than the device count)
                state = dict(zip(names, copies[i * len(params):(i + 1) * len(params)]))
                state.update({n: b.to(dev) for n, b in buffers})
                out = torch.func.functional_call(replicas[i], state, tuple(s[i] for s in scattered))
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
        return PF.Gather([o for o in outputs if o is not None], self.output_device, self.dim)
