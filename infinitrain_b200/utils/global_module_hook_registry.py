"""Process-wide module hooks (reference: infini_train/src/utils/global_module_hook_registry.cc).

Hooks registered here run for EVERY :class:`infinitrain_b200.nn.Module` call: forward-pre, forward
and full-backward.  The precision checker installs itself through this registry.
"""
from __future__ import annotations

from ..common.hook import HookHandle


class GlobalModuleHookRegistry:
    _instance = None

    def __init__(self):
        self.forward_pre_hooks: list = []
        self.forward_hooks: list = []
        self.backward_hooks: list = []

    @classmethod
    def Instance(cls) -> "GlobalModuleHookRegistry":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def RegisterModuleForwardPreHook(self, hook) -> HookHandle:
        self.forward_pre_hooks.append(hook)
        return HookHandle(self.forward_pre_hooks, hook)

    def RegisterModuleForwardHook(self, hook) -> HookHandle:
        self.forward_hooks.append(hook)
        return HookHandle(self.forward_hooks, hook)

    def RegisterModuleFullBackwardHook(self, hook) -> HookHandle:
        self.backward_hooks.append(hook)
        return HookHandle(self.backward_hooks, hook)

    def CallModuleForwardPreHooks(self, module, inputs) -> None:
        for h in list(self.forward_pre_hooks):
            h(module, inputs)

    def CallModuleForwardHooks(self, module, inputs, outputs) -> None:
        for h in list(self.forward_hooks):
            h(module, inputs, outputs)

    def CallModuleFullBackwardHooks(self, module, grad_outputs, grad_inputs) -> None:
        for h in list(self.backward_hooks):
            h(module, grad_outputs, grad_inputs)

    def HasModuleBackwardHooks(self) -> bool:
        return bool(self.backward_hooks)

    def Clear(self) -> None:
        self.forward_pre_hooks.clear()
        self.forward_hooks.clear()
        self.backward_hooks.clear()
