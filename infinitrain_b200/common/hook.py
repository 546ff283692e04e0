"""Removable hook handles (reference: infini_train/include/common/hook.h:7-28)."""
from __future__ import annotations


class HookHandle:
    """Handle returned by every ``Register*Hook`` call; ``Remove()`` detaches the hook."""

    def __init__(self, container: list, hook):
        self._container = container
        self._hook = hook

    def Remove(self) -> None:
        if self._container is not None:
            try:
                self._container.remove(self._hook)
            except ValueError:
                pass
            self._container = None

    remove = Remove


class TorchHookHandle(HookHandle):
    """Wraps a ``torch.utils.hooks.RemovableHandle``."""

    def __init__(self, handle):
        self._handle = handle

    def Remove(self) -> None:
        if self._handle is not None:
            self._handle.remove()
            self._handle = None

    remove = Remove
