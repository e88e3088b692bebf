"""Native op bindings.

``native()`` returns the compiled sm_100a extension module (``_C.so`` beside the package). On a
machine with a GPU the extension is mandatory: a missing or stale build raises instead of silently
falling back to the PyTorch oracle in :mod:`.reference`.
"""
from __future__ import annotations

import importlib.util
import threading

_lock = threading.Lock()
_mod = None


def native():
    """Load (building first if the tree changed and a compiler is present) the extension module."""
    global _mod
    if _mod is not None:
        return _mod
    with _lock:
        if _mod is not None:
            return _mod
        from .. import _build

        if not _build.SO_PATH.exists():
            _build.build()
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        spec = importlib.util.spec_from_file_location("async_grpo_nccl_b200._C", str(_build.SO_PATH))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
        return _mod


def have_native() -> bool:
    from .. import _build

    return _build.SO_PATH.exists()
