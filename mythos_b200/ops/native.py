"""Loader for the compiled sm_100a extension (``mythos_b200/_C*.so``).

The extension is built in-tree by :mod:`mythos_b200.build`. On a machine with a GPU the
kernels are the only compute path: if the extension cannot be imported there, :func:`require`
raises instead of silently falling back to PyTorch operators. On CPU-only machines the pure
PyTorch reference implementations in :mod:`mythos_b200.ops.reference` are used (they are the
numerical oracle of the kernel tests as well).
"""
from __future__ import annotations

import importlib
import threading

import torch

_lock = threading.Lock()
_ext = None
_err: Exception | None = None


def _load():
    global _ext, _err
    with _lock:
        if _ext is None and _err is None:
            try:
                _ext = importlib.import_module("mythos_b200._C")
            except Exception as e:  # noqa: BLE001 - reported by require()
                _err = e
    return _ext


def available() -> bool:
    """True when the extension imports and a CUDA device is visible."""
    return torch.cuda.is_available() and _load() is not None


def require():
    """Return the extension module or raise with the import error and the build command."""
    ext = _load()
    if ext is None:
        raise RuntimeError(
            "mythos_b200 native kernels are not built or failed to import "
            f"({_err!r}). Build them with `python -m mythos_b200.build`."
        )
    return ext


def launch_count() -> int:
    """Number of kernels launched by this library in this process (0 if not loaded)."""
    ext = _load()
    return int(ext.launch_count()) if ext is not None else 0


_status: dict = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write a non-zero code into."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
        ext = _load()
        if dev.type == "cuda" and ext is not None and hasattr(ext, "comm_set_abort_word"):
            ext.comm_set_abort_word(t)    # collective kernels stop writing once a bounded wait has expired
    return t


def check_status(device) -> None:
    """Synchronising check of the status word; raises if a bounded wait expired in a kernel."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"kernel reported status {code & 0xffff} at wait site {code >> 16} (1 = bounded wait expired)")
