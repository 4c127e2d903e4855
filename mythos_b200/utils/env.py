"""Runtime environment variables.

The reference documents ``OIL_NUM_THREADS``, ``OIL_MEMORY_POOL_SIZE``, ``OIL_SEED``,
``OIL_LOG_LEVEL``, ``OIL_VERBOSE`` and ``OIL_GPU_DEVICE`` (README.md:1335-1344) but reads none of
them. Here they are read once by ``RuntimeEnv.from_environ()`` and take effect through
``apply()``, which the command-line tools call before anything else:

* ``OIL_NUM_THREADS``  -> ``torch.set_num_threads`` (host-side ops, tokeniser, data loading)
* ``OIL_MEMORY_POOL_SIZE`` -> size in bytes of the host page pool of the native runtime
* ``OIL_SEED``         -> default seed of the tools (``torch.manual_seed``)
* ``OIL_LOG_LEVEL``    -> level of the ``mythos_b200`` logger (debug / info / warn / error)
* ``OIL_VERBOSE``      -> per-range device timing in ``utils.trace``
* ``OIL_GPU_DEVICE``   -> CUDA device index used when a tool is given ``--gpu auto``
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass

import torch

_LEVELS = {"debug": logging.DEBUG, "info": logging.INFO, "warn": logging.WARNING, "warning": logging.WARNING,
           "error": logging.ERROR}


def _int(env, key: str, default: int, lo: int = 0) -> int:
    try:
        return max(lo, int(env.get(key, default)))
    except (TypeError, ValueError):
        return default


@dataclass
class RuntimeEnv:
    num_threads: int = 0                 # 0 = leave torch's default (the core count)
    memory_pool_size: int = 64 << 20
    seed: int = 42
    log_level: str = "info"
    verbose: bool = False
    gpu_device: int = 0

    @classmethod
    def from_environ(cls, env=None) -> "RuntimeEnv":
        env = os.environ if env is None else env
        level = str(env.get("OIL_LOG_LEVEL", "info")).lower()
        return cls(num_threads=_int(env, "OIL_NUM_THREADS", 0),
                   memory_pool_size=_int(env, "OIL_MEMORY_POOL_SIZE", 64 << 20, 4096),
                   seed=_int(env, "OIL_SEED", 42),
                   log_level=level if level in _LEVELS else "info",
                   verbose=str(env.get("OIL_VERBOSE", "0")) not in ("", "0"),
                   gpu_device=_int(env, "OIL_GPU_DEVICE", 0))

    def apply(self) -> "RuntimeEnv":
        from . import trace

        if self.num_threads > 0:
            torch.set_num_threads(self.num_threads)
        torch.manual_seed(self.seed)
        logging.getLogger("mythos_b200").setLevel(_LEVELS[self.log_level])
        trace.enable_timing(self.verbose)
        return self

    def default_device(self) -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", min(self.gpu_device, torch.cuda.device_count() - 1))
        return torch.device("cpu")


_current: RuntimeEnv | None = None


def current() -> RuntimeEnv:
    """The process-wide settings (read from the environment on first use)."""
    global _current
    if _current is None:
        _current = RuntimeEnv.from_environ()
    return _current


def reset() -> None:
    global _current
    _current = None
