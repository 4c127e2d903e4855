"""Symmetric (peer-mapped) device buffers over NVLink.

Each rank allocates the same-sized buffer; after a rendezvous every rank holds the address at
which each peer's buffer is mapped in its own address space. Kernels of this framework take those
addresses and issue peer loads / stores themselves (see ``csrc/kernels/comm.cu``). Allocation and
handle exchange use ``torch.distributed._symmetric_memory``; synchronisation uses the framework's
own flag barrier with a bounded wait (never a library collective inside the fused paths).

The reference's closest notion is the file-static reduce buffer shared by thread "ranks"
(src/distributed.cpp:14-98).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import native

# ~2 s at 1.9 GHz: a rank that does not show up makes the barrier report a timeout, not hang.
DEFAULT_BARRIER_LIMIT_CYCLES = 4_000_000_000


class SymmBuffer:
    """One symmetric allocation. ``tensor`` is the local part; ``ptrs[r]`` is rank r's part."""

    def __init__(self, numel: int, dtype, device, group):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group=group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank = self.handle.rank
        self.world_size = self.handle.world_size
        # NVLS: address at which every rank's copy is mapped as one multicast object (0 when the
        # allocator could not bind one); multimem.ld_reduce / multimem.st go through it
        try:
            self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        except Exception:
            self.multicast_ptr = 0

    def zero_(self):
        self.tensor.zero_()
        return self


class LocalBuffer:
    """Stand-in used with a single rank (no peers): same attributes, ordinary device memory."""

    def __init__(self, numel: int, dtype, device):
        self.tensor = torch.zeros(numel, dtype=dtype, device=device)
        self.ptrs = [self.tensor.data_ptr()]
        self.rank, self.world_size = 0, 1
        self.multicast_ptr = 0

    def zero_(self):
        self.tensor.zero_()
        return self


def nvls_enabled() -> bool:
    """In-switch reductions and multicast stores (``multimem`` on NVLS multicast mappings) are opt-in:
    ``MYTHOS_NVLS=1``. The default, and what the failure tests use, is plain peer loads and stores: a
    rank that dies while its memory is bound to a multicast object can fault its peers' GPUs."""
    import os

    return os.environ.get("MYTHOS_NVLS", "0") == "1"


def make_buffer(numel: int, dtype, device, group=None):
    if group is None or dist.get_world_size(group) == 1:
        return LocalBuffer(numel, dtype, device)
    return SymmBuffer(numel, dtype, device, group)


class FlagBarrier:
    """Epoch-counting flag barrier between ranks, executed by a one-warp kernel on the current
    stream. ``sync(send)`` optionally delivers one float from every rank to every rank
    (``self.slots`` then holds the world's values in rank order)."""

    def __init__(self, device, group=None, limit_cycles: int = DEFAULT_BARRIER_LIMIT_CYCLES,
                 device_epoch: bool = False):
        self.device = torch.device(device)
        # device-resident epoch: the barrier launch becomes replayable from a CUDA graph
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device) if device_epoch else None
        self.limit = limit_cycles
        self.epoch = 0
        self._flags = make_buffer(64, torch.int32, self.device, group).zero_()
        self._slots = make_buffer(64, torch.float32, self.device, group).zero_()
        self.rank, self.world_size = self._flags.rank, self._flags.world_size
        self.slots = self._slots.tensor
        if group is not None and self.world_size > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)  # flags are zeroed everywhere before the first epoch

    def sync(self, send: torch.Tensor | None = None) -> None:
        self.epoch += 1
        native.require().symm_barrier(self._flags.ptrs, self._slots.ptrs, send, self.rank, self.epoch, self.limit,
                                      native.status_word(self.device), self.epoch_dev)
