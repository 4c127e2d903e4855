"""Flat parameter storage for the native training path.

All parameters of a model are re-homed into three flat buffers:

* ``master``  fp32  the weights the optimizer updates (``param.data`` becomes a view of it),
* ``grad``    fp32  gradient accumulator; kernels add into ``param.main_grad`` views of it,
* ``compute`` bf16  what the forward/backward GEMMs read: the fake-quantised (STE) image of the
  master weight for ``OILLinear`` parameters, a plain cast for norms and embeddings.

Flat buffers are what the sharded optimizer and the fused reduce-scatter / all-gather kernels
operate on: rank r owns the contiguous slice ``[r*shard, (r+1)*shard)`` of ``master`` (and of the
Adam moments); ``grad`` and ``compute`` are full-size on every rank. Each parameter starts on a
256-element boundary so that shards and vector accesses stay aligned.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..models.layers import OILLinear
from ..ops import native

ALIGN = 256


@dataclass
class Slot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    module: nn.Module | None  # the OILLinear owning the weight, if any


class ParamStore:
    @staticmethod
    def plan(model: nn.Module, world_size: int = 1):
        """Flat layout of the trainable parameters: (slots, total elements). ``total`` is padded so
        that every rank's shard is a whole number of 256-element segments."""
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not params:
            raise ValueError("model has no trainable parameters")
        owners = {}
        for m in model.modules():
            if isinstance(m, OILLinear):
                owners[id(m.weight)] = m
        slots: list[Slot] = []
        off = 0
        for n, p in params:
            slots.append(Slot(n, p, off, p.numel(), owners.get(id(p))))
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        unit = ALIGN * world_size
        return slots, (off + unit - 1) // unit * unit

    def __init__(self, model: nn.Module, device=None, world_size: int = 1, grad_buffer: torch.Tensor | None = None,
                 compute_buffer: torch.Tensor | None = None):
        self.slots, self.total = self.plan(model, world_size)
        device = torch.device(device) if device is not None else self.slots[0].param.device
        self.world_size = world_size
        self.shard = self.total // world_size
        self.device = device
        self.master = torch.zeros(self.total, device=device, dtype=torch.float32)
        self.grad = grad_buffer if grad_buffer is not None else torch.zeros(self.total, device=device,
                                                                             dtype=torch.float32)
        self.compute = compute_buffer if compute_buffer is not None else torch.zeros(
            self.total, device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
        assert self.grad.numel() >= self.total and self.compute.numel() >= self.total
        # On CPU the model runs the reference operators under ordinary autograd (STE inside
        # OILLinear), so parameters are only re-homed; gradients are gathered from ``.grad``.
        self.bound = device.type == "cuda"
        for s in self.slots:
            view = self.master[s.offset:s.offset + s.numel].view(s.param.shape)
            view.copy_(s.param.data.to(device))
            s.param.data = view
            if self.bound:
                s.param.main_grad = self.grad[s.offset:s.offset + s.numel].view(s.param.shape)
                # The compute image is a leaf that "requires grad" so autograd records the graph of
                # the custom functions; their backward adds into main_grad and returns no gradient.
                s.param.compute = self.compute[s.offset:s.offset + s.numel].view(s.param.shape).requires_grad_()
        model.to(device)  # buffers (codebooks, maps); parameters already live in the flat buffer
        for s in self.slots:  # .to() may have rebound param.data; restore the views
            s.param.data = self.master[s.offset:s.offset + s.numel].view(s.param.shape)
        self.model = model

    # ------------------------------------------------------------------ per-step operations
    def zero_grad(self) -> None:
        self.grad[: self.total].zero_()
        if not self.bound:
            for s in self.slots:
                s.param.grad = None

    def gather_autograd_grads(self) -> None:
        """CPU path: add each parameter's autograd ``.grad`` into the flat gradient buffer."""
        for s in self.slots:
            if s.param.grad is not None:
                self.grad[s.offset:s.offset + s.numel].add_(s.param.grad.reshape(-1).float())
                s.param.grad = None

    def refresh_compute(self, lo: int = 0, hi: int | None = None) -> None:
        """Recompute the bf16 compute image of every parameter overlapping ``[lo, hi)`` from the
        master weights (STE fake-quantisation for OIL formats, cast otherwise)."""
        hi = self.total if hi is None else hi
        cuda = self.device.type == "cuda"
        C = native.require() if cuda else None
        for s in self.slots:
            if s.offset + s.numel <= lo or s.offset >= hi:
                continue
            src = self.master[s.offset:s.offset + s.numel]
            dst = self.compute[s.offset:s.offset + s.numel]
            m = s.module
            if m is not None and m.fmt in ("oil8", "oil4", "i2s", "mixed"):
                m.quantize_now(src, out=dst) if cuda else dst.copy_(m.quantize_now(src))
            elif cuda:
                C.cast_f32_to_bf16(src, dst)
            else:
                dst.copy_(src)

    def grad_sumsq(self, out: torch.Tensor | None = None, lo: int = 0, hi: int | None = None) -> torch.Tensor:
        from ..ops import functional as F

        hi = self.total if hi is None else hi
        if out is None:
            out = torch.zeros(1, device=self.device, dtype=torch.float32)
        return F.sumsq(self.grad[lo:hi], out)

    def state_dict_flat(self):
        return {"master": self.master, "total": self.total, "names": [s.name for s in self.slots],
                "offsets": [s.offset for s in self.slots], "numels": [s.numel for s in self.slots]}
