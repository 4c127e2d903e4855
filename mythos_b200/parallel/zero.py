"""ZeRO-style sharded data parallelism.

Rank r owns slice r of the flat fp32 master weights and Adam moments. Every rank holds a full
fp32 gradient buffer (the GEMM epilogues accumulate into it) and a full bf16 compute image of the
weights. One optimizer step is

    grads of all ranks --reduce-scatter--> my gradient slice --AdamW--> my master slice
        --STE fake-quant--> my slice of the compute image --all-gather--> everyone

Two implementations:

``fused`` (the product): gradient and compute buffers live in symmetric memory; three kernels of
    this framework do everything with peer loads/stores over NVLink
    (``csrc/kernels/comm.cu``): flag barrier -> reduce-scatter + norm partial -> flag barrier that
    also exchanges the norm partials -> clip + AdamW + fake-quant + all-gather -> flag barrier.
    With ``MYTHOS_NVLS=1`` the reduce-scatter reads through the NVLS multicast mapping of the
    gradient buffers (``multimem.ld_reduce``: the sum is formed inside the NVSwitch) and the
    all-gather is one ``multimem.st`` per 16 bytes. The reduce-scatter is overlapped with the
    backward pass of the last micro-batch: as soon as a layer's gradients are complete (a hook on
    the layer's input gradient) a side stream runs barrier + reduce-scatter for that layer's slice
    of the flat buffer, so only the embedding's slice, the norm exchange and the optimizer kernel
    remain after the backward pass.
``nccl`` (the baseline it is measured against): ``reduce_scatter_tensor``, ``all_reduce`` of the
    norm, the single-GPU AdamW kernel, ``all_gather_into_tensor`` of the master slice and a local
    re-quantisation.

The fused kernel quantises per 256-element segment of the flat buffer, so it needs quantisation
blocks that are multiples of 256 weights (exactly 256 for I2_S); other models fall back to
``nccl`` with a warning.

The reference's data parallelism is a per-parameter blocking all-reduce through a shared host
buffer with no averaging and no sharding (``DDPWrapper``, src/distributed.cpp:102-138).
"""
from __future__ import annotations

import warnings

import torch
import torch.distributed as dist

from ..models.layers import OILLinear
from ..ops import functional as F
from ..ops import native
from ..train.param_store import ALIGN, ParamStore
from . import symm

FMT_CAST, FMT_OIL8, FMT_OIL4, FMT_I2S, FMT_BINARY = 0, 1, 2, 3, 4


class ZeroEngine:
    def __init__(self, group, device, mode: str = "fused"):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.mode = mode
        self.store: ParamStore | None = None

    # ------------------------------------------------------------------ setup
    def build_store(self, model, device) -> ParamStore:
        slots, total = ParamStore.plan(model, self.world_size)
        if self.mode == "fused" and not self._fusable(slots):
            warnings.warn("quantisation blocks are not multiples of 256 weights: using the NCCL data-parallel path")
            self.mode = "nccl"
        if self.mode == "fused":
            self.grad_buf = symm.make_buffer(total, torch.float32, self.device, self.group)
            self.compute_buf = symm.make_buffer(total, torch.bfloat16, self.device, self.group)
            self.barrier_obj = symm.FlagBarrier(self.device, self.group)
            store = ParamStore(model, device, self.world_size, self.grad_buf.tensor, self.compute_buf.tensor)
            self._build_tables(store)
            self.part = torch.zeros(1, device=self.device, dtype=torch.float32)
            use_mc = symm.nvls_enabled() and self.world_size > 1
            self.grad_mc = self.grad_buf.multicast_ptr if use_mc else 0
            self.compute_mc = self.compute_buf.multicast_ptr if use_mc else 0
            self.comm_stream = torch.cuda.Stream(device=self.device)
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            # per-block partials of the gradient norm (+ a ticket word): added in a fixed order
            self.rs_scratch = torch.zeros(sms * 8 + 2, device=self.device, dtype=torch.float32)
            self._plan_buckets(model, store)
            self._reduced: list[tuple[int, int]] = []   # slices of the flat buffer already reduce-scattered this step
        else:
            store = ParamStore(model, device, self.world_size)
        self.gshard = torch.zeros(store.shard, device=self.device, dtype=torch.float32)
        self.norm_sq = torch.zeros(1, device=self.device, dtype=torch.float32)
        self.store = store
        self.first_refresh_done = False
        # every rank starts from rank 0's weights
        dist.broadcast(store.master, src=dist.get_global_rank(self.group, 0), group=self.group)
        return store

    # ------------------------------------------------------------------ overlap with the backward pass
    def _plan_buckets(self, model, store: ParamStore) -> None:
        """One bucket per transformer block (its contiguous slice of the flat buffer) plus one for
        everything after the last block (final norm, head). ``bucket[i]`` is complete when the
        gradient of block i's input has been computed."""
        self.buckets: dict[int, tuple[int, int]] = {}
        layers = getattr(model, "layers", None)
        if layers is None or not hasattr(model, "grad_ready_callback"):
            return
        by_param = {id(s.param): s for s in store.slots}
        spans = []
        for blk in layers:
            sl = [by_param[id(p)] for p in blk.parameters() if id(p) in by_param]
            if not sl:
                return
            spans.append((min(x.offset for x in sl), max(x.offset + (x.numel + ALIGN - 1) // ALIGN * ALIGN for x in sl)))
        if any(a >= b for a, b in spans) or any(spans[i][1] > spans[i + 1][0] for i in range(len(spans) - 1)):
            return                                  # blocks are not laid out one after another: no overlap
        for i, sp in enumerate(spans):
            self.buckets[i] = sp
        if spans[-1][1] < store.total:
            self.buckets[len(spans)] = (spans[-1][1], store.total)

    def arm_overlap(self, model) -> None:
        """Call before the backward pass of the step's LAST micro-batch."""
        if self.mode != "fused" or not self.buckets or self.world_size == 1:
            return
        self.part.zero_()
        self._reduced = []
        model.grad_ready_callback = self._on_bucket_ready

    def disarm_overlap(self, model) -> None:
        if hasattr(model, "grad_ready_callback"):
            model.grad_ready_callback = None

    def _on_bucket_ready(self, index: int) -> None:
        span = self.buckets.get(index)
        if span is None:
            return
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ev)
            self.barrier_obj.sync()                      # every rank has finished this bucket's gradients
            self._reduce_span(span[0], span[1], max_blocks=64)
        self._reduced.append(span)

    def _reduce_span(self, a: int, b: int, max_blocks: int = 0) -> None:
        """Reduce-scatter of flat elements [a, b): this rank sums the part that lies in its shard."""
        lo = self.rank * self.store.shard
        s0, e0 = max(a, lo), min(b, lo + self.store.shard)
        if s0 >= e0:
            return
        native.require().zero_reduce_scatter(self.grad_buf.ptrs, self.gshard[s0 - lo:e0 - lo], s0, self.part,
                                             self.grad_mc, max_blocks, self.rs_scratch)

    @staticmethod
    def _fusable(slots) -> bool:
        for s in slots:
            m = s.module
            if m is None:
                continue
            if m.fmt in ("oil8", "oil4") and m.block_size % ALIGN != 0:
                return False
            if m.fmt in ("i2s", "mixed") and m.block_size != ALIGN:
                return False
        return True

    def _build_tables(self, store: ParamStore) -> None:
        """Per-segment format / codebook tables and one global codebook table per format; module
        codebooks become views of the tables so EMA updates are seen by the fused kernel."""
        nseg = store.total // ALIGN
        seg_fmt = torch.zeros(nseg, dtype=torch.uint8)
        seg_cb = torch.zeros(nseg, dtype=torch.int32)
        n8 = n4 = 0
        mods = []
        for s in store.slots:
            m = s.module
            if m is None or m.fmt not in ("oil8", "oil4", "i2s", "mixed"):
                continue
            s0, ns = s.offset // ALIGN, (s.numel + ALIGN - 1) // ALIGN
            if m.fmt == "i2s":
                seg_fmt[s0:s0 + ns] = FMT_I2S
                continue
            if m.fmt == "mixed":
                # one 256-weight block per segment: the segment's format is the block's format; both
                # codebook families of the layer go into the global tables
                code = m.block_formats.cpu().long()[:ns]
                local = m.cb_map.cpu().long()[:ns]
                seg_fmt[s0:s0 + ns] = torch.where(code == 3, FMT_OIL8, torch.where(code == 2, FMT_OIL4, torch.where(code == 0, FMT_BINARY, FMT_I2S))).to(torch.uint8)
                seg_cb[s0:s0 + ns] = torch.where(code == 3, local + n8, local + n4).to(torch.int32)
                mods.append((m, "oil8", n8))
                mods.append((m, "mixed4", n4))
                n8 += m.codebooks.shape[0]
                n4 += m.codebooks4.shape[0]
                continue
            blocks = (torch.arange(ns) * ALIGN) // m.block_size
            local = blocks if m.cb_map is None else m.cb_map.cpu().long()[blocks.clamp(max=m.n_blocks - 1)]
            if m.fmt == "oil8":
                seg_fmt[s0:s0 + ns] = FMT_OIL8
                seg_cb[s0:s0 + ns] = (local + n8).to(torch.int32)
                mods.append((m, "oil8", n8))
                n8 += m.codebooks.shape[0]
            else:
                seg_fmt[s0:s0 + ns] = FMT_OIL4
                seg_cb[s0:s0 + ns] = (local + n4).to(torch.int32)
                mods.append((m, "oil4", n4))
                n4 += m.codebooks.shape[0]
        dev = self.device
        self.cb8 = torch.zeros(max(n8, 1), 256, device=dev, dtype=torch.float32)
        self.cb4 = torch.zeros(max(n4, 1), 16, device=dev, dtype=torch.float32)
        for m, kind, base in mods:
            if kind == "mixed4":
                view = self.cb4[base:base + m.codebooks4.shape[0]]
                view.copy_(m.codebooks4)
                m.codebooks4 = view
                continue
            table = self.cb8 if kind == "oil8" else self.cb4
            view = table[base:base + m.codebooks.shape[0]]
            view.copy_(m.codebooks)
            m.codebooks = view  # registered buffer now aliases the global table
        self.seg_fmt = seg_fmt.to(dev)
        self.seg_cb = seg_cb.to(dev)

    # ------------------------------------------------------------------ per-step hooks used by Trainer
    def refresh_compute(self, trainer) -> None:
        """Full local re-quantisation. With the fused path this is only needed before the first
        step and after codebook updates: every later step refreshes the image inside the optimizer
        kernel."""
        if self.mode == "fused" and self.first_refresh_done and not getattr(trainer, "_force_refresh", False):
            return
        self.store.refresh_compute()
        self.first_refresh_done = True
        trainer._force_refresh = False
        if self.mode == "fused":
            self.barrier_obj.sync()

    def step(self, trainer, lr: float) -> None:
        st, c = self.store, trainer.cfg
        lo = self.rank * st.shard
        if self.mode == "fused":
            C = native.require()
            done = sorted(getattr(self, "_reduced", []))
            if done:
                torch.cuda.current_stream().wait_stream(self.comm_stream)   # the overlapped buckets have landed
            else:
                self.part.zero_()
            self._reduced = []
            self.barrier_obj.sync()                                   # every rank's gradients are complete
            pos = 0
            for a, b in done + [(st.total, st.total)]:                # whatever the backward pass did not cover
                if a > pos:
                    self._reduce_span(pos, a)
                pos = max(pos, b)
            self.barrier_obj.sync(self.part)                          # norm partials exchanged; peers done reading
            C.zero_adamw_ste_allgather(st.master[lo:lo + st.shard], trainer.m, trainer.v, self.gshard,
                                       self.compute_buf.ptrs, lo, self.seg_fmt, self.seg_cb, self.cb8, self.cb4,
                                       self.barrier_obj.slots, trainer._last_grad_norm, c.max_grad_norm, lr,
                                       c.beta1, c.beta2, c.eps, c.weight_decay, trainer.step, 1.0, self.rank,
                                       self.compute_mc)
            self.barrier_obj.sync()                                   # every rank's compute image is complete
        else:
            dist.reduce_scatter_tensor(self.gshard, st.grad[: st.total], op=dist.ReduceOp.SUM, group=self.group)
            self.norm_sq.zero_()
            F.sumsq(self.gshard, self.norm_sq)
            dist.all_reduce(self.norm_sq, group=self.group)
            clip = trainer._clip_coef(self.norm_sq)
            F.adamw_step(st.master[lo:lo + st.shard], trainer.m, trainer.v, self.gshard, lr=lr, beta1=c.beta1,
                         beta2=c.beta2, eps=c.eps, weight_decay=c.weight_decay, step=trainer.step, clip_coef=clip)
            self.gather_master()
            st.refresh_compute()
            self.first_refresh_done = True

    def gather_master(self) -> None:
        """All-gather the master slices so every rank holds the full fp32 weights (checkpointing,
        codebook statistics, the NCCL path's re-quantisation)."""
        st = self.store
        lo = self.rank * st.shard
        dist.all_gather_into_tensor(st.master[: st.total], st.master[lo:lo + st.shard].clone(), group=self.group)

    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        t = t.clone()
        dist.all_reduce(t, group=self.group)
        return t

    def all_reduce_(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    def release(self) -> None:
        """Drop the symmetric gradient / compute buffers and the shard state (collective: every rank
        calls it at the same point, with no kernel of the engine in flight)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.grad_mc = self.compute_mc = 0
        for name in ("grad_buf", "compute_buf", "barrier_obj", "gshard", "store", "cb8", "cb4", "seg_fmt", "seg_cb"):
            if hasattr(self, name):
                setattr(self, name, None)
