"""Training loop.

``Trainer`` covers the reference's ``Trainer`` (src/trainer.cpp:403-855): ``train_step``,
``fit`` over a data loader with gradient accumulation, global-norm clipping, warm-up/cosine
schedule, periodic codebook EMA, metrics callbacks, validation and checkpointing — with the
differences a GPU framework needs: micro-batches are distinct slices of the batch (the reference
re-runs the same batch ``accum`` times, src/trainer.cpp:493-495), compute is bf16 with fp32
master weights and fp32 gradient accumulation (no loss scaling), and quantisation is in the loop
(STE), which the reference only declares.

A step on the CUDA path:

1. refresh the bf16 compute image of the weights (STE fake-quant kernels),
2. per micro-batch: pinned-host -> device copy, forward, fused CE, backward; weight gradients are
   accumulated in fp32 by the GEMM epilogues into the flat gradient buffer,
3. data-parallel: reduce-scatter of the flat gradient (see :mod:`mythos_b200.parallel.zero`),
4. global-norm clip coefficient computed on the device, fused AdamW on the local shard,
5. data-parallel: all-gather of the refreshed compute image.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Callable

import torch

from ..models.layers import OILLinear
from ..ops import functional as F
from ..ops import native
from ..utils import trace
from . import sched
from .param_store import ParamStore


@dataclass
class TrainConfig:
    batch_size: int = 8            # sequences per optimizer step on this rank
    seq_length: int = 512
    micro_batch_size: int = 0      # sequences per forward/backward (0 = batch_size)
    epochs: int = 3
    max_steps: int = 10000
    lr: float = 3e-4
    weight_decay: float = 1e-2
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    warmup_steps: int = 100
    schedule: str = "warmup_cosine"
    max_grad_norm: float = 1.0     # 0 disables clipping
    activation_checkpointing: bool = False   # recompute block activations in backward (less memory, +1 forward)
    codebook_ema_interval: int = 100
    codebook_ema_decay: float = 0.999
    log_interval: int = 10
    val_interval: int = 0
    save_interval: int = 0
    output_path: str = ""
    seed: int = 42
    extras: dict = field(default_factory=dict)


@dataclass
class TrainMetrics:
    loss: float = 0.0
    perplexity: float = 0.0
    val_loss: float = 0.0
    val_perplexity: float = 0.0
    lr: float = 0.0
    grad_norm: float = 0.0
    tokens_per_sec: float = 0.0
    step: int = 0
    epoch: int = 0


class Trainer:
    def __init__(self, model, cfg: TrainConfig, device=None, dp=None):
        """``dp``: optional data-parallel engine (``mythos_b200.parallel.zero.ZeroEngine``). Without
        it the trainer runs on one device."""
        self.cfg = cfg
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.dp = dp
        world = dp.world_size if dp is not None else 1
        if dp is not None:
            self.store = dp.build_store(model, self.device)
        else:
            self.store = ParamStore(model, self.device, world)
        self.model = model
        if cfg.activation_checkpointing and hasattr(model, "activation_checkpointing"):
            model.activation_checkpointing = True
        n = self.store.shard
        self.m = torch.zeros(n, device=self.device, dtype=torch.float32)
        self.v = torch.zeros(n, device=self.device, dtype=torch.float32)
        self.step = 0
        self.epoch = 0
        self._norm_sq = torch.zeros(1, device=self.device, dtype=torch.float32)
        self._clip = torch.ones(1, device=self.device, dtype=torch.float32)
        self._last_grad_norm = torch.zeros(1, device=self.device, dtype=torch.float32)
        self._ema = {}
        self.log_callbacks: list[Callable[[TrainMetrics], None]] = []
        self.step_callbacks: list[Callable[[TrainMetrics], None]] = []
        self.epoch_callbacks: list[Callable[[TrainMetrics], None]] = []
        self._stale = True  # compute image needs a refresh before the next forward

    # ------------------------------------------------------------------ schedule
    def current_lr(self) -> float:
        c = self.cfg
        return sched.builtin_lr(c.schedule, c.lr, self.step, c.warmup_steps, c.max_steps)

    # ------------------------------------------------------------------ one optimizer step
    def train_step(self, ids, targets) -> torch.Tensor:
        """ids, targets: int32 [B, S] (pinned host tensors or device tensors). Returns the mean
        token loss of the step as a 0-d device tensor (read it with ``.item()`` when needed)."""
        cfg, st = self.cfg, self.store
        cuda = self.device.type == "cuda"
        if cuda:
            self._check_posted_status()
        B = ids.shape[0]
        mb = cfg.micro_batch_size or B
        n_micro = (B + mb - 1) // mb
        tokens = ids.numel() * (self.dp.world_size if self.dp is not None else 1)
        loss_scale = 1.0 / tokens
        if self._stale:
            with trace.span("requantize", self.device):
                self._refresh()
        st.zero_grad()
        total = None
        for i in range(n_micro):
            xi = ids[i * mb:(i + 1) * mb]
            ti = targets[i * mb:(i + 1) * mb]
            if xi.device != self.device:
                xi = xi.to(self.device, non_blocking=True)
                ti = ti.to(self.device, non_blocking=True)
            with trace.span("forward", self.device):
                loss = self.model(xi, ti, loss_scale=loss_scale)
            overlap = self.dp is not None and i == n_micro - 1 and hasattr(self.dp, "arm_overlap")
            if overlap:
                self.dp.arm_overlap(self.model)      # gradient reduce-scatter per layer, under this backward pass
            with trace.span("backward", self.device):
                loss.backward()
            if overlap:
                self.dp.disarm_overlap(self.model)
            if not st.bound:
                st.gather_autograd_grads()
            total = loss.detach() if total is None else total + loss.detach()
        self.step += 1
        lr = self.current_lr()
        with trace.span("optimizer", self.device):
            if self.dp is not None:
                self.dp.step(self, lr)
                total = self.dp.all_reduce_scalar(total)
            else:
                self._local_optimizer_step(lr, 0, st.total)
        self._stale = True
        if cfg.codebook_ema_interval and self.step % cfg.codebook_ema_interval == 0:
            self.update_codebooks()
        if cuda:
            self._post_status_read()
        return total

    def _post_status_read(self):
        """Copies the device status word to pinned host memory without waiting; the next step looks
        at it before launching anything. Kernels that consume barrier-guarded data refuse to write
        once the word is set, so a step whose barrier timed out changes no weights, and the step
        after it raises here."""
        if getattr(self, "_status_host", None) is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(native.status_word(self.device), non_blocking=True)
        self._status_event.record()

    def _check_posted_status(self):
        ev = getattr(self, "_status_event", None)
        if ev is None:
            return
        ev.synchronize()
        code = int(self._status_host[0])
        if code != 0:
            native.status_word(self.device).zero_()
            self._status_host.zero_()
            raise RuntimeError(f"the previous training step reported kernel status {code & 0xffff} at wait site "
                               f"{code >> 16} (1 = a bounded wait expired, e.g. a rank did not reach a barrier); "
                               "its optimizer update was not applied")

    def _refresh(self):
        if self.dp is not None:
            self.dp.refresh_compute(self)
        else:
            self.store.refresh_compute()
        self._stale = False

    def _clip_coef(self, norm_sq: torch.Tensor) -> torch.Tensor:
        """scale = max_norm / (||g|| + 1e-8) if ||g|| > max_norm else 1, on the device."""
        norm = norm_sq.sqrt()
        self._last_grad_norm.copy_(norm)
        if self.cfg.max_grad_norm <= 0:
            self._clip.fill_(1.0)
        else:
            torch.clamp(self.cfg.max_grad_norm / (norm + 1e-8), max=1.0, out=self._clip)
        return self._clip

    def _local_optimizer_step(self, lr: float, lo: int, hi: int):
        st, c = self.store, self.cfg
        self._norm_sq.zero_()
        st.grad_sumsq(self._norm_sq, lo, hi)
        clip = self._clip_coef(self._norm_sq)
        F.adamw_step(st.master[lo:hi], self.m, self.v, st.grad[lo:hi], lr=lr, beta1=c.beta1, beta2=c.beta2,
                     eps=c.eps, weight_decay=c.weight_decay, step=self.step, clip_coef=clip)

    # ------------------------------------------------------------------ codebooks
    @torch.no_grad()
    def update_codebooks(self):
        """EMA update of every OIL8/OIL4 codebook from the current assignment of its weights
        (reference: every 100 steps, decay 0.999, src/trainer.cpp:507-512)."""
        from ..oil.codebook import EMAState

        if self.dp is not None:
            self.dp.gather_master()  # statistics are taken over the full, current master weights
            self._force_refresh = True
        for mod in self.model.modules():
            if not isinstance(mod, OILLinear) or mod.codebooks is None:
                continue
            w = mod.weight.detach().reshape(-1)
            _, idx = F.oil_fake_quant(w, mod.codebooks, mod.cb_map, mod.block_size, want_idx=True)
            counts = torch.zeros_like(mod.codebooks, dtype=torch.float32)
            sums = torch.zeros_like(mod.codebooks, dtype=torch.float32)
            if w.is_cuda:
                native.require().oil_codebook_stats(w, idx, mod.cb_map, mod.codebooks.shape[-1], mod.block_size,
                                                    counts, sums)
            else:
                nb = mod.n_blocks
                cbi = (torch.arange(nb) if mod.cb_map is None else mod.cb_map.long())
                slot = cbi.repeat_interleave(mod.block_size)[: w.numel()] * mod.codebooks.shape[-1] + idx.long()
                counts.view(-1).index_add_(0, slot, torch.ones_like(w))
                sums.view(-1).index_add_(0, slot, w.float())
            # data parallel: every rank sees the same gathered weights, so the statistics agree
            ema = self._ema.get(id(mod))
            if ema is None:
                ema = self._ema[id(mod)] = EMAState(mod.codebooks, self.cfg.codebook_ema_decay)
            ema.update(mod.codebooks, counts, sums)
        self._stale = True

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def eval_loss(self, ids, targets) -> float:
        if self._stale:
            self._refresh()
        ids = ids.to(self.device)
        targets = targets.to(self.device)
        return float(self.model(ids, targets))

    # ------------------------------------------------------------------ epochs
    def fit(self, loader, val_loader=None, max_steps: int | None = None) -> TrainMetrics:
        """Runs ``cfg.epochs`` passes over ``loader`` (an iterable of (ids, targets) batches with a
        ``reset(epoch)`` method) or until ``max_steps``."""
        cfg = self.cfg
        limit = max_steps if max_steps is not None else cfg.max_steps
        metrics = TrainMetrics()
        t_last, tok_since = time.perf_counter(), 0
        done = False
        for epoch in range(cfg.epochs):
            self.epoch = epoch
            if hasattr(loader, "reset"):
                loader.reset(epoch)
            for ids, targets in loader:
                loss = self.train_step(ids, targets)
                tok_since += ids.numel()
                if self.step % max(1, cfg.log_interval) == 0 or self.step >= limit:
                    lv = float(loss)
                    now = time.perf_counter()
                    metrics = TrainMetrics(loss=lv, perplexity=math.exp(min(lv, 30.0)), lr=self.current_lr(),
                                           grad_norm=float(self._last_grad_norm), step=self.step, epoch=epoch,
                                           tokens_per_sec=tok_since / max(1e-9, now - t_last),
                                           val_loss=metrics.val_loss, val_perplexity=metrics.val_perplexity)
                    t_last, tok_since = now, 0
                    for cb in self.log_callbacks:
                        cb(metrics)
                for cb in self.step_callbacks:
                    cb(metrics)
                if val_loader is not None and cfg.val_interval and self.step % cfg.val_interval == 0:
                    vl = [self.eval_loss(a, b) for a, b in val_loader]
                    metrics.val_loss = sum(vl) / max(1, len(vl))
                    metrics.val_perplexity = math.exp(min(metrics.val_loss, 30.0))
                if cfg.save_interval and cfg.output_path and self.step % cfg.save_interval == 0:
                    self.save_checkpoint(cfg.output_path)
                if self.step >= limit:
                    done = True
                    break
            for cb in self.epoch_callbacks:
                cb(metrics)
            if done:
                break
        if cfg.output_path:
            self.save_checkpoint(cfg.output_path)
        return metrics

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, path: str):
        from . import checkpoint

        checkpoint.save_training_state(self, path)

    def load_checkpoint(self, path: str):
        from . import checkpoint

        checkpoint.load_training_state(self, path)
        self._stale = True
