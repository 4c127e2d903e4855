"""Optimizers over flat fp32 parameter buffers.

The nine optimizers of the reference (src/optimizer.cpp: SGD with momentum / Nesterov, Adam,
AdamW, Adamax, NAdam, RAdam, Lion, Adafactor, RMSProp) as functional update rules on flat tensors,
so they work on a ZeRO shard as well as on a whole model. AdamW on CUDA runs the fused kernel
(``ops.functional.adamw_step``); the others are expressed with in-place foreach-style tensor
operations (they are not on any benchmark's hot path). Every ``step`` takes an optional gradient
scale (accumulation average x clip coefficient).
"""
from __future__ import annotations

import math

import torch

from ..ops import functional as F


class FlatOptimizer:
    def __init__(self, n: int, device, lr: float = 3e-4, weight_decay: float = 0.0):
        self.n, self.device, self.lr, self.weight_decay = n, torch.device(device), lr, weight_decay
        self.t = 0
        self.state: dict[str, torch.Tensor] = {}

    def _buf(self, name: str) -> torch.Tensor:
        if name not in self.state:
            self.state[name] = torch.zeros(self.n, device=self.device, dtype=torch.float32)
        return self.state[name]

    def step(self, p: torch.Tensor, g: torch.Tensor, lr: float | None = None, grad_scale: float = 1.0) -> None:
        raise NotImplementedError

    def state_dict(self):
        return {"t": self.t, **{k: v.clone() for k, v in self.state.items()}}

    def load_state_dict(self, sd):
        self.t = int(sd.get("t", 0))
        for k, v in sd.items():
            if k != "t":
                self._buf(k).copy_(v)


class SGD(FlatOptimizer):
    def __init__(self, n, device, lr=1e-2, momentum=0.0, nesterov=False, weight_decay=0.0):
        super().__init__(n, device, lr, weight_decay)
        self.momentum, self.nesterov = momentum, nesterov

    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0):
        lr = self.lr if lr is None else lr
        self.t += 1
        g = g * grad_scale + self.weight_decay * p
        if self.momentum > 0:
            buf = self._buf("momentum")
            buf.mul_(self.momentum).add_(g)
            g = g + self.momentum * buf if self.nesterov else buf
        p.add_(g, alpha=-lr)


class Adam(FlatOptimizer):
    decoupled = False

    def __init__(self, n, device, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        super().__init__(n, device, lr, weight_decay)
        self.beta1, self.beta2, self.eps = beta1, beta2, eps

    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0, clip_coef=None):
        lr = self.lr if lr is None else lr
        self.t += 1
        m, v = self._buf("m"), self._buf("v")
        if self.decoupled:
            F.adamw_step(p, m, v, g, lr=lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                         weight_decay=self.weight_decay, step=self.t, grad_scale=grad_scale, clip_coef=clip_coef)
            return
        g = g * grad_scale + self.weight_decay * p  # classic Adam: L2 folded into the gradient
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1, bc2 = 1 - self.beta1 ** self.t, 1 - self.beta2 ** self.t
        p.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-lr)


class AdamW(Adam):
    decoupled = True

    def __init__(self, n, device, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2):
        super().__init__(n, device, lr, beta1, beta2, eps, weight_decay)


class Adamax(Adam):
    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0, clip_coef=None):
        lr = self.lr if lr is None else lr
        self.t += 1
        g = g * grad_scale + self.weight_decay * p
        m, u = self._buf("m"), self._buf("u")
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        torch.maximum(u.mul_(self.beta2), g.abs(), out=u)
        p.addcdiv_(m, u + self.eps, value=-lr / (1 - self.beta1 ** self.t))


class NAdam(Adam):
    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0, clip_coef=None):
        lr = self.lr if lr is None else lr
        self.t += 1
        g = g * grad_scale + self.weight_decay * p
        m, v = self._buf("m"), self._buf("v")
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1, bc2 = 1 - self.beta1 ** self.t, 1 - self.beta2 ** self.t
        mhat = self.beta1 * m / (1 - self.beta1 ** (self.t + 1)) + (1 - self.beta1) * g / bc1
        p.addcdiv_(mhat, (v / bc2).sqrt_().add_(self.eps), value=-lr)


class RAdam(Adam):
    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0, clip_coef=None):
        lr = self.lr if lr is None else lr
        self.t += 1
        g = g * grad_scale + self.weight_decay * p
        m, v = self._buf("m"), self._buf("v")
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1 = 1 - self.beta1 ** self.t
        rho_inf = 2 / (1 - self.beta2) - 1
        rho = rho_inf - 2 * self.t * self.beta2 ** self.t / (1 - self.beta2 ** self.t)
        if rho > 5:
            r = math.sqrt((rho - 4) * (rho - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho))
            p.addcdiv_(m / bc1, (v / (1 - self.beta2 ** self.t)).sqrt_().add_(self.eps), value=-lr * r)
        else:
            p.add_(m / bc1, alpha=-lr)


class Lion(FlatOptimizer):
    def __init__(self, n, device, lr=1e-4, beta1=0.9, beta2=0.99, weight_decay=0.0):
        super().__init__(n, device, lr, weight_decay)
        self.beta1, self.beta2 = beta1, beta2

    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0, clip_coef=None):
        lr = self.lr if lr is None else lr
        self.t += 1
        g = g * grad_scale
        m = self._buf("m")
        update = (self.beta1 * m + (1 - self.beta1) * g).sign_()
        p.mul_(1 - lr * self.weight_decay).add_(update, alpha=-lr)
        m.mul_(self.beta2).add_(g, alpha=1 - self.beta2)


class RMSProp(FlatOptimizer):
    def __init__(self, n, device, lr=1e-3, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0):
        super().__init__(n, device, lr, weight_decay)
        self.alpha, self.eps, self.momentum = alpha, eps, momentum

    @torch.no_grad()
    def step(self, p, g, lr=None, grad_scale=1.0, clip_coef=None):
        lr = self.lr if lr is None else lr
        self.t += 1
        g = g * grad_scale + self.weight_decay * p
        sq = self._buf("sq")
        sq.mul_(self.alpha).addcmul_(g, g, value=1 - self.alpha)
        upd = g / (sq.sqrt() + self.eps)
        if self.momentum > 0:
            buf = self._buf("momentum")
            buf.mul_(self.momentum).add_(upd)
            upd = buf
        p.add_(upd, alpha=-lr)


class Adafactor:
    """Row/column factored second moments for 2-D parameters (vector state for the rest).
    Operates on a list of parameter tensors because the factorisation needs their shapes."""

    def __init__(self, params, lr=1e-3, beta2=0.999, eps=1e-30, clip_threshold=1.0, weight_decay=0.0):
        self.params = list(params)
        self.lr, self.beta2, self.eps, self.clip, self.weight_decay = lr, beta2, eps, clip_threshold, weight_decay
        self.t = 0
        self.state = [{} for _ in self.params]

    @torch.no_grad()
    def step(self, grads, lr=None, grad_scale=1.0):
        lr = self.lr if lr is None else lr
        self.t += 1
        for p, g, st in zip(self.params, grads, self.state):
            g = g.float() * grad_scale
            sq = g * g + self.eps
            if g.dim() == 2:
                r = st.setdefault("row", torch.zeros(g.shape[0], device=g.device))
                c = st.setdefault("col", torch.zeros(g.shape[1], device=g.device))
                r.mul_(self.beta2).add_(sq.mean(1), alpha=1 - self.beta2)
                c.mul_(self.beta2).add_(sq.mean(0), alpha=1 - self.beta2)
                v = torch.outer(r, c) / r.mean().clamp(min=self.eps)
            else:
                v = st.setdefault("v", torch.zeros_like(g))
                v.mul_(self.beta2).add_(sq, alpha=1 - self.beta2)
            u = g / v.sqrt().clamp(min=1e-30)
            u = u / max(1.0, float(u.pow(2).mean().sqrt()) / self.clip)
            p.mul_(1 - lr * self.weight_decay).add_(u.to(p.dtype), alpha=-lr)


OPTIMIZERS = {"sgd": SGD, "adam": Adam, "adamw": AdamW, "adamax": Adamax, "nadam": NAdam, "radam": RAdam,
              "lion": Lion, "rmsprop": RMSProp}


def make_optimizer(name: str, n: int, device, **kw) -> FlatOptimizer:
    try:
        return OPTIMIZERS[name.lower()](n, device, **kw)
    except KeyError:
        raise ValueError(f"unknown optimizer {name!r}; choose from {sorted(OPTIMIZERS)} or adafactor") from None


def clip_coefficient(norm: float, max_norm: float) -> float:
    """scale = max_norm / (norm + 1e-8) when norm > max_norm, else 1 (src/trainer.cpp:608-630)."""
    return max_norm / (norm + 1e-8) if max_norm > 0 and norm > max_norm else 1.0


class DynamicLossScale:
    """Halve (min 1) when the gradient norm overflows or exceeds ``max_norm``, double (max 65536)
    every ``interval`` good steps (src/trainer.cpp:841-853). bf16 training does not need it; kept
    for fp16 compute."""

    def __init__(self, init: float = 128.0, interval: int = 1000, max_norm: float = 1e4):
        self.scale, self.interval, self.max_norm, self.good = init, interval, max_norm, 0

    def update(self, grad_norm: float) -> float:
        if not math.isfinite(grad_norm) or grad_norm > self.max_norm:
            self.scale = max(1.0, self.scale / 2)
            self.good = 0
        else:
            self.good += 1
            if self.good >= self.interval:
                self.scale = min(65536.0, self.scale * 2)
                self.good = 0
        return self.scale


class ModelEMA:
    """Exponential moving average of the flat master weights with swap-in / swap-out for evaluation."""

    def __init__(self, master: torch.Tensor, decay: float = 0.999):
        self.decay = decay
        self.shadow = master.detach().clone()
        self._backup = None

    @torch.no_grad()
    def step(self, master: torch.Tensor) -> None:
        self.shadow.mul_(self.decay).add_(master, alpha=1 - self.decay)

    @torch.no_grad()
    def swap_in(self, master: torch.Tensor) -> None:
        self._backup = master.clone()
        master.copy_(self.shadow)

    @torch.no_grad()
    def swap_out(self, master: torch.Tensor) -> None:
        if self._backup is not None:
            master.copy_(self._backup)
            self._backup = None
