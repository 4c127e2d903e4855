"""Learning-rate schedules.

Two families, as in the reference: the five schedules built into its AdamW
(CONSTANT / COSINE / LINEAR / WARMUP_COSINE / COSINE_RESTART, src/optimizer.cpp:57-90) exposed
through :func:`builtin_lr`, and the ten stand-alone scheduler classes of src/scheduler.cpp
(Constant, LinearDecay, CosineDecay, ExponentialDecay, StepDecay, ReduceLROnPlateau, OneCycle,
Warmup wrapper, Sequential, Lambda). All are pure functions of the step (plus the metric for
ReduceLROnPlateau) so they can be evaluated on the host without touching the device.
"""
from __future__ import annotations

import math
from typing import Callable, Sequence

LR_FLOOR = 1e-8


def builtin_lr(kind: str, base_lr: float, step: int, warmup: int = 0, total: int = 10000, restart_period: int = 1000):
    kind = kind.lower()
    if kind == "constant":
        return base_lr
    if kind == "cosine":
        t = min(1.0, step / max(1, total))
        return max(LR_FLOOR, base_lr * 0.5 * (1.0 + math.cos(math.pi * t)))
    if kind == "linear":
        t = min(1.0, step / max(1, total))
        return max(LR_FLOOR, base_lr * (1.0 - t))
    if kind == "warmup_cosine":
        if warmup > 0 and step < warmup:
            return max(LR_FLOOR, base_lr * step / warmup)
        t = min(1.0, (step - warmup) / max(1, total - warmup))
        return max(LR_FLOOR, base_lr * 0.5 * (1.0 + math.cos(math.pi * t)))
    if kind == "cosine_restart":
        t = (step % max(1, restart_period)) / max(1, restart_period)
        return max(LR_FLOOR, base_lr * 0.5 * (1.0 + math.cos(math.pi * t)))
    raise ValueError(f"unknown schedule {kind!r}")


class Scheduler:
    def __init__(self, base_lr: float):
        self.base_lr = base_lr

    def lr(self, step: int) -> float:  # pragma: no cover - interface
        raise NotImplementedError

    def __call__(self, step: int) -> float:
        return self.lr(step)


class Constant(Scheduler):
    def lr(self, step):
        return self.base_lr


class LinearDecay(Scheduler):
    def __init__(self, base_lr, total_steps, end_lr=0.0):
        super().__init__(base_lr)
        self.total, self.end = total_steps, end_lr

    def lr(self, step):
        t = min(1.0, step / max(1, self.total))
        return self.base_lr + (self.end - self.base_lr) * t


class CosineDecay(Scheduler):
    def __init__(self, base_lr, total_steps, min_lr=0.0):
        super().__init__(base_lr)
        self.total, self.min = total_steps, min_lr

    def lr(self, step):
        t = min(1.0, step / max(1, self.total))
        return self.min + (self.base_lr - self.min) * 0.5 * (1.0 + math.cos(math.pi * t))


class ExponentialDecay(Scheduler):
    def __init__(self, base_lr, gamma):
        super().__init__(base_lr)
        self.gamma = gamma

    def lr(self, step):
        return self.base_lr * self.gamma ** step


class StepDecay(Scheduler):
    def __init__(self, base_lr, step_size, gamma=0.1):
        super().__init__(base_lr)
        self.step_size, self.gamma = step_size, gamma

    def lr(self, step):
        return self.base_lr * self.gamma ** (step // max(1, self.step_size))


class ReduceLROnPlateau(Scheduler):
    """Stateful: call :meth:`observe` with the monitored metric; ``lr`` returns the current value."""

    def __init__(self, base_lr, factor=0.5, patience=5, min_lr=0.0, threshold=1e-4):
        super().__init__(base_lr)
        self.factor, self.patience, self.min_lr, self.threshold = factor, patience, min_lr, threshold
        self.best = math.inf
        self.bad = 0
        self.current = base_lr

    def observe(self, metric: float) -> float:
        if metric < self.best - self.threshold:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.current = max(self.min_lr, self.current * self.factor)
                self.bad = 0
        return self.current

    def lr(self, step):
        return self.current


class OneCycle(Scheduler):
    def __init__(self, max_lr, total_steps, pct_start=0.3, div_factor=25.0, final_div_factor=1e4):
        super().__init__(max_lr)
        self.total, self.pct = total_steps, pct_start
        self.initial = max_lr / div_factor
        self.final = self.initial / final_div_factor

    def lr(self, step):
        up = max(1, int(self.total * self.pct))
        if step < up:
            t = step / up
            return self.initial + (self.base_lr - self.initial) * 0.5 * (1.0 - math.cos(math.pi * t))
        t = min(1.0, (step - up) / max(1, self.total - up))
        return self.final + (self.base_lr - self.final) * 0.5 * (1.0 + math.cos(math.pi * t))


class Warmup(Scheduler):
    """Linear warm-up for ``warmup_steps`` steps, then the wrapped scheduler (shifted)."""

    def __init__(self, inner: Scheduler, warmup_steps: int):
        super().__init__(inner.base_lr)
        self.inner, self.warmup = inner, warmup_steps

    def lr(self, step):
        if self.warmup > 0 and step < self.warmup:
            return self.inner.lr(0) * (step + 1) / self.warmup
        return self.inner.lr(step - self.warmup)


class Sequential(Scheduler):
    def __init__(self, schedulers: Sequence[Scheduler], milestones: Sequence[int]):
        super().__init__(schedulers[0].base_lr)
        assert len(milestones) == len(schedulers) - 1
        self.scheds, self.miles = list(schedulers), list(milestones)

    def lr(self, step):
        start = 0
        for s, m in zip(self.scheds, self.miles):
            if step < m:
                return s.lr(step - start)
            start = m
        return self.scheds[-1].lr(step - start)


class Lambda(Scheduler):
    def __init__(self, base_lr, fn: Callable[[int], float]):
        super().__init__(base_lr)
        self.fn = fn

    def lr(self, step):
        return self.base_lr * self.fn(step)
