"""Tracing: named ranges that show up in profilers (NVTX) and, when switched on, per-range device
time from CUDA events.

The reference only has wall-clock timers around whole loops (tokens/s in ``Trainer::fit``,
src/trainer.cpp:514-517; ``Generator::generate_full``, src/generator.cpp:132-143;
``backend::benchmark_operation``, src/backend.cpp:737-829) and documents an ``OIL_VERBOSE`` switch
for kernel timing that nothing reads. Here ``OIL_VERBOSE=1`` (or ``enable_timing()``) makes every
``span`` record a CUDA-event pair on the current stream; ``summary()`` turns them into totals per
name after one synchronisation. Without it a span is one NVTX push / pop on CUDA and nothing on CPU.
"""
from __future__ import annotations

import contextlib
import os
import time
from collections import defaultdict

import torch

_timing = os.environ.get("OIL_VERBOSE", "0") not in ("", "0")
_pending: list = []          # (name, start_event, end_event) on CUDA; (name, seconds) on CPU
_MAX_PENDING = 1 << 16


def enable_timing(on: bool = True) -> None:
    global _timing
    _timing = on


def timing_enabled() -> bool:
    return _timing


@contextlib.contextmanager
def span(name: str, device=None):
    """``with span("forward"): ...`` — an NVTX range on CUDA, plus an event pair when timing is on."""
    cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
    if cuda:
        torch.cuda.nvtx.range_push(name)
    if not _timing:
        try:
            yield
        finally:
            if cuda:
                torch.cuda.nvtx.range_pop()
        return
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            torch.cuda.nvtx.range_pop()
            if len(_pending) < _MAX_PENDING:
                _pending.append((name, a, b))
    else:
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if len(_pending) < _MAX_PENDING:
                _pending.append((name, time.perf_counter() - t0))


def summary(reset: bool = True) -> dict:
    """{name: {"calls": n, "ms": total}} over the spans recorded so far (synchronises once)."""
    if any(len(p) == 3 for p in _pending):
        torch.cuda.synchronize()
    out = defaultdict(lambda: {"calls": 0, "ms": 0.0})
    for p in _pending:
        ms = p[1].elapsed_time(p[2]) if len(p) == 3 else p[1] * 1e3
        out[p[0]]["calls"] += 1
        out[p[0]]["ms"] += ms
    if reset:
        _pending.clear()
    return dict(out)


def format_summary(rows: dict) -> str:
    total = sum(v["ms"] for v in rows.values()) or 1.0
    lines = [f"{'range':<28}{'calls':>8}{'ms':>12}{'share':>8}"]
    for name, v in sorted(rows.items(), key=lambda kv: -kv[1]["ms"]):
        lines.append(f"{name:<28}{v['calls']:>8}{v['ms']:>12.3f}{v['ms'] / total:>8.1%}")
    return "\n".join(lines)
