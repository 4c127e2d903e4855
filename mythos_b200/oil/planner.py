"""Format planner: assign one format per quantisation block to hit a target bits-per-weight.

Reference: ``FormatPlanner`` (src/format_planner.cpp:11-176). Importance of a block is
``mean(|w| * |a|)`` (magnitude, with optional activation scales) or the Fisher proxy
``sqrt(mean g^2) * |w[start]|``; blocks are sorted by importance and the most important get OIL8,
then OIL4, ternary, binary. The reference finds the mix by an O(n^3) triple loop over block counts
(:81-98); here the counts come from the documented percentile recipe (top 1 % OIL8, next 4 % OIL4,
rest ternary) or from a closed-form solve over two adjacent formats, both O(n log n).
"""
from __future__ import annotations

import numpy as np
import torch

from .formats import FORMAT_BPW, Format


def block_importance(w: torch.Tensor, block_size: int, act_scale: torch.Tensor | None = None,
                     grad: torch.Tensor | None = None, method: str = "magnitude") -> torch.Tensor:
    flat = w.detach().float().reshape(-1)
    n = flat.numel()
    nb = (n + block_size - 1) // block_size
    pad = nb * block_size - n
    wf = torch.nn.functional.pad(flat, (0, pad)).reshape(nb, block_size)
    if method == "fisher":
        if grad is None:
            raise ValueError("fisher importance needs gradients")
        gf = torch.nn.functional.pad(grad.detach().float().reshape(-1), (0, pad)).reshape(nb, block_size)
        return gf.pow(2).mean(1).sqrt() * wf[:, 0].abs()
    a = wf.abs()
    if act_scale is not None:
        cols = w.shape[-1]
        idx = torch.arange(nb * block_size, device=w.device) % cols
        a = a * act_scale.float().abs()[idx].reshape(nb, block_size)
    return a.mean(1)


def compute_format_mix(n_blocks: int, target_bpw: float, salient: float = 0.01, moderate: float = 0.04) -> dict:
    """Block counts per format whose average bpw is as close to ``target_bpw`` as the block count
    allows. Starts from the percentile recipe (``salient`` OIL8, ``moderate`` OIL4, rest ternary)
    and moves blocks between adjacent formats to close the gap."""
    order = [Format.OIL8, Format.OIL4, Format.TERNARY, Format.BINARY]
    bpw = [FORMAT_BPW[f] for f in order]
    counts = [int(round(n_blocks * salient)), int(round(n_blocks * moderate)), 0, 0]
    counts[2] = n_blocks - counts[0] - counts[1]

    def avg(c):
        return sum(x * b for x, b in zip(c, bpw)) / max(1, n_blocks)

    for _ in range(4 * n_blocks + 8):
        cur = avg(counts)
        if abs(cur - target_bpw) <= 0.05:
            break
        moved = False
        if cur < target_bpw:      # promote one block from the cheapest populated format
            for i in (3, 2, 1):
                if counts[i] > 0:
                    counts[i] -= 1
                    counts[i - 1] += 1
                    moved = True
                    break
        else:                     # demote one block from the most expensive populated format
            for i in (0, 1, 2):
                if counts[i] > 0:
                    counts[i] -= 1
                    counts[i + 1] += 1
                    moved = True
                    break
        if not moved:
            break
    return {f: c for f, c in zip(order, counts)}


def allocate(importance: torch.Tensor, mix: dict) -> np.ndarray:
    """Per-block format codes (uint8): blocks sorted by importance, OIL8 first."""
    n = importance.numel()
    order = torch.argsort(importance, descending=True).cpu().numpy()
    out = np.full(n, int(Format.TERNARY), dtype=np.uint8)
    pos = 0
    for fmt in (Format.OIL8, Format.OIL4, Format.TERNARY, Format.BINARY):
        c = int(mix.get(fmt, 0))
        out[order[pos:pos + c]] = int(fmt)
        pos += c
    return out


def plan(w: torch.Tensor, target_bpw: float, block_size: int = 256, **kw) -> tuple[np.ndarray, float]:
    imp = block_importance(w, block_size, **kw)
    mix = compute_format_mix(imp.numel(), target_bpw)
    fmts = allocate(imp, mix)
    achieved = float(sum(FORMAT_BPW[Format(int(f))] for f in fmts) / max(1, len(fmts)))
    return fmts, achieved


def quantize_mixed(w: torch.Tensor, formats: np.ndarray, block_size: int = 256):
    """Mixed-per-block quantisation of a flat tensor (the reference's ``forward_mixed``,
    src/ste_quantizer.cpp:84-194). Returns (dequantised fp32 tensor, list of BlockData)."""
    from . import codebook as cbk
    from .container import BlockData
    from .formats import encode_block, decode_block, quantize_binary, quantize_ternary

    flat = w.detach().float().reshape(-1).cpu().numpy()
    out = np.empty_like(flat)
    blocks = []
    cb8 = cb4 = None
    for b, fmt in enumerate(formats):
        seg = flat[b * block_size:(b + 1) * block_size]
        fmt = Format(int(fmt))
        if fmt == Format.OIL8:
            std = float(seg.std()) or 0.02
            cb8 = cbk.quantile_codebook(256, std).numpy()
            idx = np.abs(seg[:, None] - cb8[None]).argmin(1).astype(np.uint8)
            cb, ix = encode_block(fmt, None, cb8, idx)
        elif fmt == Format.OIL4:
            std = float(seg.std()) or 0.02
            cb4 = cbk.quantile_codebook(16, std, fp16=True).numpy()
            idx = np.abs(seg[:, None] - cb4[None]).argmin(1).astype(np.uint8)
            cb, ix = encode_block(fmt, None, cb4, idx)
        elif fmt == Format.TERNARY:
            codes, s = quantize_ternary(seg)
            cb, ix = encode_block(fmt, None, None, codes, s)
        elif fmt == Format.BINARY:
            bits, s = quantize_binary(seg)
            cb, ix = encode_block(fmt, None, None, bits, s)
        else:
            cb, ix = encode_block(fmt, seg)
        blocks.append(BlockData(fmt, seg.size, cb, ix))
        out[b * block_size:(b + 1) * block_size] = decode_block(fmt, seg.size, cb, ix)
    return torch.from_numpy(out).view(w.shape), blocks
