"""Codebooks for the OIL8 (256 x fp32) and OIL4 (16 x fp16) vector-free scalar quantisers.

Capabilities of the reference's ``CodebookOIL8`` / ``CodebookOIL4`` (include/oil/codebook.h:28-87,
src/codebook.cpp): training by k-means (at most 20 iterations, stop when no centroid moves more
than 1e-7, src/codebook.cpp:70-135), nearest-centroid quantisation with the first minimum
winning ties (:172-186), exponential-moving-average updates from per-centroid counts and sums
(:137-170), and the serialised form ``u32 magic + raw centroids`` (:192-212, :344-364) with magic
0x4F494C38 ("OIL8") / 0x4F494C34 ("OIL4"). OIL4 centroids are stored as IEEE half bit patterns.

Codebooks in this framework are always kept sorted ascending: quantile initialisation is sorted,
and k-means / EMA updates of a scalar quantiser preserve order. Sorted codebooks let the CUDA
quantiser use a binary search instead of 256 comparisons per weight.
"""
from __future__ import annotations

import math
import struct

import numpy as np
import torch

OIL8_MAGIC = 0x4F494C38
OIL4_MAGIC = 0x4F494C34
OIL8_SIZE = 256
OIL4_SIZE = 16


def _norm_ppf(p: torch.Tensor) -> torch.Tensor:
    return math.sqrt(2.0) * torch.erfinv(2.0 * p - 1.0)


def quantile_codebook(size: int, std: float = 0.02, fp16: bool = False) -> torch.Tensor:
    """Centroids at the (i + 0.5)/size quantiles of N(0, std^2); ascending fp32 [size]."""
    p = (torch.arange(size, dtype=torch.float64) + 0.5) / size
    cb = (_norm_ppf(p) * std).float()
    if fp16:
        cb = cb.half().float()
    return cb


def kmeans_codebook(data: torch.Tensor, size: int, iters: int = 20, tol: float = 1e-7, seed: int = 42,
                    fp16: bool = False) -> torch.Tensor:
    """1-D k-means. Initial centroids are ``size`` samples drawn without replacement with a seeded
    generator (the reference draws a Fisher-Yates sample with RNG(42)); returned sorted."""
    x = data.reshape(-1).float()
    n = x.numel()
    if n == 0:
        return torch.zeros(size)
    g = torch.Generator(device="cpu").manual_seed(seed)
    if n >= size:
        perm = torch.randperm(n, generator=g)[:size]
        cb = x[perm.to(x.device)].clone()
    else:
        cb = torch.cat([x, x.new_zeros(size - n)])
    cb, _ = torch.sort(cb)
    for _ in range(iters):
        # sorted centroids: the nearest one is found from the midpoints
        mid = (cb[1:] + cb[:-1]) * 0.5
        assign = torch.bucketize(x, mid, right=False)
        sums = torch.zeros(size, device=x.device).index_add_(0, assign, x)
        cnts = torch.zeros(size, device=x.device).index_add_(0, assign, torch.ones_like(x))
        new = torch.where(cnts > 0, sums / cnts.clamp(min=1), cb)
        new, _ = torch.sort(new)
        moved = (new - cb).abs().max()
        cb = new
        if float(moved) <= tol:
            break
    if fp16:
        cb = cb.half().float()
    return cb


def quantize(data: torch.Tensor, cb: torch.Tensor):
    """Nearest centroid (first minimum on ties). Returns (indices u8, counts, sums) like the
    reference's ``quantize`` which also collects batch statistics."""
    x = data.reshape(-1).float()
    d = (x[:, None] - cb[None, :].float()).abs()
    idx = d.argmin(dim=1)
    size = cb.numel()
    cnts = torch.zeros(size, device=x.device).index_add_(0, idx, torch.ones_like(x))
    sums = torch.zeros(size, device=x.device).index_add_(0, idx, x)
    return idx.to(torch.uint8), cnts, sums


class EMAState:
    """Running per-centroid counts and sums for one tensor's codebooks:
    ``running = running * decay + batch * (1 - decay)``; ``centroid = sums / counts``."""

    def __init__(self, codebooks: torch.Tensor, decay: float = 0.999):
        self.decay = decay
        self.counts = torch.zeros_like(codebooks, dtype=torch.float32)
        self.sums = torch.zeros_like(codebooks, dtype=torch.float32)
        self.initialised = False

    def update(self, codebooks: torch.Tensor, batch_counts: torch.Tensor, batch_sums: torch.Tensor) -> None:
        if not self.initialised:
            self.counts.copy_(batch_counts)
            self.sums.copy_(batch_sums)
            self.initialised = True
        else:
            self.counts.mul_(self.decay).add_(batch_counts, alpha=1.0 - self.decay)
            self.sums.mul_(self.decay).add_(batch_sums, alpha=1.0 - self.decay)
        live = self.counts > 1e-6
        new = torch.where(live, self.sums / self.counts.clamp(min=1e-6), codebooks)
        # a scalar quantiser's cell means are ordered; sorting only repairs empty-cell leftovers
        codebooks.copy_(torch.sort(new, dim=-1).values)


# ------------------------------------------------------------------------------ serialisation
def serialize_oil8(cb: torch.Tensor) -> bytes:
    a = cb.detach().cpu().float().numpy().astype("<f4")
    assert a.size == OIL8_SIZE
    return struct.pack("<I", OIL8_MAGIC) + a.tobytes()


def serialize_oil4(cb: torch.Tensor) -> bytes:
    a = cb.detach().cpu().float().numpy().astype("<f2")
    assert a.size == OIL4_SIZE
    return struct.pack("<I", OIL4_MAGIC) + a.tobytes()


def deserialize(blob: bytes) -> tuple[str, np.ndarray]:
    """Returns (format name, fp32 centroids). Accepts blobs with or without the magic word."""
    if len(blob) >= 4:
        (magic,) = struct.unpack_from("<I", blob, 0)
        if magic == OIL8_MAGIC and len(blob) >= 4 + 4 * OIL8_SIZE:
            return "oil8", np.frombuffer(blob, dtype="<f4", count=OIL8_SIZE, offset=4).astype(np.float32)
        if magic == OIL4_MAGIC and len(blob) >= 4 + 2 * OIL4_SIZE:
            return "oil4", np.frombuffer(blob, dtype="<f2", count=OIL4_SIZE, offset=4).astype(np.float32)
    if len(blob) == 4 * OIL8_SIZE:
        return "oil8", np.frombuffer(blob, dtype="<f4").astype(np.float32)
    if len(blob) == 2 * OIL4_SIZE:
        return "oil4", np.frombuffer(blob, dtype="<f2").astype(np.float32)
    raise ValueError(f"unrecognised codebook blob of {len(blob)} bytes")
