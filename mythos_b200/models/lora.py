"""Low-rank adapters: LoRA, DoRA and the quantised-base variant (QLoRA).

The reference ships forward-only, unbuilt adapters (src/adapters/lora.cpp:9-83 ``base + alpha/r *
B A x`` with A uniform * 1/sqrt(in), B = 0; qlora.cpp NF4 base; dora.cpp row-norm magnitude). Here
they train: the base ``OILLinear`` is frozen in its storage format (OIL4 / I2_S / OIL8 — a
quantised base is what QLoRA means), the adapter matrices are ordinary parameters, and both
low-rank products run on the tcgen05 GEMM with autograd.

Because attention projections are fused (q | k | v rows in one matrix), an adapter can target row
ranges of the base's output: ``targets=("q", "v")`` attaches one (A, B) pair to the q rows and one
to the v rows of ``qkv_proj``.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as F
from .layers import OILLinear

NF4_LEVELS = [-1.0, -0.6961928, -0.5250730, -0.3949175, -0.2844414, -0.1847734, -0.0910500, 0.0,
              0.0795803, 0.1609302, 0.2461123, 0.3379152, 0.4407098, 0.5626170, 0.7229568, 1.0]


def nf4_codebook(absmax: float = 1.0) -> torch.Tensor:
    """The 16 NormalFloat4 levels scaled to ``[-absmax, absmax]`` (usable as an OIL4 codebook)."""
    return torch.tensor(NF4_LEVELS, dtype=torch.float32) * absmax


class LoRALinear(nn.Module):
    def __init__(self, base: OILLinear, rank: int = 8, alpha: float = 16.0, out_slices=None, dora: bool = False):
        super().__init__()
        self.base = base
        base.weight.requires_grad_(False)
        self.rank, self.alpha, self.scale = rank, alpha, alpha / rank
        self.out_slices = list(out_slices) if out_slices else [(0, base.out_features)]
        bound = 1.0 / math.sqrt(base.in_features)
        self.lora_A = nn.ParameterList([nn.Parameter(torch.empty(rank, base.in_features).uniform_(-bound, bound))
                                        for _ in self.out_slices])
        self.lora_B = nn.ParameterList([nn.Parameter(torch.zeros(size, rank)) for _, size in self.out_slices])
        self.dora = dora
        if dora:
            with torch.no_grad():
                mags = [base.weight[s:s + n].float().norm(dim=1) for s, n in self.out_slices]
            self.magnitude = nn.ParameterList([nn.Parameter(m.clone()) for m in mags])
        self.merged = False

    def __getattr__(self, name):
        # attributes of the wrapped layer (weight, fmt, block_size, codebooks, ...) stay reachable
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("base"), name)

    def _cast(self, p, like):
        c = getattr(p, "compute", None)
        if c is not None:
            return c, getattr(p, "main_grad", None)
        return (p.to(like.dtype) if like.is_cuda else p), None

    def forward(self, x):
        y = self.base(x)
        if self.merged:
            return y
        parts, cursor = [], 0
        for i, (start, size) in enumerate(self.out_slices):
            if start > cursor:
                parts.append(y[..., cursor:start])
            a, ga = self._cast(self.lora_A[i], x)
            b, gb = self._cast(self.lora_B[i], x)
            delta = F.linear(F.linear(x, a, ga), b, gb) * self.scale
            seg = y[..., start:start + size] + delta
            if self.dora:
                w = self.base.weight[start:start + size].float() + self.scale * (self.lora_B[i].float() @ self.lora_A[i].float())
                ratio = (self.magnitude[i].float() / w.norm(dim=1).clamp(min=1e-8)).to(seg.dtype)
                seg = seg * ratio
            parts.append(seg)
            cursor = start + size
        if cursor < y.shape[-1]:
            parts.append(y[..., cursor:])
        return torch.cat(parts, dim=-1) if len(parts) > 1 else parts[0]

    @torch.no_grad()
    def delta_weight(self, i: int) -> torch.Tensor:
        return self.scale * (self.lora_B[i].float() @ self.lora_A[i].float())

    @torch.no_grad()
    def merge(self) -> None:
        """Fold the adapters into the base master weights (they are re-quantised on next use)."""
        if self.merged:
            return
        for i, (start, size) in enumerate(self.out_slices):
            self.base.weight[start:start + size] += self.delta_weight(i).to(self.base.weight.dtype)
        self.base._frozen_image = None
        self.merged = True

    @torch.no_grad()
    def unmerge(self) -> None:
        if not self.merged:
            return
        for i, (start, size) in enumerate(self.out_slices):
            self.base.weight[start:start + size] -= self.delta_weight(i).to(self.base.weight.dtype)
        self.base._frozen_image = None
        self.merged = False

    def adapter_state(self, prefix: str = "") -> dict:
        """Tensors in the reference adapter's naming (``lora.A`` / ``lora.B`` per target)."""
        out = {}
        for i in range(len(self.out_slices)):
            out[f"{prefix}lora.{i}.A"] = self.lora_A[i].detach().float().cpu()
            out[f"{prefix}lora.{i}.B"] = self.lora_B[i].detach().float().cpu()
            if self.dora:
                out[f"{prefix}lora.{i}.magnitude"] = self.magnitude[i].detach().float().cpu()
        return out


def apply_lora(model, rank: int = 16, alpha: float = 32.0, targets=("q", "v"), dora: bool = False):
    """Freeze the model and attach adapters. targets: any of q, k, v, o, gate, up, down."""
    for p in model.parameters():
        p.requires_grad_(False)
    cfg = model.cfg
    qd, kvd = cfg.q_dim, cfg.kv_dim
    wrapped = []
    for blk in model.layers:
        att = blk.attention
        sl = []
        if "q" in targets:
            sl.append((0, qd))
        if "k" in targets:
            sl.append((qd, kvd))
        if "v" in targets:
            sl.append((qd + kvd, kvd))
        if sl:
            att.qkv_proj = LoRALinear(att.qkv_proj, rank, alpha, sl, dora)
            wrapped.append(att.qkv_proj)
        if "o" in targets:
            att.o_proj = LoRALinear(att.o_proj, rank, alpha, None, dora)
            wrapped.append(att.o_proj)
        ffn = blk.ffn
        if hasattr(ffn, "up_proj"):
            f = ffn.up_proj.out_features // (2 if ffn.gated else 1)
            sl = []
            if "gate" in targets and ffn.gated:
                sl.append((0, f))
            if "up" in targets:
                sl.append((f if ffn.gated else 0, f))
            if sl:
                ffn.up_proj = LoRALinear(ffn.up_proj, rank, alpha, sl, dora)
                wrapped.append(ffn.up_proj)
            if "down" in targets:
                ffn.down_proj = LoRALinear(ffn.down_proj, rank, alpha, None, dora)
                wrapped.append(ffn.down_proj)
    return wrapped


def merge_all(model) -> None:
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.merge()


def save_adapters(model, path: str) -> None:
    """Adapters as an ``.oil`` file of FP32 tensors (one block per tensor <= 32768 weights)."""
    from ..oil.container import write_oil
    from ..oil.model_io import _fp32_blocks

    tensors = []
    for name, m in model.named_modules():
        if isinstance(m, LoRALinear):
            for k, v in m.adapter_state(name + ".").items():
                tensors.append((k, _fp32_blocks(v.numpy())))
    write_oil(path, tensors, config=b"", write_idx=True, idx_version=1)


def load_adapters(model, path: str) -> int:
    from ..oil.container import OILReader

    rd = OILReader(path)
    n = 0
    with torch.no_grad():
        for name, m in model.named_modules():
            if not isinstance(m, LoRALinear):
                continue
            for i in range(len(m.out_slices)):
                for tag, plist in (("A", m.lora_A), ("B", m.lora_B)):
                    v = rd.read_tensor(f"{name}.lora.{i}.{tag}")
                    if v.size == plist[i].numel():
                        plist[i].copy_(torch.from_numpy(v.copy()).view(plist[i].shape))
                        n += 1
    return n


# ------------------------------------------------------------------------------------------ QLoRA
def nf4_quantize(w: torch.Tensor, block: int = 64):
    """NF4 with an affine map per block: the 16 NormalFloat levels (in [-1, 1]) are stretched onto
    ``[min, max]`` of each block of ``block`` weights, every weight takes the nearest level, and two
    4-bit codes share a byte (low nibble first). Returns (packed uint8 [n/2], lo [blocks], hi
    [blocks]). Same scheme as the reference's QLoRA base (src/adapters/qlora.cpp:23-96)."""
    flat = w.detach().float().reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.cat([flat, flat[-1:].expand(pad)])
    blocks = flat.view(-1, block)
    lo, hi = blocks.amin(dim=1), blocks.amax(dim=1)
    span = (hi - lo).clamp(min=1e-12)
    levels = torch.tensor(NF4_LEVELS, device=w.device)
    unit = (blocks - lo[:, None]) / span[:, None] * 2.0 - 1.0          # block mapped onto [-1, 1]
    codes = (unit[..., None] - levels).abs().argmin(dim=-1).to(torch.uint8).view(-1)
    packed = codes[0::2] | (codes[1::2] << 4)
    return packed, lo, hi


def nf4_dequantize(packed: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, numel: int, block: int = 64):
    codes = torch.stack([packed & 0xF, packed >> 4], dim=1).reshape(-1).long()
    levels = torch.tensor(NF4_LEVELS, device=packed.device)
    unit = levels[codes].view(-1, block)
    vals = (unit + 1.0) * 0.5 * (hi - lo)[:, None] + lo[:, None]
    return vals.reshape(-1)[:numel]


class QLoRALinear(nn.Module):
    """Linear layer whose frozen base lives in packed NF4 (4.5 bits per weight with block 64) and
    whose update is a trainable rank-``r`` pair: ``y = x deq(W)^T + (alpha / r) * (x A^T) B^T``.
    A is uniform in +-1/sqrt(in), B starts at zero, so the layer starts out equal to its quantised
    base. The reference's ``QLoRAAdapter`` is forward-only (GEMV); this one trains A and B (the
    dequantised base is rebuilt per call in bf16 and is not kept)."""

    def __init__(self, weight: torch.Tensor, rank: int = 8, alpha: float = 16.0, block: int = 64):
        super().__init__()
        self.out_features, self.in_features = weight.shape
        self.rank, self.alpha, self.scale, self.block = rank, alpha, alpha / rank, block
        packed, lo, hi = nf4_quantize(weight, block)
        self.register_buffer("packed", packed)
        self.register_buffer("lo", lo)
        self.register_buffer("hi", hi)
        bound = 1.0 / math.sqrt(self.in_features)
        self.lora_A = nn.Parameter(torch.empty(rank, self.in_features, device=weight.device).uniform_(-bound, bound))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, rank, device=weight.device))

    def base_weight(self) -> torch.Tensor:
        n = self.out_features * self.in_features
        return nf4_dequantize(self.packed, self.lo, self.hi, n, self.block).view(self.out_features, self.in_features)

    def base_bytes(self) -> int:
        return self.packed.numel() + 4 * (self.lo.numel() + self.hi.numel())

    def forward(self, x):
        dt = torch.bfloat16 if x.is_cuda else x.dtype
        w = self.base_weight().to(dt)
        y = F.linear(x.to(dt), w)
        delta = F.linear(F.linear(x.to(dt), self.lora_A.to(dt)), self.lora_B.to(dt))
        return y + self.scale * delta

    @torch.no_grad()
    def merged_weight(self) -> torch.Tensor:
        """fp32 ``deq(W) + (alpha / r) * B A`` for export."""
        return self.base_weight() + self.scale * (self.lora_B.float() @ self.lora_A.float())

    def adapter_state(self, prefix: str = "") -> dict:
        """``qlora.A`` / ``qlora.B`` plus the packed base and its block ranges."""
        return {f"{prefix}qlora.A": self.lora_A.detach().float().cpu(), f"{prefix}qlora.B": self.lora_B.detach().float().cpu(),
                f"{prefix}qlora.packed": self.packed.cpu(), f"{prefix}qlora.lo": self.lo.cpu(),
                f"{prefix}qlora.hi": self.hi.cpu()}

    @torch.no_grad()
    def load_adapter_state(self, state: dict, prefix: str = "") -> None:
        self.lora_A.copy_(state[f"{prefix}qlora.A"])
        self.lora_B.copy_(state[f"{prefix}qlora.B"])
        for k in ("packed", "lo", "hi"):
            getattr(self, k).copy_(state[f"{prefix}qlora.{k}"])
