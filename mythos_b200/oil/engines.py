"""Quantisation engines beside the OIL codebook formats: FP8 (E4M3 / E5M2), NF4, AWQ and
GPTQ-style group INT4 fake quantisers, block ternary (I2S code = trit + 1), binary, affine U8
and symmetric INT8. All functions are vectorised torch code and run on CPU or GPU tensors.

Behaviour follows the reference's ``oil::engines`` namespace (src/oil_engines.cpp:15-517), the
OIL8 engine's block quantisers (engines/OIL8/quantize.cpp:14-191) and the INT8 helpers
(src/int8_quant.cpp:8-41). Two encodings of ternary values exist in the reference; both are here
under their own names: ``i2s_*`` (code = trit + 1, block abs-max scale, threshold 0.33) and
``ternary_block_*`` (0 -> 0, 1 -> +s, 2 -> -s, threshold 0.577 max|w|, scale = mean |w| of the
non-zeros).
"""
from __future__ import annotations

import torch

# --------------------------------------------------------------------------- FP8


# Encoding is the OCP FP8 definition as implemented by torch's float8 dtypes: round to nearest
# even, gradual underflow, saturation at +-448 (E4M3, no infinities) / +-57344 (E5M2). The
# reference's loop-based encoder (src/oil_engines.cpp:31-49, 78-96) rounds half away from zero,
# never carries a rounded-up mantissa into the exponent and writes biased exponent 0 for values in
# [2^-7, 2^-6) which its own decoder then reads as subnormals; those defects are not reproduced.


def fp8_e4m3_quantize(x: torch.Tensor) -> torch.Tensor:
    return x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def fp8_e4m3_dequantize(bits: torch.Tensor) -> torch.Tensor:
    return bits.view(torch.float8_e4m3fn).float()


def fp8_e5m2_quantize(x: torch.Tensor) -> torch.Tensor:
    return x.float().clamp(-57344.0, 57344.0).to(torch.float8_e5m2).view(torch.uint8)


def fp8_e5m2_dequantize(bits: torch.Tensor) -> torch.Tensor:
    return bits.view(torch.float8_e5m2).float()


# --------------------------------------------------------------------------- NF4

NF4_CODEBOOK = torch.tensor([-1.0, -0.6961928, -0.525073, -0.39497948, -0.28444138, -0.18477343, -0.09105138, 0.0,
                             0.07958097, 0.16092212, 0.24611243, 0.33712566, 0.43570983, 0.54554284, 0.67132018,
                             1.0])


def nf4_quantize(x: torch.Tensor, block_size: int = 64):
    """Per-block abs-max scale, nearest of the 16 normal-float levels (first minimum on ties).
    Returns (indices u8 [n], scales f32 [blocks])."""
    flat = x.float().reshape(-1)
    n = flat.numel()
    pad = (-n) % block_size
    blocks = torch.nn.functional.pad(flat, (0, pad)).view(-1, block_size)
    scales = blocks.abs().amax(dim=1)
    norm = (blocks / (scales[:, None] + 1e-10)).clamp(-1, 1)
    idx = (norm[..., None] - NF4_CODEBOOK.to(x.device)).abs().argmin(dim=-1)
    return idx.reshape(-1)[:n].to(torch.uint8), scales


def nf4_dequantize(idx: torch.Tensor, scales: torch.Tensor, block_size: int = 64) -> torch.Tensor:
    n = idx.numel()
    s = scales.repeat_interleave(block_size)[:n]
    return NF4_CODEBOOK.to(idx.device)[idx.long()] * s


# --------------------------------------------------------------------------- AWQ / GPTQ style


class AWQQuantizer:
    """Activation-aware scaling: per output channel ``s = max|a|^alpha / max|w_row|`` (clamped to
    [1e-8, 1e4]), then symmetric INT4 per group of ``group_size`` inputs on ``w * s``; the result
    is returned de-scaled (a fake quantiser, as in the reference)."""

    def __init__(self, group_size: int = 128, alpha: float = 0.5):
        self.group_size, self.alpha = group_size, alpha
        self.scales: torch.Tensor | None = None

    def compute_scales(self, weight: torch.Tensor, activation: torch.Tensor) -> torch.Tensor:
        max_w = weight.float().abs().amax(dim=1)
        max_a = activation.float().abs().max()
        self.scales = (max_a.pow(self.alpha) / (max_w + 1e-10)).clamp(1e-8, 1e4)
        return self.scales

    def quantize(self, weight: torch.Tensor) -> torch.Tensor:
        N, K = weight.shape
        s = self.scales if self.scales is not None else torch.ones(N, device=weight.device)
        w = weight.float() * s[:, None]
        out = torch.empty_like(w)
        for g0 in range(0, K, self.group_size):
            blk = w[:, g0:g0 + self.group_size]
            scale = (blk.abs().amax(dim=1, keepdim=True) / 7.0).clamp_min(1e-10)
            q = _round_half_away(blk / scale).clamp(-8, 7)
            out[:, g0:g0 + self.group_size] = q * scale
        return out / s[:, None]

    dequantize = staticmethod(lambda q: q)


class GPTQQuantizer:
    """Group quantiser whose step comes from ``max |w| / (h + 1e-8)`` over the group, with ``h``
    an elementwise second-order proxy of the same shape as the weight."""

    def __init__(self, group_size: int = 128, bits: int = 4):
        self.group_size, self.bits = group_size, bits
        self.max_q, self.min_q = float((1 << (bits - 1)) - 1), -float(1 << (bits - 1))

    def quantize(self, weight: torch.Tensor, hessian: torch.Tensor) -> torch.Tensor:
        w, h = weight.float(), hessian.float()
        out = torch.empty_like(w)
        for g0 in range(0, w.shape[1], self.group_size):
            sl = slice(g0, g0 + self.group_size)
            scale = ((w[:, sl].abs() / (h[:, sl] + 1e-8)).amax(dim=1, keepdim=True) / self.max_q).clamp_min(1e-10)
            out[:, sl] = _round_half_away(w[:, sl] / scale).clamp(self.min_q, self.max_q) * scale
        return out

    dequantize = staticmethod(lambda q: q)


def _round_half_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


# --------------------------------------------------------------------------- ternary / binary


def _pack_bits(codes: torch.Tensor, bits: int) -> torch.Tensor:
    per = 8 // bits
    n = codes.numel()
    c = torch.nn.functional.pad(codes.reshape(-1).to(torch.int32), (0, (-n) % per)).view(-1, per)
    shifts = torch.arange(per, device=codes.device, dtype=torch.int32) * bits
    return (c << shifts).sum(dim=1).to(torch.uint8)


def _unpack_bits(packed: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    per = 8 // bits
    shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
    return ((packed.to(torch.int32)[:, None] >> shifts) & ((1 << bits) - 1)).reshape(-1)[:n]


def i2s_quantize(weight: torch.Tensor, block_size: int = 128, threshold: float = 0.33):
    """Block abs-max scale; trit = sign(w/scale) where |w/scale| > threshold; code = trit + 1,
    four codes per byte, first weight in bits 0-1. Returns (packed u8, scales f32)."""
    flat = weight.float().reshape(-1)
    n = flat.numel()
    blocks = torch.nn.functional.pad(flat, (0, (-n) % block_size)).view(-1, block_size)
    scales = blocks.abs().amax(dim=1)
    safe = torch.where(scales < 1e-10, torch.ones_like(scales), scales)
    norm = blocks / safe[:, None]
    trit = (norm > threshold).to(torch.int32) - (norm < -threshold).to(torch.int32)
    return _pack_bits((trit + 1).reshape(-1)[:n], 2), scales


def i2s_dequantize(packed: torch.Tensor, scales: torch.Tensor, n: int, block_size: int = 128) -> torch.Tensor:
    codes = _unpack_bits(packed, 2, n)
    trit = (codes == 2).float() - (codes == 0).float()
    return trit * scales.repeat_interleave(block_size)[:n]


def ternary_block_quantize(block: torch.Tensor):
    """One block: threshold 0.577 max|w|, scale = mean |w| over the kept weights, codes
    0 -> 0, 1 -> +scale, 2 -> -scale (2 bits, LSB first). Returns (packed u8, scale)."""
    w = block.float().reshape(-1)
    thr = 0.577 * w.abs().max()
    keep = w.abs() > thr
    scale = w[keep].abs().mean() if bool(keep.any()) else w.new_zeros(())
    codes = torch.where(keep & (w > 0), 1, torch.where(keep & (w < 0), 2, 0))
    return _pack_bits(codes, 2), float(scale)


def ternary_block_dequantize(packed: torch.Tensor, scale: float, n: int) -> torch.Tensor:
    codes = _unpack_bits(packed, 2, n)
    return ((codes == 1).float() - (codes == 2).float()) * scale


def binary_block_quantize(block: torch.Tensor):
    """scale = mean |w|, bit = w > 0 (LSB first)."""
    w = block.float().reshape(-1)
    return _pack_bits((w > 0).to(torch.int32), 1), float(w.abs().mean())


def binary_block_dequantize(packed: torch.Tensor, scale: float, n: int) -> torch.Tensor:
    bits = _unpack_bits(packed, 1, n)
    return (bits.float() * 2 - 1) * scale


def binary_tensor_quantize(weight: torch.Tensor):
    """Whole-tensor variant: scale = max |w|, bit = w >= 0."""
    w = weight.float().reshape(-1)
    return _pack_bits((w >= 0).to(torch.int32), 1), float(w.abs().max())


# --------------------------------------------------------------------------- integer


def affine_u8_quantize(x: torch.Tensor):
    """Asymmetric per-tensor U8: scale = (max - min) / 255, zero point = round(-min / scale)."""
    x = x.float()
    lo, hi = float(x.min()), float(x.max())
    scale = max((hi - lo) / 255.0, 1e-10)
    zp = int(round(-lo / scale))
    q = (_round_half_away(x / scale) + zp).clamp(0, 255).to(torch.uint8)
    return q, scale, zp


def affine_u8_dequantize(q: torch.Tensor, scale: float, zp: int) -> torch.Tensor:
    return (q.float() - zp) * scale


def int8_quantize_per_tensor(x: torch.Tensor):
    scale = float(x.float().abs().max()) / 127.0
    scale = scale if scale > 0 else 1.0
    return _round_half_away(x.float() / scale).clamp(-127, 127).to(torch.int8), scale


def int8_quantize_per_token(x: torch.Tensor):
    """Row-wise symmetric abs-max / 127 (rows = tokens)."""
    s = x.float().abs().amax(dim=-1, keepdim=True) / 127.0
    s = torch.where(s > 0, s, torch.ones_like(s))
    return _round_half_away(x.float() / s).clamp(-127, 127).to(torch.int8), s.squeeze(-1)


def int8_dequantize(q: torch.Tensor, scale) -> torch.Tensor:
    if isinstance(scale, torch.Tensor):
        return q.float() * scale.unsqueeze(-1)
    return q.float() * scale


# --------------------------------------------------------------------------- codebook engines


class CodebookEngine:
    """Scalar k-means codebook over a whole tensor (10 Lloyd iterations from a fixed grid:
    256 entries ``(i - 128) * 0.01`` for OIL8, 16 entries ``(i - 8) * 0.1`` for OIL4)."""

    def __init__(self, entries: int):
        self.entries = entries
        if entries == 256:
            self.codebook = (torch.arange(256).float() - 128) * 0.01
        else:
            self.codebook = (torch.arange(entries).float() - entries // 2) * 0.1

    def train_codebook(self, data: torch.Tensor, iters: int = 10) -> None:
        x = data.float().reshape(-1)
        cb = self.codebook.to(x.device)
        for _ in range(iters):
            idx = (x[:, None] - cb[None, :]).abs().argmin(dim=1)
            sums = torch.zeros_like(cb, dtype=torch.float64).index_add_(0, idx, x.double())
            cnt = torch.zeros_like(cb, dtype=torch.float64).index_add_(0, idx, torch.ones_like(x, dtype=torch.float64))
            cb = torch.where(cnt > 0, (sums / cnt.clamp_min(1)).float(), cb)
        self.codebook = cb

    def quantize(self, data: torch.Tensor) -> torch.Tensor:
        x = data.float().reshape(-1)
        return (x[:, None] - self.codebook.to(x.device)[None, :]).abs().argmin(dim=1).to(torch.uint8)

    def dequantize(self, idx: torch.Tensor) -> torch.Tensor:
        return self.codebook.to(idx.device)[idx.long()]


def OIL8Engine() -> CodebookEngine:
    return CodebookEngine(256)


def OIL4Engine() -> CodebookEngine:
    return CodebookEngine(16)


def compute_quant_error(original: torch.Tensor, dequantized: torch.Tensor) -> float:
    """Largest absolute element error."""
    return float((original.float().reshape(-1) - dequantized.float().reshape(-1)).abs().max())
