"""Look-up-table GEMMs over ternary weights with int8 activations (TL1: weight pairs, 9-entry
table per pair; TL2: weight triples, 27-entry table per triple) and the int8-activation I2_S GEMM.

All use a weight-shared layout ``W[N, K]`` (one packed row per output feature) and compute
``y[m, n] = (sum_k t(W[n, k]) * q(x[m, k])) / s_m`` with ``q`` = per-row abs-max int8 quantisation
(``s_m = 127 / max|x_m|``, round half away from zero) and exact int32 accumulation, which is the
arithmetic of the reference kernels (src/kernel_tl.cpp:13-168, src/kernel_i2s.cpp:156-235). The
reference indexes a distinct weight row per (m, n) output and its TL1 loop reads the 9-entry
table with a single weight's 2-bit code; both are artefacts of its test harness and are not
reproduced. CUDA tensors run the table kernels of ``csrc/kernels/ternary_lut.cu`` (tables of the
activation row in shared memory, one table read per weight pair / triple); CPU tensors run the same
arithmetic as tensor code, which is the oracle of the kernel test. The production ternary path is
the I2_S dequant GEMM / GEMV on tensor cores (``csrc/kernels/dequant_gemm.cu``, ``paged_attn.cu``).

Packing: trits are stored as 2-bit codes ``t + 1`` (0 = -1, 1 = 0, 2 = +1), four per byte, first
weight in bits 0-1: the I2_S / ``kernel_i2s`` encoding. TL1 reads them as pairs, TL2 as triples
inside 12-weight groups (3 bytes).
"""
from __future__ import annotations

import torch


def quantize_activations_int8(x: torch.Tensor):
    """Per-row symmetric int8: returns (q int8 [M, K], scale [M]) with q = round(x * scale)."""
    xf = x.float()
    amax = xf.abs().amax(dim=1).clamp_min(1e-10)
    scale = 127.0 / amax
    q = torch.sign(xf) * torch.floor(xf.abs() * scale[:, None] + 0.5)
    return q.clamp(-127, 127).to(torch.int8), scale


def pack_trits(trits: torch.Tensor) -> torch.Tensor:
    """[N, K] values in {-1, 0, 1} (K % 4 == 0) -> uint8 [N, K/4]."""
    c = (trits.to(torch.int32) + 1).reshape(trits.shape[0], -1, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).to(torch.uint8)


def unpack_trits(packed: torch.Tensor, K: int) -> torch.Tensor:
    p = packed.to(torch.int32)
    codes = torch.stack([(p >> s) & 3 for s in (0, 2, 4, 6)], dim=-1).reshape(packed.shape[0], -1)[:, :K]
    return codes - 1


def _group_lut(q: torch.Tensor, g: int) -> torch.Tensor:
    """q int8 [M, K] -> int32 table [M, K/g, 3^g]: entry (w_0..w_{g-1}) = sum_j w_j * a_j with the
    first weight as the most significant base-3 digit."""
    M, K = q.shape
    a = q.to(torch.int32).view(M, K // g, g)
    digits = torch.tensor([[(e // 3 ** (g - 1 - j)) % 3 - 1 for j in range(g)] for e in range(3 ** g)],
                          dtype=torch.int32, device=q.device)                # [3^g, g]
    return torch.einsum("mkg,eg->mke", a, digits)


def _group_index(trits: torch.Tensor, g: int) -> torch.Tensor:
    N, K = trits.shape
    t = (trits.to(torch.int64) + 1).view(N, K // g, g)
    w = torch.tensor([3 ** (g - 1 - j) for j in range(g)], dtype=torch.int64, device=trits.device)
    return (t * w).sum(-1)                                                  # [N, K/g]


def _lut_gemm(packed: torch.Tensor, x: torch.Tensor, K: int, g: int) -> torch.Tensor:
    if x.is_cuda:
        from ..ops import native

        y = torch.empty(x.shape[0], packed.shape[0], device=x.device, dtype=torch.float32)
        native.require().tl_gemm(packed.contiguous(), x.float().contiguous(), y, g)
        return y
    q, scale = quantize_activations_int8(x)
    lut = _group_lut(q, g)                                                  # [M, K/g, 3^g]
    idx = _group_index(unpack_trits(packed, K), g)                          # [N, K/g]
    M, G, E = lut.shape
    # y[m, n] = sum_G lut[m, G, idx[n, G]]
    gathered = torch.gather(lut.unsqueeze(1).expand(M, idx.shape[0], G, E), 3,
                            idx.unsqueeze(0).unsqueeze(-1).expand(M, -1, -1, 1)).squeeze(-1)
    return gathered.sum(dim=-1).float() / scale[:, None]


def tl1_gemm(packed: torch.Tensor, x: torch.Tensor, K: int) -> torch.Tensor:
    """x [M, K] float, packed ternary W [N, K/4] -> y [M, N]; pair tables (K % 4 == 0)."""
    return _lut_gemm(packed, x, K, 2)


def tl2_gemm(packed: torch.Tensor, x: torch.Tensor, K: int) -> torch.Tensor:
    """Triple tables; K must be a multiple of 12 (four triples per 3 packed bytes)."""
    if K % 12:
        raise ValueError("tl2_gemm: K must be a multiple of 12")
    return _lut_gemm(packed, x, K, 3)


def i2s_gemm_int8(packed: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, K: int, block_size: int = 128):
    """Ternary weights with one float scale per ``block_size`` weights along K, int8 activations:
    ``y[m, n] = sum_b scale[n, b] * (sum_{k in b} t * q) / s_m``."""
    q, s = quantize_activations_int8(x)
    t = unpack_trits(packed, K).to(torch.int32)
    N = t.shape[0]
    nb = K // block_size
    part = torch.einsum("mbk,nbk->mnb", q.to(torch.float64).view(-1, nb, block_size),
                        t.to(torch.float64).view(N, nb, block_size))          # exact: |sum| < 2^53
    return (part * scales.view(N, nb).double()[None]).sum(-1).float() / s[:, None]


def ternary_reference(trits: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """The same int8-activation arithmetic by direct integer matmul (oracle for the LUT paths)."""
    q, s = quantize_activations_int8(x)
    return (q.to(torch.int64) @ trits.to(torch.int64).t()).float() / s[:, None]
