"""Packed OIL weights for inference.

A ``QuantLinear`` holds one ``[N, K]`` weight matrix in its storage format — OIL8 byte indices,
OIL4 nibble pairs (even index in the low nibble), I2_S 2-bit trits (four per byte, first weight
in bits 0-1) with a per-block absmean scale — plus the codebooks as bf16 tables, exactly what the
dequant-GEMM kernels consume. Matrices are packed once (from fp32 weights, from a trained
``OILLinear``, or from ``.oil`` blocks) and never expanded in HBM on the decode path.

``matmul`` picks the execution path by token count: up to 256 tokens run the codebook-dequant
GEMM (weights are the tensor-core A operand, read once); larger batches (prefill) dequantise the
matrix once into a bf16 scratch buffer and run the dense tcgen05 GEMM.
"""
from __future__ import annotations

import torch

from ..oil import codebook as cbk
from ..ops import functional as F
from ..ops import native, reference as ref

QFMT = {"oil8": 3, "oil4": 2, "i2s": 1}
DECODE_MAX_TOKENS = 256

# fp32 split-K accumulators, one per device, kept all-zero between uses (the finalize kernel zeroes
# what it reads). Grown outside CUDA-graph capture only.
_ACC: dict = {}
_SMS: dict = {}


def _norm_device(device) -> torch.device:
    d = torch.device(device)
    if d.type == "cuda" and d.index is None:
        d = torch.device("cuda", torch.cuda.current_device())
    return d


def reserve_accumulator(device, numel: int) -> None:
    """Make the split-K accumulator of ``device`` hold at least ``numel`` floats."""
    device = _norm_device(device)
    cur = _ACC.get(device)
    if cur is None or cur.numel() < numel:
        _ACC[device] = torch.zeros(numel, device=device, dtype=torch.float32)


def _sm_count(device) -> int:
    device = _norm_device(device)
    if device not in _SMS:
        _SMS[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SMS[device]


def _pack_nibbles(idx: torch.Tensor) -> torch.Tensor:
    a = idx.reshape(-1, 2)
    return (a[:, 0] | (a[:, 1] << 4)).to(torch.uint8)


def _pack_trits(codes: torch.Tensor) -> torch.Tensor:
    a = codes.reshape(-1, 4).to(torch.uint8)
    return (a[:, 0] | (a[:, 1] << 2) | (a[:, 2] << 4) | (a[:, 3] << 6)).to(torch.uint8)


class QuantLinear:
    def __init__(self, fmt: str, N: int, K: int, block_size: int, packed: torch.Tensor, codebooks=None, cb_map=None,
                 scales=None, dense=None):
        self.fmt, self.N, self.K, self.block_size = fmt, N, K, block_size
        self.packed, self.codebooks, self.cb_map, self.scales = packed, codebooks, cb_map, scales
        self.dense = dense  # bf16 [N, K] for unquantised formats (fp16 / fp32 models)
        self._scratch = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_float(cls, w: torch.Tensor, fmt: str, block_size: int = 256, codebook_group: int = 1, codebooks=None,
                   cb_map=None) -> "QuantLinear":
        """Quantise an fp32 ``[N, K]`` matrix. For OIL formats ``codebooks`` (fp32 ``[n_cb, C]``,
        ascending) default to N(0, std(w)) quantile codebooks shared by ``codebook_group`` blocks."""
        N, K = w.shape
        dev = w.device
        if fmt in ("fp32", "fp16", "bf16"):
            return cls(fmt, N, K, block_size, None, dense=w.to(torch.bfloat16).contiguous())
        if K % block_size != 0 or block_size % 64 != 0:
            raise ValueError(f"block size {block_size} must be a multiple of 64 and divide K={K}")
        flat = w.detach().float().reshape(-1).contiguous()
        nb = flat.numel() // block_size
        if fmt == "i2s":
            _, codes, scales = F.i2s_fake_quant(flat, block_size, want_codes=True)
            return cls(fmt, N, K, block_size, _pack_trits(codes), scales=scales.contiguous())
        size = 256 if fmt == "oil8" else 16
        if codebooks is None:
            g = max(1, codebook_group)
            n_cb = (nb + g - 1) // g
            std = float(flat.std()) if flat.numel() > 1 else 0.02
            base = cbk.quantile_codebook(size, std if std > 0 else 0.02, fp16=(fmt == "oil4")).to(dev)
            codebooks = base[None].repeat(n_cb, 1).contiguous()
            cb_map = (torch.arange(nb, device=dev) // g).to(torch.int32) if g > 1 else None
        _, idx = F.oil_fake_quant(flat, codebooks.float().contiguous(), cb_map, block_size, want_idx=True)
        packed = idx if fmt == "oil8" else _pack_nibbles(idx)
        return cls(fmt, N, K, block_size, packed.contiguous(), codebooks=codebooks.to(torch.bfloat16).contiguous(),
                   cb_map=cb_map)

    @classmethod
    def random(cls, fmt: str, N: int, K: int, block_size: int = 256, codebook_group: int = 128, device="cuda",
               generator=None, std: float = 0.02) -> "QuantLinear":
        """Synthetic weights directly in storage format: N(0, std) quantile codebooks with uniform
        random indices (OIL8 / OIL4), trits drawn with p = (0.25, 0.5, 0.25) and an absmean-like
        scale per block (I2_S). No fp32 matrix is ever materialised."""
        n = N * K
        nb = n // block_size
        dev = torch.device(device)
        if fmt == "i2s":
            u = torch.rand(n, device=dev, generator=generator)
            codes = (u >= 0.25).to(torch.uint8) + (u >= 0.75).to(torch.uint8)      # 0: -1, 1: 0, 2: +1
            scales = torch.full((nb,), std * 0.8, device=dev, dtype=torch.float32)
            return cls(fmt, N, K, block_size, _pack_trits(codes), scales=scales)
        size = 256 if fmt == "oil8" else 16
        g = max(1, codebook_group)
        n_cb = (nb + g - 1) // g
        base = cbk.quantile_codebook(size, std, fp16=(fmt == "oil4")).to(dev)
        codebooks = base[None].repeat(n_cb, 1).to(torch.bfloat16).contiguous()
        cb_map = (torch.arange(nb, device=dev) // g).to(torch.int32) if g > 1 else None
        idx = torch.randint(0, size, (n,), device=dev, generator=generator, dtype=torch.uint8)
        packed = idx if fmt == "oil8" else _pack_nibbles(idx)
        return cls(fmt, N, K, block_size, packed.contiguous(), codebooks=codebooks, cb_map=cb_map)

    @classmethod
    def from_oil_linear(cls, mod, rows: slice | None = None) -> "QuantLinear":
        """Pack a trained ``OILLinear`` with its own codebooks (optionally a row range, for
        tensor-parallel shards whose row boundaries fall on block boundaries)."""
        w = mod.weight.detach()
        if mod.fmt == "mixed":
            # per-block formats: the layer's quantised image as dense bf16 (the dequant GEMM kernels
            # take one format per matrix; values are exact, the memory saving is given up)
            img = mod.quantize_now(w.float()).float()
            return cls.from_float(img if rows is None else img[rows], "bf16")
        if mod.fmt not in QFMT:
            wv = w if rows is None else w[rows]
            return cls.from_float(wv.float(), "bf16")
        if rows is None:
            return cls.from_float(w.float(), mod.fmt, mod.block_size, mod.codebook_group,
                                  None if mod.codebooks is None else mod.codebooks.float(), mod.cb_map)
        K = w.shape[1]
        b0 = rows.start * K // mod.block_size
        b1 = rows.stop * K // mod.block_size
        if mod.codebooks is None:
            return cls.from_float(w[rows].float(), mod.fmt, mod.block_size)
        cmap = (torch.arange(b0, b1, device=w.device, dtype=torch.int32) if mod.cb_map is None
                else mod.cb_map[b0:b1].contiguous())
        return cls.from_float(w[rows].float(), mod.fmt, mod.block_size, 1, mod.codebooks.float(), cmap)

    # ------------------------------------------------------------------ compute
    def nbytes(self) -> int:
        t = [self.packed, self.codebooks, self.cb_map, self.scales, self.dense]
        return sum(x.numel() * x.element_size() for x in t if x is not None)

    def dequantize(self) -> torch.Tensor:
        """bf16 [N, K] image of the weights (CUDA kernel on GPU, reference unpacking on CPU)."""
        if self.dense is not None:
            return self.dense
        if self.packed.is_cuda:
            out = torch.empty(self.N, self.K, device=self.packed.device, dtype=torch.bfloat16)
            native.require().dequant_to_bf16(self.packed, self.codebooks, self.cb_map, self.scales, QFMT[self.fmt],
                                             self.N, self.K, self.block_size, out)
            return out
        return self._dequantize_reference().to(torch.bfloat16)

    def gather_rows(self, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Embedding look-up through the quantised table: ``out[t] = dequant(W[ids[t]])`` (bf16
        [tokens, K]); ids int32, clamped to the table. Only the addressed rows are expanded."""
        ids = ids.reshape(-1)
        if out is None:
            out = torch.empty(ids.numel(), self.K, device=ids.device, dtype=torch.bfloat16)
        if self.dense is not None:
            if ids.is_cuda:
                native.require().embedding_fwd(ids, self.dense, out)
            else:
                out.copy_(self.dense[ids.long().clamp(0, self.N - 1)])
            return out
        if ids.is_cuda:
            native.require().dequant_gather_rows(ids, self.packed, self.codebooks, self.cb_map, self.scales,
                                                 QFMT[self.fmt], self.N, self.K, self.block_size, out)
        else:
            out.copy_(self._dequantize_reference()[ids.long().clamp(0, self.N - 1)].to(torch.bfloat16))
        return out

    def _dequantize_reference(self) -> torch.Tensor:
        n = self.N * self.K
        nb = n // self.block_size
        if self.fmt == "i2s":
            p = self.packed.long()
            codes = torch.stack([(p >> (2 * j)) & 3 for j in range(4)], dim=1).reshape(-1)[:n]
            s = self.scales.repeat_interleave(self.block_size)[:n]
            return ((codes.float() - 1.0) * s).reshape(self.N, self.K)
        if self.fmt == "oil8":
            idx = self.packed.long()
        else:
            p = self.packed.long()
            idx = torch.stack([p & 0xF, p >> 4], dim=1).reshape(-1)[:n]
        cbi = (torch.arange(nb, device=idx.device) if self.cb_map is None else self.cb_map.long())
        size = self.codebooks.shape[-1]
        flat_cb = self.codebooks.float().reshape(-1)
        return flat_cb[cbi.repeat_interleave(self.block_size)[:n] * size + idx].reshape(self.N, self.K)

    def matmul(self, x: torch.Tensor, out=None, peer_ptrs=None, k_splits: int = 0,
               peer_bf16_offset: int = -1) -> torch.Tensor:
        """``x [M, K] @ W^T -> [M, N]`` (bf16). With ``peer_ptrs`` the partial result goes to the
        listed peer buffers instead and ``None`` is returned: added as fp32 into every buffer, or,
        with ``peer_bf16_offset >= 0``, stored as bf16 at that element offset of every buffer."""
        M = x.shape[0]
        if not x.is_cuda:
            return (x.float() @ self._dequantize_reference().t().float() if self.dense is None
                    else x.float() @ self.dense.float().t()).to(x.dtype)
        if self.dense is not None:
            assert peer_ptrs is None
            return F.gemm(x, self.dense, out=out)
        C = native.require()
        st = native.status_word(x.device)
        if peer_ptrs is not None:
            C.dequant_gemm(x, self.packed, self.codebooks, self.cb_map, self.scales, QFMT[self.fmt], self.N, self.K,
                           self.block_size, None, list(peer_ptrs), k_splits, st, peer_bf16_offset)
            return None
        if M <= DECODE_MAX_TOKENS:
            if out is None:
                out = torch.empty(M, self.N, device=x.device, dtype=torch.bfloat16)
            if M == 1 and self.fmt == "i2s" and self.K % 64 == 0 and self.K * 4 <= 200 * 1024 and x.is_contiguous() \
                    and out.is_contiguous():
                # single-token ternary decode: one warp per output row over the packed trits, no tensor-core
                # tile to fill (a 128 x 8 MMA tile would be 7/8 padding)
                C.i2s_gemv(x.view(-1), self.packed, self.scales, self.N, self.K, self.block_size, out.view(-1))
                return out
            # One CTA covers 128 output features. Too few of them to fill the GPU (narrow or
            # tensor-parallel layers): split K across CTAs into the fp32 accumulator instead.
            n_ctas = (self.N + 127) // 128
            if n_ctas * 4 < 3 * _sm_count(x.device) and self.K >= 1024 and out.is_contiguous():
                if not torch.cuda.is_current_stream_capturing():
                    reserve_accumulator(x.device, M * self.N)
                acc = _ACC.get(_norm_device(x.device))
                if acc is not None and acc.numel() >= M * self.N:
                    acc = acc[: M * self.N].view(M, self.N)
                    C.dequant_gemm(x, self.packed, self.codebooks, self.cb_map, self.scales, QFMT[self.fmt], self.N,
                                   self.K, self.block_size, acc, [], k_splits, st)
                    C.finalize_acc(acc, None, out)
                    return out
            C.dequant_gemm(x, self.packed, self.codebooks, self.cb_map, self.scales, QFMT[self.fmt], self.N, self.K,
                           self.block_size, out, [], 1, st)
            return out
        return F.gemm(x, self.dequantize(), out=out)

    def matmul_acc(self, x: torch.Tensor) -> torch.Tensor:
        """Split-K product left in the device's fp32 accumulator: returns the ``[M, N]`` view, which
        the caller must consume with a kernel that zeroes it again (finalize / tp_push)."""
        M = x.shape[0]
        if not torch.cuda.is_current_stream_capturing():
            reserve_accumulator(x.device, M * self.N)
        acc = _ACC[_norm_device(x.device)][: M * self.N].view(M, self.N)
        native.require().dequant_gemm(x, self.packed, self.codebooks, self.cb_map, self.scales, QFMT[self.fmt],
                                      self.N, self.K, self.block_size, acc, [], 0, native.status_word(x.device))
        return acc
