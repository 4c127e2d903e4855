"""Weight formats of the OIL container and their bit-level packings.

Numeric values of ``Format`` are those of the reference (include/oil/types.h:17-24) and are what
the 9-byte format-table entries of a ``.oil`` file store.

Block payloads (``cb`` = codebook bytes, ``idx`` = index bytes), as written by the reference tools:

* FP32     cb empty; idx = raw little-endian float32                     (src/model.cpp:126-141)
* FP16     cb empty; idx = raw little-endian float16
* OIL8     cb = u32 0x4F494C38 + 256 x f32; idx = one byte per weight   (src/codebook.cpp:192-212)
* OIL4     cb = u32 0x4F494C34 + 16 x f16; idx = two weights per byte, even index in the low
           nibble                                                        (src/oil_format.cpp:436-450)
* TERNARY  cb = 3 x f32 {-s, 0, +s}; idx = 2-bit codes (trit + 1) packed LSB first, four per byte
           (tools/convert.cpp:329-378 writes {-1,0,+1}; this framework carries the per-block
           absmean scale ``s`` of I2_S in the same three slots, so any reader that dequantises
           ``cb[code]`` gets the right value)
* BINARY   cb = 2 x f32 {-s, +s}; idx = one bit per weight, LSB first (bit = w > 0)

The ternary code assignment (00 = -1, 01 = 0, 10 = +1) is the one of the reference's I2_S kernels
(src/kernel_i2s.cpp:13-21), its converter and its compressed KV cache; the alternative encoding
used by its ``STEQuantizer`` is not written by this framework.
"""
from __future__ import annotations

import enum

import numpy as np


class Format(enum.IntEnum):
    BINARY = 0
    TERNARY = 1
    OIL4 = 2
    OIL8 = 3
    FP16 = 4
    FP32 = 5


FORMAT_BPW = {Format.BINARY: 1.0, Format.TERNARY: 1.58, Format.OIL4: 4.0, Format.OIL8: 8.0, Format.FP16: 16.0,
              Format.FP32: 32.0}

NAME_TO_FORMAT = {"binary": Format.BINARY, "ternary": Format.TERNARY, "i2s": Format.TERNARY, "oil4": Format.OIL4,
                  "oil8": Format.OIL8, "fp16": Format.FP16, "fp32": Format.FP32}
FORMAT_TO_NAME = {Format.BINARY: "binary", Format.TERNARY: "i2s", Format.OIL4: "oil4", Format.OIL8: "oil8",
                  Format.FP16: "fp16", Format.FP32: "fp32"}


def format_bpw(fmt) -> float:
    return FORMAT_BPW[Format(int(fmt))]


# ------------------------------------------------------------------------------ OIL4 nibbles
def pack_nibbles(idx: np.ndarray) -> bytes:
    """Two 4-bit indices per byte, even position in the low nibble."""
    a = np.asarray(idx, dtype=np.uint8)
    if a.size % 2:
        a = np.concatenate([a, np.zeros(1, dtype=np.uint8)])
    return ((a[0::2] & 0xF) | ((a[1::2] & 0xF) << 4)).astype(np.uint8).tobytes()


def unpack_nibbles(data: bytes, n: int) -> np.ndarray:
    a = np.frombuffer(data, dtype=np.uint8)
    out = np.empty(a.size * 2, dtype=np.uint8)
    out[0::2] = a & 0xF
    out[1::2] = a >> 4
    return out[:n]


# ------------------------------------------------------------------------------ ternary 2-bit codes
def pack_trits(codes: np.ndarray) -> bytes:
    """Codes in {0,1,2} (= trit + 1), four per byte, first weight in bits 0-1."""
    a = np.asarray(codes, dtype=np.uint8)
    pad = (-a.size) % 4
    if pad:
        a = np.concatenate([a, np.full(pad, 1, dtype=np.uint8)])  # pad with the zero trit
    a = a.reshape(-1, 4)
    return (a[:, 0] | (a[:, 1] << 2) | (a[:, 2] << 4) | (a[:, 3] << 6)).astype(np.uint8).tobytes()


def unpack_trits(data: bytes, n: int) -> np.ndarray:
    a = np.frombuffer(data, dtype=np.uint8)
    out = np.empty((a.size, 4), dtype=np.uint8)
    for j in range(4):
        out[:, j] = (a >> (2 * j)) & 3
    return out.reshape(-1)[:n]


# ------------------------------------------------------------------------------ binary
def pack_bits(bits: np.ndarray) -> bytes:
    return np.packbits(np.asarray(bits, dtype=np.uint8), bitorder="little").tobytes()


def unpack_bits(data: bytes, n: int) -> np.ndarray:
    return np.unpackbits(np.frombuffer(data, dtype=np.uint8), bitorder="little")[:n]


# ------------------------------------------------------------------------------ block codecs (numpy, host side)
def encode_block(fmt: Format, values: np.ndarray, codebook: np.ndarray | None = None,
                 indices: np.ndarray | None = None, scale: float | None = None) -> tuple[bytes, bytes]:
    """Returns (cb_bytes, idx_bytes) of one block. For OIL8/OIL4 pass ``codebook`` and
    ``indices``; for TERNARY pass codes in ``indices`` and ``scale``; for BINARY bits and scale."""
    from . import codebook as cbk
    import torch

    fmt = Format(int(fmt))
    if fmt == Format.FP32:
        return b"", np.asarray(values, dtype="<f4").tobytes()
    if fmt == Format.FP16:
        return b"", np.asarray(values, dtype="<f2").tobytes()
    if fmt == Format.OIL8:
        return cbk.serialize_oil8(torch.as_tensor(codebook)), np.asarray(indices, dtype=np.uint8).tobytes()
    if fmt == Format.OIL4:
        return cbk.serialize_oil4(torch.as_tensor(codebook)), pack_nibbles(indices)
    if fmt == Format.TERNARY:
        s = np.float32(scale)
        return np.array([-s, 0.0, s], dtype="<f4").tobytes(), pack_trits(indices)
    if fmt == Format.BINARY:
        s = np.float32(scale)
        return np.array([-s, s], dtype="<f4").tobytes(), pack_bits(indices)
    raise ValueError(fmt)


def decode_block(fmt: Format, n: int, cb: bytes, idx: bytes) -> np.ndarray:
    """Dequantise one block to float32 (all six formats; the reference reader returns zeros for
    TERNARY/BINARY, src/oil_format.cpp:451-455)."""
    from . import codebook as cbk

    fmt = Format(int(fmt))
    if fmt == Format.FP32:
        return np.frombuffer(idx, dtype="<f4", count=n).astype(np.float32)
    if fmt == Format.FP16:
        return np.frombuffer(idx, dtype="<f2", count=n).astype(np.float32)
    if fmt == Format.OIL8:
        _, c = cbk.deserialize(cb)
        return c[np.frombuffer(idx, dtype=np.uint8, count=n)]
    if fmt == Format.OIL4:
        _, c = cbk.deserialize(cb)
        return c[unpack_nibbles(idx, n)]
    if fmt == Format.TERNARY:
        c = np.frombuffer(cb, dtype="<f4", count=3).astype(np.float32) if len(cb) >= 12 else np.array(
            [-1.0, 0.0, 1.0], dtype=np.float32)
        return c[np.minimum(unpack_trits(idx, n), 2)]
    if fmt == Format.BINARY:
        c = np.frombuffer(cb, dtype="<f4", count=2).astype(np.float32) if len(cb) >= 8 else np.array(
            [-1.0, 1.0], dtype=np.float32)
        return c[unpack_bits(idx, n)]
    raise ValueError(fmt)


def quantize_binary(values: np.ndarray) -> tuple[np.ndarray, float]:
    """scale = mean(|w|), bit = w > 0 (reference engines/OIL8/quantize.cpp:148-164)."""
    v = np.asarray(values, dtype=np.float32)
    return (v > 0).astype(np.uint8), float(np.abs(v).mean()) if v.size else 0.0


def quantize_ternary(values: np.ndarray) -> tuple[np.ndarray, float]:
    """I2_S: scale = mean(|w|) of the block, trit = clamp(round(w / scale), -1, 1); codes = trit + 1."""
    v = np.asarray(values, dtype=np.float32)
    s = float(np.abs(v).mean()) if v.size else 0.0
    if s == 0.0:
        return np.ones(v.size, dtype=np.uint8), 0.0
    t = np.clip(np.rint(v / np.float32(s)), -1, 1).astype(np.int8)
    return (t + 1).astype(np.uint8), s


def quantize_affine_u8(values: np.ndarray) -> tuple[np.ndarray, float, int]:
    """Asymmetric affine uint8 quantisation (reference engines/OIL8/quantize.cpp:14-60):
    returns (q, scale, zero_point) with value ~= (q - zero_point) * scale."""
    v = np.asarray(values, dtype=np.float32)
    lo, hi = float(v.min(initial=0.0)), float(v.max(initial=0.0))
    scale = (hi - lo) / 255.0 if hi > lo else 1.0
    zp = int(round(-lo / scale)) if hi > lo else 0
    q = np.clip(np.rint(v / scale) + zp, 0, 255).astype(np.uint8)
    return q, scale, zp


def quantize_int8_symmetric(values: np.ndarray, per_row: bool = False):
    """Symmetric absmax/127 int8 (reference src/int8_quant.cpp:8-41): per tensor or per row."""
    v = np.asarray(values, dtype=np.float32)
    if per_row:
        amax = np.abs(v).max(axis=-1, keepdims=True)
    else:
        amax = np.abs(v).max(initial=0.0)
    scale = np.where(amax > 0, amax / 127.0, 1.0)
    q = np.clip(np.rint(v / scale), -127, 127).astype(np.int8)
    return q, scale
