"""Core types, host memory helpers and the host tensor wire format.

Counterparts of the reference's ``include/oil/types.h`` (``DType``, ``format_to_dtype``,
``dtype_size``, ``Shape`` with at most 8 dims, ``Status``, ``Config``, ``Error`` / ``OIL_CHECK``,
:17-149), ``include/oil/memory.h`` (64-byte aligned allocations, a reference-counted ``Buffer``
with ``slice``, a bump ``MemoryPool``, :13-147) and ``Tensor::serialize / deserialize``
(``i32 rank, i64 dims[rank], u8 dtype, raw bytes``, src/tensor.cpp:297-334). Device tensors are
``torch.Tensor``; these host-side pieces exist for file formats, staging buffers and embedders.
"""
from __future__ import annotations

import enum
import struct
from dataclasses import dataclass

import numpy as np
import torch

from .oil.formats import Format

ALIGNMENT = 64
MAX_DIMS = 8


class DType(enum.IntEnum):
    I64 = 0
    U8 = 1
    U4 = 2      # two per byte
    I2 = 3      # four per byte (ternary)
    I1 = 4      # eight per byte (binary)
    F16 = 5
    F32 = 6


_DTYPE_BITS = {DType.I64: 64, DType.U8: 8, DType.U4: 4, DType.I2: 2, DType.I1: 1, DType.F16: 16, DType.F32: 32}
_FORMAT_DTYPE = {Format.BINARY: DType.I1, Format.TERNARY: DType.I2, Format.OIL4: DType.U4, Format.OIL8: DType.U8,
                 Format.FP16: DType.F16, Format.FP32: DType.F32}


def format_to_dtype(fmt) -> DType:
    """Storage element type of a block format (unknown formats read as F32, as in the reference)."""
    try:
        return _FORMAT_DTYPE[Format(int(fmt))]
    except ValueError:
        return DType.F32


def dtype_bits(dt: DType) -> int:
    return _DTYPE_BITS[DType(dt)]


def packed_nbytes(dt: DType, count: int) -> int:
    """Bytes that ``count`` elements of ``dt`` occupy when packed (sub-byte types round up)."""
    return (count * dtype_bits(dt) + 7) // 8


class OilError(RuntimeError):
    """The framework's error type (``oil::Error``)."""


def check(cond, msg: str) -> None:
    """``OIL_CHECK``: raise :class:`OilError` with ``msg`` unless ``cond`` holds."""
    if not cond:
        raise OilError(msg)


@dataclass(frozen=True)
class Status:
    ok: bool = True
    msg: str = ""

    @staticmethod
    def success() -> "Status":
        return Status()

    @staticmethod
    def error(msg: str) -> "Status":
        return Status(False, msg)

    def __bool__(self) -> bool:
        return self.ok


@dataclass
class Config:
    """Process-wide settings (``oil::Config``); ``utils.env.RuntimeEnv`` fills one from ``OIL_*``."""
    num_threads: int = 1
    seed: int = 42
    pool_size: int = 64 << 20
    verbose: bool = False

    @classmethod
    def from_environ(cls, env=None) -> "Config":
        from .utils.env import RuntimeEnv

        rt = RuntimeEnv.from_environ(env)
        return cls(max(1, rt.num_threads), rt.seed, rt.memory_pool_size, rt.verbose)


class Shape(tuple):
    """Up to 8 non-negative dimensions; ``numel`` and a ``[a, b, c]`` rendering like the reference's."""

    def __new__(cls, *dims):
        if len(dims) == 1 and not isinstance(dims[0], int):
            dims = tuple(dims[0])
        check(len(dims) <= MAX_DIMS, f"shape has {len(dims)} dimensions, at most {MAX_DIMS} are supported")
        check(all(isinstance(d, (int, np.integer)) and d >= 0 for d in dims), "dimensions must be non-negative integers")
        return super().__new__(cls, (int(d) for d in dims))

    @property
    def rank(self) -> int:
        return len(self)

    def numel(self) -> int:
        n = 1
        for d in self:
            n *= d
        return n

    def __str__(self) -> str:
        return "[" + ", ".join(str(d) for d in self) + "]"


# ------------------------------------------------------------------------------ memory
def aligned_empty(nbytes: int, alignment: int = ALIGNMENT) -> np.ndarray:
    """A uint8 array of ``nbytes`` whose first byte sits on an ``alignment`` boundary."""
    raw = np.empty(nbytes + alignment, dtype=np.uint8)
    off = (-raw.ctypes.data) % alignment
    return raw[off:off + nbytes]


class Buffer:
    """Reference-counted, 64-byte aligned host bytes. ``slice`` returns a view that shares the
    allocation and keeps it alive; ``retain`` / ``release`` count explicit owners."""

    def __init__(self, nbytes: int, _base: "Buffer | None" = None, _view: np.ndarray | None = None):
        self._root = _base._root if _base is not None else self
        self.data = _view if _view is not None else aligned_empty(nbytes)
        if _base is None:
            self._refs = 1
        else:
            self._root._refs += 1

    @property
    def nbytes(self) -> int:
        return int(self.data.nbytes)

    @property
    def address(self) -> int:
        return int(self.data.ctypes.data)

    @property
    def refcount(self) -> int:
        return self._root._refs

    def slice(self, offset: int, nbytes: int) -> "Buffer":
        check(0 <= offset and offset + nbytes <= self.nbytes, "slice outside the buffer")
        return Buffer(nbytes, _base=self, _view=self.data[offset:offset + nbytes])

    def retain(self) -> "Buffer":
        self._root._refs += 1
        return self

    def release(self) -> int:
        check(self._root._refs > 0, "buffer released more often than retained")
        self._root._refs -= 1
        return self._root._refs

    def as_array(self, dtype, count: int | None = None) -> np.ndarray:
        return self.data.view(np.uint8)[: None if count is None else count * np.dtype(dtype).itemsize].view(dtype)


class MemoryPool:
    """Bump allocator over one aligned block: ``alloc`` hands out 64-byte aligned views until the
    block is full (then raises), ``reset`` makes everything available again."""

    def __init__(self, capacity: int = 64 << 20):
        self.capacity = int(capacity)
        self._block = aligned_empty(self.capacity)
        self._used = 0
        self.peak = 0

    def alloc(self, nbytes: int) -> np.ndarray:
        start = (self._used + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
        if start + nbytes > self.capacity:
            raise OilError(f"memory pool exhausted: {nbytes} bytes requested, {self.capacity - start} left")
        self._used = start + nbytes
        self.peak = max(self.peak, self._used)
        return self._block[start:start + nbytes]

    def alloc_array(self, shape, dtype=np.float32) -> np.ndarray:
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return self.alloc(n).view(dtype).reshape(shape)

    @property
    def used(self) -> int:
        return self._used

    def reset(self) -> None:
        self._used = 0


# ------------------------------------------------------------------------------ tensor wire format
_WIRE_NP = {DType.I64: np.int64, DType.U8: np.uint8, DType.F16: np.float16, DType.F32: np.float32}
_WIRE_ID = {torch.int64: DType.I64, torch.uint8: DType.U8, torch.float16: DType.F16, torch.float32: DType.F32}


def serialize_tensor(t: torch.Tensor) -> bytes:
    """``i32 rank, i64 dims[rank], u8 dtype (reference DType numbering), raw little-endian data``.
    Types outside {int64, uint8, float16, float32} are stored as float32."""
    t = t.detach().cpu().contiguous()
    if t.dtype not in _WIRE_ID:
        t = t.float()
    Shape(*t.shape)
    head = struct.pack("<i", t.dim()) + struct.pack(f"<{t.dim()}q", *t.shape) + struct.pack("<B", int(_WIRE_ID[t.dtype]))
    return head + t.numpy().tobytes()


def deserialize_tensor(data: bytes, offset: int = 0):
    """Inverse of :func:`serialize_tensor`; returns ``(tensor, next_offset)``."""
    check(len(data) >= offset + 4, "truncated tensor header")
    (rank,) = struct.unpack_from("<i", data, offset)
    check(0 <= rank <= MAX_DIMS, f"bad tensor rank {rank}")
    offset += 4
    check(len(data) >= offset + 8 * rank + 1, "truncated tensor header")
    dims = struct.unpack_from(f"<{rank}q", data, offset) if rank else ()
    offset += 8 * rank
    dt = DType(data[offset])
    offset += 1
    check(dt in _WIRE_NP, f"dtype {dt.name} has no dense wire form")
    n = Shape(*dims).numel()
    nbytes = n * np.dtype(_WIRE_NP[dt]).itemsize
    check(len(data) >= offset + nbytes, "truncated tensor data")
    arr = np.frombuffer(data, dtype=_WIRE_NP[dt], count=n, offset=offset).copy()
    return torch.from_numpy(arr).reshape(tuple(dims)), offset + nbytes
