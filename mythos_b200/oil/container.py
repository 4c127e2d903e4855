"""The ``.oil`` container and its ``.oilidx`` sidecar, byte-compatible with the reference.

File layout (all little-endian, packed; reference writer src/oil_format.cpp:188-277, reader
:283-507):

    "OIL1" | u32 version | u32 flags | u32 config_size | config bytes
    u32 n_blocks   | n_blocks x { u32 block_id, u8 format, u32 cb_bytes }          (9 bytes each)
    u32 n_tensors  | n_tensors x { u16 name_len, name, u32 block_start, u32 num_blocks }
    blocks, in block-id order: { u32 num_weights, u32 cb_bytes, cb, u32 idx_bytes, idx }

Sidecar version 1 (src/oil_format.cpp:513-602): ``"MYTHOSIDX\\0"`` | u32 version | u32 n |
n x { u16 name_len, name, sha256(name) }. A reader recomputes every hash and raises, naming the
tensor, on the first mismatch or truncation.

Sidecar version 2 (this framework; same magic, so version-1 readers stop at the version field or
fail cleanly): after the version-1 body it appends, per tensor, { u8 rank, i64 dims[rank],
u64 offset, u64 nbytes, sha256(stored block bytes) } — shapes, byte ranges for sharded loading,
and a real content digest.

Differences from the reference reader, all on the read side and all compatible: block offsets are
indexed once (the reference walks from the first block on every read, O(blocks^2)); TERNARY and
BINARY blocks are dequantised (the reference returns zeros); shapes come from the config tail or
the v2 sidecar when present.
"""
from __future__ import annotations

import hashlib
import io
import os
import struct
from dataclasses import dataclass

import numpy as np

from .formats import Format, decode_block

MAGIC = b"OIL1"
IDX_MAGIC = b"MYTHOSIDX\x00"


class OILError(Exception):
    """Malformed or corrupt container / sidecar."""


@dataclass
class BlockData:
    format: Format
    num_weights: int
    codebook: bytes = b""
    indices: bytes = b""

    def nbytes(self) -> int:
        return 12 + len(self.codebook) + len(self.indices)


@dataclass
class TensorEntry:
    name: str
    block_start: int
    num_blocks: int


def sha256(data: bytes) -> bytes:
    return hashlib.sha256(data).digest()


def file_sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


# =============================================================================== writer
class OILWriter:
    """Streaming writer. Call order: ``write_header`` -> ``write_format_table`` ->
    ``write_tensor_table`` -> ``write_block`` for every block in id order -> ``close``.
    :func:`write_oil` does all of it from a list of tensors."""

    def __init__(self, path: str):
        self.path = path
        self._tmp = path + ".tmp"
        self._f = open(self._tmp, "wb")
        self._blob_index: dict[str, tuple[int, int]] = {}

    def write_header(self, config: bytes = b"", version: int = 1, flags: int = 0) -> None:
        self._f.write(MAGIC + struct.pack("<III", version, flags, len(config)) + config)

    def write_format_table(self, entries) -> None:
        """entries: iterable of (block_id, format, cb_bytes)."""
        entries = list(entries)
        out = [struct.pack("<I", len(entries))]
        out += [struct.pack("<IBI", bid, int(fmt), cbb) for bid, fmt, cbb in entries]
        self._f.write(b"".join(out))

    def write_tensor_table(self, entries) -> None:
        entries = list(entries)
        out = [struct.pack("<I", len(entries))]
        for e in entries:
            nb = e.name.encode("utf-8")
            if len(nb) > 0xFFFF:
                raise OILError(f"tensor name too long: {e.name[:40]}...")
            out.append(struct.pack("<H", len(nb)) + nb + struct.pack("<II", e.block_start, e.num_blocks))
        self._f.write(b"".join(out))

    def write_block(self, block: BlockData) -> int:
        off = self._f.tell()
        self._f.write(struct.pack("<II", block.num_weights, len(block.codebook)))
        self._f.write(block.codebook)
        self._f.write(struct.pack("<I", len(block.indices)))
        self._f.write(block.indices)
        return off

    def write_dedup(self, data: bytes) -> int:
        """Content-addressed blob: identical bytes are stored once; returns the file offset."""
        if not data:
            return -1
        key = hashlib.sha256(data).hexdigest()
        hit = self._blob_index.get(key)
        if hit is not None:
            return hit[0]
        off = self._f.tell()
        self._f.write(data)
        self._blob_index[key] = (off, len(data))
        return off

    def close(self) -> None:
        if self._f is not None:
            self._f.flush()
            os.fsync(self._f.fileno())
            self._f.close()
            self._f = None
            os.replace(self._tmp, self.path)  # data first, then the name: readers never see a torn file

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if exc[0] is None:
            self.close()
        elif self._f is not None:
            self._f.close()
            self._f = None
            try:
                os.unlink(self._tmp)
            except OSError:
                pass


def write_oil(path: str, tensors, config: bytes = b"", version: int = 1, flags: int = 0, write_idx: bool = True,
              idx_version: int = 2, shapes: dict | None = None) -> None:
    """tensors: list of (name, [BlockData, ...]). Writes the container and (optionally) its sidecar
    ``path + 'idx'`` (e.g. ``model.oil`` -> ``model.oilidx``)."""
    fmt_entries, tensor_entries = [], []
    bid = 0
    for name, blocks in tensors:
        tensor_entries.append(TensorEntry(name, bid, len(blocks)))
        for b in blocks:
            fmt_entries.append((bid, b.format, len(b.codebook)))
            bid += 1
    ranges = {}
    with OILWriter(path) as w:
        w.write_header(config, version, flags)
        w.write_format_table(fmt_entries)
        w.write_tensor_table(tensor_entries)
        for name, blocks in tensors:
            start = None
            h = hashlib.sha256()
            nbytes = 0
            for b in blocks:
                off = w.write_block(b)
                start = off if start is None else start
                nbytes += b.nbytes()
                h.update(struct.pack("<II", b.num_weights, len(b.codebook)) + b.codebook +
                         struct.pack("<I", len(b.indices)) + b.indices)
            ranges[name] = (start or 0, nbytes, h.digest())
    if write_idx:
        write_idx_file(idx_path_for(path), [n for n, _ in tensors], version=idx_version, ranges=ranges,
                       shapes=shapes or {})


# =============================================================================== reader
class OILReader:
    def __init__(self, path: str):
        self.path = path
        try:
            self._mm = np.memmap(path, dtype=np.uint8, mode="r")
        except (OSError, ValueError) as e:
            raise OILError(f"cannot open {path}: {e}") from e
        data = self._mm
        if data.size < 16 or bytes(data[:4]) != MAGIC:
            raise OILError(f"{path}: not an OIL1 container")
        self.version, self.flags, self.config_size = struct.unpack_from("<III", data, 4)
        off = 16
        self._need(off + self.config_size, "config")
        self.config = bytes(data[off:off + self.config_size])
        off += self.config_size
        self._need(off + 4, "format table")
        (nb,) = struct.unpack_from("<I", data, off)
        off += 4
        self._need(off + 9 * nb, "format table")
        ft = np.frombuffer(bytes(data[off:off + 9 * nb]), dtype=np.dtype([("id", "<u4"), ("fmt", "u1"), ("cb", "<u4")]))
        self.block_formats = ft["fmt"].astype(np.uint8)
        self.block_cb_bytes = ft["cb"].astype(np.uint32)
        off += 9 * nb
        self._need(off + 4, "tensor table")
        (nt,) = struct.unpack_from("<I", data, off)
        off += 4
        self.tensors: dict[str, TensorEntry] = {}
        self.tensor_order: list[str] = []
        for i in range(nt):
            self._need(off + 2, f"tensor entry {i}")
            (ln,) = struct.unpack_from("<H", data, off)
            off += 2
            self._need(off + ln + 8, f"tensor entry {i}")
            name = bytes(data[off:off + ln]).decode("utf-8", errors="replace")
            off += ln
            bs, nbk = struct.unpack_from("<II", data, off)
            off += 8
            self.tensors[name] = TensorEntry(name, bs, nbk)
            self.tensor_order.append(name)
        self.data_offset = off
        # one pass over the block headers gives every block's offset
        self.block_offsets = np.zeros(nb + 1, dtype=np.int64)
        self.block_weights = np.zeros(nb, dtype=np.int64)
        for b in range(nb):
            self.block_offsets[b] = off
            self._need(off + 8, f"block {b}")
            nw, cbb = struct.unpack_from("<II", data, off)
            self._need(off + 12 + cbb, f"block {b}")
            (ib,) = struct.unpack_from("<I", data, off + 8 + cbb)
            self.block_weights[b] = nw
            off += 12 + cbb + ib
            self._need(off, f"block {b}")
        self.block_offsets[nb] = off

    def _need(self, end: int, what: str) -> None:
        if end > self._mm.size:
            raise OILError(f"{self.path}: truncated in {what} (need {end} bytes, have {self._mm.size})")

    # ------------------------------------------------------------------ accessors
    @property
    def num_blocks(self) -> int:
        return len(self.block_formats)

    def tensor_names(self) -> list[str]:
        return list(self.tensor_order)

    def tensor_formats(self, name: str) -> list[Format]:
        e = self.tensors[name]
        return [Format(int(self.block_formats[b])) if self.block_formats[b] <= 5 else Format.FP32
                for b in range(e.block_start, e.block_start + e.num_blocks)]

    def read_block(self, block_id: int) -> BlockData:
        if not 0 <= block_id < self.num_blocks:
            raise OILError(f"block {block_id} out of range")
        off = int(self.block_offsets[block_id])
        nw, cbb = struct.unpack_from("<II", self._mm, off)
        cb = bytes(self._mm[off + 8:off + 8 + cbb])
        (ib,) = struct.unpack_from("<I", self._mm, off + 8 + cbb)
        idx = bytes(self._mm[off + 12 + cbb:off + 12 + cbb + ib])
        f = int(self.block_formats[block_id])
        return BlockData(Format(f) if f <= 5 else Format.FP32, nw, cb, idx)

    def tensor_byte_range(self, name: str) -> tuple[int, int]:
        e = self.tensors[name]
        lo = int(self.block_offsets[e.block_start])
        hi = int(self.block_offsets[e.block_start + e.num_blocks])
        return lo, hi - lo

    def tensor_sha256(self, name: str) -> bytes:
        lo, n = self.tensor_byte_range(name)
        return hashlib.sha256(bytes(self._mm[lo:lo + n])).digest()

    def read_tensor(self, name: str) -> np.ndarray:
        """Dequantised flat float32 array of the tensor (empty array when the name is unknown,
        like the reference's empty Tensor)."""
        e = self.tensors.get(name)
        if e is None:
            return np.zeros(0, dtype=np.float32)
        parts = []
        for b in range(e.block_start, e.block_start + e.num_blocks):
            bd = self.read_block(b)
            parts.append(decode_block(bd.format, bd.num_weights, bd.codebook, bd.indices))
        return np.concatenate(parts) if parts else np.zeros(0, dtype=np.float32)

    def read_tensor_blocks(self, name: str) -> list[BlockData]:
        e = self.tensors[name]
        return [self.read_block(b) for b in range(e.block_start, e.block_start + e.num_blocks)]

    def close(self):
        self._mm = None


# =============================================================================== sidecar
def idx_path_for(oil_path: str) -> str:
    return oil_path + "idx" if oil_path.endswith(".oil") else oil_path + ".oilidx"


def write_idx_file(path: str, names, version: int = 1, ranges: dict | None = None, shapes: dict | None = None) -> None:
    buf = io.BytesIO()
    names = list(names)
    buf.write(IDX_MAGIC + struct.pack("<II", version, len(names)))
    for n in names:
        nb = n.encode("utf-8")
        buf.write(struct.pack("<H", len(nb)) + nb + sha256(nb))
    if version >= 2:
        ranges, shapes = ranges or {}, shapes or {}
        for n in names:
            shape = tuple(int(d) for d in shapes.get(n, ()))
            off, nbytes, digest = ranges.get(n, (0, 0, b"\x00" * 32))
            buf.write(struct.pack("<B", len(shape)) + struct.pack(f"<{len(shape)}q", *shape) +
                      struct.pack("<QQ", off, nbytes) + digest)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(buf.getvalue())
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


@dataclass
class IdxRecord:
    name: str
    shape: tuple = ()
    offset: int = 0
    nbytes: int = 0
    sha256: bytes = b""


def read_idx_file(path: str) -> tuple[int, list[IdxRecord]]:
    """Returns (version, records). Raises :class:`OILError` naming the corrupt tensor (hash of the
    name does not match) or the index at which the file is truncated."""
    try:
        with open(path, "rb") as f:
            data = f.read()
    except OSError as e:
        raise OILError(f"OILIdxReader: invalid idx file: {e}") from e
    if len(data) < 18 or data[:9] != IDX_MAGIC[:9]:
        raise OILError("OILIdxReader: invalid idx file")
    version, n = struct.unpack_from("<II", data, 10)
    off = 18
    recs = []
    for i in range(n):
        if off + 2 > len(data):
            raise OILError(f"OILIdxReader: corrupt idx - truncated before tensor name length at index {i}")
        (ln,) = struct.unpack_from("<H", data, off)
        off += 2
        if off + ln + 32 > len(data):
            raise OILError(f"OILIdxReader: corrupt idx - truncated tensor name/hash at index {i}")
        raw = data[off:off + ln]
        off += ln
        stored = data[off:off + 32]
        off += 32
        name = raw.decode("utf-8", errors="replace")
        if sha256(raw) != stored:
            disp = name if name else "<empty>"
            raise OILError(f'OILIdxReader: corrupt idx - name hash mismatch for tensor "{disp}" at index {i}')
        recs.append(IdxRecord(name))
    if version >= 2:
        for i, r in enumerate(recs):
            if off + 1 > len(data):
                raise OILError(f'OILIdxReader: corrupt idx - truncated v2 record for tensor "{r.name}" at index {i}')
            rank = data[off]
            off += 1
            need = 8 * rank + 16 + 32
            if off + need > len(data):
                raise OILError(f'OILIdxReader: corrupt idx - truncated v2 record for tensor "{r.name}" at index {i}')
            r.shape = struct.unpack_from(f"<{rank}q", data, off)
            off += 8 * rank
            r.offset, r.nbytes = struct.unpack_from("<QQ", data, off)
            off += 16
            r.sha256 = data[off:off + 32]
            off += 32
    return version, recs


def verify(oil_path: str, idx_path: str | None = None) -> list[str]:
    """Checks every tensor of the container against the v2 sidecar digests. Returns the list of
    verified names; raises :class:`OILError` naming the first tensor whose bytes do not match."""
    idx_path = idx_path or idx_path_for(oil_path)
    version, recs = read_idx_file(idx_path)
    rd = OILReader(oil_path)
    ok = []
    for r in recs:
        if r.name not in rd.tensors:
            raise OILError(f'verify: tensor "{r.name}" listed in the sidecar is missing from {oil_path}')
        if version >= 2 and r.sha256 and r.sha256 != b"\x00" * 32:
            if rd.tensor_sha256(r.name) != r.sha256:
                raise OILError(f'verify: content hash mismatch for tensor "{r.name}"')
        ok.append(r.name)
    return ok
