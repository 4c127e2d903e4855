"""Importers: safetensors, GGUF (F32 / F16 / Q4_0 / Q4_1 / Q8_0), raw fp32.

Reference: the GGUF reader of ``oil_convert`` (tools/convert.cpp:93-309) and the unbuilt
``SafetensorsImporter`` / ``GGUFImporter`` (src/adapters/safetensors.cpp, gguf_import.cpp — the
latter never reads tensor data). Both importers here return ``{name: float32 ndarray}`` with
shapes; safetensors additionally accepts BF16 and F16.
"""
from __future__ import annotations

import json
import struct

import numpy as np

GGUF_MAGIC = 0x46554747  # "GGUF"
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q8_0 = 0, 1, 2, 3, 8
_GGUF_SCALAR = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}


def read_raw_fp32(path: str) -> dict:
    return {"weights": np.fromfile(path, dtype="<f4")}


def read_safetensors(path: str) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        base = 8 + n
        out = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            lo, hi = meta["data_offsets"]
            f.seek(base + lo)
            raw = f.read(hi - lo)
            dt = meta["dtype"]
            if dt == "F32":
                a = np.frombuffer(raw, dtype="<f4")
            elif dt == "F16":
                a = np.frombuffer(raw, dtype="<f2").astype(np.float32)
            elif dt == "BF16":
                a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
            elif dt == "F64":
                a = np.frombuffer(raw, dtype="<f8").astype(np.float32)
            else:
                continue  # integer tensors are not weights
            out[name] = a.reshape(meta["shape"]).astype(np.float32)
    return out


def write_safetensors(path: str, tensors: dict) -> None:
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        b = np.ascontiguousarray(a, dtype="<f4").tobytes()
        header[name] = {"dtype": "F32", "shape": list(np.shape(a)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode("utf-8")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


class _Cursor:
    def __init__(self, data: bytes):
        self.d, self.o = data, 0

    def take(self, fmt: str):
        v = struct.unpack_from("<" + fmt, self.d, self.o)
        self.o += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def string(self, v1: bool) -> str:
        n = self.take("I" if v1 else "Q")
        s = self.d[self.o:self.o + n].decode("utf-8", errors="replace")
        self.o += n
        return s

    def skip_value(self, t: int, v1: bool):
        if t in _GGUF_SCALAR:
            return self.take(_GGUF_SCALAR[t])
        if t == 8:
            return self.string(v1)
        if t == 9:
            et = self.take("I")
            n = self.take("I" if v1 else "Q")
            return [self.skip_value(et, v1) for _ in range(n)]
        raise ValueError(f"unknown GGUF metadata type {t}")


def _dequant_q4_0(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 18)
    d = blk[:, :2].copy().view("<f2").astype(np.float32)
    q = blk[:, 2:]
    lo = (q & 0xF).astype(np.int8) - 8
    hi = (q >> 4).astype(np.int8) - 8
    return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)[:n]


def _dequant_q4_1(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 20)
    d = blk[:, :2].copy().view("<f2").astype(np.float32)
    m = blk[:, 2:4].copy().view("<f2").astype(np.float32)
    q = blk[:, 4:]
    vals = np.concatenate([(q & 0xF), (q >> 4)], axis=1).astype(np.float32)
    return (vals * d + m).reshape(-1)[:n]


def _dequant_q8_0(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 34)
    d = blk[:, :2].copy().view("<f2").astype(np.float32)
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    return (q * d).reshape(-1)[:n]


def read_gguf(path: str) -> tuple[dict, dict]:
    """Returns (tensors, metadata). GGUF versions 1-3."""
    with open(path, "rb") as f:
        data = f.read()
    c = _Cursor(data)
    magic, version = c.take("I"), c.take("I")
    if magic != GGUF_MAGIC:
        raise ValueError(f"{path}: not a GGUF file")
    v1 = version == 1
    n_tensors = c.take("I" if v1 else "Q")
    n_kv = c.take("I" if v1 else "Q")
    meta = {}
    for _ in range(n_kv):
        k = c.string(v1)
        t = c.take("I")
        meta[k] = c.skip_value(t, v1)
    infos = []
    for _ in range(n_tensors):
        name = c.string(v1)
        nd = c.take("I")
        dims = [c.take("I" if v1 else "Q") for _ in range(nd)]
        typ = c.take("I")
        off = c.take("Q")
        infos.append((name, dims, typ, off))
    align = int(meta.get("general.alignment", 32))
    base = (c.o + align - 1) // align * align
    sizes = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20), GGML_Q8_0: (32, 34)}
    out = {}
    for name, dims, typ, off in infos:
        n = int(np.prod(dims)) if dims else 1
        if typ not in sizes:
            continue
        per, nb = sizes[typ]
        nbytes = (n + per - 1) // per * nb
        raw = np.frombuffer(data, dtype=np.uint8, count=nbytes, offset=base + off)
        if typ == GGML_F32:
            a = raw.view("<f4").astype(np.float32)
        elif typ == GGML_F16:
            a = raw.view("<f2").astype(np.float32)
        elif typ == GGML_Q4_0:
            a = _dequant_q4_0(raw, n)
        elif typ == GGML_Q4_1:
            a = _dequant_q4_1(raw, n)
        else:
            a = _dequant_q8_0(raw, n)
        out[name] = a[:n].reshape(list(reversed(dims))) if dims else a[:n]
    return out, meta
