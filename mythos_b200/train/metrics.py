"""Training logs: TensorBoard-framed event files and JSONL (reference: src/log_writer.cpp).

``EventWriter`` writes TFRecord framing — ``u64 length, u32 masked_crc32c(length), payload, u32
masked_crc32c(payload)`` — around real ``Event`` protobufs with one ``Summary.Value{tag,
simple_value}`` (the reference writes a ``"tag\\nvalue"`` text payload that TensorBoard cannot
parse; the framing and file naming are the same). ``JsonlLogger`` is the reference's
``WandBLogger``: one JSON object per line under ``wandb/<project>/<run>/metrics.json``.
"""
from __future__ import annotations

import json
import os
import struct
import time

_CRC_TABLE = []


def _crc32c(data: bytes) -> int:
    if not _CRC_TABLE:
        for i in range(256):
            crc = i
            for _ in range(8):
                crc = (crc >> 1) ^ (0x82F63B78 if crc & 1 else 0)
            _CRC_TABLE.append(crc)
    crc = 0xFFFFFFFF
    for b in data:
        crc = (crc >> 8) ^ _CRC_TABLE[(crc ^ b) & 0xFF]
    return crc ^ 0xFFFFFFFF


def masked_crc32c(data: bytes) -> int:
    crc = _crc32c(data)
    return (((crc >> 15) | (crc << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _event_proto(wall_time: float, step: int, tag: str, value: float) -> bytes:
    tagb = tag.encode("utf-8")
    val = b"\x0a" + _varint(len(tagb)) + tagb + b"\x15" + struct.pack("<f", value)      # Summary.Value
    summary = b"\x0a" + _varint(len(val)) + val                                          # Summary
    return (b"\x09" + struct.pack("<d", wall_time) + b"\x10" + _varint(step) +           # Event
            b"\x2a" + _varint(len(summary)) + summary)


class EventWriter:
    def __init__(self, logdir: str):
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, f"events.out.tfevents.{int(time.time())}.localhost")
        self._f = open(self.path, "wb")
        self._record(b"\x09" + struct.pack("<d", time.time()) + b"\x1a\x0dbrain.Event:2")  # file_version

    def _record(self, payload: bytes) -> None:
        head = struct.pack("<Q", len(payload))
        self._f.write(head + struct.pack("<I", masked_crc32c(head)) + payload +
                      struct.pack("<I", masked_crc32c(payload)))

    def write_event(self, tag: str, value: float, step: int, wall_time: float | None = None) -> None:
        self._record(_event_proto(wall_time if wall_time is not None else time.time(), step, tag, float(value)))

    def write_metrics(self, metrics, step: int | None = None) -> None:
        d = metrics if isinstance(metrics, dict) else vars(metrics)
        step = int(d.get("step", 0)) if step is None else step
        for k, v in d.items():
            if isinstance(v, (int, float)) and k not in ("step", "epoch"):
                self.write_event(k, v, step)

    def flush(self) -> None:
        self._f.flush()

    def close(self) -> None:
        self._f.close()


def read_events(path: str):
    """Yields the raw payloads of an event file after checking both CRCs of every record."""
    with open(path, "rb") as f:
        data = f.read()
    off = 0
    while off + 12 <= len(data):
        (n,) = struct.unpack_from("<Q", data, off)
        (c1,) = struct.unpack_from("<I", data, off + 8)
        if masked_crc32c(data[off:off + 8]) != c1:
            raise ValueError("length CRC mismatch")
        payload = data[off + 12:off + 12 + n]
        (c2,) = struct.unpack_from("<I", data, off + 12 + n)
        if masked_crc32c(payload) != c2:
            raise ValueError("payload CRC mismatch")
        yield payload
        off += 16 + n


class JsonlLogger:
    def __init__(self, project: str, run: str, root: str = "wandb"):
        d = os.path.join(root, project, run)
        os.makedirs(d, exist_ok=True)
        self.path = os.path.join(d, "metrics.json")
        self._f = open(self.path, "a")

    def log(self, metrics, step: int | None = None) -> None:
        d = dict(metrics if isinstance(metrics, dict) else vars(metrics))
        if step is not None:
            d["step"] = step
        d["_timestamp"] = time.time()
        self._f.write(json.dumps(d) + "\n")
        self._f.flush()

    def close(self) -> None:
        self._f.close()


# The reference calls its JSONL writer ``WandBLogger`` (src/log_writer.cpp:88-121): same file
# layout, ``wandb/<project>/<run>/metrics.json``, nothing is sent anywhere.
WandBLogger = JsonlLogger
