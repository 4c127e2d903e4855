"""Training checkpoints: ``<path>`` (the model as ``.oil``) + ``<path>.opt`` (optimizer state) +
``<path>.master`` (fp32 master weights of the quantised layers).

``.opt`` keeps the reference's layout (src/trainer.cpp:632-664) so its tools can read the common
prefix: ``i32 step, f32 lr, i32 num_params`` then per parameter ``i64 n_m, m[n_m] f32, i64 n_v,
v[n_v] f32``. A trailer the reference ignores follows: magic ``"MB2\\0"``, u32 JSON length, JSON with
what the reference forgets (optimizer step for bias correction, epoch, RNG state, parameter
names). State is stored per parameter, not per rank, so a checkpoint written at one data-parallel
size loads at any other: each rank reads the slices that overlap its shard.

The ``.oil`` file holds quantised layers in their storage format (OIL8 / OIL4 indices, I2_S trits),
which is what inference needs but not what straight-through training continues from: the fp32
master weight carries the sub-step updates that have not yet moved a weight to another centroid.
``.master`` therefore stores the fp32 master of every parameter whose layer uses a lossy format
(magic ``"MBM1"``, u32 count, then ``u16 name length, name, i64 numel, f32 data`` per parameter);
``load_training_state`` puts it back, so a resumed run follows the trajectory of an uninterrupted
one. A checkpoint without the file (written by an older version or by the reference) still loads,
with the masters at their dequantised values.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

from ..oil import model_io

TRAILER_MAGIC = b"MB2\x00"
MASTER_MAGIC = b"MBM1"
LOSSY_FORMATS = ("oil8", "oil4", "i2s", "fp16")


def _lossy_slots(store):
    return [s for s in store.slots if s.module is not None and getattr(s.module, "fmt", "fp32") in LOSSY_FORMATS]


def write_master_file(path: str, store) -> None:
    slots = _lossy_slots(store)
    with open(path, "wb") as f:
        f.write(MASTER_MAGIC + struct.pack("<I", len(slots)))
        for s in slots:
            name = s.name.encode("utf-8")
            a = store.master[s.offset:s.offset + s.numel].detach().cpu().numpy().astype("<f4")
            f.write(struct.pack("<H", len(name)) + name + struct.pack("<q", a.size))
            f.write(a.tobytes())


def read_master_file(path: str) -> dict:
    """{parameter name: flat fp32 numpy array}; raises ValueError on a malformed file."""
    with open(path, "rb") as f:
        data = f.read()
    if data[:4] != MASTER_MAGIC or len(data) < 8:
        raise ValueError(f"{path}: not a master-weight file")
    (n,) = struct.unpack_from("<I", data, 4)
    off, out = 8, {}
    for _ in range(n):
        if off + 2 > len(data):
            raise ValueError(f"{path}: truncated")
        (ln,) = struct.unpack_from("<H", data, off)
        off += 2
        if off + ln + 8 > len(data):
            raise ValueError(f"{path}: truncated")
        name = data[off:off + ln].decode("utf-8")
        off += ln
        (cnt,) = struct.unpack_from("<q", data, off)
        off += 8
        if cnt < 0 or off + 4 * cnt > len(data):
            raise ValueError(f"{path}: truncated in {name}")
        out[name] = np.frombuffer(data, dtype="<f4", count=cnt, offset=off)
        off += 4 * cnt
    return out


def _full_moments(trainer):
    """(m, v) as full-length fp32 tensors on the host (gathered across data-parallel ranks)."""
    st = trainer.store
    if trainer.dp is None:
        return trainer.m.detach().cpu(), trainer.v.detach().cpu()
    import torch.distributed as dist

    out = []
    for t in (trainer.m, trainer.v):
        full = torch.empty(st.total, device=t.device, dtype=torch.float32)
        dist.all_gather_into_tensor(full, t.contiguous(), group=trainer.dp.group)
        out.append(full.cpu())
    return out[0], out[1]


def save_training_state(trainer, path: str) -> None:
    if trainer.dp is not None:
        trainer.dp.gather_master()
    m, v = _full_moments(trainer)
    rank = trainer.dp.rank if trainer.dp is not None else 0
    if rank != 0:
        return
    model_io.save_model(trainer.model, path)
    st = trainer.store
    write_master_file(path + ".master", st)
    with open(path + ".opt", "wb") as f:
        f.write(struct.pack("<ifi", trainer.step, float(trainer.current_lr()), len(st.slots)))
        for s in st.slots:
            for t in (m, v):
                a = t[s.offset:s.offset + s.numel].numpy().astype("<f4")
                f.write(struct.pack("<q", a.size))
                f.write(a.tobytes())
        meta = {"step": trainer.step, "epoch": trainer.epoch, "names": [s.name for s in st.slots],
                "torch_rng": torch.get_rng_state().numpy().tobytes().hex()}
        blob = json.dumps(meta).encode("utf-8")
        f.write(TRAILER_MAGIC + struct.pack("<I", len(blob)) + blob)


def read_opt_file(path: str):
    """Returns (step, lr, [(m, v) numpy arrays per parameter], meta dict)."""
    with open(path, "rb") as f:
        data = f.read()
    step, lr, n = struct.unpack_from("<ifi", data, 0)
    off = 12
    moments = []
    for _ in range(n):
        pair = []
        for _k in range(2):
            (cnt,) = struct.unpack_from("<q", data, off)
            off += 8
            pair.append(np.frombuffer(data, dtype="<f4", count=cnt, offset=off))
            off += 4 * cnt
        moments.append(tuple(pair))
    meta = {}
    if data[off:off + 4] == TRAILER_MAGIC:
        (ln,) = struct.unpack_from("<I", data, off + 4)
        meta = json.loads(data[off + 8:off + 8 + ln].decode("utf-8"))
    return step, lr, moments, meta


def load_training_state(trainer, path: str) -> None:
    """Restores weights (from the ``.oil``), Adam moments, step and epoch into an existing trainer
    whose model has the same architecture; works across data-parallel sizes."""
    loaded, _ = model_io.load_model(path, device="cpu", model_cls=type(trainer.model))
    st = trainer.store
    src = dict(loaded.named_parameters())
    src_mods = dict(loaded.named_modules())
    with torch.no_grad():
        for s in st.slots:
            if s.name in src:
                st.master[s.offset:s.offset + s.numel].copy_(src[s.name].detach().reshape(-1).to(st.device))
        for name, mod in trainer.model.named_modules():
            cb = getattr(mod, "codebooks", None)
            other = getattr(src_mods.get(name), "codebooks", None)
            if cb is not None and other is not None:
                cb.copy_(other.to(cb.device))
    if os.path.exists(path + ".master"):
        masters = read_master_file(path + ".master")
        with torch.no_grad():
            for s in st.slots:
                a = masters.get(s.name)
                if a is not None and a.size == s.numel:
                    st.master[s.offset:s.offset + s.numel].copy_(torch.from_numpy(a.copy()).to(st.device))
    step, _, moments, meta = read_opt_file(path + ".opt")
    lo = (trainer.dp.rank if trainer.dp is not None else 0) * st.shard
    hi = lo + st.shard
    trainer.m.zero_()
    trainer.v.zero_()
    for s, (m, v) in zip(st.slots, moments):
        a, b = max(lo, s.offset), min(hi, s.offset + s.numel)
        if a >= b or m.size != s.numel:
            continue
        trainer.m[a - lo:b - lo].copy_(torch.from_numpy(m[a - s.offset:b - s.offset].copy()))
        trainer.v[a - lo:b - lo].copy_(torch.from_numpy(v[a - s.offset:b - s.offset].copy()))
    trainer.step = int(meta.get("step", step))
    trainer.epoch = int(meta.get("epoch", 0))
    trainer._stale = True
    trainer._force_refresh = True
