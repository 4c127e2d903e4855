"""Training checkpoints: ``<path>`` (the model as ``.oil``) + ``<path>.opt`` (optimizer state).

``.opt`` keeps the reference's layout (src/trainer.cpp:632-664) so its tools can read the common
prefix: ``i32 step, f32 lr, i32 num_params`` then per parameter ``i64 n_m, m[n_m] f32, i64 n_v,
v[n_v] f32``. A trailer the reference ignores follows: magic ``"MB2\\0"``, u32 JSON length, JSON with
what the reference forgets (optimizer step for bias correction, epoch, RNG state, parameter
names). State is stored per parameter, not per rank, so a checkpoint written at one data-parallel
size loads at any other: each rank reads the slices that overlap its shard.
"""
from __future__ import annotations

import json
import struct

import numpy as np
import torch

from ..oil import model_io

TRAILER_MAGIC = b"MB2\x00"


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
