"""Core types, host buffers / pool and the tensor wire format."""
import struct

import numpy as np
import pytest
import torch

from mythos_b200 import core
from mythos_b200.oil.formats import Format


def test_types_status_shape_and_config():
    assert [int(d) for d in core.DType] == list(range(7)) and core.DType.F32 == 6
    assert core.format_to_dtype(Format.TERNARY) == core.DType.I2 and core.format_to_dtype(Format.OIL4) == core.DType.U4
    assert core.format_to_dtype(99) == core.DType.F32
    assert core.packed_nbytes(core.DType.I2, 9) == 3 and core.packed_nbytes(core.DType.U4, 3) == 2
    assert core.packed_nbytes(core.DType.I1, 8) == 1 and core.packed_nbytes(core.DType.F16, 3) == 6
    assert core.Status.success() and not core.Status.error("bad") and core.Status.error("bad").msg == "bad"
    with pytest.raises(core.OilError, match="nope"):
        core.check(False, "nope")
    core.check(True, "fine")
    s = core.Shape(2, 3, 4)
    assert s.rank == 3 and s.numel() == 24 and str(s) == "[2, 3, 4]" and core.Shape([5]).numel() == 5
    assert core.Shape().numel() == 1
    with pytest.raises(core.OilError):
        core.Shape(*range(1, 10))
    with pytest.raises(core.OilError):
        core.Shape(2, -1)
    cfg = core.Config.from_environ({"OIL_NUM_THREADS": "6", "OIL_SEED": "9", "OIL_VERBOSE": "1"})
    assert (cfg.num_threads, cfg.seed, cfg.verbose, cfg.pool_size) == (6, 9, True, 64 << 20)
    assert core.Config().num_threads == 1


def test_aligned_buffer_slices_and_pool():
    b = core.Buffer(1000)
    assert b.address % 64 == 0 and b.nbytes == 1000 and b.refcount == 1
    s = b.slice(128, 256)
    assert s.address == b.address + 128 and s.nbytes == 256 and b.refcount == 2
    s.as_array(np.float32)[:] = 1.5
    assert float(b.as_array(np.float32)[32]) == 1.5 and float(b.as_array(np.float32, 4).size) == 4
    assert s.slice(0, 8).refcount == 3
    with pytest.raises(core.OilError):
        b.slice(900, 200)
    assert b.release() == 2 and b.retain().refcount == 3
    pool = core.MemoryPool(4096)
    a = pool.alloc(100)
    c = pool.alloc_array((10, 4), np.float32)
    assert a.ctypes.data % 64 == 0 and c.ctypes.data % 64 == 0 and c.shape == (10, 4)
    assert pool.used == 128 + 160 and pool.peak == pool.used
    with pytest.raises(core.OilError, match="exhausted"):
        pool.alloc(4096)
    pool.reset()
    assert pool.used == 0 and pool.alloc(4096).nbytes == 4096 and pool.peak == 4096


def test_tensor_wire_format_matches_the_reference_layout():
    t = torch.arange(6, dtype=torch.float32).view(2, 3)
    raw = core.serialize_tensor(t)
    assert raw[:4] == struct.pack("<i", 2) and raw[4:20] == struct.pack("<2q", 2, 3) and raw[20] == int(core.DType.F32)
    assert raw[21:] == t.numpy().tobytes() and len(raw) == 21 + 24
    parts = [t, torch.tensor([1, 2, 3], dtype=torch.int64), torch.tensor(2.5, dtype=torch.float16),
             torch.zeros(0, 4), torch.tensor([1.5, -2.0], dtype=torch.bfloat16)]
    blob = b"".join(core.serialize_tensor(p) for p in parts)
    off, got = 0, []
    for _ in parts:
        x, off = core.deserialize_tensor(blob, off)
        got.append(x)
    assert off == len(blob)
    assert torch.equal(got[0], t) and torch.equal(got[1], parts[1]) and got[2].dtype == torch.float16 and got[2].dim() == 0
    assert got[3].shape == (0, 4) and got[4].dtype == torch.float32 and torch.equal(got[4], parts[4].float())
    with pytest.raises(core.OilError, match="truncated"):
        core.deserialize_tensor(raw[:-3])
    with pytest.raises(core.OilError):
        core.deserialize_tensor(struct.pack("<i", 40))
