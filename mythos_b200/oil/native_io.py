"""ctypes front end of the C++ host runtime (``liboil_host.so``, built from ``csrc/host``): mmap
container reader with dequantisation, streaming writer, SHA-256, sidecar check, BPE, RNG and page
allocator. The pure-Python modules (`container.py`, `train/bpe.py`) define the behaviour; these
native twins are used for large files and corpora, and the tests check that both agree."""
from __future__ import annotations

import ctypes
import os

import numpy as np

_lib = None


def lib():
    global _lib
    if _lib is None:
        # MYTHOS_HOST_LIB points at another build of the same library (the sanitizer build in the tests)
        path = os.environ.get("MYTHOS_HOST_LIB") or os.path.join(
            os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "liboil_host.so")
        if not os.path.exists(path):
            raise RuntimeError("liboil_host.so is not built; run `python -m mythos_b200.build`")
        L = ctypes.CDLL(path)
        vp, cp, u8p = ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint8)
        L.oil_last_error.restype = cp
        L.oil_sha256.argtypes = [vp, ctypes.c_size_t, vp]
        L.oil_sha256_file.argtypes = [cp, vp]
        L.oil_open.restype = vp
        L.oil_open.argtypes = [cp]
        L.oil_close.argtypes = [vp]
        for n in ("oil_version", "oil_config_size", "oil_num_tensors", "oil_num_blocks"):
            getattr(L, n).restype = ctypes.c_uint32
            getattr(L, n).argtypes = [vp]
        L.oil_config.restype = vp
        L.oil_config.argtypes = [vp]
        L.oil_tensor_name.restype = cp
        L.oil_tensor_name.argtypes = [vp, ctypes.c_uint32]
        L.oil_tensor_numel.restype = ctypes.c_int64
        L.oil_tensor_numel.argtypes = [vp, cp]
        L.oil_read_tensor_f32.restype = ctypes.c_int64
        L.oil_read_tensor_f32.argtypes = [vp, cp, vp, ctypes.c_int64]
        L.oil_tensor_sha256.argtypes = [vp, cp, vp]
        L.oil_writer_create.restype = vp
        L.oil_writer_create.argtypes = [cp, vp, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]
        L.oil_writer_add_tensor.argtypes = [vp, cp]
        L.oil_writer_add_block.argtypes = [vp, ctypes.c_uint8, ctypes.c_uint32, vp, ctypes.c_uint32, vp, ctypes.c_uint32]
        L.oil_writer_finish.argtypes = [vp]
        L.oil_idx_check.argtypes = [cp, ctypes.c_char_p, ctypes.c_size_t]
        L.oil_bpe_train.restype = vp
        L.oil_bpe_train.argtypes = [vp, ctypes.c_size_t, ctypes.c_int]
        L.oil_bpe_load.restype = vp
        L.oil_bpe_load.argtypes = [cp]
        L.oil_bpe_save.argtypes = [vp, cp]
        L.oil_bpe_free.argtypes = [vp]
        L.oil_bpe_vocab_size.argtypes = [vp]
        L.oil_bpe_encode.restype = ctypes.c_int64
        L.oil_bpe_encode.argtypes = [vp, vp, ctypes.c_size_t, vp, ctypes.c_int64]
        L.oil_bpe_decode.restype = ctypes.c_int64
        L.oil_bpe_decode.argtypes = [vp, vp, ctypes.c_int64, vp, ctypes.c_int64]
        L.oil_rng_create.restype = vp
        L.oil_rng_create.argtypes = [ctypes.c_uint64]
        L.oil_rng_free.argtypes = [vp]
        L.oil_rng_next.restype = ctypes.c_uint64
        L.oil_rng_next.argtypes = [vp]
        L.oil_rng_uniform.restype = ctypes.c_double
        L.oil_rng_uniform.argtypes = [vp]
        L.oil_rng_normal.restype = ctypes.c_double
        L.oil_rng_normal.argtypes = [vp]
        L.oil_rng_fill_uniform.argtypes = [vp, vp, ctypes.c_int64, ctypes.c_float, ctypes.c_float]
        L.oil_pages_create.restype = vp
        L.oil_pages_create.argtypes = [ctypes.c_int32]
        L.oil_pages_free.argtypes = [vp]
        L.oil_pages_alloc.argtypes = [vp]
        L.oil_pages_retain.argtypes = [vp, ctypes.c_int32]
        L.oil_pages_release.argtypes = [vp, ctypes.c_int32]
        L.oil_pages_used.argtypes = [vp]
        L.oil_loader_create.restype = vp
        L.oil_loader_create.argtypes = [vp, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint64,
                                        ctypes.c_int]
        L.oil_loader_num_batches.restype = ctypes.c_int64
        L.oil_loader_num_batches.argtypes = [vp]
        L.oil_loader_reset.argtypes = [vp, ctypes.c_int]
        L.oil_loader_next.argtypes = [vp, vp, vp]
        L.oil_loader_free.argtypes = [vp]
        _lib = L
    return _lib


def available() -> bool:
    try:
        lib()
        return True
    except (RuntimeError, OSError, AttributeError):     # missing, unloadable, or an older build of the library
        return False


def sha256(data: bytes) -> bytes:
    out = ctypes.create_string_buffer(32)
    lib().oil_sha256(data, len(data), out)
    return out.raw


def sha256_file(path: str) -> str:
    out = ctypes.create_string_buffer(32)
    if lib().oil_sha256_file(path.encode(), out) != 0:
        raise OSError(lib().oil_last_error().decode())
    return out.raw.hex()


class NativeReader:
    def __init__(self, path: str):
        self._h = lib().oil_open(path.encode())
        if not self._h:
            from .container import OILError

            raise OILError(lib().oil_last_error().decode())

    def close(self):
        if self._h:
            lib().oil_close(self._h)
            self._h = None

    def __del__(self):
        self.close()

    @property
    def config(self) -> bytes:
        n = lib().oil_config_size(self._h)
        return ctypes.string_at(lib().oil_config(self._h), n) if n else b""

    def tensor_names(self):
        return [lib().oil_tensor_name(self._h, i).decode() for i in range(lib().oil_num_tensors(self._h))]

    def num_blocks(self) -> int:
        return lib().oil_num_blocks(self._h)

    def read_tensor(self, name: str) -> np.ndarray:
        n = lib().oil_tensor_numel(self._h, name.encode())
        if n < 0:
            return np.zeros(0, dtype=np.float32)
        out = np.empty(n, dtype=np.float32)
        got = lib().oil_read_tensor_f32(self._h, name.encode(), out.ctypes.data, n)
        if got < 0:
            from .container import OILError

            raise OILError(lib().oil_last_error().decode())
        return out

    def tensor_sha256(self, name: str) -> bytes:
        out = ctypes.create_string_buffer(32)
        if lib().oil_tensor_sha256(self._h, name.encode(), out) != 0:
            from .container import OILError

            raise OILError(lib().oil_last_error().decode())
        return out.raw


def write_oil_native(path: str, tensors, config: bytes = b"", version: int = 1, flags: int = 0) -> None:
    """Same file as ``container.write_oil(..., write_idx=False)``. tensors: [(name, [BlockData])]."""
    L = lib()
    w = L.oil_writer_create(path.encode(), config, len(config), version, flags)
    for name, blocks in tensors:
        L.oil_writer_add_tensor(w, name.encode())
        for b in blocks:
            L.oil_writer_add_block(w, int(b.format), b.num_weights, b.codebook, len(b.codebook), b.indices,
                                   len(b.indices))
    if L.oil_writer_finish(w) != 0:
        raise OSError(L.oil_last_error().decode())


def idx_check(path: str) -> int:
    """Number of tensors in a valid sidecar; raises OILError naming the corrupt tensor otherwise."""
    from .container import OILError

    buf = ctypes.create_string_buffer(512)
    rc = lib().oil_idx_check(path.encode(), buf, 512)
    if rc < 0:
        name = buf.value.decode(errors="replace")
        raise OILError(f"OILIdxReader: corrupt idx - {lib().oil_last_error().decode()}" +
                       (f' for tensor "{name}"' if name else ""))
    return rc


class NativeBPE:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def train(cls, text: bytes, vocab_size: int) -> "NativeBPE":
        return cls(lib().oil_bpe_train(text, len(text), vocab_size))

    @classmethod
    def load(cls, path: str) -> "NativeBPE":
        h = lib().oil_bpe_load(path.encode())
        if not h:
            raise OSError(f"cannot load {path}")
        return cls(h)

    def save(self, path: str) -> None:
        lib().oil_bpe_save(self._h, path.encode())

    @property
    def vocab_size(self) -> int:
        return lib().oil_bpe_vocab_size(self._h)

    def encode(self, text: bytes) -> list[int]:
        out = np.empty(max(1, len(text)), dtype=np.int32)
        n = lib().oil_bpe_encode(self._h, text, len(text), out.ctypes.data, out.size)
        return out[:n].tolist()

    def decode(self, ids) -> bytes:
        a = np.asarray(ids, dtype=np.int32)
        cap = 64 * max(1, a.size)
        out = ctypes.create_string_buffer(cap)
        n = lib().oil_bpe_decode(self._h, a.ctypes.data, a.size, out, cap)
        return out.raw[:max(0, n)]

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oil_bpe_free(self._h)
            self._h = None


class NativeRNG:
    """splitmix64-seeded xoroshiro128+; 53-bit uniforms; Box-Muller normals."""

    def __init__(self, seed: int):
        self._h = lib().oil_rng_create(seed)

    def next_u64(self) -> int:
        return lib().oil_rng_next(self._h)

    def uniform(self) -> float:
        return lib().oil_rng_uniform(self._h)

    def normal(self) -> float:
        return lib().oil_rng_normal(self._h)

    def fill_uniform(self, n: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().oil_rng_fill_uniform(self._h, out.ctypes.data, n, lo, hi)
        return out

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oil_rng_free(self._h)
            self._h = None


class NativePageAllocator:
    def __init__(self, num_pages: int):
        self._h = lib().oil_pages_create(num_pages)
        self.num_pages = num_pages

    def alloc(self) -> int:
        p = lib().oil_pages_alloc(self._h)
        if p < 0:
            raise MemoryError("KV cache is out of pages")
        return p

    def retain(self, p: int) -> None:
        lib().oil_pages_retain(self._h, p)

    def release(self, p: int) -> None:
        lib().oil_pages_release(self._h, p)

    @property
    def used(self) -> int:
        return lib().oil_pages_used(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oil_pages_free(self._h)
            self._h = None


class NativeTokenLoader:
    """``TokenDataset`` served by the C++ loader: a worker thread assembles ``[B, S]`` batches into a
    ring while the training step runs; iteration copies a finished batch straight into (optionally
    pinned) torch tensors. Window-level shuffle, deterministic in (seed, epoch); the permutation is
    the runtime's own, not numpy's."""

    def __init__(self, tokens, batch: int, seq: int, shuffle: bool = True, seed: int = 42, prefetch: int = 2,
                 pin: bool = False):
        import torch

        arr = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        self.batch, self.seq = batch, seq
        self._h = lib().oil_loader_create(arr.ctypes.data, arr.size, batch, seq, 1 if shuffle else 0, seed, prefetch)
        if not self._h:
            raise ValueError("NativeTokenLoader: need at least two tokens and positive batch / sequence sizes")
        self.pin = bool(pin and torch.cuda.is_available())

    def __len__(self) -> int:
        return int(lib().oil_loader_num_batches(self._h))

    def reset(self, epoch: int = 0) -> None:
        lib().oil_loader_reset(self._h, epoch)

    def __iter__(self):
        import torch

        while True:
            ids = torch.empty(self.batch, self.seq, dtype=torch.int32, pin_memory=self.pin)
            tgt = torch.empty(self.batch, self.seq, dtype=torch.int32, pin_memory=self.pin)
            if not lib().oil_loader_next(self._h, ids.data_ptr(), tgt.data_ptr()):
                return
            yield ids, tgt

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().oil_loader_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

