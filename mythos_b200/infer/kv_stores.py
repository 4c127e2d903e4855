"""Stand-alone KV stores beside the engine's paged cache: a contiguous per-layer cache with an
optional int8 block mode, and a sparse very-long-context store with a three-level page table and
least-recently-used spill of pages to disk.

Reference counterparts: ``KVCache`` (contiguous ``[1, H, max_seq, D]`` per layer; "FP8" mode is int8
abs-max per 64-value block, ``FP8_BLOCK_SIZE = 64``, ``FP8_MAX = 127``; append / get_range / get_all
/ clear / resize / size_bytes; src/kv_cache.cpp:13-238) and ``PagedKVCache1T`` (three-level table
with 4096 entries per level and 16-token blocks, i.e. 2^40+ addressable tokens; physical blocks
``[block, heads, head_dim]`` in a map; LRU eviction to ``paged_kv_l{L}_b{id}.bin`` files, reload on
access, ``flush_to_disk``, ``verify_retrieval``; src/kv_cache.cpp:244-642). The reference sizes the
generator's cache with ``num_heads`` instead of ``num_kv_heads`` and ignores the batch index in
the key/value base address; neither is reproduced. The decode path of the engine uses
``infer/kv_paged.py`` (device pages + block tables consumed by the attention kernels).
"""
from __future__ import annotations

import os
import tempfile
from collections import OrderedDict

import torch

from .kv_paged import dequantize_kv_int8, quantize_kv_int8

INT8_BLOCK = 64


class KVCache:
    def __init__(self, num_layers: int, max_seq_len: int, kv_heads: int, head_dim: int, device="cpu",
                 dtype=torch.float32, int8: bool = False, batch: int = 1):
        self.L, self.max_seq, self.H, self.D, self.B = num_layers, max_seq_len, kv_heads, head_dim, batch
        self.device, self.dtype, self.int8 = torch.device(device), dtype, int8
        self.len = 0
        self._alloc()

    def _alloc(self):
        shape = (self.L, self.B, self.H, self.max_seq, self.D)
        if self.int8:
            if self.D % INT8_BLOCK and INT8_BLOCK % self.D:
                raise ValueError("head_dim must divide or be a multiple of the 64-value quantisation block")
            self.k = torch.zeros(shape, dtype=torch.int8, device=self.device)
            self.v = torch.zeros(shape, dtype=torch.int8, device=self.device)
            nblk = max(1, self.D // INT8_BLOCK)
            self.k_scale = torch.zeros(shape[:-1] + (nblk,), dtype=torch.float32, device=self.device)
            self.v_scale = torch.zeros_like(self.k_scale)
        else:
            self.k = torch.zeros(shape, dtype=self.dtype, device=self.device)
            self.v = torch.zeros(shape, dtype=self.dtype, device=self.device)

    def context_len(self) -> int:
        return self.len

    def _store(self, buf, scale, layer, pos, x):
        """x: [B, H, T, D]."""
        T = x.shape[2]
        if not self.int8:
            buf[layer, :, :, pos:pos + T] = x.to(buf.dtype)
            return
        blk = min(INT8_BLOCK, self.D)
        q, s = quantize_kv_int8(x.reshape(-1), blk)
        buf[layer, :, :, pos:pos + T] = q.view(x.shape)
        scale[layer, :, :, pos:pos + T] = s.view(*x.shape[:-1], -1)

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, advance: bool | None = None) -> None:
        """k, v: [B, H, T, D] for positions [len, len + T). The length advances after the last layer
        (or when ``advance`` is given explicitly)."""
        T = k.shape[2]
        if self.len + T > self.max_seq:
            raise ValueError(f"KV cache overflow: {self.len} + {T} > {self.max_seq}")
        self._store(self.k, getattr(self, "k_scale", None), layer, self.len, k)
        self._store(self.v, getattr(self, "v_scale", None), layer, self.len, v)
        if advance if advance is not None else layer == self.L - 1:
            self.len += T

    def _load(self, buf, scale, layer, a, b):
        if not self.int8:
            return buf[layer, :, :, a:b]
        q = buf[layer, :, :, a:b]
        blk = min(INT8_BLOCK, self.D)
        return dequantize_kv_int8(q.reshape(-1), scale[layer, :, :, a:b].reshape(-1), blk).view(q.shape)

    def get_range(self, layer: int, start: int, end: int):
        return (self._load(self.k, getattr(self, "k_scale", None), layer, start, end),
                self._load(self.v, getattr(self, "v_scale", None), layer, start, end))

    def get_all(self, layer: int, upto: int | None = None):
        return self.get_range(layer, 0, self.len if upto is None else upto)

    def clear(self) -> None:
        self.len = 0

    def resize(self, new_max: int) -> None:
        old_k, old_v = self.k, self.v
        old_s = (self.k_scale, self.v_scale) if self.int8 else None
        keep = min(self.len, new_max)
        self.max_seq = new_max
        self._alloc()
        self.k[..., :keep, :] = old_k[..., :keep, :]
        self.v[..., :keep, :] = old_v[..., :keep, :]
        if old_s is not None:
            self.k_scale[..., :keep, :] = old_s[0][..., :keep, :]
            self.v_scale[..., :keep, :] = old_s[1][..., :keep, :]
        self.len = keep

    def size_bytes(self) -> int:
        n = self.k.numel() * self.k.element_size() * 2
        if self.int8:
            n += self.k_scale.numel() * 4 * 2
        return n


class PagedKVCache1T:
    """Sparse KV store addressed by absolute token position. A three-level radix table
    (``fanout`` entries per level) maps a logical block number to a physical block; blocks hold
    ``block_size`` tokens of ``[heads, head_dim]`` for K and V. At most ``max_resident`` blocks stay
    in memory; the least recently used one is written to ``spill_dir`` and reloaded on access."""

    def __init__(self, num_layers: int, kv_heads: int, head_dim: int, block_size: int = 16, fanout: int = 4096,
                 max_resident: int = 1024, spill_dir: str | None = None, device="cpu", dtype=torch.float32):
        self.L, self.H, self.D, self.bs, self.fanout = num_layers, kv_heads, head_dim, block_size, fanout
        self.max_resident = max_resident
        self.device, self.dtype = torch.device(device), dtype
        self.spill_dir = spill_dir or tempfile.mkdtemp(prefix="mythos_paged_kv_")
        os.makedirs(self.spill_dir, exist_ok=True)
        self.root: list = [dict() for _ in range(num_layers)]      # level 1 -> level 2 -> level 3 -> block id
        self.resident: OrderedDict = OrderedDict()                 # (layer, id) -> [K, V] tensors, LRU order
        self.on_disk: set = set()
        self.next_id = 0
        self.max_pos = [0] * num_layers
        self.stats = {"evictions": 0, "reloads": 0}

    def capacity_tokens(self) -> int:
        return self.fanout ** 3 * self.bs

    def _indices(self, block_no: int):
        f = self.fanout
        return block_no // (f * f), (block_no // f) % f, block_no % f

    def _lookup(self, layer: int, block_no: int, create: bool):
        i, j, k = self._indices(block_no)
        if i >= self.fanout:
            raise ValueError("position beyond the addressable range")
        l2 = self.root[layer].get(i)
        if l2 is None:
            if not create:
                return None
            l2 = self.root[layer][i] = {}
        l3 = l2.get(j)
        if l3 is None:
            if not create:
                return None
            l3 = l2[j] = {}
        bid = l3.get(k)
        if bid is None and create:
            bid = l3[k] = self.next_id
            self.next_id += 1
            self._install(layer, bid, [torch.zeros(self.bs, self.H, self.D, dtype=self.dtype, device=self.device)
                                       for _ in range(2)])
        return bid

    def _path(self, layer: int, bid: int) -> str:
        return os.path.join(self.spill_dir, f"paged_kv_l{layer}_b{bid}.bin")

    def _install(self, layer, bid, kv):
        self.resident[(layer, bid)] = kv
        self.resident.move_to_end((layer, bid))
        while len(self.resident) > self.max_resident:
            (el, eb), ekv = self.resident.popitem(last=False)
            torch.save([t.cpu() for t in ekv], self._path(el, eb))
            self.on_disk.add((el, eb))
            self.stats["evictions"] += 1

    def get_block(self, layer: int, bid: int):
        key = (layer, bid)
        kv = self.resident.get(key)
        if kv is not None:
            self.resident.move_to_end(key)
            return kv
        if key not in self.on_disk:
            raise KeyError(f"block {bid} of layer {layer} does not exist")
        kv = [t.to(self.device) for t in torch.load(self._path(layer, bid))]
        self.on_disk.discard(key)
        self.stats["reloads"] += 1
        self._install(layer, bid, kv)
        return kv

    def append(self, layer: int, pos: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v: [heads, head_dim] of the token at absolute position ``pos``."""
        bid = self._lookup(layer, pos // self.bs, create=True)
        kv = self.get_block(layer, bid)
        kv[0][pos % self.bs] = k.to(self.dtype)
        kv[1][pos % self.bs] = v.to(self.dtype)
        self.max_pos[layer] = max(self.max_pos[layer], pos + 1)

    def get_range(self, layer: int, start: int, end: int):
        """K, V of positions [start, end): [end - start, heads, head_dim]; never-written positions read as zero."""
        ks = torch.zeros(end - start, self.H, self.D, dtype=self.dtype, device=self.device)
        vs = torch.zeros_like(ks)
        p = start
        while p < end:
            b, off = p // self.bs, p % self.bs
            n = min(self.bs - off, end - p)
            bid = self._lookup(layer, b, create=False)
            if bid is not None:
                kv = self.get_block(layer, bid)
                ks[p - start:p - start + n] = kv[0][off:off + n]
                vs[p - start:p - start + n] = kv[1][off:off + n]
            p += n
        return ks, vs

    def flush_to_disk(self) -> int:
        n = 0
        while self.resident:
            (l, b), kv = self.resident.popitem(last=False)
            torch.save([t.cpu() for t in kv], self._path(l, b))
            self.on_disk.add((l, b))
            n += 1
        return n

    def verify_retrieval(self, layer: int, pos: int, k: torch.Tensor, v: torch.Tensor, atol: float = 0.0) -> bool:
        ks, vs = self.get_range(layer, pos, pos + 1)
        return bool(torch.allclose(ks[0], k.to(self.dtype), atol=atol) and torch.allclose(vs[0], v.to(self.dtype), atol=atol))

    def resident_bytes(self) -> int:
        return len(self.resident) * 2 * self.bs * self.H * self.D * torch.empty((), dtype=self.dtype).element_size()
