"""Paged KV cache: fixed-size token pages, per-sequence block tables, a free-list allocator with
reference counts (shared prefix pages), optional host offload of cold pages.

Covers the reference's ``KVCache`` (contiguous, src/kv_cache.cpp:44-238), ``PagedAttention`` block
pool (src/inference_opt.cpp:14-57), ``PagedKVCache1T`` (hierarchical table + LRU offload to disk,
src/kv_cache.cpp:244-642) and ``PrefixCache`` (src/inference_opt.cpp:460-520) with one design: a
flat page pool per layer on the GPU (``[pages, page_size, kv_heads, head_dim]`` bf16), an int32
block table ``[max_seqs, max_pages_per_seq]`` that the attention kernels index directly, and an
offload tier in pinned host memory (the disk files of the reference are replaced by host RAM;
``save_pages`` / ``load_pages`` still give a file tier when asked for).
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict

import torch


class PageAllocator:
    """Free list with reference counts. Page ids are ints in [0, num_pages)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free = list(range(num_pages - 1, -1, -1))
        self.refs = [0] * num_pages
        self.gen = [0] * num_pages      # bumped on every allocation: tells a re-used page from the original

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("KV cache is out of pages")
        p = self.free.pop()
        self.refs[p] = 1
        self.gen[p] += 1
        return p

    def retain(self, p: int) -> None:
        self.refs[p] += 1

    def release(self, p: int) -> None:
        self.refs[p] -= 1
        if self.refs[p] == 0:
            self.free.append(p)

    @property
    def used(self) -> int:
        return self.num_pages - len(self.free)


class PagedKVCache:
    def __init__(self, num_layers: int, kv_heads: int, head_dim: int, num_pages: int, page_size: int = 16,
                 max_seqs: int = 64, max_pages_per_seq: int = 256, device="cuda", dtype=torch.bfloat16):
        self.num_layers, self.kv_heads, self.head_dim = num_layers, kv_heads, head_dim
        self.page_size, self.max_seqs, self.max_pages = page_size, max_seqs, max_pages_per_seq
        self.device = torch.device(device)
        shape = (num_pages, page_size, kv_heads, head_dim)
        self.k = [torch.zeros(shape, device=self.device, dtype=dtype) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, device=self.device, dtype=dtype) for _ in range(num_layers)]
        # int8 pages carry one fp32 scale (max|x| / 127) per (token, kv head); the append kernel
        # writes them and the decode kernel folds them into the score and the probability
        self.int8 = dtype == torch.int8
        srows = (num_pages * page_size, kv_heads)
        self.k_scale = [torch.zeros(srows, device=self.device) for _ in range(num_layers)] if self.int8 else None
        self.v_scale = [torch.zeros(srows, device=self.device) for _ in range(num_layers)] if self.int8 else None
        self.alloc = PageAllocator(num_pages)
        self.block_table_host = torch.full((max_seqs, max_pages_per_seq), -1, dtype=torch.int32)
        self.block_table = self.block_table_host.to(self.device)
        self.lens = [0] * max_seqs           # tokens stored per sequence slot
        self.active = [False] * max_seqs
        self.prefix_index: "OrderedDict[bytes, list[int]]" = OrderedDict()
        self._dirty = False

    # ------------------------------------------------------------------ sequence management
    def new_sequence(self) -> int:
        for s in range(self.max_seqs):
            if not self.active[s]:
                self.active[s] = True
                self.lens[s] = 0
                self.block_table_host[s].fill_(-1)
                self._dirty = True
                return s
        raise MemoryError("no free sequence slot")

    def reserve(self, seq: int, new_tokens: int) -> None:
        """Make sure pages exist for ``lens[seq] + new_tokens`` tokens."""
        need = (self.lens[seq] + new_tokens + self.page_size - 1) // self.page_size
        if need > self.max_pages:
            raise MemoryError(f"sequence needs {need} pages, table holds {self.max_pages}")
        row = self.block_table_host[seq]
        for i in range(need):
            if row[i] < 0:
                row[i] = self.alloc.alloc()
                self._dirty = True

    def advance(self, seq: int, new_tokens: int) -> None:
        self.lens[seq] += new_tokens

    def free_sequence(self, seq: int) -> None:
        row = self.block_table_host[seq]
        for i in range(self.max_pages):
            p = int(row[i])
            if p >= 0:
                self.alloc.release(p)
                row[i] = -1
        self.active[seq] = False
        self.lens[seq] = 0
        self._dirty = True

    def sync_tables(self) -> torch.Tensor:
        """Upload the block table if it changed; returns the device table."""
        if self._dirty:
            self.block_table.copy_(self.block_table_host, non_blocking=True)
            self._dirty = False
        return self.block_table

    # ------------------------------------------------------------------ prefix sharing
    def _prefix_key(self, tokens) -> bytes:
        return hashlib.sha256(bytes(memoryview(torch.as_tensor(tokens, dtype=torch.int32).numpy()))).digest()

    def share_prefix(self, seq: int, tokens) -> int:
        """If full pages holding a prefix of ``tokens`` are cached, map them into ``seq`` (their
        reference counts go up) and return the number of tokens covered; else 0."""
        n_full = len(tokens) // self.page_size
        for n in range(n_full, 0, -1):
            entry = self.prefix_index.get(self._prefix_key(tokens[: n * self.page_size]))
            # an entry is valid while every page is still held by someone and has not been handed
            # out again since it was published
            if entry is not None and all(self.alloc.refs[p] > 0 and self.alloc.gen[p] == g for p, g in entry):
                pages = [p for p, _ in entry]
                for i, p in enumerate(pages):
                    self.alloc.retain(p)
                    self.block_table_host[seq, i] = p
                self.lens[seq] = n * self.page_size
                self._dirty = True
                return self.lens[seq]
        return 0

    def publish_prefix(self, seq: int, tokens, max_entries: int = 1024) -> None:
        n_full = min(len(tokens), self.lens[seq]) // self.page_size
        if n_full == 0:
            return
        pages = [int(self.block_table_host[seq, i]) for i in range(n_full)]
        self.prefix_index[self._prefix_key(tokens[: n_full * self.page_size])] = [(p, self.alloc.gen[p]) for p in pages]
        while len(self.prefix_index) > max_entries:
            self.prefix_index.popitem(last=False)

    # ------------------------------------------------------------------ statistics / offload
    def utilization(self) -> float:
        return self.alloc.used / max(1, self.alloc.num_pages)

    def size_bytes(self) -> int:
        n = 2 * self.num_layers * self.k[0].numel() * self.k[0].element_size()
        if self.int8:
            n += 2 * self.num_layers * self.k_scale[0].numel() * 4
        return n

    def offload_sequence(self, seq: int):
        """Copy a sequence's pages to pinned host memory and release them. Returns a handle for
        :meth:`restore_sequence`."""
        pages = [int(p) for p in self.block_table_host[seq] if p >= 0]
        idx = torch.tensor(pages, device=self.device, dtype=torch.long)
        host = []
        for layer in range(self.num_layers):
            hk = torch.empty((len(pages),) + tuple(self.k[layer].shape[1:]), dtype=self.k[layer].dtype,
                             pin_memory=self.device.type == "cuda")
            hv = torch.empty_like(hk, pin_memory=self.device.type == "cuda")
            hk.copy_(self.k[layer][idx], non_blocking=True)
            hv.copy_(self.v[layer][idx], non_blocking=True)
            if self.int8:
                ks = self.k_scale[layer].view(-1, self.page_size, self.kv_heads)[idx].cpu()
                vs = self.v_scale[layer].view(-1, self.page_size, self.kv_heads)[idx].cpu()
                host.append((hk, hv, ks, vs))
            else:
                host.append((hk, hv))
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        length = self.lens[seq]
        self.free_sequence(seq)
        return {"len": length, "pages": host}

    def restore_sequence(self, handle) -> int:
        seq = self.new_sequence()
        self.reserve(seq, handle["len"])
        pages = [int(p) for p in self.block_table_host[seq] if p >= 0]
        idx = torch.tensor(pages, device=self.device, dtype=torch.long)
        for layer, rec in enumerate(handle["pages"]):
            self.k[layer][idx] = rec[0].to(self.device, non_blocking=True)
            self.v[layer][idx] = rec[1].to(self.device, non_blocking=True)
            if self.int8:
                self.k_scale[layer].view(-1, self.page_size, self.kv_heads)[idx] = rec[2].to(self.device)
                self.v_scale[layer].view(-1, self.page_size, self.kv_heads)[idx] = rec[3].to(self.device)
        self.lens[seq] = handle["len"]
        return seq

    def save_pages(self, seq: int, path: str) -> None:
        """File tier: write a sequence's pages to ``path`` (torch.save of the offload handle)."""
        h = self.offload_sequence(seq)
        torch.save({"len": h["len"], "pages": [tuple(t.clone() for t in rec) for rec in h["pages"]]}, path)

    def load_pages(self, path: str) -> int:
        return self.restore_sequence(torch.load(path))


def quantize_kv_int8(x: torch.Tensor, block: int = 64):
    """int8 block quantisation of K/V vectors: scale = absmax/127 per 64-value block, q = round(x/scale)
    clamped to +-127 (the reference's "FP8" cache mode, src/kv_cache.cpp:13-42)."""
    flat = x.float().reshape(-1, block)
    amax = flat.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(flat / scale).clamp(-127, 127).to(torch.int8)
    return q.reshape(x.shape), scale.reshape(*x.shape[:-1], -1)


def dequantize_kv_int8(q: torch.Tensor, scale: torch.Tensor, block: int = 64) -> torch.Tensor:
    flat = q.float().reshape(-1, block) * scale.reshape(-1, 1)
    return flat.reshape(q.shape)


def compress_kv_ternary(x: torch.Tensor, threshold: float = 0.1) -> torch.Tensor:
    """2-bit ternary KV compression (code = sign + 1 with a dead zone of +-threshold), four codes per
    byte — the reference's lossy ``CompressedKVCache`` (src/inference_opt.cpp:378-455)."""
    t = torch.where(x > threshold, 2, torch.where(x < -threshold, 0, 1)).to(torch.uint8).reshape(-1)
    pad = (-t.numel()) % 4
    if pad:
        t = torch.cat([t, t.new_ones(pad)])
    t = t.reshape(-1, 4)
    return t[:, 0] | (t[:, 1] << 2) | (t[:, 2] << 4) | (t[:, 3] << 6)


def decompress_kv_ternary(packed: torch.Tensor, numel: int, magnitude: float = 0.1) -> torch.Tensor:
    p = packed.long()
    codes = torch.stack([(p >> (2 * j)) & 3 for j in range(4)], dim=1).reshape(-1)[:numel]
    return (codes.float() - 1.0) * magnitude
