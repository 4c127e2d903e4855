"""Data sources for training.

* :class:`ZipfStream` — the synthetic token stream of the benchmark configurations: seeded
  Zipf(s) draws over the vocabulary, delivered as pinned-host int32 ``(ids, targets)`` batches.
* :class:`TokenDataset` — contiguous ``[B, S]`` windows over a token array with next-token
  targets, sequence-level shuffling and a background prefetch thread (the reference's
  ``DataLoader`` shuffles individual tokens, src/trainer.cpp:320-325, which destroys the text;
  windows are shuffled here instead).
"""
from __future__ import annotations

import queue
import threading

import numpy as np
import torch


def zipf_probs(vocab: int, s: float = 1.1) -> np.ndarray:
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    p = ranks ** (-s)
    return p / p.sum()


class ZipfStream:
    """Infinite iterator of (ids, targets) with ``targets[t] = ids[t+1]`` inside each sequence."""

    def __init__(self, vocab: int, batch: int, seq: int, s: float = 1.1, seed: int = 0, pin: bool = True):
        self.vocab, self.batch, self.seq = vocab, batch, seq
        self.rng = np.random.default_rng(seed)
        self.cdf = np.cumsum(zipf_probs(vocab, s))
        self.pin = pin and torch.cuda.is_available()

    def draw(self, n: int) -> np.ndarray:
        u = self.rng.random(n)
        return np.minimum(np.searchsorted(self.cdf, u, side="right"), self.vocab - 1).astype(np.int32)

    def next_batch(self):
        raw = self.draw(self.batch * (self.seq + 1)).reshape(self.batch, self.seq + 1)
        ids = torch.from_numpy(np.ascontiguousarray(raw[:, :-1]))
        tgt = torch.from_numpy(np.ascontiguousarray(raw[:, 1:]))
        if self.pin:
            ids, tgt = ids.pin_memory(), tgt.pin_memory()
        return ids, tgt

    def __iter__(self):
        while True:
            yield self.next_batch()


class TokenDataset:
    """Windows of ``seq+1`` tokens over a 1-D token array; one epoch = all full windows once."""

    def __init__(self, tokens, batch: int, seq: int, shuffle: bool = True, seed: int = 42, prefetch: int = 2,
                 drop_last: bool = True, pin: bool = False):
        self.tokens = np.asarray(tokens, dtype=np.int32)
        self.batch, self.seq, self.shuffle, self.seed = batch, seq, shuffle, seed
        self.prefetch, self.drop_last, self.pin = prefetch, drop_last, pin and torch.cuda.is_available()
        self.n_windows = max(0, (len(self.tokens) - 1) // seq)
        self.order = np.arange(self.n_windows)
        self.epoch = 0

    def __len__(self):
        if self.drop_last:
            return self.n_windows // self.batch
        return (self.n_windows + self.batch - 1) // self.batch

    def reset(self, epoch: int = 0):
        self.epoch = epoch
        self.order = np.arange(self.n_windows)
        if self.shuffle:
            np.random.default_rng(self.seed + epoch).shuffle(self.order)

    def _make(self, b: int):
        sel = self.order[b * self.batch:(b + 1) * self.batch]
        ids = np.stack([self.tokens[w * self.seq: w * self.seq + self.seq] for w in sel])
        tgt = np.stack([self.tokens[w * self.seq + 1: w * self.seq + self.seq + 1] for w in sel])
        ids, tgt = torch.from_numpy(ids), torch.from_numpy(tgt)
        if self.pin:
            ids, tgt = ids.pin_memory(), tgt.pin_memory()
        return ids, tgt

    def __iter__(self):
        n = len(self)
        if self.prefetch <= 0:
            for b in range(n):
                yield self._make(b)
            return
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)

        def worker():
            for b in range(n):
                q.put(self._make(b))
            q.put(None)

        th = threading.Thread(target=worker, daemon=True)
        th.start()
        while True:
            item = q.get()
            if item is None:
                break
            yield item
        th.join()


# ------------------------------------------------------------------------------ streaming corpus
class StreamingTokenDataset:
    """Batches from a text file that is never held in memory whole: the file is read in chunks of
    ``chunk_bytes`` (4 MB, as the reference's streaming mode, src/trainer.cpp:262-296; memory-mapped
    when ``mmap`` is set), each chunk is tokenised and appended to a token buffer, and ``[B, S]``
    windows with next-token targets are cut from the buffer. A background thread keeps up to
    ``prefetch`` batches ready in a bounded queue. One pass over the file is one epoch."""

    def __init__(self, path: str, tokenizer, batch: int, seq: int, chunk_bytes: int = 4 << 20, prefetch: int = 2,
                 mmap: bool = False, vocab_limit: int | None = None):
        self.path, self.tok, self.batch, self.seq = path, tokenizer, batch, seq
        self.chunk_bytes, self.prefetch, self.use_mmap, self.vocab_limit = chunk_bytes, prefetch, mmap, vocab_limit
        self.chunks_read = 0

    def _chunks(self):
        if self.use_mmap:
            import mmap as _mmap

            with open(self.path, "rb") as f, _mmap.mmap(f.fileno(), 0, access=_mmap.ACCESS_READ) as m:
                for off in range(0, len(m), self.chunk_bytes):
                    yield bytes(m[off:off + self.chunk_bytes])
        else:
            with open(self.path, "rb") as f:
                while True:
                    data = f.read(self.chunk_bytes)
                    if not data:
                        return
                    yield data

    def _batches(self):
        need = self.batch * self.seq
        buf = np.empty(0, dtype=np.int32)
        for data in self._chunks():
            self.chunks_read += 1
            ids = np.asarray(self.tok.encode(data) if self.tok is not None else list(data), dtype=np.int32)
            if self.vocab_limit:
                ids = np.minimum(ids, self.vocab_limit - 1)
            buf = np.concatenate([buf, ids])
            while len(buf) >= need + 1:
                win = buf[:need + 1]
                ids_t = torch.from_numpy(win[:-1].reshape(self.batch, self.seq).copy())
                tgt_t = torch.from_numpy(win[1:].reshape(self.batch, self.seq).copy())
                yield ids_t, tgt_t
                buf = buf[need:]

    def __iter__(self):
        if self.prefetch <= 0:
            yield from self._batches()
            return
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)

        def worker():
            try:
                for item in self._batches():
                    q.put(item)
            finally:
                q.put(None)

        th = threading.Thread(target=worker, daemon=True)
        th.start()
        while True:
            item = q.get()
            if item is None:
                break
            yield item
        th.join()


# ------------------------------------------------------------------------------ augmentation, curriculum
def augment_batch(ids: torch.Tensor, targets: torch.Tensor, vocab: int, mask_prob: float = 0.0,
                  replace_prob: float = 0.0, label_mask_prob: float = 0.0, mask_id: int = 0, generator=None):
    """Token-level augmentation of the reference's loader (src/trainer.cpp:241-259): each input id
    becomes ``mask_id`` with ``mask_prob`` or a uniformly random id with ``replace_prob``; each
    label becomes ``mask_id`` with ``label_mask_prob``. (The reference also adds Gaussian noise to
    the float-typed ids, which has no meaning for integer ids and is left out.) Returns new tensors."""
    ids, targets = ids.clone(), targets.clone()
    if mask_prob > 0:
        ids[torch.rand(ids.shape, generator=generator) < mask_prob] = mask_id
    if replace_prob > 0:
        sel = torch.rand(ids.shape, generator=generator) < replace_prob
        ids[sel] = torch.randint(0, vocab, (int(sel.sum()),), generator=generator, dtype=ids.dtype)
    if label_mask_prob > 0:
        targets[torch.rand(targets.shape, generator=generator) < label_mask_prob] = mask_id
    return ids, targets


class Curriculum:
    """Sequence-length curriculum: training starts on prefixes of ``min_fraction`` of the full
    sequence and grows linearly to the full length over ``total_epochs`` epochs (the reference keeps
    this state, ``set_curriculum`` / ``curriculum_step``, but its ``next_batch`` never uses it)."""

    def __init__(self, seq_length: int, total_epochs: int = 3, min_fraction: float = 0.25, multiple: int = 8):
        self.seq_length, self.total_epochs, self.min_fraction, self.multiple = seq_length, total_epochs, min_fraction, multiple
        self.current_epoch = 0

    def step(self, epoch: int) -> None:
        self.current_epoch = epoch

    def length(self) -> int:
        if self.total_epochs <= 1:
            return self.seq_length
        t = min(1.0, self.current_epoch / (self.total_epochs - 1))
        frac = self.min_fraction + (1.0 - self.min_fraction) * t
        n = int(self.seq_length * frac) // self.multiple * self.multiple
        return max(self.multiple, min(self.seq_length, n))

    def apply(self, ids: torch.Tensor, targets: torch.Tensor):
        n = self.length()
        return ids[:, :n].contiguous(), targets[:, :n].contiguous()


class AugmentedLoader:
    """Wraps a loader: per batch, the curriculum cut first, then token augmentation. ``reset(epoch)``
    is passed on and advances the curriculum."""

    def __init__(self, loader, vocab: int, mask_prob: float = 0.0, replace_prob: float = 0.0,
                 label_mask_prob: float = 0.0, curriculum: Curriculum | None = None, seed: int = 0):
        self.loader, self.vocab, self.curriculum = loader, vocab, curriculum
        self.mask_prob, self.replace_prob, self.label_mask_prob = mask_prob, replace_prob, label_mask_prob
        self.gen = torch.Generator().manual_seed(seed)

    def reset(self, epoch: int = 0) -> None:
        if hasattr(self.loader, "reset"):
            self.loader.reset(epoch)
        if self.curriculum is not None:
            self.curriculum.step(epoch)

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        for ids, tgt in self.loader:
            if self.curriculum is not None:
                ids, tgt = self.curriculum.apply(ids, tgt)
            if self.mask_prob or self.replace_prob or self.label_mask_prob:
                ids, tgt = augment_batch(ids, tgt, self.vocab, self.mask_prob, self.replace_prob, self.label_mask_prob,
                                         generator=self.gen)
            yield ids, tgt
