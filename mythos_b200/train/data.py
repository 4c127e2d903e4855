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
