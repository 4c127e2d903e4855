"""Byte-level BPE tokenizer (the reference's ``BPETokenizer``, src/bpe_tokenizer.cpp).

256 byte tokens, then greedy merges of the most frequent adjacent pair until ``vocab_size``;
ids 0/1/2 double as unk/bos/eos as in the reference. The ``.vocab`` file keeps the reference's
binary layout (src/bpe_tokenizer.cpp:111-146): ``i32 vocab_size, {i32 len, bytes}*, i32 merges,
{i32 a, i32 b, i32 id}*``. Training uses pair counts maintained incrementally with a heap instead
of recounting the corpus per merge; encoding applies merges by rank (lowest id first), which for a
vocabulary trained here gives the same segmentation as the reference's repeated first-match scan.
The C++ implementation in ``csrc/host/bpe.cpp`` is used for large corpora when the host library
is built.
"""
from __future__ import annotations

import heapq
import struct
from collections import defaultdict


class BPETokenizer:
    UNK, BOS, EOS = 0, 1, 2

    def __init__(self):
        self.vocab: list[bytes] = [bytes([i]) for i in range(256)]
        self.merges: dict[tuple[int, int], int] = {}

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    def bos_id(self) -> int:
        return self.BOS

    def eos_id(self) -> int:
        return self.EOS

    # ------------------------------------------------------------------ training
    def train(self, text, vocab_size: int, max_train_bytes: int = 4 << 20) -> None:
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        ids = list(data[:max_train_bytes])
        self.vocab = [bytes([i]) for i in range(256)]
        self.merges = {}
        n = len(ids)
        if n < 2 or vocab_size <= 256:
            return
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        counts: dict[tuple[int, int], int] = defaultdict(int)
        where: dict[tuple[int, int], set] = defaultdict(set)
        for i in range(n - 1):
            p = (ids[i], ids[i + 1])
            counts[p] += 1
            where[p].add(i)
        heap = [(-c, p) for p, c in counts.items()]
        heapq.heapify(heap)
        while len(self.vocab) < vocab_size and heap:
            negc, pair = heapq.heappop(heap)
            c = counts.get(pair, 0)
            if c <= 0 or -negc != c:
                if c > 0:
                    heapq.heappush(heap, (-c, pair))
                continue
            if c < 2:
                break
            new_id = len(self.vocab)
            self.vocab.append(self.vocab[pair[0]] + self.vocab[pair[1]])
            self.merges[pair] = new_id
            touched = set()
            for i in sorted(where.pop(pair, ())):
                j = nxt[i] if alive[i] else -1
                if not alive[i] or j < 0 or not alive[j] or ids[i] != pair[0] or ids[j] != pair[1]:
                    continue
                pi, nj = prev[i], nxt[j]
                if pi >= 0:
                    old = (ids[pi], ids[i])
                    counts[old] -= 1
                    where[old].discard(pi)
                    touched.add(old)
                if nj >= 0:
                    old = (ids[j], ids[nj])
                    counts[old] -= 1
                    where[old].discard(j)
                    touched.add(old)
                ids[i] = new_id
                alive[j] = False
                nxt[i] = nj
                if nj >= 0:
                    prev[nj] = i
                if pi >= 0:
                    new = (ids[pi], new_id)
                    counts[new] += 1
                    where[new].add(pi)
                    touched.add(new)
                if nj >= 0:
                    new = (new_id, ids[nj])
                    counts[new] += 1
                    where[new].add(i)
                    touched.add(new)
            counts.pop(pair, None)
            for p in touched:
                if counts.get(p, 0) > 0:
                    heapq.heappush(heap, (-counts[p], p))

    # ------------------------------------------------------------------ encode / decode
    def encode(self, text, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        ids = list(data)
        if self.merges and len(ids) > 1:
            while True:
                best, best_rank = None, None
                for a, b in zip(ids, ids[1:]):
                    r = self.merges.get((a, b))
                    if r is not None and (best_rank is None or r < best_rank):
                        best, best_rank = (a, b), r
                if best is None:
                    break
                out, i = [], 0
                while i < len(ids):
                    if i + 1 < len(ids) and ids[i] == best[0] and ids[i + 1] == best[1]:
                        out.append(best_rank)
                        i += 2
                    else:
                        out.append(ids[i])
                        i += 1
                ids = out
                if len(ids) < 2:
                    break
        if add_bos:
            ids = [self.BOS] + ids
        if add_eos:
            ids = ids + [self.EOS]
        return ids

    def decode_bytes(self, ids) -> bytes:
        return b"".join(self.vocab[i] for i in ids if 0 <= i < len(self.vocab))

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    # ------------------------------------------------------------------ .vocab file
    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(struct.pack("<i", len(self.vocab)))
            for v in self.vocab:
                f.write(struct.pack("<i", len(v)) + v)
            f.write(struct.pack("<i", len(self.merges)))
            for (a, b), c in sorted(self.merges.items()):  # the reference iterates a std::map: sorted by (a, b)
                f.write(struct.pack("<iii", a, b, c))

    @classmethod
    def load(cls, path: str) -> "BPETokenizer":
        tok = cls()
        with open(path, "rb") as f:
            data = f.read()
        (vs,) = struct.unpack_from("<i", data, 0)
        off = 4
        tok.vocab = []
        for _ in range(vs):
            (ln,) = struct.unpack_from("<i", data, off)
            off += 4
            tok.vocab.append(data[off:off + ln])
            off += ln
        (ms,) = struct.unpack_from("<i", data, off)
        off += 4
        tok.merges = {}
        for _ in range(ms):
            a, b, c = struct.unpack_from("<iii", data, off)
            off += 12
            tok.merges[(a, b)] = c
        return tok
