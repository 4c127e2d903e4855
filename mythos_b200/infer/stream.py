"""Streaming text output: pieces are held back until a natural break.

The reference's ``engine::InferenceEngine::generate_stream`` wraps the per-token callback in a
buffer that is flushed when the text so far ends in white space, sentence punctuation, a closing
bracket or a quote (engines/inference/stream.cpp:10-48); the tail that never reached a break is
dropped there when generation ends. Here the tail is flushed by ``close()``, and bytes of an
unfinished UTF-8 sequence are held back so that a multi-byte character split over two tokens is
never emitted as replacement characters.
"""
from __future__ import annotations

from typing import Callable, Iterable, Iterator

FLUSH_CHARS = frozenset(" \n\t\r.,!?;:)}]\"'")


class StreamBuffer:
    """Collects decoded pieces; calls ``on_text`` with the buffered text whenever it ends in one of
    ``FLUSH_CHARS`` (or grows past ``max_chars``)."""

    def __init__(self, on_text: Callable[[str], None], max_chars: int = 256):
        self.on_text = on_text
        self.max_chars = max_chars
        self.buffer = ""
        self.flushes = 0

    def should_flush(self) -> bool:
        return bool(self.buffer) and (self.buffer[-1] in FLUSH_CHARS or len(self.buffer) >= self.max_chars)

    def flush(self) -> None:
        if self.buffer:
            text, self.buffer = self.buffer, ""
            self.flushes += 1
            self.on_text(text)

    def append(self, piece: str) -> None:
        self.buffer += piece
        if self.should_flush():
            self.flush()

    def close(self) -> None:
        """End of generation: emit whatever is still buffered."""
        self.flush()


class Utf8Assembler:
    """Turns a stream of byte chunks into text, holding back an unfinished multi-byte sequence."""

    def __init__(self):
        self.pending = b""

    def feed(self, data: bytes) -> str:
        data = self.pending + data
        cut = len(data)
        # look at up to 3 trailing bytes for a lead byte whose sequence is not complete yet
        for back in range(1, min(4, len(data)) + 1):
            b = data[-back]
            if b & 0xC0 == 0x80:
                continue                      # continuation byte: keep looking for its lead
            need = 2 if b & 0xE0 == 0xC0 else 3 if b & 0xF0 == 0xE0 else 4 if b & 0xF8 == 0xF0 else 1
            if need > back:
                cut = len(data) - back
            break
        self.pending = data[cut:]
        return data[:cut].decode("utf-8", errors="replace")

    def finish(self) -> str:
        tail, self.pending = self.pending, b""
        return tail.decode("utf-8", errors="replace")


def buffered(pieces: Iterable[str], max_chars: int = 256) -> Iterator[str]:
    """Generator form: regroups an iterator of text pieces at the flush points."""
    out: list[str] = []
    buf = StreamBuffer(out.append, max_chars)
    for p in pieces:
        buf.append(p)
        while out:
            yield out.pop(0)
    buf.close()
    while out:
        yield out.pop(0)
