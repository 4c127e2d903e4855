"""Remaining inference extras of the reference (src/inference_opt.cpp, include/oil/inference_opt.h):

* ``INT8Inference`` / ``FP8Inference`` (D8 / D9, :669-778). The reference round-trips the *token id
  tensor* through int8 / fp8, which only perturbs the ids; what those classes are named for is
  reduced-precision activations, and that is what these do: every linear layer's input is
  quantised per token (int8, scale = max|x| / 127) or per 32-value block (e4m3, scale = max|x| /
  448) and dequantised again before the layer runs, so a model can be scored under int8 / fp8
  activation error without another kernel.
* ``InferenceMemoryPool`` (D13, inference_opt.h:188-201): fixed-size blocks carved out of one device
  allocation, ``alloc`` / ``free`` / ``used`` / ``capacity``, thread-safe.
* ``StreamConfig`` / ``DecodeResult`` (D14-D16, inference_opt.h:204-217) and ``decode_with_config``,
  which applies them (token budget, EOS, stop on newline, stop sequences, per-token log-probs,
  perplexity) on top of any ``step(ids) -> logits`` callable.
"""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.nn as nn

FP8_BLOCK = 32
FP8_MAX = 448.0


# ------------------------------------------------------------------------------ D8 / D9
def quantize_per_token_int8(x: torch.Tensor):
    """Rows of ``x`` -> (int8 codes, fp32 scale per row); scale = max|x| / 127, zero rows keep scale 1."""
    flat = x.float().reshape(-1, x.shape[-1])
    amax = flat.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(flat / scale).clamp(-127, 127).to(torch.int8)
    return q.view(x.shape), scale.view(*x.shape[:-1], 1)


def fake_quant_int8(x: torch.Tensor) -> torch.Tensor:
    q, s = quantize_per_token_int8(x)
    return (q.float() * s).to(x.dtype)


def fake_quant_fp8(x: torch.Tensor, block: int = FP8_BLOCK) -> torch.Tensor:
    """e4m3 with one scale per ``block`` consecutive values (scale = max|x| / 448)."""
    flat = x.float().reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    b = flat.view(-1, block)
    amax = b.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (b / scale).to(torch.float8_e4m3fn).float() * scale
    return q.reshape(-1)[: x.numel()].view(x.shape).to(x.dtype)


class _ActivationQuantised:
    """Runs ``model`` with every ``nn.Linear``-like leaf (anything with ``in_features``) seeing
    fake-quantised inputs. Hooks are installed for the duration of a call only."""

    quant: Callable[[torch.Tensor], torch.Tensor] = staticmethod(lambda x: x)

    def __init__(self, model: nn.Module):
        self.model = model
        self.is_quantized = False
        self.layers_seen = 0

    def _targets(self):
        return [m for m in self.model.modules() if hasattr(m, "in_features") and not list(m.children())]

    def forward(self, *args, **kw):
        def pre(_mod, inputs):
            self.layers_seen += 1
            return (self.quant(inputs[0]),) + tuple(inputs[1:])

        self.layers_seen = 0
        handles = [m.register_forward_pre_hook(pre) for m in self._targets()]
        try:
            with torch.no_grad():
                out = self.model(*args, **kw)
        finally:
            for h in handles:
                h.remove()
        self.is_quantized = True
        return out

    __call__ = forward


class INT8Inference(_ActivationQuantised):
    quant = staticmethod(fake_quant_int8)


class FP8Inference(_ActivationQuantised):
    quant = staticmethod(fake_quant_fp8)


# ------------------------------------------------------------------------------ D13
class InferenceMemoryPool:
    """``num_blocks`` blocks of ``block_size`` bytes out of one allocation on ``device``. ``alloc``
    returns a uint8 view of a free block (or raises ``MemoryError``), ``free`` takes it back."""

    def __init__(self, block_size: int, num_blocks: int, device="cpu"):
        self.block_size, self.capacity = int(block_size), int(num_blocks)
        self.pool = torch.empty(self.capacity * self.block_size, dtype=torch.uint8, device=device)
        self._free = list(range(self.capacity - 1, -1, -1))
        self._out: set[int] = set()
        self._lock = threading.Lock()

    def alloc(self) -> torch.Tensor:
        with self._lock:
            if not self._free:
                raise MemoryError("inference memory pool exhausted")
            i = self._free.pop()
            self._out.add(i)
        return self.pool[i * self.block_size:(i + 1) * self.block_size]

    def free(self, block: torch.Tensor) -> None:
        off = block.data_ptr() - self.pool.data_ptr()
        i, rem = divmod(off, self.block_size)
        with self._lock:
            if rem or i not in self._out:
                raise ValueError("not a live block of this pool")
            self._out.remove(i)
            self._free.append(i)

    @property
    def used(self) -> int:
        return len(self._out)


# ------------------------------------------------------------------------------ D14 - D16
@dataclass
class StreamConfig:
    stream: bool = False
    max_tokens: int = 512
    eos_id: int = -1
    stop_on_newline: bool = False
    stop_sequences: list = field(default_factory=list)


@dataclass
class DecodeResult:
    text: str = ""
    tokens: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)      # per generated token: log-probability of the token
    perplexity: float = 0.0
    finish_reason: str = "length"


def decode_with_config(step: Callable[[list], torch.Tensor], prompt_ids, cfg: StreamConfig,
                       detokenize: Callable[[list], str], on_text: Callable[[str], None] | None = None,
                       choose: Callable[[torch.Tensor], int] | None = None) -> DecodeResult:
    """Greedy (or ``choose``-driven) decoding under a ``StreamConfig``. ``step(ids)`` returns the
    next-token logits [V] for the whole sequence ``ids``. Generation stops at ``max_tokens``, at
    ``eos_id``, after a newline when ``stop_on_newline``, or as soon as the text ends with one of
    ``stop_sequences`` (the stop text is cut from the result). With ``cfg.stream`` every new piece
    of text goes to ``on_text`` as it appears."""
    ids = list(prompt_ids)
    res = DecodeResult()
    nll = 0.0
    for _ in range(cfg.max_tokens):
        logits = step(ids).float()
        tok = int(choose(logits)) if choose is not None else int(logits.argmax())
        lp = float(torch.log_softmax(logits, dim=-1)[tok])
        if tok == cfg.eos_id:
            res.finish_reason = "eos"
            break
        ids.append(tok)
        res.tokens.append(tok)
        res.logprobs.append(lp)
        nll -= lp
        piece = detokenize([tok])
        text = res.text + piece
        hit = next((s for s in cfg.stop_sequences if s and text.endswith(s)), None)
        if hit is not None:
            res.text = text[: -len(hit)]
            res.finish_reason = "stop"
            break
        res.text = text
        if cfg.stream and on_text is not None:
            on_text(piece)
        if cfg.stop_on_newline and piece.endswith("\n"):
            res.finish_reason = "newline"
            break
    res.perplexity = math.exp(nll / len(res.tokens)) if res.tokens else 0.0
    return res
