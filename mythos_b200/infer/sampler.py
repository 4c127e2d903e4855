"""Sampling configuration and the sampler front end.

``SamplerConfig`` mirrors the reference (include/oil/sampler.h:9-15: temperature 1.0, top_k 40,
top_p 0.9, repetition_penalty 1.0, max_tokens 2048). ``sample`` runs the CUDA sampler kernel for
device logits and a PyTorch restatement of the reference algorithm (src/sampler.cpp:12-120) for
CPU logits; the latter is the oracle of the kernel test.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import native


@dataclass
class SamplerConfig:
    temperature: float = 1.0
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    max_tokens: int = 2048
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5


def adjusted_logits(logits, history, cfg: SamplerConfig, allow_mask=None):
    """Repetition penalty (divide positive, multiply negative logits of seen tokens), vocabulary
    mask, temperature. logits [rows, V] float; history [rows, L] int (-1 = empty)."""
    lg = logits.float().clone()
    if history is not None and cfg.repetition_penalty != 1.0:
        for r in range(lg.shape[0]):
            seen = history[r][history[r] >= 0].long().unique()
            v = lg[r, seen]
            lg[r, seen] = torch.where(v > 0, v / cfg.repetition_penalty, v * cfg.repetition_penalty)
    if allow_mask is not None:
        lg = lg.masked_fill(~allow_mask.bool(), float("-inf"))
    if not cfg.greedy:
        lg = lg / cfg.temperature
    return lg


def nucleus_keep_mask(probs: torch.Tensor, top_p: float) -> torch.Tensor:
    """Tokens kept by top-p: in decreasing probability until the cumulative sum exceeds p, inclusive."""
    sp, si = torch.sort(probs, dim=-1, descending=True)
    cum = sp.cumsum(-1)
    keep_sorted = (cum - sp) < top_p  # the token that crosses p is kept
    keep = torch.zeros_like(probs, dtype=torch.bool)
    keep.scatter_(-1, si, keep_sorted)
    return keep


def sample_reference(logits, history, cfg: SamplerConfig, allow_mask=None, generator=None):
    lg = adjusted_logits(logits, history, cfg, allow_mask)
    if cfg.greedy:
        return lg.argmax(-1).to(torch.int32)
    probs = torch.softmax(lg, -1)
    if cfg.top_p < 1.0:
        keep = nucleus_keep_mask(probs, cfg.top_p)
    elif 0 < cfg.top_k < lg.shape[-1]:
        kth = torch.topk(probs, cfg.top_k, dim=-1).values[:, -1:]
        keep = probs >= kth
    else:
        keep = torch.ones_like(probs, dtype=torch.bool)
    p = torch.where(keep, probs, torch.zeros_like(probs))
    p = p / p.sum(-1, keepdim=True)
    return torch.multinomial(p, 1, generator=generator).squeeze(-1).to(torch.int32)


def sample(logits, cfg: SamplerConfig, history=None, allow_mask=None, step: int = 0, out=None, logprobs=None):
    """One token per row. logits: [rows, V] (bf16 on CUDA). Returns int32 [rows]."""
    if logits.is_cuda:
        if out is None:
            out = torch.empty(logits.shape[0], device=logits.device, dtype=torch.int32)
        native.require().sample_tokens(logits, history, allow_mask, cfg.temperature, cfg.top_k, cfg.top_p,
                                       cfg.repetition_penalty, (cfg.seed * 1000003 + step) & 0x7FFFFFFFFFFFFFFF, out,
                                       logprobs)
        return out
    g = torch.Generator().manual_seed(cfg.seed * 1000003 + step)
    return sample_reference(logits, history, cfg, allow_mask, g)
