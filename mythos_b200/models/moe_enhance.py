"""Mixture-of-experts utilities around the layers: capacity planning, dense-to-MoE conversion,
expert files, expert dropout, balance monitoring, Switch-style and expert-choice routers, expert
merging and a growable expert pool.

Reference counterparts: include/oil/moe_enhance.h, src/moe_enhance.cpp (``ExpertCapacity::adaptive``,
``DenseToMoEPruner``, ``MoEOILFormat::save/load_experts`` with its own binary layout (:125-195),
``ExpertDropout``, ``compute_balance``, ``SwitchV2Router`` (:275-347), ``ExpertChoiceV2``,
``ExpertMerger`` (cosine-similarity averaging), ``DynamicExpertPool``). ``ExpertParallel`` lives in
``models/moe.py`` (the reference's version only slices the hidden dimension and runs no experts).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import torch


def adaptive_capacity(num_experts: int, tokens: int, importance=None, slack: float = 1.25) -> list[int]:
    """Per-expert token capacity proportional to ``importance`` (uniform when absent), with slack,
    at least 1 each."""
    imp = torch.ones(num_experts) if importance is None else torch.as_tensor(importance, dtype=torch.float32).clamp_min(0)
    share = imp / imp.sum().clamp_min(1e-12)
    return [max(1, int(c)) for c in torch.ceil(share * tokens * slack).tolist()]


class DenseToMoEPruner:
    """Split a dense gated FFN into ``n_experts`` experts by partitioning its hidden units: units
    are ranked by ``|gate row| * |up row| * |down column|`` and dealt round-robin so every expert
    receives strong and weak units; with ``sparsity`` > 0 the weakest fraction is dropped."""

    def __init__(self, hidden: int, n_experts: int, sparsity: float = 0.5):
        self.hidden, self.n_experts, self.sparsity = hidden, n_experts, sparsity

    def prune_ffn(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor):
        score = gate.float().norm(dim=1) * up.float().norm(dim=1) * down.float().norm(dim=0)
        order = torch.argsort(score, descending=True)
        keep = order[: max(self.n_experts, int(round(order.numel() * (1.0 - self.sparsity))))]
        experts = []
        for e in range(self.n_experts):
            idx = keep[e::self.n_experts]
            experts.append({"gate": gate[idx].clone(), "up": up[idx].clone(), "down": down[:, idx].clone(),
                            "units": idx})
        return experts


def save_experts(tensors, path: str) -> None:
    """Expert tensor file: i32 count, then per tensor i32 rank, i64 dims[rank], u8 dtype, raw bytes
    (the host tensor serialisation of the reference, src/tensor.cpp:297-334, with its ``DType``
    numbering: int64 0, uint8 1, float16 5, float32 6; int32 tensors are widened to int64, other
    types stored as float32)."""
    from ..core import serialize_tensor

    with open(path, "wb") as f:
        f.write(struct.pack("<i", len(tensors)))
        for t in tensors:
            if t.dtype in (torch.int32, torch.int16, torch.int8):
                t = t.long()
            f.write(serialize_tensor(t))


def load_experts(path: str) -> list[torch.Tensor]:
    from ..core import OilError, deserialize_tensor

    data = open(path, "rb").read()
    if len(data) < 4:
        raise ValueError(f"{path}: truncated expert file")
    (n,) = struct.unpack_from("<i", data, 0)
    out, off = [], 4
    try:
        for _ in range(n):
            t, off = deserialize_tensor(data, off)
            out.append(t)
    except OilError as e:
        raise ValueError(f"{path}: truncated expert file ({e})") from None
    return out


class ExpertDropout:
    def __init__(self, rate: float = 0.1, seed: int = 0):
        self.rate = rate
        self.gen = torch.Generator().manual_seed(seed)

    def get_active_count(self, total: int) -> int:
        return max(1, int(round(total * (1.0 - self.rate))))

    def get_mask(self, total: int) -> list[bool]:
        keep = torch.randperm(total, generator=self.gen)[: self.get_active_count(total)]
        mask = torch.zeros(total, dtype=torch.bool)
        mask[keep] = True
        return mask.tolist()


@dataclass
class ExpertBalance:
    token_counts: list
    load_balance_loss: float
    stddev: float


def compute_balance(assignments, n_experts: int) -> ExpertBalance:
    """Counts per expert, ``E * sum f_e^2`` (1.0 when uniform) and the standard deviation of the counts."""
    a = torch.as_tensor(assignments).reshape(-1).long()
    counts = torch.bincount(a, minlength=n_experts).float()
    f = counts / counts.sum().clamp_min(1)
    return ExpertBalance(counts.long().tolist(), float(n_experts * (f * f).sum()), float(counts.std(unbiased=False)))


class SwitchV2Router:
    """Top-1 routing with a capacity of ``capacity_factor * tokens / experts`` per expert; overflow
    tokens get index -1 (dropped; the caller passes them through on the residual path)."""

    def __init__(self, n_experts: int, capacity_factor: float = 1.25):
        self.n_experts, self.capacity_factor = n_experts, capacity_factor

    def forward(self, logits: torch.Tensor, tokens: int | None = None):
        T = logits.shape[0] if tokens is None else tokens
        probs = torch.softmax(logits.float(), dim=-1)
        gate, idx = probs.max(dim=-1)
        cap = max(1, int(self.capacity_factor * T / self.n_experts))
        onehot = torch.nn.functional.one_hot(idx, self.n_experts)
        pos = (torch.cumsum(onehot, dim=0) * onehot).sum(-1)            # 1-based arrival order within the expert
        idx = torch.where(pos <= cap, idx, torch.full_like(idx, -1))
        return idx, torch.where(idx >= 0, gate, torch.zeros_like(gate))

    __call__ = forward


class ExpertChoiceV2:
    """Two-sided matching: a (token, expert) pair is kept when the expert is among the token's
    top-k AND the token is among the expert's top-capacity tokens."""

    def __init__(self, n_experts: int, top_k: int = 2, capacity_factor: float = 2.0):
        self.n_experts, self.top_k, self.capacity_factor = n_experts, top_k, capacity_factor

    def forward(self, x: torch.Tensor, logits: torch.Tensor):
        T = logits.shape[0]
        probs = torch.softmax(logits.float(), dim=-1)
        tok_pick = torch.zeros_like(probs, dtype=torch.bool).scatter_(1, probs.topk(min(self.top_k, self.n_experts), 1).indices, True)
        cap = max(1, min(T, int(self.capacity_factor * T * self.top_k / self.n_experts)))
        exp_pick = torch.zeros_like(probs, dtype=torch.bool).scatter_(0, probs.topk(cap, 0).indices, True)
        keep = tok_pick & exp_pick
        return keep, probs * keep

    __call__ = forward


class ExpertMerger:
    """Greedy merging of experts whose flattened weights have cosine similarity above the
    threshold: each group is replaced by its mean."""

    def __init__(self, similarity_threshold: float = 0.9):
        self.threshold = similarity_threshold

    def merge(self, experts):
        flat = [e.float().reshape(-1) for e in experts]
        used = [False] * len(experts)
        out = []
        for i in range(len(experts)):
            if used[i]:
                continue
            group = [i]
            used[i] = True
            for j in range(i + 1, len(experts)):
                if not used[j] and flat[i].numel() == flat[j].numel() and \
                        float(torch.nn.functional.cosine_similarity(flat[i], flat[j], dim=0)) >= self.threshold:
                    group.append(j)
                    used[j] = True
            out.append(torch.stack([experts[g].float() for g in group]).mean(0).to(experts[i].dtype))
        return out


class DynamicExpertPool:
    def __init__(self, initial: int = 0, max_experts: int = 64):
        self.experts: list[torch.Tensor] = []
        self.max_experts = max_experts
        self._initial = initial

    def add_expert(self, weights: torch.Tensor) -> int:
        if len(self.experts) >= self.max_experts:
            return -1
        self.experts.append(weights)
        return len(self.experts) - 1

    def remove_expert(self, idx: int) -> bool:
        if 0 <= idx < len(self.experts) and len(self.experts) > 1:
            del self.experts[idx]
            return True
        return False

    def count(self) -> int:
        return len(self.experts)
