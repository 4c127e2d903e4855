"""Vocabulary-parallel cross-entropy: the lm_head is split by rows (vocabulary) over the ranks of
a tensor-parallel group, each rank holds ``logits[:, v0:v1]`` and no rank ever materialises a
full row.

Same loss as the reference's ``cross_entropy_loss`` / ``cross_entropy_grad`` (src/autograd.cpp:
1166-1215: mean over rows of ``logsumexp - logit[target]``, targets clamped to the vocabulary,
gradient ``(softmax - onehot) / rows``); the reference has no sharded form.

Per rank: one kernel pass over the local columns writes a 12-byte record per row (local max, local
sum of exponentials, target logit when this shard owns the target). The records are exchanged
(``all_gather`` of ``rows x 3`` floats: 12 bytes per row and rank, against ``2 V / W`` bytes per row
for gathering logits), merged into the global log-sum-exp, and a second pass overwrites the local
logits with their gradient, so backward costs nothing. On CPU tensors the same algebra runs with
torch ops (gloo groups; used by the tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import native


def shard_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_offset: int, vocab_total: int) -> torch.Tensor:
    """[rows, 3] fp32 records {local max, sum exp(x - local max), owned target logit or 0}."""
    rows, v = logits.shape
    if logits.is_cuda:
        stats = torch.empty(rows, 3, device=logits.device, dtype=torch.float32)
        native.require().cross_entropy_shard_stats(logits, targets, stats, vocab_offset, vocab_total)
        return stats
    x = logits.float()
    m = x.max(dim=1).values
    s = torch.exp(x - m[:, None]).sum(dim=1)
    local = targets.long().clamp(0, vocab_total - 1) - vocab_offset
    owned = (local >= 0) & (local < v)
    t = torch.where(owned, x.gather(1, local.clamp(0, v - 1)[:, None])[:, 0], torch.zeros_like(m))
    return torch.stack([m, s, t], dim=1)


def merge_stats(all_stats: torch.Tensor):
    """``all_stats`` [W, rows, 3] -> (lse [rows], target_logit [rows])."""
    m, s, t = all_stats[..., 0], all_stats[..., 1], all_stats[..., 2]
    gm = m.max(dim=0).values
    gs = (s * torch.exp(m - gm[None])).sum(dim=0)
    return gm + torch.log(gs), t.sum(dim=0)


def shard_grad_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, vocab_offset: int, vocab_total: int,
                grad_scale: float) -> torch.Tensor:
    """Overwrite the local logits with ``(exp(x - lse) - onehot) * grad_scale``."""
    rows, v = logits.shape
    if logits.is_cuda:
        native.require().cross_entropy_shard_grad(logits, targets, lse.contiguous(), vocab_offset, vocab_total,
                                                  grad_scale)
        return logits
    g = torch.exp(logits.float() - lse[:, None])
    local = targets.long().clamp(0, vocab_total - 1) - vocab_offset
    owned = (local >= 0) & (local < v)
    r = torch.arange(rows)[owned]
    g[r, local[owned]] -= 1.0
    logits.copy_((g * grad_scale).to(logits.dtype))
    return logits


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, group, vocab_offset, vocab_total, grad_scale):
        world = dist.get_world_size(group) if group is not None else 1
        stats = shard_stats(logits, targets, vocab_offset, vocab_total)
        if world > 1:
            flat = torch.empty(world * stats.shape[0], 3, device=stats.device, dtype=stats.dtype)
            dist.all_gather_into_tensor(flat, stats, group=group)       # rank-major concatenation
            gathered = flat.view(world, stats.shape[0], 3)
        else:
            gathered = stats[None]
        lse, tgt = merge_stats(gathered)
        loss = (lse - tgt).sum() * grad_scale
        shard_grad_(logits, targets, lse, vocab_offset, vocab_total, grad_scale)
        ctx.save_for_backward(logits)
        return loss

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits, None, None, None, None, None


def vocab_parallel_cross_entropy(logits_shard: torch.Tensor, targets: torch.Tensor, group=None,
                                 vocab_offset: int | None = None, vocab_total: int | None = None,
                                 grad_scale: float | None = None) -> torch.Tensor:
    """``grad_scale * sum_rows(logsumexp - logit[target])`` (mean over rows by default) for logits
    sharded by columns over ``group``. Every rank gets the same loss. ``logits_shard`` [rows, V/W]
    is consumed: it holds its own gradient afterwards, and the upstream gradient must be 1.
    ``vocab_offset`` defaults to ``rank * V/W`` and ``vocab_total`` to ``W * V/W``."""
    world = dist.get_world_size(group) if group is not None else 1
    rank = dist.get_rank(group) if group is not None else 0
    v = logits_shard.shape[1]
    vocab_offset = rank * v if vocab_offset is None else vocab_offset
    vocab_total = world * v if vocab_total is None else vocab_total
    gs = (1.0 / logits_shard.shape[0]) if grad_scale is None else grad_scale
    return _VocabParallelCE.apply(logits_shard, targets, group, vocab_offset, vocab_total, gs)
