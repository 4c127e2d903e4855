"""Evaluation metrics.

* ``eval_perplexity``: sliding window (context 512, stride 256 by default, src/eval.cpp): each
  window scores only the tokens not scored by the previous window.
* ``eval_accuracy``: next-token top-1 accuracy.
* ``eval_classification``: accuracy and macro precision / recall / F1 from label lists.
* ``compute_bleu`` (uniform 1..4-gram, brevity penalty), ``compute_rouge_l`` (LCS F-measure).
* ``eval_multiple_choice``: HellaSwag-style, the ending with the lowest mean token loss wins.
"""
from __future__ import annotations

import math
from collections import Counter

import torch


def _model_device(model):
    return next(model.parameters()).device


@torch.no_grad()
def _token_losses(model, ids: torch.Tensor) -> torch.Tensor:
    """Per-position next-token losses for one sequence [S] -> [S-1] (fp32, on CPU)."""
    from ..ops import reference as ref

    dev = _model_device(model)
    x = ids[None, :-1].to(dev, torch.int32)
    logits = model(x)
    return ref.cross_entropy(logits[0].float().cpu(), ids[1:].cpu())


@torch.no_grad()
def eval_perplexity(model, tokens, context: int = 512, stride: int = 256) -> dict:
    tokens = torch.as_tensor(tokens, dtype=torch.int32)
    n = tokens.numel()
    total, count, scored_until = 0.0, 0, 1
    start = 0
    while scored_until < n:
        end = min(n, start + context + 1)
        losses = _token_losses(model, tokens[start:end])
        first_new = scored_until - (start + 1)
        total += float(losses[first_new:].sum())
        count += losses.numel() - first_new
        scored_until = end
        if end == n:
            break
        start += stride
    loss = total / max(1, count)
    return {"loss": loss, "perplexity": math.exp(min(loss, 50.0)), "tokens": count}


@torch.no_grad()
def eval_accuracy(model, tokens, context: int = 512) -> float:
    tokens = torch.as_tensor(tokens, dtype=torch.int32)
    dev = _model_device(model)
    hit = tot = 0
    for s in range(0, tokens.numel() - 1, context):
        chunk = tokens[s:s + context + 1]
        if chunk.numel() < 2:
            break
        pred = model(chunk[None, :-1].to(dev)).argmax(-1)[0].cpu()
        hit += int((pred == chunk[1:]).sum())
        tot += chunk.numel() - 1
    return hit / max(1, tot)


def eval_classification(pred, gold, num_classes: int | None = None) -> dict:
    pred, gold = list(pred), list(gold)
    k = num_classes or (max(pred + gold) + 1 if pred else 0)
    acc = sum(int(p == g) for p, g in zip(pred, gold)) / max(1, len(gold))
    ps, rs, fs = [], [], []
    for c in range(k):
        tp = sum(1 for p, g in zip(pred, gold) if p == c and g == c)
        fp = sum(1 for p, g in zip(pred, gold) if p == c and g != c)
        fn = sum(1 for p, g in zip(pred, gold) if p != c and g == c)
        pr = tp / (tp + fp) if tp + fp else 0.0
        rc = tp / (tp + fn) if tp + fn else 0.0
        ps.append(pr)
        rs.append(rc)
        fs.append(2 * pr * rc / (pr + rc) if pr + rc else 0.0)
    return {"accuracy": acc, "precision": sum(ps) / max(1, k), "recall": sum(rs) / max(1, k), "f1": sum(fs) / max(1, k)}


def compute_bleu(candidate, reference, max_n: int = 4) -> float:
    c, r = list(candidate), list(reference)
    if not c:
        return 0.0
    logp = 0.0
    for n in range(1, max_n + 1):
        cg = Counter(tuple(c[i:i + n]) for i in range(len(c) - n + 1))
        rg = Counter(tuple(r[i:i + n]) for i in range(len(r) - n + 1))
        overlap = sum(min(v, rg[g]) for g, v in cg.items())
        total = max(1, sum(cg.values()))
        if overlap == 0:
            return 0.0
        logp += math.log(overlap / total) / max_n
    bp = 1.0 if len(c) > len(r) else math.exp(1 - len(r) / max(1, len(c)))
    return bp * math.exp(logp)


def compute_rouge_l(candidate, reference) -> float:
    c, r = list(candidate), list(reference)
    if not c or not r:
        return 0.0
    dp = [0] * (len(r) + 1)
    for x in c:
        prev = 0
        for j, y in enumerate(r, 1):
            cur = dp[j]
            dp[j] = prev + 1 if x == y else max(dp[j], dp[j - 1])
            prev = cur
    lcs = dp[-1]
    if lcs == 0:
        return 0.0
    p, rec = lcs / len(c), lcs / len(r)
    return 2 * p * rec / (p + rec)


@torch.no_grad()
def eval_multiple_choice(model, items) -> float:
    """items: iterable of (context_ids, [ending_ids, ...], label). Returns accuracy."""
    hit = tot = 0
    for ctx, endings, label in items:
        scores = []
        for e in endings:
            seq = torch.tensor(list(ctx) + list(e), dtype=torch.int32)
            losses = _token_losses(model, seq)
            scores.append(float(losses[len(ctx) - 1:].mean()))
        hit += int(min(range(len(scores)), key=scores.__getitem__) == label)
        tot += 1
    return hit / max(1, tot)


class ModelEvaluator:
    """Runs the metrics that apply to the data given (``run_all`` of the reference)."""

    def __init__(self, model):
        self.model = model

    def run_all(self, tokens=None, choice_items=None, context: int = 512, stride: int = 256) -> dict:
        out = {}
        if tokens is not None:
            out.update(eval_perplexity(self.model, tokens, context, stride))
            out["accuracy"] = eval_accuracy(self.model, tokens, context)
        if choice_items is not None:
            out["multiple_choice_accuracy"] = eval_multiple_choice(self.model, choice_items)
        return out


# Names of the reference's evaluation entry points (src/eval.cpp).
eval_hellaswag = eval_multiple_choice


def load_eval_tokens(path: str, tokenizer=None, max_tokens: int | None = None, vocab_size: int | None = None):
    """Token ids of an evaluation text file: through ``tokenizer`` (anything with ``encode``), else
    its raw bytes; clipped to ``vocab_size`` and truncated to ``max_tokens`` (``load_eval_tokens`` of
    the reference)."""
    import numpy as np

    with open(path, "rb") as f:
        data = f.read()
    ids = np.asarray(tokenizer.encode(data) if tokenizer is not None else list(data), dtype=np.int32)
    if vocab_size:
        ids = np.minimum(ids, vocab_size - 1)
    if max_tokens:
        ids = ids[:max_tokens]
    return torch.from_numpy(ids)
