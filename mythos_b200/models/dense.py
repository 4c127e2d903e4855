"""Dense decoder-only transformer (the reference's ``DenseModel``, src/model.cpp:10-75).

embedding -> N pre-norm blocks -> RMSNorm -> lm_head. Tensor names follow the reference's
``collect_named_tensors`` (src/model.cpp:80-102) where a one-to-one tensor exists; fused
projections are split into the reference's names when exported (see ``export_named_tensors``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as F
from .config import TransformerConfig
from .layers import Embedding, OILLinear, RMSNorm, TransformerBlock


class DenseModel(nn.Module):
    def __init__(self, cfg: TransformerConfig):
        super().__init__()
        self.cfg = cfg
        # recompute every block's activations in the backward pass instead of keeping them
        # (memory of one block's activations + one [B, S, d] pair per block; one extra forward)
        self.activation_checkpointing = False
        # set by the data-parallel engine around the last backward pass of a step: called with i when
        # the gradients of every parameter in blocks >= i (and of the final norm / head) are complete
        self.grad_ready_callback = None
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([self._make_block(i) for i in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        if cfg.tie_embeddings:
            self.lm_head = None
        else:
            self.lm_head = OILLinear(cfg.hidden_size, cfg.vocab_size, cfg.format_for("head"), cfg.oil_block_size,
                                     cfg.codebook_group)

    def _make_block(self, index: int) -> nn.Module:
        return TransformerBlock(self.cfg)

    # ------------------------------------------------------------------ forward
    def hidden_states(self, ids, pos=None):
        """ids: int32 [B, S]. Returns the final normalised hidden states [B, S, d]."""
        B, S = ids.shape
        if pos is None:
            pos = torch.arange(S, device=ids.device, dtype=torch.int32).repeat(B)
        x = self.tok_embeddings(ids)
        branch, stream = x, None
        cb = self.grad_ready_callback if torch.is_grad_enabled() else None
        for i, blk in enumerate(self.layers):
            if cb is not None and branch.requires_grad:
                # the gradient of block i's input exists once block i (and everything after it) is done
                branch.register_hook(lambda g, i=i: cb(i))
            if self.activation_checkpointing and self.training:
                branch, stream = F.checkpoint(blk, branch, stream, pos)
            else:
                branch, stream = blk(branch, stream, pos)
        if cb is not None and branch.requires_grad:
            branch.register_hook(lambda g, i=len(self.layers): cb(i))
        h, _ = self.norm(branch, stream)
        return h

    def logits(self, h):
        if self.lm_head is not None:
            return self.lm_head(h)
        w = getattr(self.tok_embeddings.weight, "compute", None)
        if w is None:
            w = self.tok_embeddings.weight.to(h.dtype)
        return F.linear(h, w, getattr(self.tok_embeddings.weight, "main_grad", None))

    def forward(self, ids, targets=None, pos=None, loss_scale: float | None = None):
        """Without targets: logits [B, S, V]. With targets (int32 [B, S]): scalar loss
        ``loss_scale * sum(token losses)`` (``loss_scale`` defaults to 1/(B*S), the mean)."""
        h = self.hidden_states(ids, pos)
        lg = self.logits(h)
        if targets is None:
            return lg
        rows = lg.shape[0] * lg.shape[1]
        return F.cross_entropy(lg.reshape(rows, -1), targets.reshape(-1), loss_scale)

    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    # ------------------------------------------------------------------ names for the .oil container
    def export_named_tensors(self):
        """(name, fp32 tensor, module-or-None) in the reference's save order, with fused projections
        split into q/k/v and gate/up so that files use the reference's tensor names."""
        cfg = self.cfg
        out = [("tok_embeddings.weight", self.tok_embeddings.weight, None)]
        for i, blk in enumerate(self.layers):
            p = f"layers.{i}."
            out.append((p + "attention_norm.weight", blk.attention_norm.weight, None))
            out.append((p + "ffn_norm.weight", blk.ffn_norm.weight, None))
            att = blk.attention
            out.append((p + "attention.qkv_proj.weight", att.qkv_proj.weight, att.qkv_proj))
            out.append((p + "attention.o_proj.weight", att.o_proj.weight, att.o_proj))
            for name, mod in _ffn_tensors(blk.ffn):
                out.append((p + name, mod.weight, mod if isinstance(mod, OILLinear) else None))
        out.append(("norm.weight", self.norm.weight, None))
        if self.lm_head is not None:
            out.append(("lm_head.weight", self.lm_head.weight, self.lm_head))
        return out


def _ffn_tensors(ffn):
    if hasattr(ffn, "named_oil_tensors"):
        return list(ffn.named_oil_tensors())
    return [("ffn.up_proj.weight", ffn.up_proj), ("ffn.down_proj.weight", ffn.down_proj)]
