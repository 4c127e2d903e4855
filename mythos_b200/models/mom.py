"""Mixture-of-modalities block: modality classifier, modality-biased router, expert FFN bank,
cross-modal attention, and the block that chains them.

Counterparts in the reference: ``ModalityClassifier``, ``MoERouter`` (gate GEMM plus
``+10 * p(modality)`` on the experts of each modality group, softmax, top-k, load-balance
``E * sum f_i P_i`` and z-loss ``coef * mean(lse^2)``), ``MoEFFN``, ``CrossModalAttention`` and
``MoMBlock`` (engines/trainer/moe/moe.cpp:47-153, 199-213, 231-304, 318-340; defaults 16 experts,
top-3, aux 0.01, z 0.001 in moe.h:39-53). The reference runs one expert FFN call per token and
per k and has no backward; here tokens are batched per expert and everything is differentiable.
Weights are N(0, 0.02) instead of the reference's all-zero gates, which route every token to the
same experts.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .config import TransformerConfig
from .layers import Attention, RMSNorm
from .moe_variants import ExpertFFN, compute_load_balance_loss, compute_z_loss, moe_dispatch_batched

MODALITY_NAMES = ("TEXT", "VISION", "IMAGE_GEN", "VIDEO_GEN", "AUDIO", "OCR", "EMBEDDING", "CROSS_MODAL",
                  "META_COGNITION")


@dataclass
class MoMConfig:
    num_experts: int = 16
    top_k: int = 3
    expert_hidden_size: int = 2048
    load_balance_coef: float = 0.01
    z_loss_coef: float = 0.001
    text_experts: int = 4
    vision_experts: int = 3
    image_gen_experts: int = 2
    video_gen_experts: int = 2
    audio_experts: int = 2
    ocr_experts: int = 1
    cross_modal_experts: int = 2
    modality_bias: float = 10.0

    def groups(self):
        """(modality index, expert count) in expert order; modalities without experts are skipped."""
        order = [(0, self.text_experts), (1, self.vision_experts), (2, self.image_gen_experts),
                 (3, self.video_gen_experts), (4, self.audio_experts), (5, self.ocr_experts),
                 (7, self.cross_modal_experts)]
        return [(m, c) for m, c in order if c > 0]


@dataclass
class RouterOutput:
    gates: torch.Tensor            # [T, E] softmax over the biased logits
    indices: torch.Tensor          # [T, K]
    weights: torch.Tensor          # [T, K]
    modality_probs: torch.Tensor   # [T, M]
    dominant_modality: int
    load_balance_loss: torch.Tensor
    z_loss: torch.Tensor


class ModalityClassifier(nn.Module):
    def __init__(self, hidden_size: int, num_modalities: int = len(MODALITY_NAMES)):
        super().__init__()
        self.head = nn.Linear(hidden_size, num_modalities, bias=False)
        nn.init.normal_(self.head.weight, std=0.02)

    def forward(self, x):
        return self.head(x)

    @staticmethod
    def predict_modality(logits) -> int:
        """Most frequent arg-max modality over the tokens."""
        return int(torch.bincount(logits.reshape(-1, logits.shape[-1]).argmax(-1)).argmax())


class MoMRouter(nn.Module):
    def __init__(self, hidden_size: int, cfg: MoMConfig):
        super().__init__()
        self.cfg = cfg
        total = sum(c for _, c in cfg.groups())
        if total != cfg.num_experts:
            raise ValueError(f"modality allocation sums to {total}, expected {cfg.num_experts} experts")
        self.gate = nn.Linear(hidden_size, cfg.num_experts, bias=False)
        nn.init.normal_(self.gate.weight, std=0.02)
        self.modality_cls = ModalityClassifier(hidden_size)
        owner = torch.cat([torch.full((c,), m) for m, c in cfg.groups()]).long()
        self.register_buffer("expert_modality", owner)

    def forward(self, x, modality_hints=None) -> RouterOutput:
        xf = x.reshape(-1, x.shape[-1])
        m_logits = self.modality_cls(xf)
        if modality_hints is not None:
            m_probs = torch.nn.functional.one_hot(modality_hints.reshape(-1).long(), len(MODALITY_NAMES)).float()
        else:
            m_probs = torch.softmax(m_logits.float(), dim=-1)
        logits = self.gate(xf).float() + self.cfg.modality_bias * m_probs[:, self.expert_modality]
        gates = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(gates, min(self.cfg.top_k, gates.shape[-1]), dim=-1)
        lb = self.cfg.load_balance_coef * compute_load_balance_loss(logits, idx, self.cfg.num_experts)
        zl = self.cfg.z_loss_coef * compute_z_loss(logits)
        return RouterOutput(gates, idx, w, m_probs, ModalityClassifier.predict_modality(m_probs), lb, zl)


class MoMFFN(nn.Module):
    def __init__(self, hidden_size: int, cfg: MoMConfig):
        super().__init__()
        self.experts = nn.ModuleList([ExpertFFN(hidden_size, cfg.expert_hidden_size) for _ in range(cfg.num_experts)])

    def forward(self, x, route: RouterOutput):
        xf = x.reshape(-1, x.shape[-1])
        y, _ = moe_dispatch_batched(xf, self.experts, route.indices, route.weights.to(xf.dtype))
        return y.view_as(x)


class CrossModalAttention(nn.Module):
    """Queries from one stream attend over a second stream (keys/values), multi-head, no mask."""

    def __init__(self, hidden_size: int, num_heads: int):
        super().__init__()
        self.h, self.d = num_heads, hidden_size // num_heads
        self.q = nn.Linear(hidden_size, hidden_size, bias=False)
        self.kv = nn.Linear(hidden_size, 2 * hidden_size, bias=False)
        self.o = nn.Linear(hidden_size, hidden_size, bias=False)
        for lin in (self.q, self.kv, self.o):
            nn.init.normal_(lin.weight, std=0.02)

    def forward(self, x, context):
        B, S, _ = x.shape
        q = self.q(x).view(B, S, self.h, self.d).transpose(1, 2)
        k, v = self.kv(context).view(B, context.shape[1], 2, self.h, self.d).permute(2, 0, 3, 1, 4)
        att = torch.softmax((q @ k.transpose(-1, -2)).float() / self.d ** 0.5, dim=-1).to(v.dtype)
        return self.o((att @ v).transpose(1, 2).reshape(B, S, -1))


class MoMBlock(nn.Module):
    """``x + attn(norm x)`` -> router -> ``+ experts(norm x)`` -> ``+ cross-attn(norm x, context)``
    (the last step only when a context stream is given)."""

    def __init__(self, cfg: TransformerConfig, mom: MoMConfig | None = None):
        super().__init__()
        self.mom = mom or MoMConfig(expert_hidden_size=cfg.ffn_hidden_size)
        d = cfg.hidden_size
        self.attn_norm, self.ffn_norm, self.cross_norm = RMSNorm(d, cfg.norm_eps), RMSNorm(d, cfg.norm_eps), \
            RMSNorm(d, cfg.norm_eps)
        self.attention = Attention(cfg)
        self.router = MoMRouter(d, self.mom)
        self.moe = MoMFFN(d, self.mom)
        self.cross = CrossModalAttention(d, cfg.num_heads)
        self.last_route: RouterOutput | None = None

    def forward(self, x, pos=None, modality_hints=None, context=None):
        B, S, _ = x.shape
        if pos is None:
            pos = torch.arange(S, device=x.device, dtype=torch.int32).repeat(B)
        # RMSNorm returns (normed, residual stream); the stream is kept explicitly here
        x = x + self.attention(self.attn_norm(x)[0], pos)
        h = self.ffn_norm(x)[0]
        self.last_route = self.router(h, modality_hints)
        x = x + self.moe(h, self.last_route)
        if context is not None:
            x = x + self.cross(self.cross_norm(x)[0], context)
        return x

    def aux_loss(self):
        r = self.last_route
        return r.load_balance_loss + r.z_loss if r is not None else 0.0
