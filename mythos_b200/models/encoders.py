"""Modality encoders: vision (ViT patches, DETR-style object queries, scene-graph relations, video
frames), audio (mel frames), OCR patches, video tubelets, sinusoidal text, and a sentence embedder.

All encoders share one bidirectional transformer stack (pre-norm, LayerNorm, GELU MLP). On CUDA in
bf16 inference the stack uses this framework's kernels: LayerNorm, the tcgen05 GEMMs, GELU and
the flash-attention forward kernel with the causal mask off; with autograd on, or on CPU, the
same math runs through torch so the encoders can be trained. Weights are N(0, 0.02).

Reference counterparts (forward only, all weights zero-initialised there):
engines/trainer/moe/vision/vision.cpp:27-391 (``VisionEncoder``, ``ObjectDetector``,
``SceneGraphEncoder``), engines/trainer/moe/{audio,embeddings,image,ocr,text,video}/*.cpp
(``AudioEncoder``, ``SentenceEmbedder``, ``ViTEncoder``, ``OCREncoder``, ``TextEncoder``,
``VideoEncoder``).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import reference as ref


def _lin(i: int, o: int, bias: bool = True) -> nn.Linear:
    m = nn.Linear(i, o, bias=bias)
    nn.init.normal_(m.weight, std=0.02)
    if bias:
        nn.init.zeros_(m.bias)
    return m


def _native_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled()


def _proj(lin: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    if _native_ok(x) and x.shape[-1] % 8 == 0 and lin.out_features % 8 == 0:
        y = F.gemm(x.reshape(-1, x.shape[-1]).contiguous(), lin.weight.to(torch.bfloat16)).view(*x.shape[:-1], -1)
        return y if lin.bias is None else y + lin.bias.to(y.dtype)
    return torch.nn.functional.linear(x, lin.weight.to(x.dtype), None if lin.bias is None else lin.bias.to(x.dtype))


def attention(q, k, v, heads: int) -> torch.Tensor:
    """Bidirectional multi-head attention on [B, S, d] / [B, Skv, d] streams."""
    B, S, d = q.shape
    D = d // heads
    q4, k4, v4 = (t.reshape(B, t.shape[1], heads, D) for t in (q, k, v))
    if _native_ok(q) and D in (64, 128):
        o, _ = F.flash_attention(q4.contiguous(), k4.contiguous(), v4.contiguous(), causal=False)
    else:
        o, _ = ref.attention(q4, k4, v4, causal=False)
    return o.reshape(B, S, d)


class EncoderBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.heads = heads
        self.n1_w, self.n1_b = nn.Parameter(torch.ones(dim)), nn.Parameter(torch.zeros(dim))
        self.n2_w, self.n2_b = nn.Parameter(torch.ones(dim)), nn.Parameter(torch.zeros(dim))
        self.qkv, self.o = _lin(dim, 3 * dim), _lin(dim, dim)
        hidden = int(dim * mlp_ratio)
        self.fc1, self.fc2 = _lin(dim, hidden), _lin(hidden, dim)

    def forward(self, x, context=None):
        h = F.layernorm(x, self.n1_w.to(x.dtype), self.n1_b.to(x.dtype))
        if context is None:
            q, k, v = _proj(self.qkv, h).chunk(3, dim=-1)
        else:  # cross-attention: queries from x, keys/values from the context stream
            d = x.shape[-1]
            q = torch.nn.functional.linear(h, self.qkv.weight[:d].to(h.dtype), self.qkv.bias[:d].to(h.dtype))
            kv = torch.nn.functional.linear(context, self.qkv.weight[d:].to(h.dtype), self.qkv.bias[d:].to(h.dtype))
            k, v = kv.chunk(2, dim=-1)
        x = x + _proj(self.o, attention(q, k, v, self.heads))
        h = F.layernorm(x, self.n2_w.to(x.dtype), self.n2_b.to(x.dtype))
        h = _proj(self.fc1, h)
        h = F.activation(h, "gelu") if _native_ok(h) else torch.nn.functional.gelu(h)
        return x + _proj(self.fc2, h)


class EncoderStack(nn.Module):
    def __init__(self, dim: int, layers: int, heads: int):
        super().__init__()
        self.blocks = nn.ModuleList([EncoderBlock(dim, heads) for _ in range(layers)])
        self.norm_w, self.norm_b = nn.Parameter(torch.ones(dim)), nn.Parameter(torch.zeros(dim))

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return F.layernorm(x, self.norm_w.to(x.dtype), self.norm_b.to(x.dtype))


def patchify(images: torch.Tensor, patch: int) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/p)(W/p), C*p*p], channel-major inside a patch."""
    B, C, H, W = images.shape
    x = images.reshape(B, C, H // patch, patch, W // patch, patch)
    return x.permute(0, 2, 4, 1, 3, 5).reshape(B, (H // patch) * (W // patch), C * patch * patch)


class ViTEncoder(nn.Module):
    """Patch embedding + class token + learned positions + encoder stack; returns [B, 1+N, d]."""

    def __init__(self, img_size: int = 224, patch_size: int = 16, hidden: int = 768, layers: int = 12, heads: int = 12,
                 channels: int = 3):
        super().__init__()
        self.patch = patch_size
        n = (img_size // patch_size) ** 2
        self.patch_embed = _lin(channels * patch_size * patch_size, hidden)
        self.cls = nn.Parameter(torch.zeros(1, 1, hidden))
        self.pos = nn.Parameter(torch.randn(1, n + 1, hidden) * 0.02)
        self.stack = EncoderStack(hidden, layers, heads)

    def forward(self, images):
        x = _proj(self.patch_embed, patchify(images, self.patch))
        x = torch.cat([self.cls.to(x.dtype).expand(x.shape[0], -1, -1), x], dim=1)
        n = x.shape[1]
        pos = self.pos if n <= self.pos.shape[1] else torch.cat(
            [self.pos, self.pos[:, -1:].expand(-1, n - self.pos.shape[1], -1)], dim=1)   # clamp like the reference
        return self.stack(x + pos[:, :n].to(x.dtype))


class VisionEncoder(ViTEncoder):
    """ViT over images; ``forward_video`` encodes frames independently, adds a temporal position
    per frame and returns [B, T, 1+N, d]."""

    def __init__(self, *a, max_frames: int = 64, **k):
        super().__init__(*a, **k)
        self.temporal = nn.Parameter(torch.randn(max_frames, self.pos.shape[-1]) * 0.02)

    def forward_video(self, video):
        B, T = video.shape[:2]
        f = self.forward(video.reshape(B * T, *video.shape[2:])).view(B, T, -1, self.pos.shape[-1])
        return f + self.temporal[:T].to(f.dtype)[None, :, None, :]


class ObjectDetector(nn.Module):
    """DETR-like head: ``num_queries`` learned queries cross-attend over visual features, then a
    class head (incl. "no object") and a sigmoid box head (cx, cy, w, h)."""

    def __init__(self, hidden: int = 768, heads: int = 12, num_queries: int = 100, num_classes: int = 91,
                 layers: int = 2):
        super().__init__()
        self.queries = nn.Parameter(torch.randn(1, num_queries, hidden) * 0.02)
        self.blocks = nn.ModuleList([EncoderBlock(hidden, heads) for _ in range(layers)])
        self.cls_head, self.box_head = _lin(hidden, num_classes + 1), _lin(hidden, 4)

    def forward(self, visual_features):
        q = self.queries.to(visual_features.dtype).expand(visual_features.shape[0], -1, -1)
        for b in self.blocks:
            q = b(q, context=visual_features)
        return {"features": q, "logits": self.cls_head(q), "boxes": torch.sigmoid(self.box_head(q))}


class SceneGraphEncoder(nn.Module):
    """Relation scores for every ordered object pair from concatenated features (+ optional
    spatial edge features): [B, N, d] -> [B, N, N, num_relations]."""

    def __init__(self, hidden: int = 768, num_relations: int = 50, edge_dim: int = 4):
        super().__init__()
        self.edge_dim = edge_dim
        self.pair = _lin(2 * hidden + edge_dim, hidden)
        self.rel = _lin(hidden, num_relations)

    def forward(self, object_features, spatial_edges=None):
        B, N, d = object_features.shape
        a = object_features[:, :, None, :].expand(B, N, N, d)
        b = object_features[:, None, :, :].expand(B, N, N, d)
        if spatial_edges is None:
            spatial_edges = object_features.new_zeros(B, N, N, self.edge_dim)
        return self.rel(torch.nn.functional.gelu(self.pair(torch.cat([a, b, spatial_edges], dim=-1))))


class AudioEncoder(nn.Module):
    """Mel spectrogram [B, n_mels, T] -> per-frame projection + positions (clamped at 1024) -> stack."""

    def __init__(self, n_mels: int = 80, hidden: int = 512, layers: int = 6, heads: int = 8, max_pos: int = 1024):
        super().__init__()
        self.proj = _lin(n_mels, hidden)
        self.pos = nn.Parameter(torch.randn(max_pos, hidden) * 0.02)
        self.stack = EncoderStack(hidden, layers, heads)

    def forward(self, spectrogram):
        x = _proj(self.proj, spectrogram.transpose(1, 2))
        idx = torch.arange(x.shape[1], device=x.device).clamp_max(self.pos.shape[0] - 1)
        return self.stack(x + self.pos[idx].to(x.dtype))


class OCREncoder(nn.Module):
    """16x16 patches of a page image -> projection + positions -> stack (character-level features)."""

    def __init__(self, hidden: int = 512, layers: int = 4, heads: int = 8, patch_size: int = 16, max_pos: int = 4096,
                 channels: int = 3):
        super().__init__()
        self.patch = patch_size
        self.proj = _lin(channels * patch_size * patch_size, hidden)
        self.pos = nn.Parameter(torch.randn(max_pos, hidden) * 0.02)
        self.stack = EncoderStack(hidden, layers, heads)

    def forward(self, image):
        x = _proj(self.proj, patchify(image, self.patch))
        idx = torch.arange(x.shape[1], device=x.device).clamp_max(self.pos.shape[0] - 1)
        return self.stack(x + self.pos[idx].to(x.dtype))


class VideoEncoder(nn.Module):
    """Tubelet embedding: ``tube_size`` consecutive frames x one spatial patch form a token.
    [B, T, C, H, W] -> [B, (T/tube)*(H/p)*(W/p), d]."""

    def __init__(self, tube_size: int = 2, img_size: int = 224, patch_size: int = 16, hidden: int = 768,
                 layers: int = 4, heads: int = 12, channels: int = 3, max_tubes: int = 8192):
        super().__init__()
        self.tube, self.patch = tube_size, patch_size
        self.proj = _lin(channels * tube_size * patch_size * patch_size, hidden)
        self.pos = nn.Parameter(torch.randn(max_tubes, hidden) * 0.02)
        self.stack = EncoderStack(hidden, layers, heads)

    def forward(self, video):
        B, T, C, H, W = video.shape
        t, p = self.tube, self.patch
        x = video.reshape(B, T // t, t, C, H // p, p, W // p, p).permute(0, 1, 4, 6, 3, 2, 5, 7)
        x = _proj(self.proj, x.reshape(B, (T // t) * (H // p) * (W // p), C * t * p * p))
        idx = torch.arange(x.shape[1], device=x.device).clamp_max(self.pos.shape[0] - 1)
        return self.stack(x + self.pos[idx].to(x.dtype))


def sinusoidal_positions(n: int, dim: int, device=None) -> torch.Tensor:
    pos = torch.arange(n, device=device, dtype=torch.float32)[:, None]
    inv = torch.exp(torch.arange(0, dim, 2, device=device, dtype=torch.float32) * (-math.log(10000.0) / dim))
    pe = torch.zeros(n, dim, device=device)
    pe[:, 0::2] = torch.sin(pos * inv)
    pe[:, 1::2] = torch.cos(pos * inv)[:, : dim // 2]
    return pe


class TextEncoder(nn.Module):
    """Token embedding + fixed sinusoidal positions + encoder stack."""

    def __init__(self, vocab: int = 32000, hidden: int = 512, layers: int = 4, heads: int = 8):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        nn.init.normal_(self.embed.weight, std=0.02)
        self.stack = EncoderStack(hidden, layers, heads)

    def forward(self, input_ids):
        x = self.embed(input_ids.long())
        return self.stack(x + sinusoidal_positions(x.shape[1], x.shape[2], x.device).to(x.dtype))


class SentenceEmbedder(nn.Module):
    """Mean-pool token embeddings over the sequence, project, L2-normalise."""

    def __init__(self, hidden: int = 512, output: int = 256, normalize: bool = True):
        super().__init__()
        self.projection = _lin(hidden, output, bias=False)
        self.normalize = normalize

    def forward(self, token_embeddings, mask=None):
        if mask is None:
            pooled = token_embeddings.mean(dim=1)
        else:
            m = mask.to(token_embeddings.dtype)[..., None]
            pooled = (token_embeddings * m).sum(1) / m.sum(1).clamp_min(1)
        out = self.projection(pooled)
        return torch.nn.functional.normalize(out, dim=-1) if self.normalize else out
