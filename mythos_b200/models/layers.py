"""Transformer building blocks with train-in-format weights.

``OILLinear`` keeps an fp32 master weight and computes with its fake-quantised image
(straight-through estimator: the backward pass treats quantisation as identity). The reference
declares this capability (``STEQuantizer``, src/ste_quantizer.cpp:19-58; ``TrainConfig::use_ste``,
include/oil/trainer.h:32) but never wires it into training; here it is the training path.

Two ways to obtain the compute weight:

* a :class:`mythos_b200.train.param_store.ParamStore` re-homes all parameters into flat buffers
  and refreshes ``param.compute`` (bf16, quantised) once per optimizer step; gradients accumulate
  in ``param.main_grad`` (fp32) straight from the GEMM epilogue;
* without a store the weight is fake-quantised on every forward and gradients flow to
  ``param.grad`` through autograd (simple, used on CPU and in small tests).

Layer structure follows the reference model (src/transformer.cpp:142-406, src/model.cpp:45-75):
pre-norm blocks, RMSNorm, half-split RoPE, SwiGLU FFN, untied head; deviations are deliberate and
listed in the class docstrings (no biases, standard GQA grouping h // (H/Hkv), fused QKV and
gate/up projections).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..oil import codebook as cbk
from ..ops import functional as F
from .config import TransformerConfig


class _STEQuantFn(torch.autograd.Function):
    """fake_quant(w) forward, identity backward."""

    @staticmethod
    def forward(ctx, w, module):
        return module.quantize_now(w)

    @staticmethod
    def backward(ctx, g):
        return g.float(), None


class OILLinear(nn.Module):
    """Linear layer ``y = x W^T`` (no bias) whose weight lives in an OIL format.

    ``fmt``: ``oil8`` (256 fp32 centroids), ``oil4`` (16 fp16 centroids), ``i2s`` (ternary with a
    per-block absmean scale), ``fp32``/``fp16`` (no quantisation), or ``mixed``: every block has its
    own format among OIL8 / OIL4 / ternary / binary (``block_formats``, one code per block in the container's
    numbering), chosen by the format planner for a target number of bits per weight: the
    reference's ``forward_mixed`` (src/ste_quantizer.cpp:137) with the plan of
    src/format_planner.cpp:59-157. ``block_size`` weights (in row-major order of the [out, in]
    matrix) form one block; ``codebook_group`` consecutive blocks share one codebook.
    """

    def __init__(self, in_features: int, out_features: int, fmt: str = "oil8", block_size: int = 256,
                 codebook_group: int = 1, init_std: float = 0.02, target_bpw: float = 1.5):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.fmt, self.block_size, self.codebook_group = fmt, block_size, max(1, codebook_group)
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        nn.init.normal_(self.weight, mean=0.0, std=init_std)
        n = out_features * in_features
        self.n_blocks = (n + block_size - 1) // block_size
        if fmt != "mixed":
            self.codebooks4 = None
        if fmt == "mixed":
            n_cb = (self.n_blocks + self.codebook_group - 1) // self.codebook_group
            self.register_buffer("codebooks", cbk.quantile_codebook(256, init_std)[None, :].repeat(n_cb, 1).contiguous())
            self.register_buffer("codebooks4", cbk.quantile_codebook(16, init_std, fp16=True)[None, :].repeat(n_cb, 1).contiguous())
            self.register_buffer("cb_map", (torch.arange(self.n_blocks) // self.codebook_group).to(torch.int32))
            self.register_buffer("block_formats", torch.ones(self.n_blocks, dtype=torch.uint8))
            self.target_bpw = float(target_bpw)
            self.replan()
        elif fmt in ("oil8", "oil4"):
            size = 256 if fmt == "oil8" else 16
            n_cb = (self.n_blocks + self.codebook_group - 1) // self.codebook_group
            cb = cbk.quantile_codebook(size, init_std, fp16=(fmt == "oil4"))
            self.register_buffer("codebooks", cb[None, :].repeat(n_cb, 1).contiguous())
            if self.codebook_group > 1:
                self.register_buffer("cb_map", (torch.arange(self.n_blocks) // self.codebook_group).to(torch.int32))
            else:
                self.cb_map = None
        else:
            self.codebooks = None
            self.cb_map = None

    # ------------------------------------------------------------------ quantisation
    @torch.no_grad()
    def replan(self, target_bpw: float | None = None) -> float:
        """(Re)assign a format to every block from the current weights: blocks ranked by importance
        get OIL8, then OIL4, then ternary, so that the average reaches ``target_bpw`` bits per
        weight. Returns the achieved bits per weight."""
        from ..oil import planner

        if self.fmt != "mixed":
            raise ValueError("replan() applies to fmt='mixed' layers")
        if target_bpw is not None:
            self.target_bpw = float(target_bpw)
        fmts, achieved = planner.plan(self.weight.detach().float().cpu(), self.target_bpw, self.block_size)
        self.block_formats.copy_(torch.from_numpy(fmts.astype("uint8")).to(self.block_formats.device))
        return achieved

    def _quantize_mixed(self, w, out=None):
        """Per-block format: the OIL8, OIL4 and ternary images of the whole tensor, selected block by
        block (three fake-quant kernels and two selects; it runs once per optimizer step)."""
        flat = w.reshape(-1)
        bs, n = self.block_size, flat.numel()
        q8, _ = F.oil_fake_quant(flat, self.codebooks, self.cb_map, bs)
        q4, _ = F.oil_fake_quant(flat, self.codebooks4, self.cb_map, bs)
        q2, _, _ = F.i2s_fake_quant(flat, bs)
        code = self.block_formats.to(flat.device).repeat_interleave(bs)[:n]
        q = torch.where(code == 3, q8.reshape(-1), torch.where(code == 2, q4.reshape(-1), q2.reshape(-1)))
        if bool((self.block_formats == 0).any()):
            # binary blocks: sign(w) * mean|w| of the block, bit = w > 0 (engines/OIL8/quantize.cpp:148-164)
            nb = (n + bs - 1) // bs
            pad = nb * bs - n
            a = torch.nn.functional.pad(flat.float(), (0, pad)).view(nb, bs)
            cnt = torch.full((nb, 1), float(bs), device=flat.device)
            if pad:
                cnt[-1] = bs - pad
            sc = a.abs().sum(1, keepdim=True) / cnt
            q1 = torch.where(a > 0, sc, -sc).reshape(-1)[:n].to(q.dtype)
            q = torch.where(code == 0, q1, q)
        if out is not None:
            out.copy_(q)
            return out
        return q.view(w.shape)

    def quantize_now(self, w, out=None):
        """Fake-quantised image of ``w`` (bf16 on CUDA, fp32 on CPU)."""
        if self.fmt == "mixed":
            return self._quantize_mixed(w, out)
        if self.fmt in ("oil8", "oil4"):
            q, _ = F.oil_fake_quant(w, self.codebooks, self.cb_map, self.block_size, out=out)
            return q
        if self.fmt == "i2s":
            q, _, _ = F.i2s_fake_quant(w, self.block_size, out=out)
            return q
        if out is not None:
            out.copy_(w.reshape(-1))
            return out
        return w.to(torch.bfloat16) if w.is_cuda else w

    def compute_weight(self):
        c = getattr(self.weight, "compute", None)
        if c is not None:
            return c
        if torch.is_grad_enabled() and self.weight.requires_grad:
            return _STEQuantFn.apply(self.weight, self)
        if not self.weight.requires_grad:
            # frozen base (LoRA fine-tuning, evaluation): quantise once and keep the image
            key = (self.weight.data_ptr(), self.weight._version, self.weight.device)
            cached = getattr(self, "_frozen_image", None)
            if cached is None or cached[0] != key:
                cached = (key, self.quantize_now(self.weight.detach()))
                self._frozen_image = cached
            return cached[1]
        return self.quantize_now(self.weight.detach())

    def forward(self, x):
        return F.linear(x, self.compute_weight(), getattr(self.weight, "main_grad", None))

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, fmt={self.fmt}, block={self.block_size}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def _gamma(self, x):
        c = getattr(self.weight, "compute", None)
        if c is not None:
            return c
        return self.weight.to(x.dtype) if x.is_cuda else self.weight

    def forward(self, x, residual=None):
        """Returns ``(normed, h)`` with ``h = x + residual`` (the new residual stream)."""
        return F.rmsnorm(x, self._gamma(x), self.eps, residual, getattr(self.weight, "main_grad", None))


class Embedding(nn.Module):
    def __init__(self, vocab: int, dim: int, init_std: float = 0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim))
        nn.init.normal_(self.weight, mean=0.0, std=init_std)

    def forward(self, ids):
        c = getattr(self.weight, "compute", None)
        if c is not None:
            return F.embedding(ids, c, getattr(self.weight, "main_grad", None))
        if self.weight.is_cuda:
            return F.embedding(ids, self.weight.to(torch.bfloat16))
        return F.embedding(ids, self.weight)


class Attention(nn.Module):
    """Causal self-attention with fused QKV projection, half-split RoPE and GQA.

    Differences from the reference ``Attention`` (src/transformer.cpp:142-362): no biases; query
    head h reads kv head ``h // (H/Hkv)`` (the reference uses ``h % Hkv``); the S x S score matrix
    is never materialised."""

    def __init__(self, cfg: TransformerConfig):
        super().__init__()
        self.cfg = cfg
        fmt = cfg.format_for("attn")
        d = cfg.hidden_size
        self.qkv_proj = OILLinear(d, cfg.q_dim + 2 * cfg.kv_dim, fmt, cfg.oil_block_size, cfg.codebook_group)
        self.o_proj = OILLinear(cfg.q_dim, d, fmt, cfg.oil_block_size, cfg.codebook_group,
                                init_std=0.02 / math.sqrt(2 * cfg.num_layers))

    def forward(self, x, pos):
        cfg = self.cfg
        w = self.qkv_proj.compute_weight() if type(self.qkv_proj) is OILLinear else None   # not an adapter wrapper
        if w is not None and F.fused_rope_ok(x, w, cfg.head_dim, cfg.rope_theta) and x.shape[-2] <= cfg.max_seq_len:
            # RoPE in the epilogue of the projection GEMM; positions are below max_seq_len
            qkv = F.linear_rope(x, w, getattr(self.qkv_proj.weight, "main_grad", None), pos, cfg.rope_theta,
                                cfg.q_dim + cfg.kv_dim, cfg.max_seq_len)
            o = F.attention_qkv(qkv, pos, cfg.num_heads, cfg.kv_heads, cfg.head_dim, cfg.rope_theta, True,
                                rope_applied=True, rope_max_pos=cfg.max_seq_len)
        else:
            qkv = self.qkv_proj(x)
            o = F.attention_qkv(qkv, pos, cfg.num_heads, cfg.kv_heads, cfg.head_dim, cfg.rope_theta, True)
        return self.o_proj(o)


class FFN(nn.Module):
    """Gated FFN ``down(act(gate(x)) * up(x))`` with gate and up fused into one projection
    (reference: src/transformer.cpp:373-387). ``activation``: silu (SwiGLU) or relu2 (squared
    ReLU gate, BitNet style). ``gated=False`` gives ``down(act(up(x)))``."""

    def __init__(self, cfg: TransformerConfig, ffn_hidden: int | None = None):
        super().__init__()
        self.cfg = cfg
        f = ffn_hidden or cfg.ffn_hidden_size
        fmt = cfg.format_for("ffn")
        self.gated = cfg.gated_ffn
        self.act = cfg.activation
        self.up_proj = OILLinear(cfg.hidden_size, (2 if self.gated else 1) * f, fmt, cfg.oil_block_size,
                                 cfg.codebook_group)
        self.down_proj = OILLinear(f, cfg.hidden_size, fmt, cfg.oil_block_size, cfg.codebook_group,
                                   init_std=0.02 / math.sqrt(2 * cfg.num_layers))

    def forward(self, x):
        if self.gated and self.act != "relu2" and type(self.up_proj) is OILLinear and type(self.down_proj) is OILLinear:
            w_gu, w_down = self.up_proj.compute_weight(), self.down_proj.compute_weight()
            if F.fused_ffn_ok(x, w_gu, w_down):
                return F.swiglu_ffn(x, w_gu, w_down, getattr(self.up_proj.weight, "main_grad", None),
                                    getattr(self.down_proj.weight, "main_grad", None))
        u = self.up_proj(x)
        if self.gated:
            if self.act == "relu2":
                f = u.shape[-1] // 2
                h = F.relu2(u[..., :f].contiguous()) * u[..., f:]
            else:
                h = F.swiglu(u)
        else:
            h = F.relu2(u) if self.act == "relu2" else F.activation(u, self.act)
        return self.down_proj(h)


class TransformerBlock(nn.Module):
    """Pre-norm block. The residual add is fused into the following RMSNorm, so the block takes
    and returns the pair (branch output, residual stream)."""

    def __init__(self, cfg: TransformerConfig, ffn: nn.Module | None = None):
        super().__init__()
        self.attention_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.attention = Attention(cfg)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.ffn = ffn if ffn is not None else FFN(cfg)

    def forward(self, branch, stream, pos):
        n, stream = self.attention_norm(branch, stream)
        a = self.attention(n, pos)
        n, stream = self.ffn_norm(a, stream)
        out = self.ffn(n)
        return out, stream
