"""Pure-PyTorch restatements of every kernel, written from the reference's formulas.

They run on CPU (and on CUDA tensors through torch operators) and serve two purposes: the
numerical oracle that each sm_100a kernel is tested against, and the execution path of
CPU-only runs (the tiny byte-level configuration). All math is fp32 regardless of the input
dtype; results are cast back to the input dtype.

Formula sources in the reference tree: RMSNorm ``src/math.cpp:182-205``; RoPE
``src/transformer.cpp:108-135``; SiLU / SwiGLU ``src/transformer.cpp:373-387``; attention
``src/autograd.cpp:361-461``; cross-entropy ``src/autograd.cpp:1166-1215``; AdamW
``src/optimizer.cpp:91-119``; nearest-centroid quantisation ``src/codebook.cpp:172-186``;
router ``src/moe_variants.cpp:25-91``; sampler ``src/sampler.cpp:12-120``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x, gamma, eps: float = 1e-5, residual=None):
    """Returns ``(y, h)`` with ``h = x + residual`` (or ``x``) and ``y = rmsnorm(h) * gamma``."""
    h = x.float() if residual is None else (x.float() + residual.float())
    if residual is not None:
        h = h.to(x.dtype).float()  # the kernel normalises the rounded sum
    rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    y = h * rstd * gamma.float()
    return y.to(x.dtype), h.to(x.dtype)


def layernorm(x, gamma, beta=None, eps: float = 1e-5):
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps) * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(x.dtype)


def rope_tables(pos, head_dim: int, theta: float):
    j = torch.arange(head_dim // 2, device=pos.device, dtype=torch.float32)
    inv_freq = theta ** (-2.0 * j / head_dim)
    ang = pos.float()[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)


def rope(x, pos, theta: float = 10000.0, inverse: bool = False):
    """Half-split rotary embedding. x: [tokens, heads, head_dim]; pos: [tokens]."""
    d = x.shape[-1]
    cos, sin = rope_tables(pos, d, theta)
    if inverse:
        sin = -sin
    xf = x.float()
    a, b = xf[..., : d // 2], xf[..., d // 2:]
    cos, sin = cos[:, None, :], sin[:, None, :]
    out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return out.to(x.dtype)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def swiglu(gate_up):
    """gate_up: [..., 2*ffn] with gate in the first half. Returns silu(gate) * up."""
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (silu(g) * u).to(gate_up.dtype)


def relu2(x):
    return torch.relu(x.float()).pow(2).to(x.dtype)


def gelu_erf(x):
    xf = x.float()
    return (0.5 * xf * (1.0 + torch.erf(xf / math.sqrt(2.0)))).to(x.dtype)


def gelu_tanh(x):
    xf = x.float()
    return (0.5 * xf * (1.0 + torch.tanh(0.7978845608028654 * (xf + 0.044715 * xf ** 3)))).to(x.dtype)


def attention(q, k, v, causal: bool = True, scale: float | None = None):
    """Naive softmax(Q K^T * scale) V. q: [B,S,H,D]; k, v: [B,Skv,Hkv,D] (standard GQA grouping:
    query head h uses kv head h // (H/Hkv)). Returns (o [B,S,H,D], lse [B,H,S])."""
    B, S, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, Skv, dtype=torch.bool, device=q.device).tril(diagonal=Skv - S)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def cross_entropy(logits, targets):
    """Per-row loss ``logsumexp - logit[target]`` with targets clamped to [0, V-1]."""
    lf = logits.float()
    t = targets.long().clamp(0, lf.shape[-1] - 1)
    return torch.logsumexp(lf, dim=-1) - lf.gather(-1, t[:, None]).squeeze(-1)


def cross_entropy_grad(logits, targets, grad_scale: float):
    lf = logits.float()
    t = targets.long().clamp(0, lf.shape[-1] - 1)
    p = torch.softmax(lf, dim=-1)
    p.scatter_add_(-1, t[:, None], -torch.ones_like(p[:, :1]))
    return (p * grad_scale).to(logits.dtype)


def adamw_step(p, m, v, g, lr, beta1, beta2, eps, weight_decay, step, grad_scale: float = 1.0):
    """In-place AdamW in the reference's form (decoupled decay, bias-corrected moments)."""
    g = g.float() * grad_scale
    p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    p.addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    return p, m, v


def nearest_centroid(w, codebooks, cb_map, bs: int):
    """Brute-force nearest centroid, first minimum wins. w: flat fp32 [n]; codebooks [n_cb, C];
    cb_map: int [n_blocks] or None (block b uses codebook b). Returns (indices u8, dequantised fp32)."""
    n = w.numel()
    nb = (n + bs - 1) // bs
    pad = nb * bs - n
    wf = F.pad(w.float().reshape(-1), (0, pad)).reshape(nb, bs)
    cbi = torch.arange(nb, device=w.device) if cb_map is None else cb_map.long()
    idx = torch.empty(nb, bs, dtype=torch.uint8, device=w.device)
    deq = torch.empty(nb, bs, dtype=torch.float32, device=w.device)
    step = max(1, (1 << 22) // (bs * codebooks.shape[-1]))
    for s in range(0, nb, step):
        cb = codebooks[cbi[s:s + step]].float()  # [b, C]
        d = (wf[s:s + step, :, None] - cb[:, None, :]).pow(2)
        j = d.argmin(dim=-1)  # torch.argmin returns the first minimum on ties
        idx[s:s + step] = j.to(torch.uint8)
        deq[s:s + step] = torch.gather(cb, 1, j)
    return idx.reshape(-1)[:n], deq.reshape(-1)[:n]


def i2s_quant(w, bs: int):
    """I2_S ternary: per-block absmean scale, trit = clamp(round(w/scale), -1, 1).
    Returns (codes u8 in {0,1,2} = trit+1, scales fp32 [n_blocks], dequantised fp32)."""
    n = w.numel()
    nb = (n + bs - 1) // bs
    pad = nb * bs - n
    wf = F.pad(w.float().reshape(-1), (0, pad)).reshape(nb, bs)
    cnt = torch.full((nb,), bs, dtype=torch.float32, device=w.device)
    if pad:
        cnt[-1] = bs - pad
    a = wf.abs()
    amax = a.amax(-1)
    # a block that already is {-s, 0, +s} keeps s, so quantising twice equals quantising once
    exact = ((a == 0) | (a == amax[:, None])).all(-1)
    scale = torch.where(exact, amax, a.sum(-1) / cnt)
    inv = torch.where(scale > 0, 1.0 / scale, torch.zeros_like(scale))
    t = torch.round(wf * inv[:, None]).clamp(-1, 1)
    deq = t * scale[:, None]
    return (t + 1).to(torch.uint8).reshape(-1)[:n], scale, deq.reshape(-1)[:n]


def router_topk(logits, k: int):
    """softmax over all experts, top-k by probability, weights are those probabilities
    (not renormalised over the chosen k). Returns (weights [T,k], experts [T,k], probs [T,E])."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, e = torch.topk(probs, k, dim=-1)
    return w, e, probs


def load_balance_loss(probs, experts, num_experts: int):
    """E * sum_e f_e * P_e with f_e = fraction of tokens routed to e (any of the k slots) and
    P_e = mean over tokens of the probability of e when chosen."""
    T = probs.shape[0]
    onehot = torch.zeros(T, num_experts, device=probs.device, dtype=torch.float32)
    onehot.scatter_(1, experts, 1.0)
    f = onehot.sum(0) / T
    P = (probs * onehot).sum(0) / T
    return num_experts * (f * P).sum()


def z_loss(logits, coef: float):
    return coef * torch.logsumexp(logits.float(), dim=-1).pow(2).mean()
