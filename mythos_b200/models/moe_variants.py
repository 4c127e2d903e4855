"""Mixture-of-experts layer variants sharing one batched dispatch.

Every variant is an ``nn.Module`` whose ``forward`` returns a :class:`MoEOutput`. Tokens are grouped
per expert (one FFN call per expert on its token batch, weighted scatter-add back), which is the
semantics of the reference's ``moe_dispatch_batched`` (src/moe_variants.cpp:695-755); routing
helpers follow ``softmax_with_topk`` (:25-62: softmax over all experts, top-k weights NOT
renormalised), ``compute_load_balance_loss`` (:68-91: ``E * sum_e f_e * P_e``) and ``compute_z_loss``.
The 25 variants correspond to include/oil/moe_variants.h:195-600. The reference's factory returns
a null pointer for every variant (:1535-1538); :func:`create_moe` builds them.

The five "quantised" variants of the reference quantise expert *outputs* (:1333-1520); here they
quantise the expert *weights* with a straight-through estimator, which is what the names say.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as tF

from ..ops import reference as ref


@dataclass
class MoEAllConfig:
    variant: str = "sparse_topk"
    num_experts: int = 16
    top_k: int = 2
    expert_hidden_size: int = 2048
    load_balance_coef: float = 0.01
    z_loss_coef: float = 0.001
    num_groups: int = 4
    experts_per_group: int = 4
    top_groups: int = 2
    top_experts_per_group: int = 1
    group_load_balance_coef: float = 0.005
    num_slots_per_expert: int = 1
    capacity_factor: float = 2.0
    hash_bucket_size: int = 2
    num_shared_layers: int = 4
    num_tasks: int = 1
    num_shared_experts: int = 1
    num_routed_experts: int = 8
    use_shared_expert: bool = True
    capacity_strategy: str = "token_drop"
    modality_experts: dict = field(default_factory=lambda: {
        "text": 4, "vision": 3, "image_gen": 2, "video_gen": 2, "audio": 2, "ocr": 1, "cross_modal": 2})


@dataclass
class MoEOutput:
    output: torch.Tensor
    router_logits: torch.Tensor | None = None
    expert_weights: torch.Tensor | None = None
    expert_indices: torch.Tensor | None = None
    load_balance_loss: torch.Tensor | float = 0.0
    z_loss: torch.Tensor | float = 0.0
    num_activated_experts: int = 0
    tokens_dropped: int = 0


# --------------------------------------------------------------------------- shared helpers


def softmax_with_topk(logits: torch.Tensor, k: int):
    """Softmax over all experts, then the k largest probabilities (not renormalised)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, min(k, logits.shape[-1]), dim=-1)
    return idx, w


def compute_load_balance_loss(logits: torch.Tensor, indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    """``E * sum_e f_e * P_e`` with f = fraction of (token, k) assignments, P = mean router probability."""
    probs = torch.softmax(logits.float(), dim=-1)
    f = torch.zeros(num_experts, device=logits.device).index_add_(
        0, indices.reshape(-1), torch.ones(indices.numel(), device=logits.device)) / max(1, indices.numel())
    return num_experts * (f * probs.mean(dim=0)).sum()


def compute_z_loss(values: torch.Tensor) -> torch.Tensor:
    """Mean squared log-sum-exp over rows."""
    return torch.logsumexp(values.float(), dim=-1).pow(2).mean()


def _act(x, kind: str):
    if kind == "silu":
        return tF.silu(x)
    if kind == "gelu":
        return tF.gelu(x)
    if kind == "relu2":
        return torch.relu(x).pow(2)
    return torch.relu(x)


class ExpertFFN(nn.Module):
    """``down(act(gate(x)) * up(x))`` with SiLU by default (gated), or ``down(act(up(x)))``."""

    def __init__(self, hidden: int, ffn: int, activation: str = "silu", gated: bool = True, std: float = 0.02):
        super().__init__()
        self.gated, self.activation = gated, activation
        self.up = nn.Parameter(torch.randn((2 if gated else 1) * ffn, hidden) * std)
        self.down = nn.Parameter(torch.randn(hidden, ffn) * std)
        self.weight_transform = None    # callable(weight) -> weight, set by the quantised variants

    def _w(self, p):
        return p if self.weight_transform is None else self.weight_transform(p)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = x @ self._w(self.up).t().to(x.dtype)
        if self.gated:
            g, u = h.chunk(2, dim=-1)
            h = _act(g, self.activation) * u
        else:
            h = _act(h, self.activation)
        return h @ self._w(self.down).t().to(x.dtype)


def create_experts(n: int, hidden: int, ffn: int, activation: str = "silu") -> nn.ModuleList:
    return nn.ModuleList([ExpertFFN(hidden, ffn, activation) for _ in range(n)])


def moe_dispatch_batched(x: torch.Tensor, experts, indices: torch.Tensor, weights: torch.Tensor,
                         capacity: int | None = None):
    """x [T, D]; indices/weights [T, K]. Returns (out [T, D], dropped). With ``capacity`` each
    expert keeps its first ``capacity`` assignments in token order and drops the rest."""
    T, K = indices.shape
    out = torch.zeros_like(x)
    flat_e = indices.reshape(-1)
    flat_t = torch.arange(T, device=x.device).repeat_interleave(K)
    flat_w = weights.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    counts = torch.bincount(flat_e, minlength=len(experts)).tolist()
    dropped, start = 0, 0
    for e, n in enumerate(counts):
        sel = order[start:start + n]
        start += n
        if n == 0:
            continue
        if capacity is not None and n > capacity:
            dropped += n - capacity
            sel = sel[:capacity]
        tok = flat_t[sel]
        y = experts[e](x[tok])
        out.index_add_(0, tok, y * flat_w[sel, None].to(y.dtype))
    return out, dropped


class _Base(nn.Module):
    def __init__(self, hidden: int, cfg: MoEAllConfig):
        super().__init__()
        self.hidden, self.cfg = hidden, cfg

    @staticmethod
    def _flat(x):
        return x.reshape(-1, x.shape[-1])

    def _router(self, out_features: int, in_features: int | None = None) -> nn.Linear:
        lin = nn.Linear(in_features or self.hidden, out_features, bias=False)
        nn.init.normal_(lin.weight, std=0.02)
        return lin

    def _topk_route(self, xf, router, experts, k, capacity=None, logits=None):
        logits = router(xf) if logits is None else logits
        idx, w = softmax_with_topk(logits, k)
        y, dropped = moe_dispatch_batched(xf, experts, idx, w, capacity)
        lb = self.cfg.load_balance_coef * compute_load_balance_loss(logits, idx, len(experts))
        zl = self.cfg.z_loss_coef * compute_z_loss(logits)
        return y, logits, idx, w, lb, zl, dropped


# --------------------------------------------------------------------------- 1-10


class SparseMoE(_Base):
    """Top-k routing (top-1 = Switch, top-2 = GShard style) with optional expert capacity."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.router = self._router(cfg.num_experts)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x, training: bool = True):
        xf = self._flat(x)
        cap = None
        if training and self.cfg.capacity_strategy == "token_drop" and self.cfg.capacity_factor > 0:
            cap = max(1, int(math.ceil(self.cfg.capacity_factor * xf.shape[0] * self.cfg.top_k / self.cfg.num_experts)))
        y, logits, idx, w, lb, zl, dropped = self._topk_route(xf, self.router, self.experts, self.cfg.top_k, cap)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k, dropped)


class SoftMoE(_Base):
    """Every expert slot processes a softmax-weighted mix of all tokens; tokens read the slots back
    with the same weights, followed by an output projection."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.slots = cfg.num_experts * cfg.num_slots_per_expert
        self.input_mixing = self._router(self.slots)
        self.output_mixing = self._router(hidden)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        xf = self._flat(x)
        logits = self.input_mixing(xf)
        sw = torch.softmax(logits.float(), dim=-1).to(xf.dtype)                  # [T, slots]
        per_expert = sw.view(-1, self.cfg.num_experts, self.cfg.num_slots_per_expert).sum(-1)   # [T, E]
        expert_in = per_expert.t() @ xf                                          # [E, D]
        expert_out = torch.stack([self.experts[e](expert_in[e:e + 1])[0] for e in range(self.cfg.num_experts)])
        y = self.output_mixing(per_expert @ expert_out)
        zl = self.cfg.z_loss_coef * compute_z_loss(expert_out) / xf.shape[0]
        return MoEOutput(y.view_as(x), logits, None, None, 0.0, zl, self.cfg.num_experts)


class HierarchicalMoE(_Base):
    """Two-level routing: top groups, then top experts inside each chosen group; the weight of an
    expert is group probability x expert probability."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.group_router = self._router(cfg.num_groups)
        self.expert_routers = nn.ModuleList([self._router(cfg.experts_per_group) for _ in range(cfg.num_groups)])
        self.groups = nn.ModuleList([create_experts(cfg.experts_per_group, hidden, cfg.expert_hidden_size)
                                     for _ in range(cfg.num_groups)])

    def forward(self, x):
        xf = self._flat(x)
        g_logits = self.group_router(xf)
        g_idx, g_w = softmax_with_topk(g_logits, self.cfg.top_groups)
        y = torch.zeros_like(xf)
        lb = self.cfg.group_load_balance_coef * compute_load_balance_loss(g_logits, g_idx, self.cfg.num_groups)
        for g in range(self.cfg.num_groups):
            hit = (g_idx == g)
            tok = hit.any(dim=1).nonzero(as_tuple=True)[0]
            if tok.numel() == 0:
                continue
            gw = (g_w * hit).sum(dim=1)[tok]
            e_logits = self.expert_routers[g](xf[tok])
            e_idx, e_w = softmax_with_topk(e_logits, self.cfg.top_experts_per_group)
            sub, _ = moe_dispatch_batched(xf[tok], self.groups[g], e_idx, e_w * gw[:, None])
            y.index_add_(0, tok, sub)
            lb = lb + self.cfg.load_balance_coef * compute_load_balance_loss(e_logits, e_idx, self.cfg.experts_per_group) \
                / self.cfg.num_groups
        return MoEOutput(y.view_as(x), g_logits, g_w, g_idx, lb, self.cfg.z_loss_coef * compute_z_loss(g_logits),
                         self.cfg.top_groups * self.cfg.top_experts_per_group)


class MoMoE(HierarchicalMoE):
    """Mixture of mixtures: like the hierarchical variant but every group also owns a gate that
    mixes the group's result with the token itself (a residual gate per group)."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.group_gates = nn.Parameter(torch.zeros(cfg.num_groups))

    def forward(self, x):
        out = super().forward(x)
        xf = self._flat(x)
        g = torch.sigmoid(self.group_gates)[out.expert_indices]                 # [T, top_groups]
        mix = (g * out.expert_weights).sum(dim=1, keepdim=True).to(xf.dtype)
        out.output = (out.output.view_as(xf) + mix * xf).view_as(x)
        return out


class ExpertChoiceMoE(_Base):
    """Experts pick tokens: each expert takes its ``capacity`` highest-affinity tokens."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.router = self._router(cfg.num_experts)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        xf = self._flat(x)
        T, E = xf.shape[0], self.cfg.num_experts
        logits = self.router(xf)
        probs = torch.softmax(logits.float(), dim=-1)
        cap = max(1, min(T, int(self.cfg.capacity_factor * T / E)))
        w, tok = torch.topk(probs.t(), cap, dim=1)                              # [E, cap]
        y = torch.zeros_like(xf)
        for e in range(E):
            y.index_add_(0, tok[e], self.experts[e](xf[tok[e]]) * w[e, :, None].to(xf.dtype))
        covered = torch.zeros(T, dtype=torch.bool, device=xf.device)
        covered[tok.reshape(-1)] = True
        return MoEOutput(y.view_as(x), logits, w, tok, 0.0, self.cfg.z_loss_coef * compute_z_loss(logits), E,
                         int((~covered).sum()))


class HashMoE(_Base):
    """No learned router: expert = hash of the token id (``hash_bucket_size`` experts per token,
    equal weights)."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x, token_ids):
        xf = self._flat(x)
        ids = token_ids.reshape(-1).long()
        k = max(1, self.cfg.hash_bucket_size)
        idx = torch.stack([((ids * 2654435761 + j * 40503) >> 7) % self.cfg.num_experts for j in range(k)], dim=1)
        w = torch.full_like(idx, 1.0 / k, dtype=torch.float32)
        y, _ = moe_dispatch_batched(xf, self.experts, idx, w)
        return MoEOutput(y.view_as(x), None, w, idx, 0.0, 0.0, k)


class CrossLayerMoE(_Base):
    """One expert pool shared by ``num_shared_layers`` layers, each layer with its own router."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.routers = nn.ModuleList([self._router(cfg.num_experts) for _ in range(cfg.num_shared_layers)])
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x, layer_idx: int = 0):
        xf = self._flat(x)
        r = self.routers[layer_idx % len(self.routers)]
        y, logits, idx, w, lb, zl, _ = self._topk_route(xf, r, self.experts, self.cfg.top_k)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k)


MODALITIES = ("text", "vision", "image_gen", "video_gen", "audio", "ocr", "cross_modal")


class MultiModalMoE(_Base):
    """Experts are partitioned by modality; a per-token modality hint (or a learned classifier when
    no hint is given) adds a large bias to the experts of that modality before top-k."""

    def __init__(self, hidden, cfg, bias: float = 10.0):
        super().__init__(hidden, cfg)
        counts = [cfg.modality_experts.get(m, 0) for m in MODALITIES]
        self.total = sum(counts)
        owner = torch.cat([torch.full((c,), i) for i, c in enumerate(counts)]).long()
        self.register_buffer("owner", owner)
        self.bias = bias
        self.classifier = self._router(len(MODALITIES))
        self.router = self._router(self.total)
        self.experts = create_experts(self.total, hidden, cfg.expert_hidden_size)

    def forward(self, x, modality_hints=None):
        xf = self._flat(x)
        logits = self.router(xf)
        if modality_hints is not None:
            mp = tF.one_hot(modality_hints.reshape(-1).long(), len(MODALITIES)).float()
        else:
            mp = torch.softmax(self.classifier(xf).float(), dim=-1)
        logits = logits + self.bias * mp[:, self.owner].to(logits.dtype)
        y, logits, idx, w, lb, zl, _ = self._topk_route(xf, None, self.experts, self.cfg.top_k, logits=logits)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k)


class MMoE(_Base):
    """Multi-gate MoE: all experts run on every token; each task owns a softmax gate."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.gates = nn.ModuleList([self._router(cfg.num_experts) for _ in range(max(1, cfg.num_tasks))])
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x, task_id: int = 0):
        xf = self._flat(x)
        logits = self.gates[task_id % len(self.gates)](xf)
        g = torch.softmax(logits.float(), dim=-1).to(xf.dtype)
        outs = torch.stack([e(xf) for e in self.experts], dim=1)                 # [T, E, D]
        y = (g[..., None] * outs).sum(dim=1)
        return MoEOutput(y.view_as(x), logits, g, None, 0.0, 0.0, self.cfg.num_experts)


class DeepSeekMoE(_Base):
    """Always-on shared experts plus fine-grained routed experts; balancing by a per-expert bias
    that is nudged against the load after every training forward (no auxiliary loss)."""

    def __init__(self, hidden, cfg, bias_update: float = 0.001):
        super().__init__(hidden, cfg)
        self.shared = create_experts(cfg.num_shared_experts if cfg.use_shared_expert else 0, hidden,
                                     cfg.expert_hidden_size)
        self.router = self._router(cfg.num_routed_experts)
        self.experts = create_experts(cfg.num_routed_experts, hidden, cfg.expert_hidden_size)
        self.register_buffer("route_bias", torch.zeros(cfg.num_routed_experts))
        self.bias_update = bias_update

    def forward(self, x, training: bool = True):
        xf = self._flat(x)
        logits = self.router(xf)
        probs = torch.softmax(logits.float(), dim=-1)
        _, idx = torch.topk(probs + self.route_bias, min(self.cfg.top_k, probs.shape[1]), dim=-1)   # bias picks ...
        w = torch.gather(probs, 1, idx)                                                            # ... not weighs
        y, _ = moe_dispatch_batched(xf, self.experts, idx, w)
        for s in self.shared:
            y = y + s(xf)
        if training:
            with torch.no_grad():
                load = torch.bincount(idx.reshape(-1), minlength=probs.shape[1]).float()
                self.route_bias += self.bias_update * torch.sign(load.mean() - load)
        return MoEOutput(y.view_as(x), logits, w, idx, 0.0, self.cfg.z_loss_coef * compute_z_loss(logits),
                         self.cfg.top_k + len(self.shared))


# --------------------------------------------------------------------------- 11-20


class BaseLayerMoE(_Base):
    """BASE layers: balanced assignment, every expert receives exactly T/E tokens (greedy by
    affinity over a random token order in training, plain top-1 at inference)."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.router = self._router(cfg.num_experts)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x, training: bool = True):
        xf = self._flat(x)
        T, E = xf.shape[0], self.cfg.num_experts
        logits = self.router(xf)
        if not training:
            idx = logits.argmax(dim=-1, keepdim=True)
        else:
            cap = (T + E - 1) // E
            pref = torch.argsort(logits, dim=1, descending=True).tolist()
            fill = [0] * E
            choice = [0] * T
            for t in range(T):
                for e in pref[t]:
                    if fill[e] < cap:
                        fill[e] += 1
                        choice[t] = e
                        break
            idx = torch.tensor(choice, device=xf.device).view(T, 1)
        w = torch.sigmoid(torch.gather(logits, 1, idx).float())
        y, _ = moe_dispatch_batched(xf, self.experts, idx, w)
        return MoEOutput(y.view_as(x), logits, w, idx, 0.0, 0.0, 1)


class DenseMoE(_Base):
    """All experts on all tokens, softmax-weighted."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.router = self._router(cfg.num_experts)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        xf = self._flat(x)
        logits = self.router(xf)
        g = torch.softmax(logits.float(), dim=-1).to(xf.dtype)
        y = sum(g[:, e:e + 1] * self.experts[e](xf) for e in range(self.cfg.num_experts))
        return MoEOutput(y.view_as(x), logits, g, None, 0.0, 0.0, self.cfg.num_experts)


class SharedExpertMoE(SparseMoE):
    """Top-k routed experts plus one shared expert applied to every token."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.shared = ExpertFFN(hidden, cfg.expert_hidden_size)

    def forward(self, x, training: bool = True):
        out = super().forward(x, training)
        out.output = out.output + self.shared(self._flat(x)).view_as(x)
        out.num_activated_experts += 1
        return out


class ResidualMoE(SparseMoE):
    """Routed output added to a dense residual FFN with a learned mixing coefficient."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        self.dense = ExpertFFN(hidden, cfg.expert_hidden_size)
        self.mix = nn.Parameter(torch.tensor(0.5))

    def forward(self, x):
        out = super().forward(x, training=False)
        out.output = self.dense(self._flat(x)).view_as(x) + self.mix.to(x.dtype) * out.output
        return out


class GatingDropoutMoE(SparseMoE):
    """Router logits are dropped (set to -inf) with probability ``dropout_rate`` while training, so
    routing does not collapse on a few experts."""

    def __init__(self, hidden, cfg, dropout_rate: float = 0.1):
        super().__init__(hidden, cfg)
        self.dropout_rate = dropout_rate

    def forward(self, x, training: bool = True):
        xf = self._flat(x)
        logits = self.router(xf)
        if training and self.dropout_rate > 0:
            drop = torch.rand_like(logits.float()) < self.dropout_rate
            drop[torch.arange(xf.shape[0]), logits.argmax(dim=-1)] = False    # at least the best expert stays
            logits = logits.masked_fill(drop, float("-inf"))
        y, logits, idx, w, lb, zl, _ = self._topk_route(xf, None, self.experts, self.cfg.top_k, logits=logits)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k)


class DomainMoE(_Base):
    """A domain classifier weighs the outputs of per-domain MoEs (or selects one when the domain
    is given)."""

    def __init__(self, hidden, cfg, num_domains: int = 4):
        super().__init__(hidden, cfg)
        self.num_domains = num_domains
        per = max(1, cfg.num_experts // num_domains)
        self.domain_classifier = self._router(num_domains)
        self.domain_routers = nn.ModuleList([self._router(per) for _ in range(num_domains)])
        self.domain_experts = nn.ModuleList([create_experts(per, hidden, cfg.expert_hidden_size)
                                             for _ in range(num_domains)])

    def forward(self, x, domain_id: int = -1):
        xf = self._flat(x)
        dom_logits = self.domain_classifier(xf)
        dp = torch.softmax(dom_logits.float(), dim=-1)
        if domain_id >= 0:
            dp = tF.one_hot(torch.full((xf.shape[0],), domain_id, device=xf.device), self.num_domains).float()
        y = torch.zeros_like(xf)
        lb = 0.0
        for d in range(self.num_domains):
            if domain_id >= 0 and d != domain_id:
                continue
            sub, logits, idx, _, lbd, _, _ = self._topk_route(xf, self.domain_routers[d], self.domain_experts[d],
                                                              self.cfg.top_k)
            y = y + dp[:, d:d + 1].to(xf.dtype) * sub
            lb = lb + lbd / self.num_domains
        return MoEOutput(y.view_as(x), dom_logits, dp, None, lb, 0.0, self.cfg.top_k * self.num_domains)


class ProductKeyMoE(_Base):
    """Two half-size expert sets with independent routers; the outputs add."""

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        half = max(1, cfg.num_experts // 2)
        rest = max(1, cfg.num_experts - half)
        self.router_a, self.router_b = self._router(half), self._router(rest)
        self.experts_a = create_experts(half, hidden, cfg.expert_hidden_size)
        self.experts_b = create_experts(rest, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        xf = self._flat(x)
        ya, la, ia, wa, lba, zla, _ = self._topk_route(xf, self.router_a, self.experts_a, self.cfg.top_k)
        yb, _, _, _, _, zlb, _ = self._topk_route(xf, self.router_b, self.experts_b, self.cfg.top_k)
        return MoEOutput((ya + yb).view_as(x), la, wa, ia, lba, zla + zlb, 2 * self.cfg.top_k)


class AttentionMoE(_Base):
    """Routing scores are scaled dot products between a token query and learned expert keys."""

    def __init__(self, hidden, cfg, key_dim: int = 64):
        super().__init__(hidden, cfg)
        self.q_proj = self._router(key_dim)
        self.expert_keys = nn.Parameter(torch.randn(cfg.num_experts, key_dim) * 0.02)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        xf = self._flat(x)
        q = self.q_proj(xf)
        logits = q @ self.expert_keys.t().to(q.dtype) / math.sqrt(q.shape[-1])
        y, logits, idx, w, lb, zl, _ = self._topk_route(xf, None, self.experts, self.cfg.top_k, logits=logits)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k)


class MLAMoE(_Base):
    """Tokens pass through a low-rank latent bottleneck (down, up) before routing and experts."""

    def __init__(self, hidden, cfg, latent_dim: int = 64):
        super().__init__(hidden, cfg)
        self.down_proj = self._router(latent_dim)
        self.up_proj = self._router(hidden, latent_dim)
        self.router = self._router(cfg.num_experts)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        xf = self._flat(x)
        rec = self.up_proj(self.down_proj(xf))
        y, logits, idx, w, lb, zl, _ = self._topk_route(rec, self.router, self.experts, self.cfg.top_k)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k)


class MambaMoE(_Base):
    """A diagonal state-space scan over the sequence is added to the tokens before routing:
    ``h_t = a * h_{t-1} + B x_t``, ``x'_t = x_t + C h_t`` with a learned per-channel decay."""

    def __init__(self, hidden, cfg, state_dim: int = 16):
        super().__init__(hidden, cfg)
        self.in_proj = self._router(state_dim)
        self.out_proj = self._router(hidden, state_dim)
        self.decay_logit = nn.Parameter(torch.full((state_dim,), 2.0))
        self.router = self._router(cfg.num_experts)
        self.experts = create_experts(cfg.num_experts, hidden, cfg.expert_hidden_size)

    def forward(self, x):
        B, S, D = x.shape
        u = self.in_proj(x)                                   # [B, S, N]
        a = torch.sigmoid(self.decay_logit).to(u.dtype)
        h = torch.zeros(B, u.shape[-1], device=x.device, dtype=u.dtype)
        hs = []
        for t in range(S):
            h = a * h + u[:, t]
            hs.append(h)
        comb = x + self.out_proj(torch.stack(hs, dim=1))
        xf = self._flat(comb)
        y, logits, idx, w, lb, zl, _ = self._topk_route(xf, self.router, self.experts, self.cfg.top_k)
        return MoEOutput(y.view_as(x), logits, w, idx, lb, zl, self.cfg.top_k)


# --------------------------------------------------------------------------- 21-25 weight-quantised experts


class _STE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, q):
        return q

    @staticmethod
    def backward(ctx, g):
        return g, None


def _ste(w, q):
    return _STE.apply(w, q.to(w.dtype))


def _q_int8(w):
    s = w.detach().abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 127.0
    return _ste(w, torch.round(w.detach() / s).clamp(-127, 127) * s)


def _q_ternary(w, block: int = 256):
    _, _, q = ref.i2s_quant(w.detach().float().reshape(-1), block if w.numel() % block == 0 else w.shape[1])
    return _ste(w, q.view_as(w))


def _q_binary(w):
    d = w.detach()
    s = d.abs().mean(dim=1, keepdim=True)
    return _ste(w, torch.where(d >= 0, s, -s))


def _q_codebook(size: int):
    def fn(w, block: int = 256):
        from ..oil import codebook as cbk

        d = w.detach().float()
        std = float(d.std()) or 0.02
        cb = cbk.quantile_codebook(size, std, fp16=(size == 16)).to(d.device)[None]
        bs = block if d.numel() % block == 0 else d.shape[1]
        nb = d.numel() // bs
        _, q = ref.nearest_centroid(d.reshape(-1), cb, torch.zeros(nb, dtype=torch.int32, device=d.device), bs)
        return _ste(w, q.view_as(w))
    return fn


class _QuantisedMoE(SparseMoE):
    transform = None

    def __init__(self, hidden, cfg):
        super().__init__(hidden, cfg)
        for e in self.experts:
            e.weight_transform = type(self).transform

    def forward(self, x):
        return super().forward(x, training=False)


class QuantizedINT8MoE(_QuantisedMoE):
    transform = staticmethod(_q_int8)


class TernaryMoE(_QuantisedMoE):
    transform = staticmethod(_q_ternary)


class BinaryMoE(_QuantisedMoE):
    transform = staticmethod(_q_binary)


class OIL8MoE(_QuantisedMoE):
    transform = staticmethod(_q_codebook(256))


class OIL4MoE(_QuantisedMoE):
    transform = staticmethod(_q_codebook(16))


VARIANTS = {
    "sparse_topk": SparseMoE, "sparse_top1": SparseMoE, "sparse_top2": SparseMoE, "soft": SoftMoE,
    "hierarchical": HierarchicalMoE, "momoe": MoMoE, "expert_choice": ExpertChoiceMoE, "hash": HashMoE,
    "cross_layer": CrossLayerMoE, "multimodal": MultiModalMoE, "mmoe": MMoE, "deepseek": DeepSeekMoE,
    "base_layer": BaseLayerMoE, "dense": DenseMoE, "shared_expert": SharedExpertMoE, "residual": ResidualMoE,
    "gating_dropout": GatingDropoutMoE, "domain": DomainMoE, "product_key": ProductKeyMoE,
    "attention": AttentionMoE, "mla": MLAMoE, "mamba": MambaMoE, "int8": QuantizedINT8MoE, "ternary": TernaryMoE,
    "binary": BinaryMoE, "oil8": OIL8MoE, "oil4": OIL4MoE,
}


def create_moe(variant: str, hidden: int, cfg: MoEAllConfig | None = None) -> nn.Module:
    cfg = cfg or MoEAllConfig()
    cfg.variant = variant
    if variant == "sparse_top1":
        cfg.top_k = 1
    elif variant == "sparse_top2":
        cfg.top_k = 2
    return VARIANTS[variant](hidden, cfg)
