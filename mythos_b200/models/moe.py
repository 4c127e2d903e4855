"""Mixture-of-experts transformer.

``MoEFFN`` covers the reference's router and expert FFN (``MoERouter`` / ``MoEFFN``,
engines/trainer/moe/moe.cpp:47-218) with the batched dispatch semantics of
``moe_dispatch_batched`` (src/moe_variants.cpp:695-755) and, through options, the routing families
of its ``moe_variants``: top-1/2/k sparse routing, shared always-on experts (DeepSeek style),
capacity factor with token dropping or residual pass-through (Switch style), hash routing, expert
choice, dense / soft mixtures, gating dropout, router z-loss and the load-balance loss
``E * sum_e f_e P_e``. Router weights are the softmax probabilities over all experts, used without
renormalising over the chosen k (src/moe_variants.cpp:46-58).

CUDA path: probabilities -> ``moe_topk`` (top-k + slot per expert) -> ``moe_dispatch`` (permute and
send rows to the expert's owner) -> per (source rank, expert) tcgen05 GEMMs -> ``moe_combine``
(gather from the owners and weight). With expert parallelism the dispatch and combine kernels read
and write the other ranks' buffers directly (symmetric memory); only the per-expert counts (a few
integers) travel through a library all-gather. CPU path: the same arithmetic in plain PyTorch (the
oracle of the kernel tests).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import native
from .config import TransformerConfig
from .dense import DenseModel
from .layers import FFN, OILLinear, TransformerBlock


class ExpertParallel:
    """Expert-parallel context: symmetric receive/return buffers and a flag barrier."""

    def __init__(self, group, device, cap_rows: int, dim: int):
        import torch.distributed as dist

        from ..parallel import symm

        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.cap = cap_rows
        n = self.world * cap_rows * dim
        self.bufs = {k: symm.make_buffer(n, torch.bfloat16, device, group) for k in ("x", "y", "dy", "dx")}
        self.barrier = symm.FlagBarrier(device, group)

    def all_counts(self, counts: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        out = torch.empty(self.world, counts.numel(), device=counts.device, dtype=counts.dtype)
        dist.all_gather_into_tensor(out, counts, group=self.group)
        return out


class _LocalExchange:
    """Single-rank stand-in for :class:`ExpertParallel` (buffers are ordinary tensors)."""

    rank, world = 0, 1

    def __init__(self):
        self.bufs = {}
        self.cap = 0
        self.barrier = None

    def ensure(self, rows: int, dim: int, device):
        if self.cap < rows or not self.bufs or next(iter(self.bufs.values())).tensor.shape[0] < rows * dim:
            from ..parallel.symm import LocalBuffer

            self.cap = rows
            self.bufs = {k: LocalBuffer(rows * dim, torch.bfloat16, device) for k in ("x", "y", "dy", "dx")}

    def all_counts(self, counts):
        return counts[None]


class _MoEFn(torch.autograd.Function):
    """dispatch -> expert FFNs -> combine, with a hand-written backward that reuses the same two
    exchange kernels in the opposite direction."""

    @staticmethod
    def forward(ctx, x, w, moe, topk_idx, slot, send_off, groups):
        C = native.require()
        ex = moe.exchange
        T, d = x.shape
        k = topk_idx.shape[1]
        epr = moe.num_experts // ex.world
        xbuf, ybuf = ex.bufs["x"], ex.bufs["y"]
        C.moe_dispatch(x, topk_idx, slot, send_off, None, xbuf.ptrs, epr, ex.rank, ex.cap)
        if ex.barrier is not None:
            ex.barrier.sync()
        xs = xbuf.tensor.view(-1, d)
        ys = ybuf.tensor.view(-1, d)
        saved_h = []
        for (le, a, b) in groups:
            up, down = moe.experts_up[ex.rank * epr + le], moe.experts_down[ex.rank * epr + le]
            u = F.gemm(xs[a:b], up.weight.compute)
            h = torch.empty(b - a, u.shape[1] // 2, device=x.device, dtype=x.dtype)
            C.swiglu_fused_fwd(u, h)
            F.gemm(h, down.weight.compute, out=ys[a:b])
            saved_h.append((u, h))
        if ex.barrier is not None:
            ex.barrier.sync()
        out = torch.empty_like(x)
        C.moe_combine(ybuf.ptrs, topk_idx, slot, send_off, w, None, out, None, d, epr, ex.rank, ex.cap)
        ctx.moe, ctx.groups, ctx.saved_h = moe, groups, saved_h
        ctx.save_for_backward(x, w, topk_idx, slot, send_off, xs.clone() if ex.world > 1 else xs, ys.clone())
        return out

    @staticmethod
    def backward(ctx, dout):
        C = native.require()
        moe, ex = ctx.moe, ctx.moe.exchange
        x, w, topk_idx, slot, send_off, xs, ys = ctx.saved_tensors
        T, d = x.shape
        k = topk_idx.shape[1]
        epr = moe.num_experts // ex.world
        dout = dout.contiguous()
        # dw[t,j] = <dout[t], y row>; needs the forward's expert outputs where the combine reads them
        ybuf = ex.bufs["y"]
        ybuf.tensor.view(-1, d)[: ys.shape[0]].copy_(ys)
        if ex.barrier is not None:
            ex.barrier.sync()
        dw = torch.empty(T, k, device=x.device, dtype=torch.float32)
        C.moe_combine(ybuf.ptrs, topk_idx, slot, send_off, None, dout, None, dw, d, epr, ex.rank, ex.cap)
        # dy rows = w * dout[t], sent to the owners
        dybuf, dxbuf = ex.bufs["dy"], ex.bufs["dx"]
        C.moe_dispatch(dout, topk_idx, slot, send_off, w.contiguous(), dybuf.ptrs, epr, ex.rank, ex.cap)
        if ex.barrier is not None:
            ex.barrier.sync()
        dys = dybuf.tensor.view(-1, d)
        dxs = dxbuf.tensor.view(-1, d)
        for (le, a, b), (u, h) in zip(ctx.groups, ctx.saved_h):
            up, down = moe.experts_up[ex.rank * epr + le], moe.experts_down[ex.rank * epr + le]
            dh = F.gemm(dys[a:b], down.weight.compute, b_mn=True)
            F.gemm(dys[a:b], h, a_mn=True, b_mn=True, out=down.weight.main_grad, epi=F.EPI_F32_ACC)
            du = torch.empty_like(u)
            C.swiglu_fused_bwd(u, dh, du)
            F.gemm(du, up.weight.compute, b_mn=True, out=dxs[a:b])
            F.gemm(du, xs[a:b], a_mn=True, b_mn=True, out=up.weight.main_grad, epi=F.EPI_F32_ACC)
        if ex.barrier is not None:
            ex.barrier.sync()
        dx = torch.empty_like(x)
        C.moe_combine(dxbuf.ptrs, topk_idx, slot, send_off, None, None, dx, None, d, epr, ex.rank, ex.cap)
        return dx, dw, None, None, None, None, None


class MoEFFN(nn.Module):
    def __init__(self, cfg: TransformerConfig, routing: str = "topk", capacity_factor: float = 0.0,
                 drop_policy: str = "none", gating_dropout: float = 0.0, exchange=None):
        """routing: ``topk`` | ``hash`` | ``expert_choice`` | ``dense`` (all experts, probability
        weighted) | ``soft``. capacity_factor > 0 limits each expert to ``cf * T * k / E`` tokens;
        overflow tokens are dropped (``drop``) or keep their residual (``residual``)."""
        super().__init__()
        self.cfg = cfg
        self.num_experts, self.top_k = cfg.num_experts, cfg.moe_top_k
        self.routing, self.capacity_factor, self.drop_policy = routing, capacity_factor, drop_policy
        self.gating_dropout = gating_dropout
        f = cfg.moe_ffn_hidden_size or cfg.ffn_hidden_size
        fmt = cfg.format_for("ffn")
        # The router's output width is padded to a multiple of 8 (TMA rows are 16-byte multiples);
        # only the first num_experts columns are used, the rest receive zero gradients.
        self.router = OILLinear(cfg.hidden_size, (cfg.num_experts + 7) // 8 * 8, "fp32", cfg.oil_block_size)
        self.experts_up = nn.ModuleList([OILLinear(cfg.hidden_size, 2 * f, fmt, cfg.oil_block_size, cfg.codebook_group)
                                         for _ in range(cfg.num_experts)])
        self.experts_down = nn.ModuleList([OILLinear(f, cfg.hidden_size, fmt, cfg.oil_block_size, cfg.codebook_group)
                                           for _ in range(cfg.num_experts)])
        self.shared = nn.ModuleList([FFN(cfg, f) for _ in range(cfg.moe_shared_experts)])
        self.exchange = exchange if exchange is not None else _LocalExchange()
        self.last_aux = None
        self.last_stats = {}

    def named_oil_tensors(self):
        yield "moe.router.weight", self.router
        for e in range(self.num_experts):
            yield f"moe.experts.{e}.up_proj.weight", self.experts_up[e]
            yield f"moe.experts.{e}.down_proj.weight", self.experts_down[e]
        for i, s in enumerate(self.shared):
            yield f"moe.shared.{i}.up_proj.weight", s.up_proj
            yield f"moe.shared.{i}.down_proj.weight", s.down_proj

    # ------------------------------------------------------------------ routing
    def _route(self, x2):
        from ..ops import reference as ref

        logits = self.router(x2)[:, : self.num_experts].float()
        if self.training and self.gating_dropout > 0:
            logits = logits + torch.empty_like(logits).bernoulli_(self.gating_dropout) * -1e4
        probs = torch.softmax(logits, dim=-1)
        T, E = probs.shape
        if self.routing == "hash":
            idx = (torch.arange(T, device=x2.device)[:, None] * 2654435761 + torch.arange(self.top_k, device=x2.device)
                   ) % E
            idx = idx.to(torch.int64)
        elif self.routing == "expert_choice":
            cap = max(1, T * self.top_k // E)
            chosen = torch.topk(probs.t(), cap, dim=-1).indices  # [E, cap] tokens picked by each expert
            mask = torch.zeros(T, E, device=x2.device, dtype=torch.bool)
            mask[chosen.reshape(-1), torch.arange(E, device=x2.device).repeat_interleave(cap)] = True
            idx = torch.topk(torch.where(mask, probs, torch.full_like(probs, -1.0)), self.top_k, dim=-1).indices
        else:
            idx = torch.topk(probs, self.top_k, dim=-1).indices
        w = probs.gather(1, idx)
        aux = self.cfg.moe_aux_coef * ref.load_balance_loss(probs, idx, E)
        if self.cfg.moe_z_coef > 0:
            aux = aux + ref.z_loss(logits, self.cfg.moe_z_coef)
        return probs, idx, w, aux

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        T, E, k = x2.shape[0], self.num_experts, self.top_k
        if self.routing in ("dense", "soft"):
            probs = torch.softmax(self.router(x2)[:, :E].float(), dim=-1)
            out = sum(probs[:, e:e + 1].to(x2.dtype) * self._expert(e, x2) for e in range(E))
            self.last_aux = torch.zeros((), device=x.device)
        else:
            probs, idx, w, aux = self._route(x2)
            self.last_aux = aux
            if self.capacity_factor > 0:
                idx, w = self._apply_capacity(idx, w, T)
            native_ok = x2.is_cuda and getattr(self.experts_up[0].weight, "compute", None) is not None \
                and self.routing == "topk" and self.capacity_factor == 0 and self.cfg.gated_ffn \
                and self.cfg.activation != "relu2"
            out = self._forward_native(x2, probs, w) if native_ok else self._forward_reference(x2, idx, w)
            kept = idx.reshape(-1)
            counts = torch.bincount(kept[kept >= 0], minlength=E).float()
            self.last_stats.update({"tokens_per_expert": counts,
                                    "cv2": (counts.std() / counts.mean().clamp(min=1e-9)) ** 2})
        for s in self.shared:
            out = out + s(x2)
        return out.reshape(shape)

    def _expert(self, e: int, xs):
        u = self.experts_up[e](xs)
        if self.cfg.activation == "relu2":
            f = u.shape[-1] // 2
            h = F.relu2(u[..., :f].contiguous()) * u[..., f:]
        else:
            h = F.swiglu(u)
        return self.experts_down[e](h)

    def _apply_capacity(self, idx, w, T):
        cap = max(1, int(self.capacity_factor * T * self.top_k / self.num_experts))
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        ranks = torch.empty_like(order)
        sorted_e = flat[order]
        start = torch.searchsorted(sorted_e, sorted_e, right=False)
        ranks[order] = torch.arange(flat.numel(), device=idx.device) - start
        keep = (ranks < cap).reshape(idx.shape)
        self.last_stats["tokens_dropped"] = int((~keep).sum())
        return torch.where(keep, idx, torch.full_like(idx, -1)), torch.where(keep, w, torch.zeros_like(w))

    def _forward_reference(self, x2, idx, w):
        out = torch.zeros_like(x2)
        for e in range(self.num_experts):
            sel = (idx == e)
            tok = sel.any(dim=1).nonzero(as_tuple=True)[0]
            if tok.numel() == 0:
                continue
            we = (w * sel).sum(dim=1)[tok]
            out = out.index_add(0, tok, (self._expert(e, x2[tok]) * we[:, None].to(x2.dtype)))
        if self.drop_policy == "residual" and self.capacity_factor > 0:
            dropped = (idx < 0).all(dim=1)
            out = torch.where(dropped[:, None], x2, out)
        return out

    def _forward_native(self, x2, probs, w_unused):
        C = native.require()
        ex = self.exchange
        T, d = x2.shape
        E, k = self.num_experts, self.top_k
        dev = x2.device
        topk_idx = torch.empty(T, k, device=dev, dtype=torch.int32)
        slot = torch.empty(T, k, device=dev, dtype=torch.int32)
        counts = torch.zeros(E, device=dev, dtype=torch.int32)
        C.moe_topk(probs.detach().contiguous(), k, topk_idx, slot, counts)
        w = probs.gather(1, topk_idx.long())
        epr = E // ex.world
        if isinstance(ex, _LocalExchange):
            ex.ensure(T * k, d, dev)
        all_counts = ex.all_counts(counts).cpu()            # [world, E] (one small host sync per layer)
        send_off = torch.zeros(E, dtype=torch.int32)
        for r in range(ex.world):                             # my rows inside each owner's segment
            send_off[r * epr:(r + 1) * epr] = torch.cumsum(all_counts[ex.rank, r * epr:(r + 1) * epr], 0) - \
                all_counts[ex.rank, r * epr:(r + 1) * epr]
        groups = []
        for s in range(ex.world):                             # what every source sent to my experts
            off = 0
            for le in range(epr):
                c = int(all_counts[s, ex.rank * epr + le])
                if c > 0:
                    groups.append((le, s * ex.cap + off, s * ex.cap + off + c))
                off += c
        return _MoEFn.apply(x2.contiguous(), w, self, topk_idx, slot, send_off.to(dev), groups)


class MoEBlock(TransformerBlock):
    def __init__(self, cfg: TransformerConfig, exchange=None):
        super().__init__(cfg, ffn=MoEFFN(cfg, exchange=exchange))


class MoEModel(DenseModel):
    """Decoder with a MoE FFN in every block. ``forward`` with targets adds the routers' auxiliary
    losses (already scaled by their coefficients) to the language-model loss."""

    def __init__(self, cfg: TransformerConfig, exchange=None):
        self._exchange = exchange
        super().__init__(cfg)

    def _make_block(self, index: int) -> nn.Module:
        return MoEBlock(self.cfg, self._exchange)

    def aux_loss(self):
        terms = [blk.ffn.last_aux for blk in self.layers if getattr(blk.ffn, "last_aux", None) is not None]
        return sum(terms) if terms else None

    def forward(self, ids, targets=None, pos=None, loss_scale: float | None = None):
        out = super().forward(ids, targets, pos, loss_scale)
        if targets is None:
            return out
        aux = self.aux_loss()
        if aux is None:
            return out
        rows = ids.numel()
        scale = rows * (loss_scale if loss_scale is not None else 1.0 / rows)  # aux counts once per micro-batch
        return out + aux.to(out.dtype) * scale / max(1, len(self.layers))
