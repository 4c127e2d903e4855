"""Mixture-of-experts transformer.

``MoEFFN`` covers the reference's router and expert FFN (``MoERouter`` / ``MoEFFN``,
engines/trainer/moe/moe.cpp:47-218) with the batched dispatch semantics of
``moe_dispatch_batched`` (src/moe_variants.cpp:695-755) and, through options, the routing families
of its ``moe_variants``: top-1/2/k sparse routing, shared always-on experts (DeepSeek style),
capacity factor with token dropping or residual pass-through (Switch style), hash routing, expert
choice, dense / soft mixtures, gating dropout, router z-loss and the load-balance loss
``E * sum_e f_e P_e``. Router weights are the softmax probabilities over all experts, used without
renormalising over the chosen k (src/moe_variants.cpp:46-58).

CUDA path, with no host round trip inside a layer: router GEMM -> ``moe_route`` (softmax, top-k,
slot per expert, combine weights, load statistics in one kernel) -> per-expert counts exchanged
between ranks through symmetric memory -> ``moe_offsets`` (segment of every local expert in the
receive buffer, computed on the device) -> ``moe_dispatch`` (permute and store rows straight into
the owner rank's buffer) -> two grouped tcgen05 GEMM launches over all local experts (ragged M,
SwiGLU in the first epilogue) -> ``moe_combine`` (gather from the owners and weight). The backward
pass reuses the exchange kernels in the opposite direction and adds two ragged-K grouped GEMMs for
the weight gradients. CPU path and the other routing families: the same arithmetic in plain
PyTorch (the oracle of the kernel tests).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import native
from .config import TransformerConfig
from .dense import DenseModel
from .layers import FFN, OILLinear, TransformerBlock


MAX_LOCAL_EXPERTS = 16      # segments one grouped GEMM launch covers
SEG_ALIGN = 256             # segment starts are multiples of the paired GEMM's tile height


class ExpertParallel:
    """Expert-parallel context: symmetric receive / return buffers, the table through which the ranks
    exchange their per-expert token counts, and a flag barrier. ``cap_rows`` is the number of
    (token, expert) rows one rank may send per layer call; a rank can receive ``world * cap_rows``
    rows (every token of every rank routed to its experts) unless ``receive_factor`` lowers the bound,
    plus alignment padding per expert."""

    def __init__(self, group, device, cap_rows: int, dim: int, receive_factor: float | None = None):
        import math

        import torch.distributed as dist

        from ..parallel import symm

        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        # receive_factor bounds what one rank accepts per call to that multiple of a rank's own rows
        # (perfect balance = 1); None keeps the worst case, every row of every rank. The buffers and the
        # activations saved per layer scale with it. More rows than the bound raise the status word
        # (nothing is dropped silently).
        factor = self.world if receive_factor is None else min(float(self.world), max(1.0, float(receive_factor)))
        self.cap = (int(math.ceil(factor * cap_rows)) + SEG_ALIGN - 1) // SEG_ALIGN * SEG_ALIGN + SEG_ALIGN * MAX_LOCAL_EXPERTS
        self.dim = dim
        n = self.cap * dim
        self.bufs = {k: symm.make_buffer(n, torch.bfloat16, device, group) for k in ("x", "y", "dy", "dx")}
        self.count_table = symm.make_buffer(self.world * 64, torch.int32, device, group).zero_()
        self.barrier = symm.FlagBarrier(device, group)
        self.shared = True      # one set of buffers serves every layer: saved rows are copied out

    def ensure(self, rows: int, dim: int, device):
        if rows > self.cap or dim != self.dim:
            raise ValueError(f"expert-parallel buffers hold {self.cap} rows of {self.dim}; this call needs {rows} x {dim}")


class _LocalExchange:
    """Single-rank stand-in for :class:`ExpertParallel` (buffers are ordinary tensors, one set per
    layer, so the rows of a layer stay valid until its backward pass)."""

    rank, world = 0, 1
    shared = False

    def __init__(self):
        self.bufs = {}
        self.cap = 0
        self.barrier = None
        self.count_table = None

    def ensure(self, rows: int, dim: int, device):
        if self.cap < rows or not self.bufs or next(iter(self.bufs.values())).tensor.shape[0] < rows * dim:
            from ..parallel.symm import LocalBuffer

            self.cap = rows
            self.bufs = {k: LocalBuffer(rows * dim, torch.bfloat16, device) for k in ("x", "y", "dy", "dx")}


class _RouteFn(torch.autograd.Function):
    """Router on the device in one kernel: softmax over the expert logits, top-k, a slot in each
    chosen expert's batch, combine weights (the probabilities of the chosen experts, not
    renormalised: src/moe_variants.cpp:46-58) and the statistics of the load-balance loss
    ``coef * E * sum_e f_e P_e`` (engines/trainer/moe/moe.cpp:47-153). Nothing returns to the host."""

    @staticmethod
    def forward(ctx, logits, E, k, aux_coef):
        C = native.require()
        T = logits.shape[0]
        dev = logits.device
        probs = torch.empty(T, E, device=dev, dtype=torch.float32)
        topk_idx = torch.empty(T, k, device=dev, dtype=torch.int32)
        slot = torch.empty(T, k, device=dev, dtype=torch.int32)
        w = torch.empty(T, k, device=dev, dtype=torch.float32)
        counts = torch.zeros(E, device=dev, dtype=torch.int32)
        psum = torch.zeros(E, device=dev, dtype=torch.float32)
        C.moe_route(logits, E, probs, topk_idx, slot, w, counts, psum)
        f = counts.float() / float(T * k)
        aux = (aux_coef * E) * (f * (psum / float(T))).sum()
        ctx.save_for_backward(probs, topk_idx, f)
        ctx.meta = (E, k, aux_coef, T, logits.shape[1])
        ctx.mark_non_differentiable(topk_idx, slot, counts)
        return w, aux, topk_idx, slot, counts

    @staticmethod
    def backward(ctx, dw, daux, *_):
        C = native.require()
        probs, topk_idx, f = ctx.saved_tensors
        E, k, aux_coef, T, ld = ctx.meta
        if dw is None:
            dw = torch.zeros(T, k, device=probs.device, dtype=torch.float32)
        coef = None
        if daux is not None:            # d aux / d p[t, e] = coef * E * f_e / T (f is piecewise constant)
            coef = (f * (aux_coef * E / float(T))) * daux.float()
        dlogits = torch.empty(T, ld, device=probs.device, dtype=torch.bfloat16)
        C.moe_route_bwd(probs, topk_idx, dw.contiguous().float(), coef, dlogits)
        return dlogits, None, None, None


class _MoEFn(torch.autograd.Function):
    """dispatch -> grouped expert FFN -> combine without a host round trip. The receive buffer holds
    one segment per local expert (start aligned to 256 rows, tokens of all source ranks in rank
    order); segment starts and sizes are computed on the device from the exchanged counts and read
    by the grouped GEMMs' tile scheduler. Expert FFN: gate/up GEMM with SwiGLU in the epilogue,
    down GEMM; backward: down dgrad with the SwiGLU derivative in the epilogue, up dgrad, and two
    ragged-K weight-gradient GEMMs accumulating in fp32 into the experts' gradient buffers."""

    @staticmethod
    def forward(ctx, x, w, moe, topk_idx, slot, counts):
        C = native.require()
        ex = moe.exchange
        T, d = x.shape
        E = moe.num_experts
        k = topk_idx.shape[1]
        epr = E // ex.world
        dev = x.device
        st = native.status_word(dev)
        rows = T * k + SEG_ALIGN * epr if ex.world == 1 else ex.cap
        ex.ensure(rows, d, dev)
        cap = ex.cap
        if ex.world > 1:
            C.moe_publish_counts(counts, ex.count_table.ptrs, E, ex.rank)
            ex.barrier.sync()
            table = ex.count_table.tensor
        else:
            table = counts
        seg_start = torch.empty(epr, device=dev, dtype=torch.int32)
        seg_rows = torch.empty(epr, device=dev, dtype=torch.int32)
        send_base = torch.empty(E, device=dev, dtype=torch.int32)
        send_limit = torch.empty(E, device=dev, dtype=torch.int32)   # where each expert's segment ends on its owner
        C.moe_offsets(table, ex.world, E, ex.rank, cap, seg_start, seg_rows, send_base, st, send_limit)
        xbuf, ybuf = ex.bufs["x"], ex.bufs["y"]
        xs = xbuf.tensor.view(-1, d)[:cap]
        ys = ybuf.tensor.view(-1, d)[:cap]
        C.moe_zero_pad(seg_start, seg_rows, epr, xs, None)
        C.moe_dispatch(x, topk_idx, slot, send_base, None, xbuf.ptrs, epr, 0, 0, send_limit)
        if ex.barrier is not None:
            ex.barrier.sync()
        lo = ex.rank * epr
        ups = [moe.experts_up[lo + i].weight.compute for i in range(epr)]
        downs = [moe.experts_down[lo + i].weight.compute for i in range(epr)]
        f2 = ups[0].shape[0]
        gu = torch.empty(cap, f2, device=dev, dtype=torch.bfloat16)
        h = torch.empty(cap, f2 // 2, device=dev, dtype=torch.bfloat16)
        C.gemm_grouped_rows(xs, ups, False, gu, seg_start, seg_rows, 1, None, h, st)      # + SwiGLU forward
        C.gemm_grouped_rows(h, downs, False, ys, seg_start, seg_rows, 0, None, None, st)
        if ex.barrier is not None:
            ex.barrier.sync()
        out = torch.empty_like(x)
        C.moe_combine(ybuf.ptrs, topk_idx, slot, send_base, w, None, out, None, d, epr, 0, 0, send_limit)
        ctx.moe = moe
        keep_x, keep_y = (xs.clone(), ys.clone()) if ex.shared else (xs, ys)
        ctx.save_for_backward(x, w, topk_idx, slot, send_base, seg_start, seg_rows, keep_x, keep_y, gu, h, send_limit)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = native.require()
        moe, ex = ctx.moe, ctx.moe.exchange
        x, w, topk_idx, slot, send_base, seg_start, seg_rows, xs, ys, gu, h, send_limit = ctx.saved_tensors
        T, d = x.shape
        k = topk_idx.shape[1]
        epr = moe.num_experts // ex.world
        dev = x.device
        st = native.status_word(dev)
        cap = ex.cap
        dout = dout.contiguous()
        # dw[t, j] = <dout[t], y row of (t, j)>: the forward's expert outputs, where the combine reads them
        ybuf = ex.bufs["y"]
        if ex.shared:
            ybuf.tensor.view(-1, d)[:cap].copy_(ys)
            ex.barrier.sync()
        dw = torch.empty(T, k, device=dev, dtype=torch.float32)
        C.moe_combine(ybuf.ptrs, topk_idx, slot, send_base, None, dout, None, dw, d, epr, 0, 0, send_limit)
        # dy rows = w * dout[t], sent to the owners
        dybuf, dxbuf = ex.bufs["dy"], ex.bufs["dx"]
        dys = dybuf.tensor.view(-1, d)[:cap]
        dxs = dxbuf.tensor.view(-1, d)[:cap]
        C.moe_zero_pad(seg_start, seg_rows, epr, dys, None)
        C.moe_dispatch(dout, topk_idx, slot, send_base, w.contiguous(), dybuf.ptrs, epr, 0, 0, send_limit)
        if ex.barrier is not None:
            ex.barrier.sync()
        lo = ex.rank * epr
        ups = [moe.experts_up[lo + i].weight for i in range(epr)]
        downs = [moe.experts_down[lo + i].weight for i in range(epr)]
        dgu = torch.empty_like(gu)
        C.gemm_grouped_rows(dys, [p.compute for p in downs], True, dgu, seg_start, seg_rows, 2, gu, None, st)  # + SwiGLU backward
        C.gemm_grouped_k(dys, h, [p.main_grad for p in downs], seg_start, seg_rows, st)
        C.gemm_grouped_rows(dgu, [p.compute for p in ups], True, dxs, seg_start, seg_rows, 0, None, None, st)
        C.gemm_grouped_k(dgu, xs, [p.main_grad for p in ups], seg_start, seg_rows, st)
        if ex.barrier is not None:
            ex.barrier.sync()
        dx = torch.empty_like(x)
        C.moe_combine(dxbuf.ptrs, topk_idx, slot, send_base, None, None, dx, None, d, epr, 0, 0, send_limit)
        return dx, dw, None, None, None, None


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
        elif self._native_ok(x2):
            out = self._forward_native(x2)
        else:
            probs, idx, w, aux = self._route(x2)
            self.last_aux = aux
            if self.capacity_factor > 0:
                idx, w = self._apply_capacity(idx, w, T)
            out = self._forward_reference(x2, idx, w)
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

    def _native_ok(self, x2) -> bool:
        """The device-side path: plain top-k routing without capacity limit, SwiGLU experts whose width
        is a multiple of 128, weights bound to a parameter store, at most 16 experts per rank."""
        cfg = self.cfg
        f = cfg.moe_ffn_hidden_size or cfg.ffn_hidden_size
        return (x2.is_cuda and getattr(self.experts_up[0].weight, "compute", None) is not None
                and getattr(self.router.weight, "compute", None) is not None
                and self.routing == "topk" and self.capacity_factor == 0 and cfg.gated_ffn and cfg.activation != "relu2"
                and cfg.moe_z_coef == 0 and not (self.training and self.gating_dropout > 0)
                and f % 128 == 0 and cfg.hidden_size % 8 == 0 and cfg.hidden_size >= 256
                and self.num_experts % self.exchange.world == 0
                and self.num_experts // self.exchange.world <= MAX_LOCAL_EXPERTS)

    def _forward_native(self, x2):
        logits = self.router(x2)                                     # bf16 [T, E padded to 8]
        w, aux, topk_idx, slot, counts = _RouteFn.apply(logits, self.num_experts, self.top_k, float(self.cfg.moe_aux_coef))
        self.last_aux = aux
        self.last_stats.update({"tokens_per_expert": counts})        # device tensor; no host read here
        return _MoEFn.apply(x2.contiguous(), w, self, topk_idx, slot, counts)


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
