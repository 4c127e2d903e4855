"""Pipeline parallelism: 1F1B schedule over point-to-point sends and receives.

Each rank owns a contiguous range of layers (``infer.serving.ModelShard``). Activations (the block
output and the residual stream) travel forward and their gradients travel back with
``torch.distributed`` p2p (NCCL over NVLink on GPUs, gloo on CPU); transfers are posted with
``isend`` / ``irecv`` so that a stage computes while its neighbour's data is in flight. The schedule
is the usual warm-up (``stages - rank - 1`` forwards), steady one-forward-one-backward, cool-down.
By design this path uses library p2p only (it is the one communication pattern the fused kernels do
not replace).

The reference's ``PipelineParallelWrapper`` (src/distributed.cpp:182-193) never assigns its model
and runs the full model on every call; ``ModelShard`` (src/inference_opt.cpp:783-822) is the only
real piece and is what a stage is here.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..infer.serving import ModelShard


def split_layers(num_layers: int, stages: int) -> list[tuple[int, int]]:
    """Contiguous, as-even-as-possible layer ranges."""
    base, rem = divmod(num_layers, stages)
    out, start = [], 0
    for s in range(stages):
        n = base + (1 if s < rem else 0)
        out.append((start, start + n))
        start += n
    return out


class PipelineStage:
    def __init__(self, model, group=None, micro_batches: int = 4):
        self.group = group
        self.rank = dist.get_rank(group)
        self.stages = dist.get_world_size(group)
        self.micro_batches = micro_batches
        lo, hi = split_layers(len(model.layers), self.stages)[self.rank]
        self.shard = ModelShard(model, lo, hi)
        self.model = model
        self.first, self.last = self.rank == 0, self.rank == self.stages - 1
        self.prev = None if self.first else dist.get_global_rank(group, self.rank - 1) if group else self.rank - 1
        self.next = None if self.last else dist.get_global_rank(group, self.rank + 1) if group else self.rank + 1

    def parameters(self):
        """Parameters this stage trains (its layers, plus embedding / final norm + head at the ends)."""
        m = self.model
        ps = [p for blk in m.layers[self.shard.start:self.shard.end] for p in blk.parameters()]
        if self.first:
            ps += list(m.tok_embeddings.parameters())
        if self.last:
            ps += list(m.norm.parameters()) + (list(m.lm_head.parameters()) if m.lm_head is not None else [])
        return ps

    # ------------------------------------------------------------------ p2p helpers
    def _recv_pair(self, shape, dtype, device, src):
        x = torch.empty(shape, dtype=dtype, device=device)
        s = torch.empty(shape, dtype=dtype, device=device)
        reqs = [dist.irecv(x, src=src, group=self.group), dist.irecv(s, src=src, group=self.group)]
        return x, s, reqs

    def _send_pair(self, a, b, dst):
        return [dist.isend(a.contiguous(), dst=dst, group=self.group), dist.isend(b.contiguous(), dst=dst, group=self.group)]

    # ------------------------------------------------------------------ one training step
    def train_step(self, ids=None, targets=None, hidden_shape=None, dtype=torch.float32, device="cpu"):
        """Runs all micro-batches through this stage with the 1F1B order. ``ids`` (first stage) and
        ``targets`` (last stage) are ``[micro_batches, mb, S]`` int32 tensors; ``hidden_shape`` is the
        per-micro-batch activation shape ``(mb, S, d)``. Gradients accumulate in the parameters'
        ``.grad``; returns the mean loss on the last stage, else None."""
        M = self.micro_batches
        warm = min(M, self.stages - self.rank - 1)
        inputs, outputs, losses, pending = [], [], [], []
        fwd = bwd = 0

        def forward_one(i):
            nonlocal pending
            if self.first:
                x, s = self.shard(ids[i].to(device))
                inp = None
            else:
                xin, sin, reqs = self._recv_pair(hidden_shape, dtype, device, self.prev)
                for r in reqs:
                    r.wait()
                xin.requires_grad_()
                sin.requires_grad_()
                B, S = hidden_shape[0], hidden_shape[1]
                pos = torch.arange(S, device=device, dtype=torch.int32).repeat(B)
                x, s = self.shard(xin, sin, pos)
                inp = (xin, sin)
            if self.last:
                logits = x
                from ..ops import functional as F

                rows = logits.numel() // logits.shape[-1]
                # the 1/M of the micro-batch mean goes into the loss scale: the fused CUDA loss writes
                # its (scaled) gradient in the forward pass and expects an upstream gradient of 1
                loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets[i].to(device).reshape(-1),
                                       1.0 / (rows * M))
                outputs.append(loss)
                losses.append(loss.detach())
            else:
                if s is None:
                    s = torch.zeros_like(x)
                pending += self._send_pair(x.detach(), s.detach(), self.next)
                outputs.append((x, s))
            inputs.append(inp)

        def backward_one(i):
            nonlocal pending
            out, inp = outputs[i], inputs[i]
            if self.last:
                out.backward()
            else:
                gx, gs, reqs = self._recv_pair(hidden_shape, dtype, device, self.next)
                for r in reqs:
                    r.wait()
                torch.autograd.backward([out[0], out[1]], [gx, gs])
            if inp is not None:
                gxi = inp[0].grad if inp[0].grad is not None else torch.zeros_like(inp[0])
                gsi = inp[1].grad if inp[1].grad is not None else torch.zeros_like(inp[1])
                pending += self._send_pair(gxi, gsi, self.prev)
            outputs[i] = None
            inputs[i] = None

        for _ in range(warm):
            forward_one(fwd)
            fwd += 1
        while fwd < M:
            forward_one(fwd)
            fwd += 1
            backward_one(bwd)
            bwd += 1
        while bwd < M:
            backward_one(bwd)
            bwd += 1
        for r in pending:
            r.wait()
        return torch.stack(losses).sum() if self.last else None
