"""All-gather fused into the consuming GEMM (sequence-sharded activations x column-parallel weight).

Every rank owns ``M / world`` rows of an activation matrix ``A`` [M, K] and a shard ``W`` [N, K] of a
column-parallel weight; it needs ``C = A @ W.T`` for all M rows. The library form is an all-gather
followed by a GEMM (the reference's tensor-parallel layers gather with NCCL and then call the GEMM,
src/distributed.cpp:102-138). Here one launch does both: a few SM pairs copy the peers' rows over NVLink
into this rank's buffer (non-multicast TMA loads from peer memory, TMA stores locally) while the other SM
pairs multiply, starting with the rank's own rows and taking the remote 256-row tiles in the order in
which they arrive (``gemm_2cta.cu``, GROUP_GATHER). Every remote byte crosses NVLink once.

Two symmetric buffers alternate between calls: a rank rewrites its rows of a buffer only after the flag
barrier of the following call, by which time every peer has finished the launch that read them.
"""
from __future__ import annotations

import torch

from ..ops import native
from . import symm


class AllGatherGemm:
    def __init__(self, group, device, rows: int, cols: int, copier_clusters: int = 6):
        import torch.distributed as dist

        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if rows % (256 * self.world) != 0 or cols % 64 != 0:
            raise ValueError("AllGatherGemm: rows must be a multiple of 256 x world and cols of 64")
        self.rows, self.cols = rows, cols
        self.shard_rows = rows // self.world
        self.bufs = [symm.make_buffer(rows * cols, torch.bfloat16, device, group) for _ in range(2)]
        self.counts = [torch.zeros(rows // 256, device=device, dtype=torch.int32) for _ in range(2)]
        self.cur = 0
        self.copier_clusters = copier_clusters if self.world > 1 else 0
        self.barrier = symm.FlagBarrier(device, group) if self.world > 1 else None

    def _rows(self, rows):
        rows = self.rows if rows is None else rows
        if rows > self.rows or rows % (256 * self.world) != 0:
            raise ValueError(f"AllGatherGemm: {rows} rows (capacity {self.rows}, multiple of {256 * self.world} needed)")
        return rows

    def shard(self, rows: int | None = None) -> torch.Tensor:
        """This rank's rows of the buffer the next ``run`` will use: write the local activations here.
        ``rows``: total rows of this call's matrix (default: the capacity)."""
        rows = self._rows(rows)
        full = self.bufs[self.cur].tensor[: rows * self.cols].view(rows, self.cols)
        sh = rows // self.world
        return full[self.rank * sh:(self.rank + 1) * sh]

    def run(self, weight: torch.Tensor, out: torch.Tensor | None = None, rows: int | None = None):
        """``(C, A)``: C = A @ weight.T ([rows, N] bf16) and the gathered A (valid until the second next
        call). Every rank must have written ``shard(rows)`` on the current stream before calling."""
        C = native.require()
        rows = self._rows(rows)
        if out is None:
            out = torch.empty(rows, weight.shape[0], device=self.device, dtype=torch.bfloat16)
        i = self.cur
        if self.barrier is not None:
            self.barrier.sync()                       # every rank's rows are in its buffer
        # the tile counters restart at zero every call (the row count may differ from call to call)
        self.counts[i].zero_()
        C.gemm_allgather_a(self.bufs[i].ptrs, rows, self.cols, weight, out, self.rank, self.counts[i], 1,
                           self.copier_clusters, native.status_word(self.device))
        self.cur ^= 1
        return out, self.bufs[i].tensor[: rows * self.cols].view(rows, self.cols)


class ShardedWeightGemm:
    """``y = x @ W.T`` for a weight ``W`` [N, K] whose bf16 image is sharded by output rows over the ranks
    (each rank keeps and updates ``N / world`` rows): the parameter all-gather fused into the first GEMM
    that consumes the weight. Copier CTAs of the launch pull the peers' rows into this rank's full-size
    buffer while the other SM pairs multiply, own column block first (``gemm_allgather_b``); afterwards
    the buffer holds all of ``W`` until the next ``write_shard`` (the backward products can read it).
    The reference gathers parameters with a library all-gather before the layer runs
    (src/distributed.cpp:102-138)."""

    def __init__(self, group, device, out_features: int, in_features: int, copier_clusters: int = 2):
        import torch.distributed as dist

        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if out_features % (256 * self.world) != 0 or in_features % 64 != 0:
            raise ValueError("ShardedWeightGemm: out_features must be a multiple of 256 x world, in_features of 64")
        self.N, self.K = out_features, in_features
        self.buf = symm.make_buffer(out_features * in_features, torch.bfloat16, device, group)
        self.counts = torch.zeros(out_features // 256, device=device, dtype=torch.int32)
        self.copier_clusters = copier_clusters if self.world > 1 else 0
        self.barrier = symm.FlagBarrier(device, group) if self.world > 1 else None

    def weight(self) -> torch.Tensor:
        """The full [N, K] buffer (all rows valid after ``run``; before it only this rank's)."""
        return self.buf.tensor.view(self.N, self.K)

    def write_shard(self, rows: torch.Tensor) -> None:
        """Replace this rank's rows (e.g. after an optimizer step). The barrier first makes sure that no
        peer is still copying the previous values."""
        if self.barrier is not None:
            self.barrier.sync()
        sh = self.N // self.world
        self.weight()[self.rank * sh:(self.rank + 1) * sh].copy_(rows)

    def run(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        C = native.require()
        x2 = x.reshape(-1, self.K)
        if out is None:
            out = torch.empty(x2.shape[0], self.N, device=self.device, dtype=torch.bfloat16)
        if self.barrier is not None:
            self.barrier.sync()                       # every rank's rows are in its buffer
        self.counts.zero_()
        C.gemm_allgather_b(x2, self.buf.ptrs, self.N, out, self.rank, self.counts, 1, self.copier_clusters,
                           native.status_word(self.device))
        return out
