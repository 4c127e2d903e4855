"""Inference engine: paged KV cache, prefill + decode, tensor parallelism, CUDA-graph decode.

Role of the reference's ``Generator`` (src/generator.cpp:14-145), ``engine::InferenceEngine``
(engines/inference/inference.cpp) and ``ContinuousBatching`` (src/inference_opt.cpp:281-373), for
batches of sequences instead of one, with weights kept in their OIL storage format.

Per layer: RMSNorm (+ residual add) -> fused QKV projection (codebook-dequant GEMM) -> RoPE in
place -> K/V scattered into pages -> attention (tcgen05 flash attention over the prompt for
prefill, split-KV paged attention for decode) -> output projection -> RMSNorm -> gate/up
projection -> SwiGLU / ReLU^2 gate -> down projection.

Tensor parallelism (``tp``): attention heads and FFN columns are sharded; the two row-parallel
projections of a layer store their bf16 partials into this rank's slot on every peer (from the GEMM
epilogue, or from a push kernel after split-K), a flag barrier follows, and the sum over slots is
fused with the residual add and the next RMSNorm. Prefill-sized sums use a pull all-reduce kernel
or a GEMM with a fused reduce-scatter epilogue. No library collective runs inside a step. The
lm_head is vocabulary-parallel; logits are gathered with peer stores. An embedding table stored in
an OIL format is expanded row by row inside the gather kernel.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import torch

from ..models.config import TransformerConfig
from ..ops import functional as F
from ..ops import native
from ..utils import trace
from .kv_paged import PagedKVCache
from .quant_weights import QFMT, QuantLinear, reserve_accumulator
from .sampler import SamplerConfig, sample


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    new_tokens: int = 0
    ttft_s: float = 0.0            # prefill + first sample
    decode_s: float = 0.0
    tokens_per_s: float = 0.0      # generated tokens per second over the whole batch (decode phase)
    kv_bytes: int = 0
    kv_utilization: float = 0.0


@dataclass
class GenerationResult:
    tokens: list = field(default_factory=list)   # per sequence: generated token ids
    stats: GenerationStats = field(default_factory=GenerationStats)


ONESHOT_MAX_TOKENS = 256   # up to this many tokens a row-parallel sum takes the one-barrier path


class TPContext:
    """Tensor-parallel state of one rank: the symmetric buffers of the two all-reduce paths, a
    symmetric logits buffer and a flag barrier whose epoch lives on the device.

    One-shot path (decode): ``staging[b]`` holds one bf16 slot per rank; every rank writes its
    partial into its slot on all peers, one barrier, then sums its own slots. Two staging buffers
    alternate, so a peer may already write the next partial while this rank still sums.
    Two-shot path (prefill): partials sit in ``part``; after a barrier each rank pulls its slice
    from all peers, sums and stores the result into every peer's ``out[b]``; a second barrier."""

    def __init__(self, group, device, max_tokens: int, hidden: int, vocab_shard: int, max_batch: int):
        import torch.distributed as dist

        from ..parallel import symm

        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.slot_stride = ONESHOT_MAX_TOKENS * hidden
        self.staging = [symm.make_buffer(self.world * self.slot_stride, torch.bfloat16, device, group).zero_()
                        for _ in range(2)]
        self.max_tokens = max_tokens
        big = max(max_tokens, ONESHOT_MAX_TOKENS) * hidden
        self.part = symm.make_buffer(big, torch.bfloat16, device, group)
        self.out = [symm.make_buffer(big, torch.bfloat16, device, group) for _ in range(2)]
        self.logits = symm.make_buffer(max_batch * vocab_shard * self.world, torch.bfloat16, device, group)
        self.barrier = symm.FlagBarrier(device, group, device_epoch=True)
        self.which = 0
        # Prefill-sized row-parallel sums. True: GEMM whose epilogue stores each 256-row tile into the
        # owner rank's slot in full 128-byte lines, then reduce + all-gather by peer stores. False:
        # local GEMM, then the pull all-reduce kernel. Measured on B200: at 2 ranks (16384 x 4096 x
        # 4096) fused 0.48 ms, pull 0.58 ms, GEMM + NCCL all-reduce 0.64 ms; at 8 ranks (65536 x 4096
        # x 1024) fused 2.82 ms, pull 2.02 ms, NCCL 2.09 ms, and the TP8 time to first token is 0.33 s
        # fused against 0.23 s pull. So the fused epilogue is the default at 2 ranks only.
        # MYTHOS_TP_FUSED_RS=0/1 overrides.
        import os

        default = "1" if self.world <= 2 else "0"
        self.fused_reduce_scatter = os.environ.get("MYTHOS_TP_FUSED_RS", default) != "0"
        # Decode-sized sums fused with residual + RMSNorm, optional single-launch form: one kernel
        # pushes the row, signals a per-row flag on every peer, waits for the peers' flags of that
        # row and reduces (instead of push kernel + barrier kernel + sum kernel). Measured at 2 ranks
        # on a 64 x 4096 activation: 18.6 us against 17.7 us for the three launches (which overlap
        # their launch latencies on the stream; the chain of NVLink round trips is the same), so it
        # is off unless MYTHOS_TP_ROW_FLAGS=1. Flags: [2 staging buffers][world][rows] int32.
        self.row_flags = symm.make_buffer(2 * self.world * ONESHOT_MAX_TOKENS, torch.int32, device, group).zero_()
        self.row_epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.row_arrive = torch.zeros(1, dtype=torch.int32, device=device)
        self.row_signalled = os.environ.get("MYTHOS_TP_ROW_FLAGS", "0") != "0"
        # Sequence-parallel prefill: between the row-parallel and the next column-parallel projection every
        # rank keeps T / world tokens. The row-parallel sum is a reduce-scatter (from the GEMM epilogue at 2
        # ranks, by peer loads after a local GEMM above that), the owner adds the residual and normalises
        # its tokens only, and the column-parallel GEMM gathers the normalised rows from the peers while it
        # multiplies (all-gather fused into the GEMM, parallel/ag_gemm.py). No all-reduce, and residual /
        # RMSNorm work is divided by the world size. Measured time to first token, Llama-3-8B shape, 64 x
        # 1024 tokens at 8 ranks: 0.194 s against 0.223 s for the all-reduce path; at 2 ranks the two are
        # equal (0.118 s), so it is the default above 2 ranks. MYTHOS_TP_SEQ_PARALLEL=0/1 overrides.
        self.seq_parallel = os.environ.get("MYTHOS_TP_SEQ_PARALLEL", "1" if self.world > 2 else "0") != "0" \
            and self.world > 1
        self.ag = None
        if self.seq_parallel and hidden % 64 == 0:
            from ..parallel.ag_gemm import AllGatherGemm

            cap = max_tokens // (256 * self.world) * (256 * self.world)
            if cap > 0:
                self.ag = AllGatherGemm(group, device, cap, hidden,
                                        copier_clusters=int(os.environ.get("MYTHOS_AG_COPIERS", str(min(12, 2 * self.world)))))
        if self.world > 1:
            torch.cuda.synchronize(device)
            dist.barrier(group=group)      # every rank's flags are zero before anyone signals


def _embed_gather_ok(cfg: TransformerConfig) -> bool:
    """The row-gather kernel expands 16 weights per thread and needs whole 64-weight blocks per row."""
    return cfg.hidden_size % 64 == 0


def _zero_ffn_padding(up: QuantLinear, down: QuantLinear, f_loc: int, f_pad: int, gated: bool) -> None:
    """Set the padded FFN units of a shard to exact zeros: rows [f_loc, f_pad) of each half of the up
    projection and columns [f_loc, f_pad) of the down projection. I2_S only (trit code 1 is zero
    whatever the block scale; four trits per byte, so f_loc has to be a multiple of 4); codebook
    formats have no exact zero."""
    if up.fmt != "i2s" or down.fmt != "i2s" or f_loc % 4:
        raise ValueError("padding an FFN shard needs I2_S weights and a shard width that is a multiple of 4; "
                         "choose a tensor-parallel size whose FFN shard is a multiple of 64")
    zero = 0x55                                            # 01 01 01 01
    rows_up = up.packed.view(up.N, up.K // 4)
    rows_up[f_loc:f_pad] = zero
    if gated:
        rows_up[f_pad + f_loc:2 * f_pad] = zero
    down.packed.view(down.N, down.K // 4)[:, f_loc // 4:] = zero


def _zero_padded_heads(qkv: QuantLinear, o: QuantLinear, eng, cfg: TransformerConfig) -> None:
    """Synthetic engine: set the q / k / v rows and the output-projection columns of this rank's padded
    heads (global head index >= the model's head count) to exact zeros."""
    D, hl, kl = cfg.head_dim, eng.h_local, eng.hkv_local
    real_q = max(0, min(hl, cfg.num_heads - eng.rank * hl))
    real_kv = max(0, min(kl, cfg.kv_heads - eng.rank * kl))
    spans = [(real_q * D, hl * D), (hl * D + real_kv * D, (hl + kl) * D), ((hl + kl) * D + real_kv * D, (hl + 2 * kl) * D)]
    if qkv.fmt == "i2s":
        rows = qkv.packed.view(qkv.N, qkv.K // 4)
        for a, b in spans:
            rows[a:b] = 0x55                               # trit code 1 = zero, four per byte
        o.packed.view(o.N, o.K // 4)[:, real_q * D // 4:] = 0x55
    else:                                                  # unquantised weights
        for a, b in spans:
            qkv.dense[a:b] = 0
        o.dense[:, real_q * D:] = 0


def _pad_rows(w: torch.Tensor, start: int, size: int, padded: int) -> torch.Tensor:
    """Rows [start, start + size) of w followed by zero rows up to ``padded`` rows."""
    part = w[start:start + size]
    if padded == size:
        return part
    return torch.cat([part, part.new_zeros(padded - size, w.shape[1])], dim=0)


def _embed_block(cfg: TransformerConfig) -> int:
    return cfg.oil_block_size if cfg.hidden_size % cfg.oil_block_size == 0 else 64


class _Layer:
    __slots__ = ("attn_norm", "ffn_norm", "qkv", "o", "up", "down")


class InferenceEngine:
    def __init__(self, cfg: TransformerConfig, device="cuda", max_batch: int = 64, max_seq_len: int | None = None,
                 page_size: int = 16, tp: TPContext | None = None, kv_pages: int | None = None,
                 kv_dtype: str = "bf16"):
        """``kv_dtype``: "bf16", or "int8" for pages of int8 rows with one scale per (token, kv head)
        (half the KV bytes per decode step; the reference's block-quantised cache mode,
        src/kv_cache.cpp:13-42, 78-137)."""
        if kv_dtype not in ("bf16", "int8"):
            raise ValueError(f"kv_dtype must be 'bf16' or 'int8', got {kv_dtype!r}")
        self.cfg, self.device, self.tp = cfg, torch.device(device), tp
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len or cfg.max_seq_len
        self.page_size = page_size
        self.world = tp.world if tp is not None else 1
        self.rank = tp.rank if tp is not None else 0
        # Heads that do not divide by the tensor-parallel size are padded with zero heads (zero q / k / v
        # rows, zero output-projection columns: a padded head attends uniformly over zero values and adds
        # nothing). 20 heads on 8 ranks become 24, three per rank. Needs a format with an exact zero.
        group = cfg.num_heads // cfg.kv_heads
        self.hkv_eff = (cfg.kv_heads + self.world - 1) // self.world * self.world
        self.h_eff = self.hkv_eff * group
        if self.h_eff != cfg.num_heads:
            af = cfg.attn_format or cfg.weight_format
            if af not in ("i2s", "bf16", "fp16", "fp32"):
                raise ValueError(f"heads ({cfg.num_heads}/{cfg.kv_heads}) do not divide by the tensor-parallel size "
                                 f"{self.world}; zero-padding them needs I2_S or unquantised attention weights, not {af}")
        self.h_local = self.h_eff // self.world
        self.hkv_local = self.hkv_eff // self.world
        pages_per_seq = (self.max_seq_len + page_size - 1) // page_size
        self.cache = PagedKVCache(cfg.num_layers, self.hkv_local, cfg.head_dim, kv_pages or max_batch * pages_per_seq,
                                  page_size, max_batch, pages_per_seq, self.device,
                                  dtype=torch.int8 if kv_dtype == "int8" else torch.bfloat16)
        self.layers: list[_Layer] = []
        self.embed = None        # bf16 [V, d], or a QuantLinear when the table is stored in an OIL format
        self.final_norm = None
        self.head: QuantLinear | None = None
        self._graph = None
        self._static = {}
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 1
        self._sms = sm
        self._scratch = None
        self._counters = None
        self.fused_decode = True     # decode steps use the fused epilogue kernels when the model allows
        # tokens per pass of the chunked paged prefill (all sequences of the pass together); under tensor
        # parallelism a pass must also fit the symmetric all-reduce buffers
        self.prefill_chunk = 8192 if tp is None else min(8192, getattr(tp, "max_tokens", 8192))
        # generate(): equal-length batches above this many prompt tokens are prefilled in chunks
        self.prefill_chunk_threshold = 1 << 30
        self.last_prefix_hit = 0     # tokens of the latest start_sequence that came from shared pages

    # ------------------------------------------------------------------ weights
    @classmethod
    def from_model(cls, model, **kw) -> "InferenceEngine":
        """Pack a (trained or random) ``DenseModel`` into inference weights. Under tensor
        parallelism every rank packs its own shard of each matrix."""
        cfg = model.cfg
        eng = cls(cfg, **kw)
        dev = eng.device
        W, r = eng.world, eng.rank
        D, H, Hkv = cfg.head_dim, cfg.num_heads, cfg.kv_heads
        if cfg.embed_format in QFMT and _embed_gather_ok(cfg):
            eng.embed = QuantLinear.from_float(model.tok_embeddings.weight.detach().float().to(dev), cfg.embed_format,
                                               _embed_block(cfg), cfg.codebook_group)
        else:
            eng.embed = model.tok_embeddings.weight.detach().to(dev, torch.bfloat16).contiguous()
        eng.final_norm = model.norm.weight.detach().to(dev, torch.bfloat16).contiguous()
        for blk in model.layers:
            L = _Layer()
            L.attn_norm = blk.attention_norm.weight.detach().to(dev, torch.bfloat16).contiguous()
            L.ffn_norm = blk.ffn_norm.weight.detach().to(dev, torch.bfloat16).contiguous()
            att, ffn = blk.attention, blk.ffn
            if W == 1:
                L.qkv = QuantLinear.from_oil_linear(att.qkv_proj)
                L.o = QuantLinear.from_oil_linear(att.o_proj)
                L.up = QuantLinear.from_oil_linear(ffn.up_proj)
                L.down = QuantLinear.from_oil_linear(ffn.down_proj)
            elif eng.h_eff != H:
                # zero-padded heads: shard the padded float weights (formats with an exact zero only)
                wq = att.qkv_proj.weight.detach().float()
                He, Ke, hl, kl = eng.h_eff, eng.hkv_eff, eng.h_local, eng.hkv_local
                qp = _pad_rows(wq, 0, H * D, He * D)[r * hl * D:(r + 1) * hl * D]
                kp = _pad_rows(wq, H * D, Hkv * D, Ke * D)[r * kl * D:(r + 1) * kl * D]
                vp = _pad_rows(wq, (H + Hkv) * D, Hkv * D, Ke * D)[r * kl * D:(r + 1) * kl * D]
                fmt = att.qkv_proj.fmt if att.qkv_proj.fmt == "i2s" else "bf16"
                L.qkv = QuantLinear.from_float(torch.cat([qp, kp, vp]).contiguous().to(dev), fmt, att.qkv_proj.block_size)
                wo = att.o_proj.weight.detach().float()
                wo = torch.cat([wo, wo.new_zeros(wo.shape[0], (He - H) * D)], dim=1)[:, r * hl * D:(r + 1) * hl * D]
                L.o = QuantLinear.from_float(wo.contiguous().to(dev), fmt,
                                             att.o_proj.block_size if (hl * D) % att.o_proj.block_size == 0 else 64)
            else:
                L.qkv = _shard_rows_multi(att.qkv_proj, [(0, H * D), (H * D, Hkv * D), ((H + Hkv) * D, Hkv * D)], r, W)
                L.o = _shard_cols(att.o_proj, r, W)
                f = ffn.up_proj.out_features // (2 if ffn.gated else 1)
                parts = [(0, f), (f, f)] if ffn.gated else [(0, f)]
                L.up = _shard_rows_multi(ffn.up_proj, parts, r, W)
                L.down = _shard_cols(ffn.down_proj, r, W)
            eng.layers.append(L)
        head_mod = model.lm_head
        if head_mod is None:
            w = model.tok_embeddings.weight.detach().float()
            V = w.shape[0]
            rows = slice(r * V // W, (r + 1) * V // W)
            eng.head = QuantLinear.from_float(w[rows].to(dev), "bf16")
        elif W == 1:
            eng.head = QuantLinear.from_oil_linear(head_mod)
        else:
            eng.head = _shard_rows_multi(head_mod, [(0, head_mod.out_features)], r, W)
        return eng

    @classmethod
    def random(cls, cfg: TransformerConfig, seed: int = 0, **kw) -> "InferenceEngine":
        """Synthetic engine for benchmarks: every matrix is created directly in its storage format
        (quantile codebooks with uniform-random indices, trits with p = 0.25/0.5/0.25), shard by
        shard, so a large model never exists in fp32. Embeddings are random bf16."""
        ffn_multiple = int(kw.pop("ffn_multiple", 64))
        eng = cls(cfg, **kw)
        dev, W, r = eng.device, eng.world, eng.rank
        if cfg.ffn_hidden_size % W or ffn_multiple % 64:
            raise ValueError("the FFN width must divide by the tensor-parallel size and ffn_multiple by 64")
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + r)
        D, d = cfg.head_dim, cfg.hidden_size
        bs, grp = cfg.oil_block_size, cfg.codebook_group
        f = cfg.ffn_hidden_size
        ge = torch.Generator(device=dev).manual_seed(seed)           # replicated tensors: same on every rank

        def mk(fmt, N, K):
            if fmt not in QFMT:
                return QuantLinear.from_float(torch.randn(N, K, device=dev, generator=g) * 0.02, "bf16")
            return QuantLinear.random(fmt, N, K, bs if K % bs == 0 else 64, grp, device=dev, generator=g)

        af = cfg.attn_format or cfg.weight_format
        ff = cfg.ffn_format or cfg.weight_format
        if cfg.embed_format in QFMT and _embed_gather_ok(cfg):
            eng.embed = QuantLinear.random(cfg.embed_format, cfg.vocab_size, d, _embed_block(cfg), grp, device=dev,
                                           generator=ge)
        else:
            eng.embed = (torch.randn(cfg.vocab_size, d, device=dev, generator=ge) * 0.02).to(torch.bfloat16)
        eng.final_norm = torch.ones(d, device=dev, dtype=torch.bfloat16)
        for _ in range(cfg.num_layers):
            L = _Layer()
            L.attn_norm = torch.ones(d, device=dev, dtype=torch.bfloat16)
            L.ffn_norm = torch.ones(d, device=dev, dtype=torch.bfloat16)
            L.qkv = mk(af, (eng.h_local + 2 * eng.hkv_local) * D, d)
            L.o = mk(af, d, eng.h_local * D)
            if eng.h_eff != cfg.num_heads:
                _zero_padded_heads(L.qkv, L.o, eng, cfg)
            # The down projection's reduction length (this rank's FFN columns) has to be a multiple
            # of 64 for the dequant GEMM; a shard that is not (6912 / 8 = 864) is padded with zero
            # weights: zero rows of the up projection give act(0) * 0 = 0 and meet zero columns.
            f_loc = f // W
            f_pad = (f_loc + ffn_multiple - 1) // ffn_multiple * ffn_multiple
            L.up = mk(ff, (2 if cfg.gated_ffn else 1) * f_pad, d)
            L.down = mk(ff, d, f_pad)
            if f_pad != f_loc:
                _zero_ffn_padding(L.up, L.down, f_loc, f_pad, cfg.gated_ffn)
            eng.layers.append(L)
        hf = cfg.weight_format if cfg.embed_format in ("fp32", "fp16", "bf16") else cfg.embed_format
        eng.head = mk(hf, cfg.vocab_size // W, d)
        return eng

    def weight_bytes(self) -> int:
        n = self.head.nbytes()
        n += self.embed.nbytes() if isinstance(self.embed, QuantLinear) else self.embed.numel() * 2
        for L in self.layers:
            n += L.qkv.nbytes() + L.o.nbytes() + L.up.nbytes() + L.down.nbytes()
        return n

    # ------------------------------------------------------------------ building blocks
    def _embed(self, ids: torch.Tensor, x: torch.Tensor) -> None:
        """Token rows into ``x``; a quantised table is expanded row by row inside the gather."""
        if isinstance(self.embed, QuantLinear):
            self.embed.gather_rows(ids, x)
        else:
            native.require().embedding_fwd(ids, self.embed, x)

    def _row_parallel(self, lin: QuantLinear, x: torch.Tensor) -> torch.Tensor:
        """x [T, K_local] @ W_shard^T, summed over ranks -> bf16 [T, d] (the all-reduce runs in this
        framework's own kernels over peer memory)."""
        if self.tp is None:
            return lin.matmul(x)
        tp, C = self.tp, native.require()
        T, n = x.shape[0], x.shape[0] * lin.N
        b = tp.which
        tp.which ^= 1
        if lin.dense is None and T <= ONESHOT_MAX_TOKENS:
            stage = tp.staging[b]
            slot_off = tp.rank * tp.slot_stride
            if lin.K // 64 <= 16:
                # short reduction: one K split, the GEMM epilogue stores straight into the peers' slots
                lin.matmul(x, peer_ptrs=stage.ptrs, k_splits=1, peer_bf16_offset=slot_off)
            else:
                # split-K into the local fp32 accumulator, then one kernel converts and pushes it
                acc = lin.matmul_acc(x)
                C.tp_push(acc, stage.ptrs, tp.rank, slot_off)
            tp.barrier.sync()
            out = torch.empty(T, lin.N, device=x.device, dtype=torch.bfloat16)
            C.tp_reduce_slots(stage.tensor, tp.world, tp.slot_stride, None, out)
            return out
        if tp.fused_reduce_scatter and T % (tp.world * 256) == 0 and lin.N >= 256 and lin.N % 64 == 0:
            # GEMM with a fused reduce-scatter epilogue: every 256-row output tile is stored
            # straight into the owner rank's slot for this rank while the GEMM is still running;
            # after one barrier each rank sums its slots and stores the result to all peers.
            rows = T // tp.world
            n_slot = rows * lin.N
            w = lin.dense if lin.dense is not None else lin.dequantize()
            C.gemm_reduce_scatter(x, w, tp.part.ptrs, tp.rank, rows, n_slot, native.status_word(x.device))
            tp.barrier.sync()
            C.tp_reduce_slots_bcast(tp.part.tensor, tp.world, n_slot, tp.out[b].ptrs, tp.rank, tp.rank * n_slot, n_slot)
            tp.barrier.sync()
            return tp.out[b].tensor[:n].view(T, lin.N)
        # other sizes: local GEMM into the symmetric partial buffer, two-shot all-reduce
        part = tp.part.tensor[:n].view(T, lin.N)
        lin.matmul(x, out=part)
        tp.barrier.sync()
        C.tp_allreduce_pull(tp.part.ptrs, tp.out[b].ptrs, tp.rank, n)
        tp.barrier.sync()
        return tp.out[b].tensor[:n].view(T, lin.N)

    def _row_parallel_norm(self, lin: QuantLinear, x, gamma, stream):
        """Decode-sized row-parallel projection fused with what follows it: returns
        ``(rmsnorm(stream + x W^T) * gamma, stream + x W^T)``. The sum over K splits (and over
        ranks under tensor parallelism), the residual add and the normalisation are one kernel."""
        C, tp = native.require(), self.tp
        T = x.shape[0]
        normed = torch.empty(T, lin.N, device=x.device, dtype=torch.bfloat16)
        new_stream = torch.empty_like(normed)
        if tp is None:
            acc = lin.matmul_acc(x)
            C.sum_residual_rmsnorm(acc, None, 0, 0, stream, gamma, new_stream, normed, self.cfg.norm_eps)
            return normed, new_stream
        b = tp.which
        tp.which ^= 1
        stage = tp.staging[b]
        slot_off = tp.rank * tp.slot_stride
        acc = None
        if lin.K // 64 <= 16:
            lin.matmul(x, peer_ptrs=stage.ptrs, k_splits=1, peer_bf16_offset=slot_off)
        else:
            acc = lin.matmul_acc(x)
        if tp.row_signalled:
            from ..parallel.symm import DEFAULT_BARRIER_LIMIT_CYCLES

            C.tp_sum_residual_rmsnorm(acc, stage.ptrs, tp.row_flags.ptrs, tp.rank, tp.slot_stride, b,
                                      ONESHOT_MAX_TOKENS, stream, gamma, new_stream, normed, self.cfg.norm_eps,
                                      tp.row_epoch, tp.row_arrive, DEFAULT_BARRIER_LIMIT_CYCLES,
                                      native.status_word(x.device))
            return normed, new_stream
        if acc is not None:
            C.tp_push(acc, stage.ptrs, tp.rank, slot_off)
        tp.barrier.sync()
        C.sum_residual_rmsnorm(None, stage.tensor, tp.world, tp.slot_stride, stream, gamma, new_stream, normed,
                               self.cfg.norm_eps)
        return normed, new_stream

    def _fused_decode_ok(self, T: int) -> bool:
        cfg = self.cfg
        return (T <= ONESHOT_MAX_TOKENS and cfg.hidden_size % 8 == 0 and cfg.hidden_size <= 16384
                and (not self.cache.int8 or cfg.head_dim in (64, 128, 256))
                and all(m.dense is None for L in self.layers for m in (L.qkv, L.o, L.up, L.down))
                and (not cfg.gated_ffn or cfg.activation in ("silu", "relu2")))

    def _forward_decode(self, ids, pos, seq_ids, ctx_lens):
        """Decode step with the fused epilogue kernels: per layer QKV GEMM -> (finalize + RoPE + KV
        append) -> paged attention -> o GEMM -> (sum + residual + RMSNorm) -> up GEMM -> (finalize +
        gate) -> down GEMM -> (sum + residual + RMSNorm of the next layer)."""
        cfg, C = self.cfg, native.require()
        D, H, Hkv = cfg.head_dim, self.h_local, self.hkv_local
        T = ids.numel()
        scale = 1.0 / math.sqrt(D)
        table = self.cache.block_table
        dev = self.device
        x = torch.empty(T, cfg.hidden_size, device=dev, dtype=torch.bfloat16)
        self._embed(ids, x)
        n, stream = F.rmsnorm(x, self.layers[0].attn_norm, cfg.norm_eps, None)
        st = native.status_word(dev)
        for li, L in enumerate(self.layers):
            acc = L.qkv.matmul_acc(n)
            q = torch.empty(T, H, D, device=dev, dtype=torch.bfloat16)
            o = torch.empty(T, H, D, device=dev, dtype=torch.bfloat16)
            if self.cache.int8:
                ks, vs = self.cache.k_scale[li], self.cache.v_scale[li]
                C.qkv_rope_append(acc, pos, seq_ids, table, q, self.cache.k[li], self.cache.v[li], cfg.rope_theta, ks, vs)
                C.paged_attn_decode_int8(q, self.cache.k[li], self.cache.v[li], ks, vs, table, ctx_lens, o,
                                         self._scratch, self._counters, self._splits, scale, st)
            else:
                C.qkv_rope_append(acc, pos, seq_ids, table, q, self.cache.k[li], self.cache.v[li], cfg.rope_theta)
                C.paged_attn_decode(q, self.cache.k[li], self.cache.v[li], table, ctx_lens, o, self._scratch,
                                    self._counters, self._splits, scale, st)
            n, stream = self._row_parallel_norm(L.o, o.view(T, H * D), L.ffn_norm, stream)
            if cfg.gated_ffn:
                acc = L.up.matmul_acc(n)
                h = torch.empty(T, L.up.N // 2, device=dev, dtype=torch.bfloat16)
                C.finalize_gate(acc, h, 0 if cfg.activation == "silu" else 1)
            else:
                u = L.up.matmul(n)
                h = F.relu2(u) if cfg.activation == "relu2" else F.activation(u, cfg.activation)
            gamma = self.layers[li + 1].attn_norm if li + 1 < len(self.layers) else self.final_norm
            n, stream = self._row_parallel_norm(L.down, h, gamma, stream)
        return n

    def _forward(self, ids, pos, seq_ids, ctx_lens, prefill_shape=None, paged=None):
        """ids/pos/seq_ids: int32 [T]; ctx_lens int32 [B] (decode). Returns final hidden [T, d].
        ``paged`` = (cu_q, kv_lens, table_rows, max_q_len): the tokens are new tokens of several
        sequences, packed; their K/V go to the pages first and attention is the tcgen05 prefill kernel
        over the paged cache (prefix + new tokens)."""
        if prefill_shape is None and paged is None and self.fused_decode and self._fused_decode_ok(ids.numel()):
            return self._forward_decode(ids, pos, seq_ids, ctx_lens)
        if (prefill_shape is not None or paged is not None) and self._seq_parallel_ok(ids.numel()):
            return self._forward_prefill_sp(ids, pos, seq_ids, prefill_shape, paged)
        cfg, C = self.cfg, native.require()
        D, H, Hkv = cfg.head_dim, self.h_local, self.hkv_local
        scale = 1.0 / math.sqrt(D)
        table = self.cache.block_table
        x = torch.empty(ids.numel(), cfg.hidden_size, device=self.device, dtype=torch.bfloat16)
        self._embed(ids, x)
        branch, stream = x, None
        for li, L in enumerate(self.layers):
            n, stream = F.rmsnorm(branch, L.attn_norm, cfg.norm_eps, stream)
            qkv = L.qkv.matmul(n)
            T = qkv.shape[0]
            q = qkv[:, : H * D].unflatten(-1, (H, D))
            k = qkv[:, H * D:(H + Hkv) * D].unflatten(-1, (Hkv, D))
            v = qkv[:, (H + Hkv) * D:].unflatten(-1, (Hkv, D))
            if cfg.rope_theta > 0:   # q and k heads are adjacent in the fused projection: one launch
                C.rope(qkv[:, : (H + Hkv) * D].unflatten(-1, (H + Hkv, D)), pos, cfg.rope_theta, False)
            if self.cache.int8:
                C.kv_append_int8(k, v, self.cache.k[li], self.cache.v[li], self.cache.k_scale[li],
                                 self.cache.v_scale[li], table, pos, seq_ids)
            else:
                C.kv_append(k, v, self.cache.k[li], self.cache.v[li], table, pos, seq_ids)
            if paged is not None:
                cu_q, kv_lens, rows, max_q = paged
                o = torch.empty(T, H, D, device=self.device, dtype=torch.bfloat16)
                C.flash_attn_paged_prefill(q, self.cache.k[li], self.cache.v[li], rows, cu_q, kv_lens, o, max_q, scale,
                                           native.status_word(self.device))
                o = o.view(T, H * D)
            elif prefill_shape is not None:
                B, S = prefill_shape
                o = torch.empty(B, S, H, D, device=self.device, dtype=torch.bfloat16)
                lse = torch.empty(B, H, S, device=self.device, dtype=torch.float32)
                q4 = qkv.view(B, S, -1)[..., : H * D].unflatten(-1, (H, D))
                k4 = qkv.view(B, S, -1)[..., H * D:(H + Hkv) * D].unflatten(-1, (Hkv, D))
                v4 = qkv.view(B, S, -1)[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
                C.flash_attn_fwd(q4, k4, v4, o, lse, True, scale, native.status_word(self.device))
                o = o.view(T, H * D)
            else:
                o = torch.empty(T, H, D, device=self.device, dtype=torch.bfloat16)
                if self.cache.int8:
                    C.paged_attn_decode_int8(q, self.cache.k[li], self.cache.v[li], self.cache.k_scale[li],
                                             self.cache.v_scale[li], table, ctx_lens, o, self._scratch,
                                             self._counters, self._splits, scale, native.status_word(self.device))
                else:
                    C.paged_attn_decode(q, self.cache.k[li], self.cache.v[li], table, ctx_lens, o,
                                        self._scratch, self._counters, self._splits, scale,
                                        native.status_word(self.device))
                o = o.view(T, H * D)
            a = self._row_parallel(L.o, o)
            n, stream = F.rmsnorm(a, L.ffn_norm, cfg.norm_eps, stream)
            u = L.up.matmul(n)
            if cfg.gated_ffn:
                if cfg.activation == "relu2":
                    f = u.shape[-1] // 2
                    h = F.relu2(u[:, :f].contiguous()) * u[:, f:]
                else:
                    h = F.swiglu(u)
            else:
                h = F.relu2(u) if cfg.activation == "relu2" else F.activation(u, cfg.activation)
            branch = self._row_parallel(L.down, h)
        hfin, _ = F.rmsnorm(branch, self.final_norm, cfg.norm_eps, stream)
        return hfin

    def _seq_parallel_ok(self, T: int) -> bool:
        tp = self.tp
        if tp is None or tp.ag is None or T % (tp.world * 256) != 0 or T > tp.ag.rows or T > tp.max_tokens:
            return False
        cfg = self.cfg
        return (cfg.hidden_size >= 256 and cfg.hidden_size % 64 == 0
                and all(m.K % 64 == 0 for L in self.layers for m in (L.qkv, L.up)))

    def _attention_prefill(self, li, qkv, pos, seq_ids, prefill_shape, paged):
        """RoPE, K/V append and prefill attention for all tokens over this rank's heads -> [T, H_local * D]."""
        cfg, C = self.cfg, native.require()
        D, H, Hkv = cfg.head_dim, self.h_local, self.hkv_local
        scale = 1.0 / math.sqrt(D)
        T = qkv.shape[0]
        q = qkv[:, : H * D].unflatten(-1, (H, D))
        k = qkv[:, H * D:(H + Hkv) * D].unflatten(-1, (Hkv, D))
        v = qkv[:, (H + Hkv) * D:].unflatten(-1, (Hkv, D))
        if cfg.rope_theta > 0:
            C.rope(qkv[:, : (H + Hkv) * D].unflatten(-1, (H + Hkv, D)), pos, cfg.rope_theta, False)
        table = self.cache.block_table
        if self.cache.int8:
            C.kv_append_int8(k, v, self.cache.k[li], self.cache.v[li], self.cache.k_scale[li], self.cache.v_scale[li],
                             table, pos, seq_ids)
        else:
            C.kv_append(k, v, self.cache.k[li], self.cache.v[li], table, pos, seq_ids)
        if paged is not None:
            cu_q, kv_lens, rows, max_q = paged
            o = torch.empty(T, H, D, device=self.device, dtype=torch.bfloat16)
            C.flash_attn_paged_prefill(q, self.cache.k[li], self.cache.v[li], rows, cu_q, kv_lens, o, max_q, scale,
                                       native.status_word(self.device))
            return o.view(T, H * D)
        B, S = prefill_shape
        o = torch.empty(B, S, H, D, device=self.device, dtype=torch.bfloat16)
        lse = torch.empty(B, H, S, device=self.device, dtype=torch.float32)
        q4 = qkv.view(B, S, -1)[..., : H * D].unflatten(-1, (H, D))
        k4 = qkv.view(B, S, -1)[..., H * D:(H + Hkv) * D].unflatten(-1, (Hkv, D))
        v4 = qkv.view(B, S, -1)[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
        C.flash_attn_fwd(q4, k4, v4, o, lse, True, scale, native.status_word(self.device))
        return o.view(T, H * D)

    def _row_parallel_scatter(self, lin: QuantLinear, x: torch.Tensor) -> torch.Tensor:
        """x [T, K_local] @ W_shard^T summed over the ranks, this rank's T / world rows only. Two routes, as
        for the all-reduce: the GEMM's epilogue stores every 256-row tile into the owner's slot and the
        owner sums its slots (the faster one at 2 ranks), or a local GEMM into the symmetric partial
        buffer, a barrier, and one kernel that pulls this rank's rows from every peer and sums them."""
        tp, C = self.tp, native.require()
        T = x.shape[0]
        rows = T // tp.world
        out = torch.empty(rows, lin.N, device=x.device, dtype=torch.bfloat16)
        if tp.fused_reduce_scatter and lin.N >= 256 and lin.N % 64 == 0:
            n_slot = rows * lin.N
            w = lin.dense if lin.dense is not None else lin.dequantize()
            C.gemm_reduce_scatter(x, w, tp.part.ptrs, tp.rank, rows, n_slot, native.status_word(x.device))
            tp.barrier.sync()
            C.tp_reduce_slots(tp.part.tensor, tp.world, n_slot, None, out)
            return out
        n = T * lin.N
        lin.matmul(x, out=tp.part.tensor[:n].view(T, lin.N))
        tp.barrier.sync()
        C.tp_reduce_scatter_pull(tp.part.ptrs, tp.rank, n, out)
        return out

    def _forward_prefill_sp(self, ids, pos, seq_ids, prefill_shape, paged):
        """Prefill with sequence-sharded activations between the projections (see TPContext.seq_parallel).
        The slots of ``tp.part`` written by one reduce-scatter are summed before the barrier inside the
        next all-gather GEMM, so the next reduce-scatter cannot overwrite them early."""
        import torch.distributed as dist

        cfg, tp = self.cfg, self.tp
        self.sp_passes = getattr(self, "sp_passes", 0) + 1
        T = ids.numel()
        sh = T // tp.world
        lo = tp.rank * sh
        x = torch.empty(sh, cfg.hidden_size, device=self.device, dtype=torch.bfloat16)
        self._embed(ids[lo:lo + sh].contiguous(), x)
        branch, stream = x, None
        for li, L in enumerate(self.layers):
            n, stream = F.rmsnorm(branch, L.attn_norm, cfg.norm_eps, stream)
            tp.ag.shard(T).copy_(n)
            wq = L.qkv.dense if L.qkv.dense is not None else L.qkv.dequantize()
            qkv, _ = tp.ag.run(wq, rows=T)
            o = self._attention_prefill(li, qkv, pos, seq_ids, prefill_shape, paged)
            a = self._row_parallel_scatter(L.o, o)
            n, stream = F.rmsnorm(a, L.ffn_norm, cfg.norm_eps, stream)
            tp.ag.shard(T).copy_(n)
            wu = L.up.dense if L.up.dense is not None else L.up.dequantize()
            u, _ = tp.ag.run(wu, rows=T)
            if cfg.gated_ffn:
                if cfg.activation == "relu2":
                    f = u.shape[-1] // 2
                    h = F.relu2(u[:, :f].contiguous()) * u[:, f:]
                else:
                    h = F.swiglu(u)
            else:
                h = F.relu2(u) if cfg.activation == "relu2" else F.activation(u, cfg.activation)
            branch = self._row_parallel_scatter(L.down, h)
        hfin, _ = F.rmsnorm(branch, self.final_norm, cfg.norm_eps, stream)
        full = torch.empty(T, cfg.hidden_size, device=self.device, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, hfin.contiguous(), group=tp.group)   # once per pass: plumbing, not a hot op
        return full

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        lg = self.head.matmul(h)
        if self.tp is None:
            return lg
        return _gather_columns(lg, self.tp)

    # ------------------------------------------------------------------ paged / chunked prefill
    def _paged_prefill_ok(self) -> bool:
        return not self.cache.int8 and self.cfg.head_dim in (64, 128) and self.cache.page_size == 16

    @torch.no_grad()
    def _prefill_paged(self, seqs, token_lists, bases):
        """Run the new tokens ``token_lists[i]`` of sequence ``seqs[i]`` (which already holds
        ``bases[i]`` tokens; pages reserved) in one pass. Returns the hidden states of all new
        tokens, packed in the order given, and the row offsets of the sequences."""
        dev = self.device
        lens = [len(t) for t in token_lists]
        ids = torch.tensor([x for t in token_lists for x in t], dtype=torch.int32, device=dev)
        pos = torch.cat([torch.arange(b, b + n, dtype=torch.int32) for b, n in zip(bases, lens)]).to(dev)
        sid = torch.cat([torch.full((n,), s, dtype=torch.int32) for s, n in zip(seqs, lens)]).to(dev)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        cu_q = torch.tensor(cu, dtype=torch.int32, device=dev)
        kv_lens = torch.tensor([b + n for b, n in zip(bases, lens)], dtype=torch.int32, device=dev)
        rows = self.cache.block_table.index_select(0, torch.tensor(seqs, dtype=torch.long, device=dev)).contiguous()
        h = self._forward(ids, pos, sid, None, paged=(cu_q, kv_lens, rows, max(lens)))
        return h, cu

    @torch.no_grad()
    def _prefill_chunked(self, seqs, token_lists, bases=None):
        """Prefill through the paged kernel in passes of at most ``prefill_chunk`` tokens: any mix of
        prompt lengths, prompts longer than one pass, prompts that continue a cached prefix
        (``bases``). Advances the sequences; returns the hidden state of each sequence's last token."""
        cache = self.cache
        B = len(seqs)
        done = list(bases) if bases is not None else [0] * B
        start = list(done)
        total = [start[i] + len(token_lists[i]) for i in range(B)]
        last = [None] * B
        budget = max(16, getattr(self, "prefill_chunk", 8192))
        while any(done[i] < total[i] for i in range(B)):
            active = [i for i in range(B) if done[i] < total[i]]
            per = max(16, budget // len(active))
            part = [token_lists[i][done[i] - start[i]: done[i] - start[i] + per] for i in active]
            h, cu = self._prefill_paged([seqs[i] for i in active], part, [done[i] for i in active])
            for j, i in enumerate(active):
                n = len(part[j])
                cache.advance(seqs[i], n)
                done[i] += n
                if done[i] == total[i]:
                    last[i] = h[cu[j + 1] - 1]
        return torch.stack(last)

    def _prepare_decode_scratch(self, batch: int, max_ctx: int):
        pairs = max(1, batch * self.hkv_local)
        splits = max(1, min(32, (6 * self._sms + pairs - 1) // pairs, (max_ctx + 255) // 256))
        self._splits = splits
        widest = max([self.head.N] + [max(L.qkv.N, L.o.N, L.up.N, L.down.N) for L in self.layers])
        reserve_accumulator(self.device, min(batch, 256) * widest)
        need = batch * self.h_local * splits * (self.cfg.head_dim + 2)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, device=self.device, dtype=torch.float32)
            self._counters = torch.zeros(batch * self.hkv_local + 64, device=self.device, dtype=torch.int32)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts, max_new_tokens: int = 32, sampler: SamplerConfig | None = None, stream_callback=None,
                 eos_id: int | None = None, use_graph: bool = True) -> GenerationResult:
        """prompts: an int tensor [B, S] or a list of token lists, which may differ in length.
        Equal-length prompts that fit one pass run the contiguous flash-attention prefill; ragged
        batches and prompts longer than ``prefill_chunk`` tokens per pass go through the paged
        prefill kernel in chunks."""
        sampler = sampler or SamplerConfig(temperature=0.0)
        if torch.is_tensor(prompts):
            lists = [[int(x) for x in row] for row in prompts.tolist()]
        else:
            lists = [[int(x) for x in row] for row in prompts]
        lens = [len(t) for t in lists]
        B, S = len(lists), max(lens)
        if B > self.max_batch or S + max_new_tokens > self.max_seq_len or min(lens) < 1:
            raise ValueError("batch or sequence length exceeds the engine's limits")
        ragged = len(set(lens)) > 1
        cache = self.cache
        seqs = [cache.new_sequence() for _ in range(B)]
        for s, n in zip(seqs, lens):
            cache.reserve(s, n + max_new_tokens)
        cache.sync_tables()
        dev = self.device
        seq_t = torch.tensor(seqs, dtype=torch.int32, device=dev)
        stats = GenerationStats(prompt_tokens=sum(lens))
        self._prepare_decode_scratch(B, S + max_new_tokens)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        # ---- prefill
        chunked = (ragged or B * S > getattr(self, "prefill_chunk_threshold", 1 << 30)) and self._paged_prefill_ok()
        with trace.span("prefill", dev):
            if chunked:
                last = self._prefill_chunked(seqs, lists)
            elif ragged:          # int8 pages: one contiguous prefill per sequence
                rows = []
                for s, t in zip(seqs, lists):
                    n = len(t)
                    hh = self._forward(torch.tensor(t, dtype=torch.int32, device=dev),
                                       torch.arange(n, device=dev, dtype=torch.int32),
                                       torch.full((n,), s, device=dev, dtype=torch.int32), None, prefill_shape=(1, n))
                    cache.advance(s, n)
                    rows.append(hh[-1])
                last = torch.stack(rows)
            else:
                ids_d = torch.tensor(lists, dtype=torch.int32).to(dev).reshape(-1)
                pos = torch.arange(S, device=dev, dtype=torch.int32).repeat(B)
                h = self._forward(ids_d, pos, seq_t.repeat_interleave(S), None, prefill_shape=(B, S))
                last = h.view(B, S, -1)[:, -1, :].contiguous()
                for s in seqs:
                    cache.advance(s, S)
            tok = sample(self._logits(last.contiguous()), sampler, step=0)
        torch.cuda.synchronize(dev)
        stats.ttft_s = time.perf_counter() - t0
        out = [tok.clone()]
        if stream_callback is not None:
            stream_callback(0, tok)
        # ---- decode
        cur = tok.clone()
        posd = torch.tensor(lens, device=dev, dtype=torch.int32)
        ctx = posd + 1
        graph = None
        graph_ok = use_graph and sampler.greedy and stream_callback is None and eos_id is None

        def step_fn():
            hh = self._forward(cur, posd, seq_t, ctx, None)
            nt = sample(self._logits(hh), sampler, step=1)
            cur.copy_(nt)
            posd.add_(1)
            ctx.add_(1)

        t1 = time.perf_counter()
        steps = max_new_tokens - 1
        done = 0
        if graph_ok and steps > 2:
            step_fn()  # warm-up outside capture (allocations, lazy initialisation)
            out.append(cur.clone())
            done = 1
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_fn()  # recorded only: nothing runs and no state advances during capture
            for _ in range(done, steps):
                graph.replay()
                out.append(cur.clone())
        else:
            for i in range(steps):
                hh = self._forward(cur, posd, seq_t, ctx, None)
                nt = sample(self._logits(hh), sampler, step=i + 1)
                cur.copy_(nt)
                posd.add_(1)
                ctx.add_(1)
                out.append(nt.clone())
                if stream_callback is not None:
                    stream_callback(i + 1, nt)
                if eos_id is not None and bool((nt == eos_id).all()):
                    break
        torch.cuda.synchronize(dev)
        native.check_status(dev)
        stats.decode_s = time.perf_counter() - t1
        toks = torch.stack(out, dim=1).cpu()
        stats.new_tokens = toks.numel()
        stats.tokens_per_s = (toks.numel() - B) / max(stats.decode_s, 1e-9)
        stats.kv_bytes = cache.size_bytes()
        stats.kv_utilization = cache.utilization()
        for s in seqs:
            cache.free_sequence(s)
        return GenerationResult(tokens=[t.tolist() for t in toks], stats=stats)


    # ------------------------------------------------------------------ text-level API
    @classmethod
    def load(cls, path: str, device="cuda", **kw) -> "InferenceEngine":
        """Engine from an ``.oil`` file and its sibling ``.vocab`` tokenizer (byte-level ids when the
        vocabulary file is missing): the reference's ``engine::InferenceEngine::load`` + ``init``
        (engines/inference/inference.cpp)."""
        import os

        from ..oil.model_io import load_model
        from ..train.bpe import BPETokenizer

        model, _ = load_model(path, device=device)
        kw.setdefault("max_seq_len", model.cfg.max_seq_len)
        eng = cls.from_model(model, device=device, **kw)
        vocab = (path[:-4] if path.endswith(".oil") else path) + ".vocab"
        eng.tokenizer = BPETokenizer.load(vocab) if os.path.exists(vocab) else None
        return eng

    def encode(self, text: str) -> list:
        tok = getattr(self, "tokenizer", None)
        ids = tok.encode(text) if tok is not None else list(text.encode("utf-8"))
        return [min(int(i), self.cfg.vocab_size - 1) for i in ids] or [0]

    def decode_text(self, ids) -> str:
        tok = getattr(self, "tokenizer", None)
        if tok is not None:
            return tok.decode(list(ids))
        return bytes(int(i) & 0xFF for i in ids).decode("utf-8", errors="replace")

    def generate_with_stats(self, prompt: str, max_new_tokens: int = 64, sampler: SamplerConfig | None = None):
        """``(text, GenerationStats)``: tokens, seconds, tokens/s, KV bytes and KV utilisation of one
        prompt (the reference's ``generate_with_stats`` / ``InferenceStats``)."""
        ids = self.encode(prompt)
        room = self.max_seq_len - len(ids)
        if room < 1:
            raise ValueError("prompt fills the engine's context")
        tok = getattr(self, "tokenizer", None)
        res = self.generate([ids], max_new_tokens=min(max_new_tokens, room), sampler=sampler,
                            eos_id=tok.eos_id() if tok is not None else None)
        new = res.tokens[0]
        if tok is not None and tok.eos_id() in new:
            new = new[: new.index(tok.eos_id())]
        return self.decode_text(new), res.stats

    def generate_text(self, prompt: str, max_new_tokens: int = 64, sampler: SamplerConfig | None = None) -> str:
        return self.generate_with_stats(prompt, max_new_tokens, sampler)[0]

    def generate_batch(self, prompts, max_new_tokens: int = 64, sampler: SamplerConfig | None = None) -> list:
        """Texts for a list of prompts. Prompts that tokenise to the same length share one batched
        prefill + decode (up to ``max_batch`` at a time); the reference loops over them one by one."""
        enc = [self.encode(p) for p in prompts]
        out = [None] * len(prompts)
        by_len: dict[int, list[int]] = {}
        for i, ids in enumerate(enc):
            by_len.setdefault(len(ids), []).append(i)
        for n, members in by_len.items():
            for lo in range(0, len(members), self.max_batch):
                group = members[lo:lo + self.max_batch]
                res = self.generate([enc[i] for i in group], max_new_tokens=min(max_new_tokens, self.max_seq_len - n),
                                    sampler=sampler)
                for i, toks in zip(group, res.tokens):
                    out[i] = self.decode_text(toks)
        return out

    def reset_context(self) -> None:
        """Drop every live sequence and the prefix index (all pages return to the free list)."""
        cache = self.cache
        for s in range(cache.max_seqs):
            if cache.active[s]:
                cache.free_sequence(s)
        cache.prefix_index.clear()

    # ------------------------------------------------------------------ step-wise API (serving)
    @torch.no_grad()
    def generate_stream(self, prompt_ids, detokenize, on_text, max_new_tokens: int = 32,
                        sampler: SamplerConfig | None = None, eos_id: int | None = None) -> GenerationResult:
        """One sequence, text delivered while it is generated: every sampled token goes through
        ``detokenize(list[int]) -> str`` into a buffer that calls ``on_text`` when the text ends in
        white space, punctuation, a closing bracket or a quote, and once more at the end (role of
        the reference's ``generate_stream``, engines/inference/stream.cpp:35-48)."""
        from .stream import StreamBuffer

        buf = StreamBuffer(on_text)

        def on_token(step, tok):
            buf.append(detokenize([int(tok[0])]))

        res = self.generate([list(prompt_ids)], max_new_tokens, sampler, stream_callback=on_token, eos_id=eos_id,
                            use_graph=False)
        buf.close()
        return res

    def start_sequence(self, prompt_ids, reuse_prefix: bool = True):
        """Prefill one request. Returns ``(seq, logits)`` with the logits of the last prompt token
        ([1, V]). With ``reuse_prefix`` the full pages of an earlier prompt with the same head are
        mapped into the new sequence (their reference counts go up) and only the remaining tokens
        are computed: their K/V are appended to fresh pages and the tcgen05 prefill kernel attends
        over the paged cache (shared prefix + the new tokens before them). Prompts longer than
        ``prefill_chunk`` tokens run in several such passes. With int8 pages the remainder goes
        through the decode kernel instead, and a hit below half of the prompt is not used."""
        ids = [int(t) for t in prompt_ids]
        cache = self.cache
        seq = cache.new_sequence()
        S = len(ids)
        # at least the last token is always computed: its logits are the result
        covered = cache.share_prefix(seq, ids[:-1]) if reuse_prefix and S > 1 else 0
        paged_ok = self._paged_prefill_ok()
        if 0 < covered < S // 2 and not paged_ok:
            # Without the paged prefill kernel (int8 pages) the rest would go through the decode kernel
            # in chunks of max_batch tokens, each a full pass over the weights: a short hit is not
            # worth it. Recompute the whole prompt.
            cache.free_sequence(seq)
            seq = cache.new_sequence()
            covered = 0
        cache.reserve(seq, S - covered)
        cache.sync_tables()
        dev = self.device
        self._prepare_decode_scratch(self.max_batch, self.max_seq_len)
        self.last_prefix_hit = covered
        if covered == 0 and not (paged_ok and S > getattr(self, "prefill_chunk", 8192)):
            t = torch.tensor(ids, dtype=torch.int32, device=dev)
            pos = torch.arange(S, device=dev, dtype=torch.int32)
            sid = torch.full((S,), seq, device=dev, dtype=torch.int32)
            h = self._forward(t, pos, sid, None, prefill_shape=(1, S))
            cache.advance(seq, S)
        else:
            # remainder after a cached prefix, or a prompt longer than one pass: chunked paged prefill
            h = self._extend_sequence(seq, ids[covered:])
        if reuse_prefix:
            cache.publish_prefix(seq, ids)
        return seq, self._logits(h[-1:].contiguous())

    @torch.no_grad()
    def _extend_sequence(self, seq: int, new_ids) -> torch.Tensor:
        """Append ``new_ids`` to a sequence that already has tokens in the cache (pages reserved)
        and return their hidden states. Token i of a chunk is a row of a decode batch whose block
        table row is the sequence's and whose context length is its own position + 1, so the paged
        decode kernel gives causal attention over prefix and chunk."""
        cache, dev = self.cache, self.device
        if self._paged_prefill_ok():
            # the tcgen05 prefill kernel over the paged cache (shared prefix + the new tokens), in
            # passes of at most prefill_chunk tokens
            return self._prefill_chunked([seq], [list(new_ids)], bases=[cache.lens[seq]])[-1:]
        step = max(1, min(self.max_batch, ONESHOT_MAX_TOKENS))
        h = None
        for lo in range(0, len(new_ids), step):
            chunk = new_ids[lo:lo + step]
            n, base = len(chunk), cache.lens[seq]
            t = torch.tensor(chunk, dtype=torch.int32, device=dev)
            pos = torch.arange(base, base + n, device=dev, dtype=torch.int32)
            rows = cache.block_table[seq:seq + 1].expand(n, -1).contiguous()
            saved = cache.block_table
            cache.block_table = rows
            try:
                h = self._forward(t, pos, torch.arange(n, device=dev, dtype=torch.int32), pos + 1, None)
            finally:
                cache.block_table = saved
            cache.advance(seq, n)
        return h

    @torch.no_grad()
    def decode(self, seqs, tokens):
        """One decode step for the given sequences (any mix of lengths): appends ``tokens`` (one per
        sequence) and returns the next-token logits [n, V]."""
        cache, dev = self.cache, self.device
        for s in seqs:
            cache.reserve(s, 1)
        cache.sync_tables()
        n = len(seqs)
        ids = torch.as_tensor(tokens, dtype=torch.int32).to(dev).reshape(n)
        pos = torch.tensor([cache.lens[s] for s in seqs], dtype=torch.int32, device=dev)
        sid = torch.tensor(list(seqs), dtype=torch.int32, device=dev)
        # the decode kernel indexes block-table rows by position in the batch: gather the rows
        table_rows = cache.block_table.index_select(0, sid.long()).contiguous()
        saved = cache.block_table
        cache.block_table = table_rows
        try:
            h = self._forward(ids, pos, torch.arange(n, device=dev, dtype=torch.int32), pos + 1, None)
        finally:
            cache.block_table = saved
        for s in seqs:
            cache.advance(s, 1)
        return self._logits(h)

    def release(self, seq: int) -> None:
        self.cache.free_sequence(seq)


# ---------------------------------------------------------------------------------------- TP helpers
def _shard_rows_multi(mod, parts, rank: int, world: int) -> QuantLinear:
    """Column-parallel shard of a fused projection: from each (start, size) part of the output rows
    take this rank's 1/world slice, concatenate, and pack with the module's codebooks."""
    w = mod.weight.detach().float()
    if mod.fmt == "mixed":
        w = mod.quantize_now(w).float()              # dense bf16 image of the per-block formats
    K = w.shape[1]
    pieces, maps = [], []
    for start, size in parts:
        per = size // world
        lo = start + rank * per
        pieces.append(w[lo:lo + per])
        if mod.codebooks is not None:
            b0, b1 = lo * K // mod.block_size, (lo + per) * K // mod.block_size
            maps.append(torch.arange(b0, b1, device=w.device, dtype=torch.int32) if mod.cb_map is None
                        else mod.cb_map[b0:b1])
    ws = torch.cat(pieces, dim=0).contiguous()
    if mod.fmt not in ("oil8", "oil4", "i2s"):
        return QuantLinear.from_float(ws, "bf16")
    if mod.codebooks is None:
        return QuantLinear.from_float(ws, mod.fmt, mod.block_size)
    return QuantLinear.from_float(ws, mod.fmt, mod.block_size, 1, mod.codebooks.float(), torch.cat(maps).contiguous())


def _shard_cols(mod, rank: int, world: int) -> QuantLinear:
    """Row-parallel shard (input features split). Quantisation blocks run along the input
    dimension, so the shard is re-blocked: block b of the shard keeps the codebook of the original
    block it came from as long as shard boundaries fall on block boundaries; otherwise the shard
    gets fresh quantile codebooks."""
    w = mod.weight.detach().float()
    if mod.fmt == "mixed":
        w = mod.quantize_now(w).float()
    N, K = w.shape
    per = K // world
    ws = w[:, rank * per:(rank + 1) * per].contiguous()
    if mod.fmt not in ("oil8", "oil4", "i2s"):
        return QuantLinear.from_float(ws, "bf16")
    bs = mod.block_size
    if mod.codebooks is None or per % bs != 0:
        return QuantLinear.from_float(ws, mod.fmt, bs if per % bs == 0 else 64, mod.codebook_group)
    blocks_per_row, shard_blocks = K // bs, per // bs
    rows = torch.arange(N, device=w.device)[:, None]
    cols = torch.arange(shard_blocks, device=w.device)[None, :] + rank * shard_blocks
    orig = (rows * blocks_per_row + cols).reshape(-1)
    cmap = orig.to(torch.int32) if mod.cb_map is None else mod.cb_map[orig]
    return QuantLinear.from_float(ws, mod.fmt, bs, 1, mod.codebooks.float(), cmap.contiguous())


def _gather_columns(lg: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """Vocabulary-parallel logits [B, V/W] of every rank -> [B, V] on every rank (peer stores)."""
    B, Vs = lg.shape
    native.require().peer_gather_cols(lg.contiguous(), list(tp.logits.ptrs), tp.rank, tp.world)
    tp.barrier.sync()
    return tp.logits.tensor[: B * Vs * tp.world].view(B, Vs * tp.world)
