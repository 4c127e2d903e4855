"""Kernel micro-benchmarks (the role of the reference's ``oil_bench --kernel`` and
``bench/bench_kernels.cpp``): times one kernel with CUDA events after warm-up, flushing L2 between
iterations, and reports achieved TFLOP/s or GB/s next to the measured device peaks.

    python -m mythos_b200.tools.kernel_bench --kernel gemm --m 16384 --n 2048 --k 2048
    python -m mythos_b200.tools.kernel_bench --kernel attn_fwd --batch 8 --seq 2048 --heads 16
    python -m mythos_b200.tools.kernel_bench --kernel all

This is also the program profiled for the summaries under ``profiles/``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p.get("bf16_tflops", 1590.0), p.get("hbm_gbs", 6650.0), "measured"
    except OSError:
        return 1590.0, 6650.0, "fallback"


class Timer:
    def __init__(self, iters: int, warmup: int, flush: bool = True):
        self.iters, self.warmup, self.flush = iters, warmup, flush
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn) -> float:
        """Median milliseconds per call."""
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            if self.buf is not None:
                self.buf.zero_()  # 256 MB write evicts the 126 MB L2
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        times.sort()
        return times[len(times) // 2]


def graph_time(t: Timer, fn) -> float:
    """Median milliseconds of ``fn`` alone for launches of a few microseconds, where eager timing
    would measure the CPU launch path: replay a CUDA graph of [L2 flush, fn] and subtract the
    replay time of a graph holding only the flush."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(1, t.warmup)):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    buf = t.buf if t.buf is not None else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g_full, g_flush = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_full):
        buf.zero_()
        fn()
    with torch.cuda.graph(g_flush):
        buf.zero_()

    def med(g):
        times = []
        for _ in range(t.warmup + t.iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        times = sorted(times[t.warmup:])
        return times[len(times) // 2]

    return max(1e-6, med(g_full) - med(g_flush))


def bench_gemm(t: Timer, M, N, K, layout="kk", epi=0):
    from mythos_b200.ops import functional as F

    a_mn, b_mn = {"kk": (False, False), "kmn": (False, True), "mnmn": (True, True)}[layout]
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if epi == 0 else torch.float32)
    ms = t(lambda: F.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, epi=epi))
    return ms, 2.0 * M * N * K / ms / 1e9, "TFLOP/s"


def bench_fused_epilogues(t: Timer, M: int, d: int, F: int, heads: int, only: str = "", unfused: bool = True):
    """The fused-epilogue GEMMs against the launches they replace (same shapes as one layer of the
    1.3B model): gate/up GEMM + SwiGLU, down dgrad GEMM + SwiGLU backward, QKV GEMM + RoPE on q and k.
    Returns [(name, ms fused, ms unfused)]."""
    from mythos_b200.ops import functional as Fn, native

    C = native.require()
    st = native.status_word("cuda")
    x = torch.randn(M, d, device="cuda").to(torch.bfloat16)
    w_gu = (torch.randn(2 * F, d, device="cuda") * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(d, F, device="cuda") * 0.02).to(torch.bfloat16)
    gu = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    dgu = torch.empty_like(gu)
    dh = torch.empty_like(h)
    dy = torch.randn(M, d, device="cuda").to(torch.bfloat16)
    out = []
    skip = (lambda fn: 0.0) if not unfused else t        # profiling runs time the fused launch only

    def unfused_fwd():
        Fn.gemm(x, w_gu, out=gu)
        C.swiglu_fused_fwd(gu, h)

    if only in ("", "fwd"):
        out.append(("gate_up+swiglu_fwd", t(lambda: C.gemm_swiglu_fwd(x, w_gu, gu, h, st)), skip(unfused_fwd),
                    2.0 * M * 2 * F * d))

    def unfused_bwd():
        Fn.gemm(dy, w_dn, b_mn=True, out=dh)
        C.swiglu_fused_bwd(gu, dh, dgu)

    if only in ("", "bwd"):
        gu.normal_()
        out.append(("down_dgrad+swiglu_bwd", t(lambda: C.gemm_swiglu_bwd(dy, w_dn, gu, dgu, st)), skip(unfused_bwd),
                    2.0 * M * F * d))
    if only not in ("", "rope"):
        return out
    D = 128
    N = 3 * heads * D
    w_qkv = (torch.randn(N, d, device="cuda") * 0.02).to(torch.bfloat16)
    qkv = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    pos = (torch.arange(M, device="cuda") % 2048).to(torch.int32)
    table = Fn.rope_table(10000.0, 2048, x.device)

    def unfused_rope():
        Fn.gemm(x, w_qkv, out=qkv)
        C.rope(qkv[:, : heads * D].unflatten(-1, (heads, D)), pos, 10000.0, False)
        C.rope(qkv[:, heads * D: 2 * heads * D].unflatten(-1, (heads, D)), pos, 10000.0, False)

    out.append(("qkv+rope", t(lambda: C.gemm_rope(x, w_qkv, qkv, pos, table, 2 * heads * D, st)), skip(unfused_rope),
                2.0 * M * N * d))
    return out


def bench_attn(t: Timer, B, S, H, Hkv, D, backward=False):
    from mythos_b200.ops import functional as F

    W = (H + 2 * Hkv) * D
    qkv = (torch.randn(B, S, W, device="cuda") * 0.5).to(torch.bfloat16)
    pos = torch.arange(S, device="cuda", dtype=torch.int32).repeat(B)
    flops_fwd = 4.0 * B * H * S * S * D * 0.5
    if not backward:
        q = qkv[..., : H * D].unflatten(-1, (H, D))
        k = qkv[..., H * D:(H + Hkv) * D].unflatten(-1, (Hkv, D))
        v = qkv[..., (H + Hkv) * D:].unflatten(-1, (Hkv, D))
        ms = t(lambda: F.flash_attention(q, k, v, True))
        return ms, flops_fwd / ms / 1e9, "TFLOP/s"
    x = qkv.clone().requires_grad_()
    o = F.attention_qkv(x, pos, H, Hkv, D, 0.0, True)
    do = torch.randn_like(o)
    ms = t(lambda: torch.autograd.grad(o, x, do, retain_graph=True))
    return ms, 2.5 * flops_fwd / ms / 1e9, "TFLOP/s"


def bench_memory_bound(t: Timer, name: str, rows: int, dim: int):
    from mythos_b200.ops import native, reference  # noqa: F401

    C = native.require()
    x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    g = torch.ones(dim, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    if name == "rmsnorm":
        rstd = torch.empty(rows, device="cuda")
        ms = t(lambda: C.rmsnorm_fwd(x, None, g, y, None, rstd, 1e-5))
        nbytes = 2 * x.numel() * 2
    elif name == "swiglu":
        out = torch.empty(rows, dim // 2, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: C.swiglu_fused_fwd(x, out))
        nbytes = x.numel() * 2 + out.numel() * 2
    elif name == "ce":
        tg = torch.randint(0, dim, (rows,), device="cuda", dtype=torch.int32)
        losses = torch.empty(rows, device="cuda")
        ms = t(lambda: C.cross_entropy_fwd_bwd(x, tg, losses, 1.0 / rows))
        nbytes = 3 * x.numel() * 2
    elif name == "adamw":
        n = rows * dim
        p, m, v, gr = (torch.randn(n, device="cuda") for _ in range(4))
        ms = t(lambda: C.adamw_step(p, m, v, gr, None, 3e-4, 0.9, 0.999, 1e-8, 0.01, 5, 1.0, None))
        nbytes = n * 4 * 7
    elif name == "fake_quant":
        from mythos_b200.oil.codebook import quantile_codebook

        n = rows * dim
        w = torch.randn(n, device="cuda") * 0.02
        nb = n // 256
        cb = quantile_codebook(256).cuda()[None].repeat((nb + 127) // 128, 1).contiguous()
        cmap = (torch.arange(nb, device="cuda") // 128).to(torch.int32)
        out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: C.oil_fake_quant(w, cb, cmap, 256, out, None))
        nbytes = n * 6
    else:
        raise ValueError(name)
    return ms, nbytes / ms / 1e6, "GB/s"


def bench_dequant_gemm(t: Timer, fmt: str, M: int, N: int, K: int, group: int = 128):
    """Decode-shaped GEMM over packed weights; reported as packed weight bytes per second."""
    from mythos_b200.infer.quant_weights import QuantLinear

    g = torch.Generator(device="cuda").manual_seed(0)
    q = QuantLinear.random(fmt, N, K, 256, group, device="cuda", generator=g)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    q.matmul(x, out=out)   # sizes the split-K accumulator outside graph capture
    ms = graph_time(t, lambda: q.matmul(x, out=out))
    return ms, q.packed.numel() / ms / 1e6, "GB/s"


def bench_misc(t: Timer, name: str):
    """Single-kernel cases of the smaller kernels (also the programs behind their ncu summaries).
    Multi-rank kernels run over two emulated ranks' buffers on this GPU, one launch after the other
    (none of them waits on a peer). Returns (ms, GB/s of the bytes the kernel must move, unit)."""
    from mythos_b200.ops import functional as Fn, native

    C = native.require()
    st = native.status_word("cuda")
    bf = torch.bfloat16
    if name == "rope":
        T, H, D = 16384, 16, 128
        x = torch.randn(T, H, D, device="cuda").to(bf)
        pos = (torch.arange(T, device="cuda") % 2048).to(torch.int32)
        return t(lambda: C.rope(x, pos, 10000.0, False)), 2.0 * x.numel() * 2, "GB/s"
    if name == "rmsnorm_bwd":
        rows, dim = 16384, 2048
        x, dy, dres = (torch.randn(rows, dim, device="cuda").to(bf) for _ in range(3))
        g = torch.ones(dim, device="cuda", dtype=bf)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        dx = torch.empty_like(x)
        part = torch.empty(296, dim, device="cuda")
        dg = torch.zeros(dim, device="cuda")
        return t(lambda: C.rmsnorm_bwd(dy, x, g, rstd, dx, part, dg, True, dres)), 4.0 * x.numel() * 2, "GB/s"
    if name in ("layernorm_fwd", "layernorm_bwd"):
        rows, dim = 16384, 2048
        x, dy = (torch.randn(rows, dim, device="cuda").to(bf) for _ in range(2))
        g = torch.ones(dim, device="cuda", dtype=bf)
        b = torch.zeros(dim, device="cuda", dtype=bf)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        if name == "layernorm_fwd":
            return t(lambda: C.layernorm_fwd(x, g, b, y, 1e-5)), 2.0 * x.numel() * 2, "GB/s"
        part = torch.empty(444, 2 * dim, device="cuda")
        dgb = torch.empty(2 * dim, device="cuda")
        return t(lambda: C.layernorm_bwd(dy, x, g, dx, part, dgb, 1e-5)), 3.0 * x.numel() * 2, "GB/s"
    if name in ("gelu_fwd", "gelu_bwd", "softmax_fwd", "softmax_bwd"):
        rows, dim = 16384, 4096
        x, dy = (torch.randn(rows, dim, device="cuda").to(bf) for _ in range(2))
        y, dx = torch.empty_like(x), torch.empty_like(x)
        if name == "gelu_fwd":
            return t(lambda: C.act_fwd(x, y, 1)), 2.0 * x.numel() * 2, "GB/s"
        if name == "gelu_bwd":
            return t(lambda: C.act_bwd(x, dy, dx, 1)), 3.0 * x.numel() * 2, "GB/s"
        if name == "softmax_fwd":
            return t(lambda: C.softmax_rows(x, y)), 2.0 * x.numel() * 2, "GB/s"
        C.softmax_rows(x, y)
        return t(lambda: C.softmax_rows_bwd(y, dy, dx)), 3.0 * x.numel() * 2, "GB/s"
    if name in ("moe_route", "moe_dispatch", "moe_combine"):
        T, E, k, d = 16384, 8, 2, 2048
        logits = torch.randn(T, 8, device="cuda").to(bf)
        probs = torch.empty(T, E, device="cuda")
        idx = torch.empty(T, k, device="cuda", dtype=torch.int32)
        slot = torch.empty_like(idx)
        w = torch.empty(T, k, device="cuda")
        counts = torch.zeros(E, device="cuda", dtype=torch.int32)
        psum = torch.zeros(E, device="cuda")

        def route():
            counts.zero_()
            C.moe_route(logits, E, probs, idx, slot, w, counts, psum)

        if name == "moe_route":
            return t(route), T * (8 * 2 + E * 4 + k * 12.0), "GB/s"
        route()
        cap = T * k + 256 * E
        seg_start = torch.empty(E, device="cuda", dtype=torch.int32)
        seg_rows = torch.empty(E, device="cuda", dtype=torch.int32)
        send_base = torch.empty(E, device="cuda", dtype=torch.int32)
        C.moe_offsets(counts, 1, E, 0, cap, seg_start, seg_rows, send_base, st)
        x = torch.randn(T, d, device="cuda").to(bf)
        buf = torch.zeros(cap, d, device="cuda", dtype=bf)
        if name == "moe_dispatch":
            return t(lambda: C.moe_dispatch(x, idx, slot, send_base, None, [buf.data_ptr()], E, 0, 0)), \
                (1 + k) * T * d * 2.0, "GB/s"
        C.moe_dispatch(x, idx, slot, send_base, None, [buf.data_ptr()], E, 0, 0)
        out = torch.empty_like(x)
        return t(lambda: C.moe_combine([buf.data_ptr()], idx, slot, send_base, w, None, out, None, d, E, 0, 0)), \
            (1 + k) * T * d * 2.0, "GB/s"
    if name in ("zero_rs", "zero_adamw"):
        n = 64 << 20                                   # elements per emulated rank buffer
        world, shard = 2, (64 << 20) // 2
        grads = [torch.randn(n, device="cuda") * 1e-3 for _ in range(world)]
        gsh = torch.empty(shard, device="cuda")
        part = torch.zeros(1, device="cuda")
        if name == "zero_rs":
            return t(lambda: C.zero_reduce_scatter([g.data_ptr() for g in grads], gsh, 0, part)), \
                shard * 4.0 * (world + 1), "GB/s"
        from mythos_b200.oil.codebook import quantile_codebook

        master = torch.randn(shard, device="cuda") * 0.02
        m, v = torch.zeros(shard, device="cuda"), torch.zeros(shard, device="cuda")
        comp = [torch.empty(n, device="cuda", dtype=bf) for _ in range(world)]
        nseg = n // 256
        seg_fmt = torch.ones(nseg, device="cuda", dtype=torch.uint8)
        seg_cb = (torch.arange(nseg, device="cuda") // 128).to(torch.int32)
        cb8 = quantile_codebook(256).cuda()[None].repeat((nseg + 127) // 128, 1).contiguous()
        cb4 = torch.zeros(1, 16, device="cuda")
        parts = torch.ones(world, device="cuda")
        gn = torch.zeros(1, device="cuda")
        gsh.normal_(0, 1e-3)
        return t(lambda: C.zero_adamw_ste_allgather(master, m, v, gsh, [c.data_ptr() for c in comp], 0, seg_fmt, seg_cb,
                                                    cb8, cb4, parts, gn, 1.0, 1e-4, 0.9, 0.95, 1e-8, 0.1, 10, 1.0, 0, 0)), \
            shard * (28.0 + 2.0 * world), "GB/s"
    if name == "tp_pull":
        n = 16384 * 4096
        parts = [torch.randn(n, device="cuda").to(bf) for _ in range(2)]
        outs = [torch.empty(n, device="cuda", dtype=bf) for _ in range(2)]
        return t(lambda: C.tp_allreduce_pull([p.data_ptr() for p in parts], [o.data_ptr() for o in outs], 0, n)), \
            (n // 2) * 2.0 * 4, "GB/s"
    if name == "qkv_rope_append":
        T, H, Hkv, D = 64, 32, 8, 128
        acc = torch.randn(T, (H + 2 * Hkv) * D, device="cuda")
        pos = torch.full((T,), 100, device="cuda", dtype=torch.int32)
        sid = torch.arange(T, device="cuda", dtype=torch.int32)
        table = torch.arange(T * 8, device="cuda", dtype=torch.int32).view(T, 8)
        q = torch.empty(T, H, D, device="cuda", dtype=bf)
        kc = torch.zeros(T * 8, 16, Hkv, D, device="cuda", dtype=bf)
        vc = torch.zeros_like(kc)

        def run():
            acc.normal_()
            C.qkv_rope_append(acc, pos, sid, table, q, kc, vc, 500000.0, None, None)

        return t(run), acc.numel() * 6.0, "GB/s"
    if name == "paged_prefill":
        B, S, H, Hkv, D = 8, 2048, 16, 16, 128
        pages = B * S // 16
        kc = (torch.randn(pages, 16, Hkv, D, device="cuda") * 0.5).to(bf)
        vc = (torch.randn(pages, 16, Hkv, D, device="cuda") * 0.5).to(bf)
        q = (torch.randn(B * S, H, D, device="cuda") * 0.5).to(bf)
        table = torch.randperm(pages, device="cuda").to(torch.int32).view(B, S // 16)
        cu = (torch.arange(B + 1, device="cuda") * S).to(torch.int32)
        kv = torch.full((B,), S, device="cuda", dtype=torch.int32)
        o = torch.empty_like(q)
        ms = t(lambda: C.flash_attn_paged_prefill(q, kc, vc, table, cu, kv, o, S, D ** -0.5, st))
        return ms, 4.0 * B * H * S * S * D * 0.5 / 1e3, "TFLOP/s"       # value below is divided by ms * 1e6
    if name == "grouped_gemm":
        E, rows_e, d, F2 = 8, 4096, 2048, 2 * 5632
        cap = E * rows_e
        a = torch.randn(cap, d, device="cuda").to(bf)
        ws = [(torch.randn(F2, d, device="cuda") * 0.02).to(bf) for _ in range(E)]
        seg_start = (torch.arange(E, device="cuda") * rows_e).to(torch.int32)
        seg_rows = torch.full((E,), rows_e, device="cuda", dtype=torch.int32)
        gu = torch.empty(cap, F2, device="cuda", dtype=bf)
        h = torch.empty(cap, F2 // 2, device="cuda", dtype=bf)
        ms = t(lambda: C.gemm_grouped_rows(a, ws, False, gu, seg_start, seg_rows, 1, None, h, st))
        return ms, 2.0 * cap * F2 * d / 1e3, "TFLOP/s"
    if name == "tl_gemm":
        from mythos_b200.oil import ternary_kernels as tk

        N, K = 6912, 2556 // 12 * 12
        packed = tk.pack_trits(torch.randint(-1, 2, (N, K))).cuda()
        x = torch.randn(8, K, device="cuda")
        return t(lambda: tk.tl2_gemm(packed, x, K)), packed.numel() * 8.0, "GB/s"
    raise ValueError(name)


MISC_CASES = ("rope", "rmsnorm_bwd", "moe_route", "moe_dispatch", "moe_combine", "zero_rs", "zero_adamw", "tp_pull",
              "qkv_rope_append", "paged_prefill", "grouped_gemm", "tl_gemm", "layernorm_fwd", "layernorm_bwd",
              "gelu_fwd", "gelu_bwd", "softmax_fwd", "softmax_bwd")


def bench_i2s_gemv(t: Timer, N: int, K: int):
    """Single-token ternary GEMV (one warp per output row); reported as packed weight bytes per second."""
    from mythos_b200.infer.quant_weights import QuantLinear

    g = torch.Generator(device="cuda").manual_seed(0)
    q = QuantLinear.random("i2s", N, K, 256, 1, device="cuda", generator=g)
    x = (torch.randn(1, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    out = torch.empty(1, N, device="cuda", dtype=torch.bfloat16)
    ms = graph_time(t, lambda: q.matmul(x, out=out))
    return ms, q.packed.numel() / ms / 1e6, "GB/s"


def bench_sampler(t: Timer, B: int, V: int, greedy: bool):
    """Sampling kernels over bf16 logits [B, V]: greedy arg-max, or temperature + top-k + top-p."""
    from mythos_b200.infer.sampler import SamplerConfig, sample

    logits = (torch.randn(B, V, device="cuda") * 3).to(torch.bfloat16)
    cfg = SamplerConfig(temperature=0.0) if greedy else SamplerConfig(temperature=0.8, top_k=40, top_p=0.9, seed=1)
    ms = graph_time(t, lambda: sample(logits, cfg, step=1)) if greedy else t(lambda: sample(logits, cfg, step=1))
    return ms, logits.numel() * 2 / ms / 1e6, "GB/s"


def bench_paged_decode(t: Timer, B: int, ctx: int, H: int, Hkv: int, D: int, splits: int = 0, int8: bool = False):
    """Split-KV decode attention over 16-token pages; reported as KV bytes per second (for int8
    pages: the int8 rows plus their fp32 scales)."""
    from mythos_b200.ops import native

    C = native.require()
    pages_per_seq = (ctx + 15) // 16
    n_pages = B * pages_per_seq
    kc = (torch.randn(n_pages, 16, Hkv, D, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(n_pages, 16, Hkv, D, device="cuda") * 0.5).to(torch.bfloat16)
    table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(B, pages_per_seq)
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    q = torch.randn(B, H, D, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if splits <= 0:
        splits = max(1, min(32, (6 * sms + B * Hkv - 1) // (B * Hkv), (ctx + 255) // 256))
    scratch = torch.empty(B * H * splits * (D + 2), device="cuda")
    counters = torch.zeros(B * Hkv + 64, device="cuda", dtype=torch.int32)
    st = native.status_word("cuda")
    if int8:
        k8 = torch.empty(n_pages, 16, Hkv, D, device="cuda", dtype=torch.int8)
        v8 = torch.empty_like(k8)
        ks = torch.empty(n_pages * 16, Hkv, device="cuda")
        vs = torch.empty_like(ks)
        # quantise the bf16 pages with the append kernel: token j of physical page p belongs to the
        # sequence and logical page that map to p in the block table
        flat = table.long().view(-1)
        seq_of = torch.empty(n_pages, device="cuda", dtype=torch.int32)
        lpage_of = torch.empty(n_pages, device="cuda", dtype=torch.int32)
        seq_of[flat] = torch.arange(B, device="cuda", dtype=torch.int32).repeat_interleave(pages_per_seq)
        lpage_of[flat] = torch.arange(pages_per_seq, device="cuda", dtype=torch.int32).repeat(B)
        seq_ids = seq_of.repeat_interleave(16).contiguous()
        pos = (lpage_of.repeat_interleave(16) * 16 + torch.arange(16, device="cuda", dtype=torch.int32).repeat(n_pages))
        C.kv_append_int8(kc.view(-1, Hkv, D), vc.view(-1, Hkv, D), k8, v8, ks, vs, table, pos.contiguous(), seq_ids)
        ms = graph_time(t, lambda: C.paged_attn_decode_int8(q, k8, v8, ks, vs, table, lens, out, scratch, counters,
                                                            splits, D ** -0.5, st))
        return ms, 2.0 * B * ctx * Hkv * (D + 4) / ms / 1e6, "GB/s"
    ms = graph_time(t, lambda: C.paged_attn_decode(q, kc, vc, table, lens, out, scratch, counters, splits,
                                                   D ** -0.5, st))
    return ms, 2.0 * B * ctx * Hkv * D * 2 / ms / 1e6, "GB/s"


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--layout", default="kk", choices=["kk", "kmn", "mnmn"])
    ap.add_argument("--epi", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--fmt", default="oil8", choices=["oil8", "oil4", "i2s"])
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--splits", type=int, default=0, help="KV splits of paged_decode (0 = the engine's choice)")
    ap.add_argument("--coalesced-epilogue", type=int, default=1,
                    help="paired GEMM: 1 stores through a shared-memory transpose, 0 straight from registers")
    ap.add_argument("--attn-fwd-mode", type=int, default=-1, help="0 first forward kernel, 1 persistent 128x128 kernel")
    ap.add_argument("--gemm-mode", type=int, default=0, help="0 auto, 1 single-CTA kernel, 2 paired-SM kernel")
    args = ap.parse_args()
    from mythos_b200.ops import native

    native.require().set_gemm_mode(args.gemm_mode)
    native.require().set_gemm_coalesced_epilogue(args.coalesced_epilogue)
    if args.attn_fwd_mode >= 0:
        native.require().set_attn_fwd_mode(args.attn_fwd_mode)
    tf_peak, bw_peak, src = _peaks()
    t = Timer(args.iters, args.warmup, not args.no_flush)
    hkv = args.kv_heads or args.heads
    rows = []

    def report(name, res):
        ms, val, unit = res
        frac = val / (tf_peak if unit == "TFLOP/s" else bw_peak)
        rows.append({"kernel": name, "ms": round(ms, 4), "value": round(val, 1), "unit": unit,
                     f"fraction_of_{src}_peak": round(frac, 3)})
        print(json.dumps(rows[-1]), flush=True)

    k = args.kernel
    if k in ("gemm", "gemm_set", "all"):
        if k == "gemm":
            report(f"gemm_{args.layout}_{args.m}x{args.n}x{args.k}_epi{args.epi}",
                   bench_gemm(t, args.m, args.n, args.k, args.layout, args.epi))
        else:
            for (M, N, K, lay, epi) in [(16384, 6144, 2048, "kk", 0), (16384, 2048, 2048, "kk", 0),
                                        (16384, 11008, 2048, "kk", 0), (16384, 2048, 5504, "kk", 0),
                                        (16384, 32000, 2048, "kk", 0), (16384, 2048, 6144, "kmn", 0),
                                        (16384, 5504, 2048, "kmn", 0), (6144, 2048, 16384, "mnmn", 2),
                                        (11008, 2048, 16384, "mnmn", 2), (2048, 5504, 16384, "mnmn", 2),
                                        (32000, 2048, 16384, "mnmn", 2), (8192, 8192, 8192, "kk", 0)]:
                report(f"gemm_{lay}_{M}x{N}x{K}_epi{epi}", bench_gemm(t, M, N, K, lay, epi))
    if k == "wgrad_set":
        # weight-gradient shapes of the 1.3B model at 8 and 32 sequences per pass: read-add-store
        # epilogue (one tile per output block) against split-K with atomic adds
        for K in (16384, 65536):
            for (M, N) in [(6144, 2048), (11008, 2048), (2048, 5504), (2048, 2048), (32000, 2048)]:
                for epi in (2, 3):
                    report(f"gemm_mnmn_{M}x{N}x{K}_epi{epi}", bench_gemm(t, M, N, K, "mnmn", epi))
    if k in ("fused_epilogue", "fused_swiglu_fwd", "fused_swiglu_bwd", "fused_rope", "all"):
        only = {"fused_swiglu_fwd": "fwd", "fused_swiglu_bwd": "bwd", "fused_rope": "rope"}.get(k, "")
        for name, ms_f, ms_u, flops in bench_fused_epilogues(t, args.m, 2048, 5504, 16, only, unfused=not only):
            report(f"{name}_fused_m{args.m}", (ms_f, flops / ms_f / 1e9, "TFLOP/s"))
            if ms_u > 0:
                report(f"{name}_unfused_m{args.m}", (ms_u, flops / ms_u / 1e9, "TFLOP/s"))
    if k in ("attn_fwd", "all"):
        report(f"attn_fwd_b{args.batch}_s{args.seq}_h{args.heads}_d{args.head_dim}",
               bench_attn(t, args.batch, args.seq, args.heads, hkv, args.head_dim, False))
    if k in ("attn_bwd", "all"):
        report(f"attn_bwd_b{args.batch}_s{args.seq}_h{args.heads}_d128",
               bench_attn(t, args.batch, args.seq, args.heads, hkv, 128, True))
    if k == "dequant_gemm":
        report(f"dequant_gemm_{args.fmt}_{args.m}x{args.n}x{args.k}", bench_dequant_gemm(t, args.fmt, args.m, args.n, args.k))
    if k == "all":
        for fmt, M, N, K in [("oil8", 64, 28672, 4096), ("oil8", 64, 4096, 14336), ("oil4", 64, 6144, 4096),
                             ("oil4", 64, 4096, 4096), ("i2s", 8, 6912, 2560), ("oil8", 64, 128256, 4096)]:
            report(f"dequant_gemm_{fmt}_{M}x{N}x{K}", bench_dequant_gemm(t, fmt, M, N, K))
    if k in MISC_CASES or k in ("misc", "all"):
        for name in (MISC_CASES if k in ("misc", "all") else (k,)):
            ms, nbytes, unit = bench_misc(t, name)
            report(f"misc_{name}", (ms, nbytes / ms / 1e6, unit))
    if k in ("i2s_gemv", "all"):
        for N, K in [(6912 * 2, 2560), (2560, 6912), (128256, 2560)]:
            report(f"i2s_gemv_1x{N}x{K}", bench_i2s_gemv(t, N, K))
    if k in ("sampler", "all"):
        report("sampler_greedy_b64_v128256", bench_sampler(t, 64, 128256, True))
        report("sampler_topk_topp_b64_v128256", bench_sampler(t, 64, 128256, False))
    if k in ("paged_decode", "paged_decode_int8"):
        report(f"{k}_b{args.batch}_ctx{args.ctx}_h{args.heads}_kv{hkv}_d{args.head_dim}_splits{args.splits}",
               bench_paged_decode(t, args.batch, args.ctx, args.heads, hkv, args.head_dim, args.splits,
                                  int8=k.endswith("int8")))
    if k == "all":
        for B, ctx, H, Hkv in [(64, 1024, 32, 8), (64, 1024, 4, 1), (8, 32768, 20, 20)]:
            report(f"paged_decode_b{B}_ctx{ctx}_h{H}_kv{Hkv}_d128", bench_paged_decode(t, B, ctx, H, Hkv, 128))
        report("paged_decode_int8_b8_ctx32768_h32_kv8_d128", bench_paged_decode(t, 8, 32768, 32, 8, 128, int8=True))
    for name, r, d in [("rmsnorm", args.rows, args.dim), ("swiglu", args.rows, 11008), ("ce", 4096, 32000),
                       ("adamw", 16384, 4096), ("fake_quant", 16384, 4096)]:
        if k in (name, "all"):
            report(f"{name}_{r}x{d}", bench_memory_bound(t, name, r, d))


if __name__ == "__main__":
    main()
