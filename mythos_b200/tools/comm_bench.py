"""Fused compute + collective paths against their NCCL equivalents and the NVLink roofline.

Launch with torchrun on N >= 2 GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m mythos_b200.tools.comm_bench

Every case is timed with CUDA events on the launching stream after warm-up, bracketed by a process
group barrier, and reported as the maximum over ranks. For each fused path the line gives the bytes
that have to cross NVLink per rank and direction, the time that would take at the measured peer-copy
rate (770 GB/s per direction per GPU), the compute time at the measured GEMM rate where there is a
GEMM, the roofline (the slower of the two) and achieved / roofline.

Cases: ZeRO gradient reduce-scatter + norm (own kernel vs ``reduce_scatter_tensor``), ZeRO AdamW +
STE + all-gather (own kernel vs AdamW kernel + ``all_gather_into_tensor`` + local re-quantisation),
tensor-parallel one-shot all-reduce of a decode-sized activation (own kernels vs ``all_reduce``),
tensor-parallel GEMM with fused reduce-scatter + reduce/broadcast (vs GEMM + ``all_reduce``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0      # measured peer copy, per direction per GPU
GEMM_TFLOPS = 1654.5    # measured cuBLAS bf16 burst
HBM_GBS = 6549.4        # measured copy bandwidth


def _time(fn, group, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def main(argv=None) -> int:
    from ..ops import functional as F
    from ..ops import native
    from ..parallel import symm

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--params", type=int, default=256 << 20, help="flat parameter count of the ZeRO cases")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default="", help="'ag_gemm': run only the fused all-gather GEMM case")
    ap.add_argument("--copier-clusters", type=int, default=0, help="ag_gemm: SM pairs that copy (0 = sweep 2, 4, 6, 8)")
    a = ap.parse_args(argv)
    rank, local, W = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    C = native.require()
    st = native.status_word(dev)
    rows = []

    def report(name, ms, nvlink_bytes, flops=0.0, baseline_ms=None, hbm_bytes=0.0):
        t_link = nvlink_bytes / NVLINK_GBS / 1e6          # ms
        t_math = flops / GEMM_TFLOPS / 1e9                # ms
        t_hbm = hbm_bytes / HBM_GBS / 1e6                 # ms, local memory traffic of this rank
        roof = max(t_link, t_math, t_hbm)
        bound = "nvlink" if roof == t_link else ("compute" if roof == t_math else "hbm")
        row = {"case": name, "ranks": W, "ms": round(ms, 4), "nvlink_MB_per_rank_dir": round(nvlink_bytes / 1e6, 2),
               "roofline_ms": round(roof, 4), "bound": bound, "achieved_over_roofline": round(roof / ms, 3)}
        if baseline_ms is not None:
            row["nccl_ms"] = round(baseline_ms, 4)
            row["speedup_vs_nccl"] = round(baseline_ms / ms, 3)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    def ag_gemm_case():
        # ------------------------------------------------------------ all-gather fused into the GEMM (prefill, sequence-sharded)
        from ..parallel.ag_gemm import AllGatherGemm

        Ma, Ka, Na = 16384, 4096, 28672 // W            # Llama-3-8B gate/up projection, tensor parallel over W ranks
        Ma = Ma // (256 * W) * (256 * W)
        wa = (torch.randn(Na, Ka, device=dev) * 0.05).to(torch.bfloat16)
        a_loc = (torch.randn(Ma // W, Ka, device=dev) * 0.5).to(torch.bfloat16)
        a_all = torch.empty(Ma, Ka, device=dev, dtype=torch.bfloat16)
        ca = torch.empty(Ma, Na, device=dev, dtype=torch.bfloat16)

        def nccl_form():
            dist.all_gather_into_tensor(a_all, a_loc, group=group)
            F.gemm(a_all, wa, out=ca)

        t_n = _time(nccl_form, group, a.iters, a.warmup)
        want = ca.clone()
        t_g = _time(lambda: F.gemm(a_all, wa, out=ca), group, a.iters, a.warmup)
        report(f"gemm_alone_{Ma}x{Na}x{Ka}", t_g, 0.0, flops=2.0 * Ma * Na * Ka)
        for cc in ([a.copier_clusters] if a.copier_clusters > 0 else [2, 4, 6, 8]):
            ag = AllGatherGemm(group, dev, Ma, Ka, copier_clusters=cc)
            out = torch.empty(Ma, Na, device=dev, dtype=torch.bfloat16)

            def fused():
                ag.shard().copy_(a_loc)                    # stands for the producer of the local rows (8 MB copy)
                ag.run(wa, out)

            t_f = _time(fused, group, a.iters, a.warmup)
            native.check_status(dev)
            err = float((out.float() - want.float()).abs().max() / want.float().abs().max())
            assert err < 2e-2, f"fused all-gather GEMM differs from all_gather + GEMM: {err}"
            report(f"allgather_gemm_fused_{Ma}x{Na}x{Ka}_copiers{cc}", t_f, Ma * Ka * 2.0 * (W - 1) / W,
                   flops=2.0 * Ma * Na * Ka, baseline_ms=t_n)
            del ag
            torch.cuda.empty_cache()

    def sharded_weight_case():
        # ------------------------------------------------------------ parameter all-gather fused into the consuming GEMM
        from ..parallel.ag_gemm import ShardedWeightGemm

        Mw, Kw, Nw = 16384, 2048, 6144                 # QKV projection of the 1.3B model, weight sharded over W ranks
        Nw = Nw // (256 * W) * (256 * W)
        w_loc = (torch.randn(Nw // W, Kw, device=dev) * 0.05).to(torch.bfloat16)
        w_all = torch.empty(Nw, Kw, device=dev, dtype=torch.bfloat16)
        xw = (torch.randn(Mw, Kw, device=dev) * 0.5).to(torch.bfloat16)
        yw = torch.empty(Mw, Nw, device=dev, dtype=torch.bfloat16)

        def nccl_form():
            dist.all_gather_into_tensor(w_all, w_loc, group=group)
            F.gemm(xw, w_all, out=yw)

        t_n = _time(nccl_form, group, a.iters, a.warmup)
        want = yw.clone()
        t_g = _time(lambda: F.gemm(xw, w_all, out=yw), group, a.iters, a.warmup)
        report(f"gemm_alone_{Mw}x{Nw}x{Kw}", t_g, 0.0, flops=2.0 * Mw * Nw * Kw)
        for cc in (1, 2, 4):
            sw = ShardedWeightGemm(group, dev, Nw, Kw, copier_clusters=cc)
            sw.write_shard(w_loc)
            out = torch.empty(Mw, Nw, device=dev, dtype=torch.bfloat16)
            t_f = _time(lambda: sw.run(xw, out), group, a.iters, a.warmup)
            native.check_status(dev)
            err = float((out.float() - want.float()).abs().max() / want.float().abs().max())
            assert err < 2e-2, f"fused weight gather GEMM differs from all_gather + GEMM: {err}"
            report(f"weight_allgather_gemm_fused_{Mw}x{Nw}x{Kw}_copiers{cc}", t_f, Nw * Kw * 2.0 * (W - 1) / W,
                   flops=2.0 * Mw * Nw * Kw, baseline_ms=t_n)
            del sw
            torch.cuda.empty_cache()

    if a.only == "ag_gemm":
        ag_gemm_case()
        sharded_weight_case()
        if rank == 0:
            print(json.dumps({"summary": rows}))
        native.check_status(dev)
        dist.destroy_process_group()
        return 0

    bar = symm.FlagBarrier(dev, group)
    use_mc = symm.nvls_enabled()          # MYTHOS_NVLS=1: also time the multimem (in-switch) variants

    # ---------------------------------------------------------------- ZeRO reduce-scatter + norm
    n = a.params // (256 * W) * (256 * W)
    shard = n // W
    gbuf = symm.make_buffer(n, torch.float32, dev, group)
    gbuf.tensor.normal_()
    gshard = torch.empty(shard, device=dev)
    part = torch.zeros(1, device=dev)

    def rs_fused():
        bar.sync()
        C.zero_reduce_scatter(gbuf.ptrs, gshard, rank * shard, part)
        bar.sync(part)

    def rs_nccl():
        dist.reduce_scatter_tensor(gshard, gbuf.tensor, op=dist.ReduceOp.SUM, group=group)
        F.sumsq(gshard, part)
        dist.all_reduce(part, group=group)

    t_f, t_n = _time(rs_fused, group, a.iters, a.warmup), _time(rs_nccl, group, a.iters, a.warmup)
    # local memory: this rank's slice is read by every rank (W reads) and the result written once
    report("zero_reduce_scatter_norm_fp32", t_f, shard * 4.0 * (W - 1), baseline_ms=t_n, hbm_bytes=shard * 4.0 * (W + 1))
    if use_mc and gbuf.multicast_ptr:
        want = gshard.clone()
        gmc = torch.empty_like(gshard)

        def rs_nvls():
            bar.sync()
            C.zero_reduce_scatter(gbuf.ptrs, gmc, rank * shard, part, gbuf.multicast_ptr, 0)
            bar.sync(part)

        t_m = _time(rs_nvls, group, a.iters, a.warmup)
        err = float((gmc - want).abs().max() / want.abs().max())
        assert err < 1e-5, f"multimem reduce-scatter differs from the peer-load sum: {err}"
        report("zero_reduce_scatter_norm_fp32_nvls", t_m, shard * 4.0 * (W - 1), baseline_ms=t_n,
               hbm_bytes=shard * 4.0 * (W + 1))
    elif use_mc and rank == 0:
        print(json.dumps({"note": "MYTHOS_NVLS=1 but the symmetric allocation has no multicast mapping"}), flush=True)

    # ---------------------------------------------------------------- ZeRO AdamW + STE + all-gather
    cbuf = symm.make_buffer(n, torch.bfloat16, dev, group)
    master = torch.randn(shard, device=dev) * 0.02
    m, v = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    from ..oil.codebook import quantile_codebook

    nseg = n // 256
    seg_fmt = torch.ones(nseg, device=dev, dtype=torch.uint8)                       # every segment OIL8
    seg_cb = (torch.arange(nseg, device=dev) // 128).to(torch.int32)
    cb8 = quantile_codebook(256).to(dev)[None].repeat((nseg + 127) // 128, 1).contiguous()
    cb4 = torch.zeros(1, 16, device=dev)
    gnorm = torch.zeros(1, device=dev)

    def ag_fused(mc=0):
        C.zero_adamw_ste_allgather(master, m, v, gshard, cbuf.ptrs, rank * shard, seg_fmt, seg_cb, cb8, cb4, bar.slots,
                                   gnorm, 1.0, 1e-4, 0.9, 0.95, 1e-8, 0.1, 10, 1.0, rank, mc)
        bar.sync()

    full = torch.empty(n, device=dev)
    qout = torch.empty(n, device=dev, dtype=torch.bfloat16)
    clip = torch.ones(1, device=dev)

    def ag_nccl():
        F.adamw_step(master, m, v, gshard, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=10,
                     clip_coef=clip)
        dist.all_gather_into_tensor(full, master, group=group)
        C.oil_fake_quant(full, cb8, seg_cb, 256, qout, None)

    t_f, t_n = _time(ag_fused, group, a.iters, a.warmup), _time(ag_nccl, group, a.iters, a.warmup)
    # local memory: p, m, v, g read and p, m, v written in fp32, plus the bf16 image written by all W ranks
    report("zero_adamw_ste_allgather_bf16", t_f, shard * 2.0 * (W - 1), baseline_ms=t_n,
           hbm_bytes=shard * (28.0 + 2.0 * W))
    if use_mc and cbuf.multicast_ptr:
        t_m = _time(lambda: ag_fused(cbuf.multicast_ptr), group, a.iters, a.warmup)
        # every rank's image must be identical after a multicast all-gather
        digest = cbuf.tensor.view(torch.int16).long().sum().reshape(1)
        digs = [torch.zeros_like(digest) for _ in range(W)]
        dist.all_gather(digs, digest, group=group)
        assert all(int(d) == int(digs[0]) for d in digs), "multicast all-gather left different images on the ranks"
        report("zero_adamw_ste_allgather_bf16_nvls", t_m, shard * 2.0 * (W - 1), baseline_ms=t_n,
               hbm_bytes=shard * (28.0 + 2.0 * W))
    del gbuf, cbuf, full, qout
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- TP one-shot all-reduce (decode)
    T, N = 64, 4096
    stride = 256 * N
    staging = symm.make_buffer(W * stride, torch.bfloat16, dev, group).zero_()
    acc = torch.randn(T, N, device=dev)
    out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
    fbar = symm.FlagBarrier(dev, group)

    def tp_oneshot():
        C.tp_push(acc, staging.ptrs, rank, rank * stride)
        fbar.sync()
        C.tp_reduce_slots(staging.tensor, W, stride, None, out)

    xb = torch.randn(T, N, device=dev).to(torch.bfloat16)

    def tp_nccl():
        dist.all_reduce(xb, group=group)

    t_f, t_n = _time(tp_oneshot, group, a.iters * 5, a.warmup), _time(tp_nccl, group, a.iters * 5, a.warmup)
    report("tp_allreduce_oneshot_64x4096_bf16", t_f, T * N * 2.0 * (W - 1), baseline_ms=t_n)

    # the same sum followed by residual add + RMSNorm: three kernels + barrier vs one signalled kernel
    gamma = torch.ones(N, device=dev, dtype=torch.bfloat16)
    resid = torch.randn(T, N, device=dev).to(torch.bfloat16)
    s_out, n_out = torch.empty_like(resid), torch.empty_like(resid)
    row_flags = symm.make_buffer(2 * W * 256, torch.int32, dev, group).zero_()
    row_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    row_arrive = torch.zeros(1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    dist.barrier(group=group)
    parity = [0]

    def tp_norm_unfused():
        C.tp_push(acc, staging.ptrs, rank, rank * stride)
        fbar.sync()
        C.sum_residual_rmsnorm(None, staging.tensor, W, stride, resid, gamma, s_out, n_out, 1e-5)

    def tp_norm_signalled():
        C.tp_sum_residual_rmsnorm(acc, staging.ptrs, row_flags.ptrs, rank, stride, parity[0], 256, resid, gamma, s_out,
                                  n_out, 1e-5, row_epoch, row_arrive, symm.DEFAULT_BARRIER_LIMIT_CYCLES, st)
        parity[0] ^= 1

    def tp_norm_nccl():
        dist.all_reduce(xb, group=group)
        F.rmsnorm(xb, gamma, 1e-5, resid)

    t_u = _time(tp_norm_unfused, group, a.iters * 5, a.warmup)
    t_s = _time(tp_norm_signalled, group, a.iters * 5, a.warmup)
    t_n = _time(tp_norm_nccl, group, a.iters * 5, a.warmup)
    report("tp_sum_residual_rmsnorm_push_barrier_sum_64x4096", t_u, T * N * 2.0 * (W - 1), baseline_ms=t_n)
    report("tp_sum_residual_rmsnorm_row_signalled_64x4096", t_s, T * N * 2.0 * (W - 1), baseline_ms=t_n)

    # ---------------------------------------------------------------- TP GEMM + fused reduce-scatter (prefill)
    Tp, K = 8192 * W if W <= 4 else 65536, 4096 // W * 2
    Tp = Tp // (W * 256) * (W * 256)
    rows_per = Tp // W
    n_slot = rows_per * N
    partb = symm.make_buffer(W * n_slot, torch.bfloat16, dev, group)
    outb = symm.make_buffer(Tp * N, torch.bfloat16, dev, group)
    x = (torch.randn(Tp, K, device=dev) * 0.1).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)

    def tp_fused_gemm():
        C.gemm_reduce_scatter(x, w, partb.ptrs, rank, rows_per, n_slot, st)
        fbar.sync()
        C.tp_reduce_slots_bcast(partb.tensor, W, n_slot, outb.ptrs, rank, rank * n_slot, n_slot)
        fbar.sync()

    partc = symm.make_buffer(Tp * N, torch.bfloat16, dev, group)

    def tp_gemm_pull():        # unfused variant of the own path: local GEMM, then pull-sum-store between two barriers
        F.gemm(x, w, out=partc.tensor.view(Tp, N))
        fbar.sync()
        C.tp_allreduce_pull(partc.ptrs, outb.ptrs, rank, Tp * N)
        fbar.sync()

    yb = torch.empty(Tp, N, device=dev, dtype=torch.bfloat16)

    def tp_gemm_nccl():
        F.gemm(x, w, out=yb)
        dist.all_reduce(yb, group=group)

    t_f, t_n = _time(tp_fused_gemm, group, a.iters, a.warmup), _time(tp_gemm_nccl, group, a.iters, a.warmup)
    t_p = _time(tp_gemm_pull, group, a.iters, a.warmup)
    if use_mc and partc.multicast_ptr and outb.multicast_ptr:
        want = outb.tensor.clone()

        def tp_gemm_nvls():    # local GEMM, then the all-reduce inside the switch: multimem.ld_reduce + multimem.st
            F.gemm(x, w, out=partc.tensor.view(Tp, N))
            fbar.sync()
            C.tp_allreduce_multimem(partc.multicast_ptr, outb.multicast_ptr, W, rank, Tp * N)
            fbar.sync()

        t_m = _time(tp_gemm_nvls, group, a.iters, a.warmup)
        err = float((outb.tensor.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < 2e-2, f"multimem all-reduce differs from the pull all-reduce: {err}"
        # in-switch reduction: each direction carries the output once ((W-1)/W up, the same down)
        report(f"tp_gemm_then_nvls_allreduce_{Tp}x{N}x{K}", t_m, Tp * N * 2.0 * (W - 1) / W * 1.0 + Tp * N * 2.0 / W,
               flops=2.0 * Tp * N * K, baseline_ms=t_n)
    t_g = _time(lambda: F.gemm(x, w, out=yb), group, a.iters, a.warmup)
    report(f"tp_gemm_then_pull_allreduce_{Tp}x{N}x{K}", t_p, 2.0 * Tp * N * 2.0 * (W - 1) / W, flops=2.0 * Tp * N * K,
           baseline_ms=t_n)
    report(f"gemm_alone_{Tp}x{N}x{K}", t_g, 0.0, flops=2.0 * Tp * N * K)
    # reduce-scatter then all-gather: each direction carries (W-1)/W of the output twice
    report(f"tp_gemm_reduce_scatter_allgather_{Tp}x{N}x{K}", t_f, 2.0 * Tp * N * 2.0 * (W - 1) / W,
           flops=2.0 * Tp * N * K, baseline_ms=t_n)
    del partb, outb, partc
    torch.cuda.empty_cache()
    ag_gemm_case()
    sharded_weight_case()

    if rank == 0:
        print(json.dumps({"summary": rows}))
    native.check_status(dev)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
