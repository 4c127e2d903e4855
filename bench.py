#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s over the whole job) of the dense 1.3B
OIL8-STE model — 24 layers, d 2048, 16 heads, SwiGLU 5504, vocab 32000, seq 2048 — with bf16
compute, fp32 master weights, STE fake-quantised linear weights, fused AdamW, ZeRO-style data
parallel. Weak scaling: 64 sequences per GPU per optimizer step (global batch 512 at 8 GPUs).
Synthetic seeded Zipf(1.1) tokens, random-init N(0, 0.02) weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Prints one JSON line on rank 0. ``--impl reference`` reports why the reference cannot run this
configuration (CPU-only FP32 C++ engine without a Python package, a GPU path or multi-process
communication).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

SEQ = 2048
PER_GPU_BATCH = 64
MICRO_BATCH = 32     # sequences per forward/backward pass; measured 104.0k / 110.5k / 112.4k tokens/s at 8 / 16 / 32 (peak 124 GB at 32)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # the busiest half of the samples is "under load"
        sm_sorted = sorted(sm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "sm_mhz_min": sm_sorted[0] if sm else None, "samples": len(sm), "reasons": sorted(reasons)}


def model_flops_per_token(cfg) -> float:
    d, L, f, V, S = cfg.hidden_size, cfg.num_layers, cfg.ffn_hidden_size, cfg.vocab_size, SEQ
    lin = L * (d * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * d + 3 * d * f) + V * d
    attn = L * 2 * S * cfg.q_dim * 0.5 * 2  # QK^T and PV, causal half
    return 6.0 * lin + 3.0 * attn


def run_reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a CPU-only FP32 C++ engine (no setup.py/pyproject: pip install fails; no GPU "
                      "path, no bf16, no multi-process data parallel), so the 1.3B bf16 ZeRO config cannot run on it"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--per-gpu-batch", type=int, default=PER_GPU_BATCH)
    ap.add_argument("--micro-batch", type=int, default=MICRO_BATCH)
    ap.add_argument("--dp-mode", default="fused", choices=["fused", "nccl"],
                    help="data-parallel gradient path: fused peer-memory kernels or plain NCCL collectives")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm()

    import torch

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from mythos_b200.models import DenseModel
    from mythos_b200.models.config import llama_1p3b_config
    from mythos_b200.ops import native
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    native.require()

    dp = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        from mythos_b200.parallel.zero import ZeroEngine

        dp = ZeroEngine(dist.group.WORLD, device, mode=args.dp_mode)

    cfg = llama_1p3b_config()
    torch.manual_seed(1234)
    with torch.device(device):
        model = DenseModel(cfg)
    tcfg = TrainConfig(batch_size=args.per_gpu_batch, micro_batch_size=args.micro_batch, seq_length=SEQ, lr=3e-4,
                       warmup_steps=100, max_steps=10000, max_grad_norm=1.0, codebook_ema_interval=0)
    trainer = Trainer(model, tcfg, device=device, dp=dp)
    stream = ZipfStream(cfg.vocab_size, args.per_gpu_batch, SEQ, s=1.1, seed=100 + rank, pin=True)

    def barrier():
        if dp is not None:
            dp.barrier()
        torch.cuda.synchronize()

    # device-resident batches for the kernel-only measurement, pinned-host batches for end-to-end
    dev_batches = [tuple(t.to(device) for t in stream.next_batch()) for _ in range(2)]
    host_batches = [stream.next_batch() for _ in range(2)]

    for i in range(args.warmup):
        ids, tg = dev_batches[i % 2]
        trainer.train_step(ids, tg)
    barrier()
    native.check_status(device)

    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        ids, tg = dev_batches[i % 2]
        loss = trainer.train_step(ids, tg)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = native.launch_count() - launches0

    # end to end through the public API: pinned host -> device each step, loss read back each step
    barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        ids, tg = host_batches[i % 2]
        last = trainer.train_step(ids, tg).item()
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    native.check_status(device)

    t = torch.tensor([dev_ms, e2e_s * 1e3], device=device, dtype=torch.float64)
    if dp is not None:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    tokens_per_step = args.per_gpu_batch * SEQ * world
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    peak_tflops = peaks.get("bf16_tflops_sustained", 1400.0)
    mfu = value / world * model_flops_per_token(cfg) / (peak_tflops * 1e12)
    if rank == 0:
        h2d = 2 * args.per_gpu_batch * SEQ * 4
        out = {
            "metric": "train tok/s/box (1.3B OIL8-STE)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic seeded Zipf(1.1) tokens, random-init N(0,0.02) weights and quantile codebooks",
            "config": {"model": "dense-1.3B (24L d2048 16h ffn5504 v32000) OIL8 STE on all linear weights",
                       "global_batch": args.per_gpu_batch * world, "seq_len": SEQ,
                       "micro_batch": args.micro_batch,
                       "parallelism": f"dp{world}-zero" + (f"-{args.dp_mode}" if world > 1 else ""),
                       "l2": "working set (weights 2.6 GB + activations) far exceeds the 126 MB L2; no flush needed",
                       "optimizer": "AdamW fp32 master, global-norm clip 1.0, every step inside the timed region"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": int(launches),
            "model_flops_per_token": model_flops_per_token(cfg),
            "fraction_of_measured_bf16_sustained": mfu,
            "final_loss": last,
            "peak_memory_gb": torch.cuda.max_memory_allocated(device) / 2 ** 30,
        }
        print(json.dumps(out))
    if dp is not None:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
