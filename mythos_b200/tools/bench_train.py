"""Training-step throughput of any named configuration on one GPU (tokens/s, CUDA events).

    python -m mythos_b200.tools.bench_train --preset moe-8x --batch 16 --micro-batch 4 --seq 2048
    python -m mythos_b200.tools.bench_train --preset bitnet-2.4b --lora-rank 16 --batch 4 --micro-batch 1 --seq 4096

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m mythos_b200.tools.bench_train --preset moe-8x

``bench.py`` at the repository root is the fixed headline benchmark (dense 1.3B, 1-8 GPUs); this
tool covers the other training configurations: the 8-expert MoE and LoRA fine-tuning of q / v on a
frozen quantised base. On one GPU all experts are local (routing, dispatch, grouped expert GEMMs and
combine run through the same kernels as under expert parallelism, with the exchange buffers in
local memory). Under torchrun with N ranks the MoE runs expert-parallel over the N GPUs (E / N
experts computed per rank, dispatch / combine over peer memory) with ZeRO data parallelism for the
optimizer; ``--batch`` is then per rank (weak scaling) and times are the maximum over ranks. Synthetic seeded Zipf(1.1) tokens, random-init weights, optimizer step inside the
timed region, W warm-up steps, K timed steps bracketed by synchronisation.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None) -> int:
    from ..models import DenseModel
    from ..models.config import NAMED_CONFIGS
    from ..ops import native
    from ..train.data import ZipfStream
    from ..train.trainer import TrainConfig, Trainer

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="moe-8x", choices=sorted(NAMED_CONFIGS))
    ap.add_argument("--layers", type=int, default=0, help="use only this many layers (0 = all)")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lora-rank", type=int, default=0, help="> 0: freeze the base and train rank-r adapters")
    ap.add_argument("--lora-targets", default="q,v")
    ap.add_argument("--activation-checkpointing", action="store_true",
                    help="keep only each block's input and recompute the block in the backward pass")
    ap.add_argument("--ep-receive-factor", type=float, default=2.0,
                    help="expert parallel: rows a rank accepts per micro-batch, as a multiple of its own (0 = worst case)")
    a = ap.parse_args(argv)
    import os

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    native.require()
    dp = exchange = None
    if world > 1:
        import torch.distributed as dist

        from ..parallel.zero import ZeroEngine

        dist.init_process_group("nccl", device_id=dev)
        dp = ZeroEngine(dist.group.WORLD, dev, mode="fused")
    cfg = NAMED_CONFIGS[a.preset]()
    if a.layers:
        cfg.num_layers = a.layers
    cfg.max_seq_len = max(a.seq, min(cfg.max_seq_len, a.seq))
    torch.manual_seed(1234)
    if cfg.num_experts > 0:
        from ..models.moe import MoEModel as Model
    else:
        Model = DenseModel
    if world > 1 and cfg.num_experts > 0:
        from ..models.moe import ExpertParallel

        # a rank accepts up to --ep-receive-factor times its own (token, expert) rows per micro-batch
        # (0 = every row of every rank); more than that raises the status word, nothing is dropped
        exchange = ExpertParallel(dist.group.WORLD, dev, cap_rows=a.micro_batch * a.seq * cfg.moe_top_k,
                                  dim=cfg.hidden_size, receive_factor=a.ep_receive_factor or None)
    with torch.device(dev):
        model = Model(cfg, exchange=exchange) if cfg.num_experts > 0 else Model(cfg)
    if a.lora_rank > 0:
        from ..models.lora import apply_lora

        apply_lora(model, a.lora_rank, 2.0 * a.lora_rank, tuple(a.lora_targets.split(",")))
    n_params = sum(p.numel() for p in model.parameters())
    n_train = sum(p.numel() for p in model.parameters() if p.requires_grad)
    tr = Trainer(model, TrainConfig(batch_size=a.batch, micro_batch_size=a.micro_batch, seq_length=a.seq, lr=3e-4,
                                    warmup_steps=100, max_steps=10000, max_grad_norm=1.0, codebook_ema_interval=0,
                                    activation_checkpointing=a.activation_checkpointing),
                 device=dev, dp=dp)
    stream = ZipfStream(cfg.vocab_size, a.batch, a.seq, s=1.1, seed=100 + rank)
    batches = [tuple(t.to(dev) for t in stream.next_batch()) for _ in range(2)]
    for i in range(a.warmup):
        tr.train_step(*batches[i % 2])
    torch.cuda.synchronize()
    native.check_status(dev)
    l0 = native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = tr.train_step(*batches[i % 2])
    e1.record()
    torch.cuda.synchronize()
    native.check_status(dev)
    ms = e0.elapsed_time(e1) / a.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    if rank == 0:
        print(json.dumps({"metric": "train tokens/s (whole job)", "preset": a.preset, "layers": cfg.num_layers,
                      "n_gpus": world, "parallelism": (f"ep{world}+zero-dp{world}" if exchange is not None else f"dp{world}"),
                      "value": world * a.batch * a.seq / (ms / 1e3), "ms_per_step": ms, "batch": a.batch,
                      "micro_batch": a.micro_batch, "activation_checkpointing": a.activation_checkpointing, "seq_len": a.seq, "steps": a.steps, "warmup": a.warmup,
                      "parameters": n_params, "trainable_parameters": n_train, "lora_rank": a.lora_rank,
                      "gpu_launches_per_step": (native.launch_count() - l0) // a.steps, "loss": float(loss),
                      "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
                      "data": "synthetic seeded Zipf(1.1) tokens, random-init weights"}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
