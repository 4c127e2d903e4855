"""Decode benchmark: batch decode tokens/s and time to first token of the inference engine, on one
GPU or tensor-parallel over N GPUs (launch with torchrun for N > 1).

    python -m mythos_b200.tools.bench_decode --preset llama3-8b --batch 64 --prompt 1024 --new 256
    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m mythos_b200.tools.bench_decode --tp 8

Weights are random-init in the configuration's formats (OIL4 attention / OIL8 FFN for the 8B
shape, I2_S for the 2.4B shape), prompts are uniform-random tokens, sampling is greedy. Timing:
TTFT = prefill + first sample (wall clock around a device synchronise, max over ranks); decode
tokens/s over the remaining steps (CUDA-graph replay), max-over-ranks time. ``--layers`` trims the
depth for quick runs; the JSON line says so.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    from ..infer.engine import InferenceEngine, TPContext
    from ..models.config import NAMED_CONFIGS
    from ..ops import native

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="llama3-8b", choices=sorted(NAMED_CONFIGS))
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="use only this many layers (0 = all)")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary size (0 = preset)")
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "int8"], help="KV page storage")
    ap.add_argument("--no-graph", action="store_true", help="launch decode steps one by one (for launch lists)")
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    native.require()
    cfg = NAMED_CONFIGS[a.preset]()
    if a.layers:
        cfg.num_layers = a.layers
    if a.vocab:
        cfg.vocab_size = a.vocab
    cfg.max_seq_len = a.prompt + a.new + 16
    tp = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
        tp = TPContext(dist.group.WORLD, dev, max_tokens=max(a.batch * a.prompt, 256), hidden=cfg.hidden_size,
                       vocab_shard=cfg.vocab_size // world, max_batch=a.batch)
    torch.manual_seed(1234)
    # weights are created shard by shard directly in their storage format
    eng = InferenceEngine.random(cfg, seed=1234, device=dev, max_batch=a.batch, max_seq_len=cfg.max_seq_len, tp=tp,
                                 kv_dtype=a.kv_dtype)
    wbytes = eng.weight_bytes()
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(7)
    prompts = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=g, dtype=torch.int32)
    ttfts, rates = [], []
    for it in range(a.repeat):
        res = eng.generate(prompts, max_new_tokens=a.new, use_graph=not a.no_graph)
        t = torch.tensor([res.stats.ttft_s, res.stats.decode_s], device=dev, dtype=torch.float64)
        if world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if it > 0 or a.repeat == 1:
            ttfts.append(float(t[0]))
            rates.append(a.batch * (a.new - 1) / float(t[1]))
    if rank == 0:
        ttfts.sort()
        print(json.dumps({"metric": "decode tok/s and p50 TTFT", "preset": a.preset, "tp": world, "batch": a.batch,
                          "prompt": a.prompt, "new_tokens": a.new, "layers": cfg.num_layers,
                          "full_depth": cfg.num_layers == NAMED_CONFIGS[a.preset]().num_layers, "decode_tok_s": max(rates), "decode_tok_s_runs": [round(r, 1) for r in rates],
                          "p50_ttft_s": ttfts[len(ttfts) // 2], "ttft_s_runs": [round(t, 4) for t in ttfts],
                          "weight_bytes_per_rank": wbytes, "kv_bytes_per_rank": eng.cache.size_bytes(), "kv_dtype": a.kv_dtype,
                          "data": "random-init weights in format, uniform-random prompts, greedy"}))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
