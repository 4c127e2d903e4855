"""Tiny byte-level configuration (4 layers, d 256, 4 heads, FFN 1024, vocab 256, context 128, batch 16,
AdamW 3e-4, seeded Zipf(1.1) tokens) on this machine's CPU: the reference's stock trainer (FP32, no
straight-through quantiser in its loop) against this framework's CPU path (fp32 master weights with
OIL8 STE fake-quantisation, 64-weight blocks). Prints one JSON line per arm.

    python baseline/build_reference.py && python baseline/run_config1.py --steps 3
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def ours(steps: int, warmup: int) -> dict:
    import torch

    from mythos_b200.models import DenseModel
    from mythos_b200.models.config import tiny_byte_config
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(0)
    cfg = tiny_byte_config()
    tr = Trainer(DenseModel(cfg), TrainConfig(batch_size=16, seq_length=128, lr=3e-4, warmup_steps=0), device="cpu")
    data = ZipfStream(cfg.vocab_size, 16, 128, s=1.1, seed=1234)
    loss = 0.0
    for _ in range(warmup):
        loss = float(tr.train_step(*data.next_batch()))
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = float(tr.train_step(*data.next_batch()))
    sec = time.perf_counter() - t0
    return {"impl": "mythos_b200 (CPU path)", "config": "tiny-byte 4L d256 4h ffn1024 v256 ctx128 batch16, OIL8 STE, fp32 cpu",
            "steps": steps, "tokens_per_s": round(steps * 16 * 128 / sec, 1), "ms_per_step": round(sec / steps * 1e3, 2),
            "last_loss": round(loss, 4), "threads": torch.get_num_threads()}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--ours-steps", type=int, default=20)
    a = ap.parse_args()
    exe = os.path.join(HERE, "_ref", "ref_config1")
    if os.path.exists(exe):
        out = subprocess.run([exe, str(a.steps), str(a.warmup)], capture_output=True, text=True)
        print(out.stdout.strip() or json.dumps({"impl": "reference", "error": out.stderr[-300:]}))
    else:
        print(json.dumps({"impl": "reference", "unavailable": "run baseline/build_reference.py first"}))
    print(json.dumps(ours(a.ours_steps, a.warmup)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
