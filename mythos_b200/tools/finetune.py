"""oil-finetune: continue training a ``.oil`` model on new text, fully or with adapters.

Reference flags (tools/finetune.cpp:22-45): ``--model --data --output --lr --epochs --batch-size
--seq-length``; documented extras: ``--method {full,lora,qlora,dora} --lora-rank --lora-alpha
--target-modules --freeze-base --log-interval --save-interval --gpu --seed``. ``qlora`` = LoRA on
a base that is stored quantised (the model's own OIL format); steps whose gradient norm is below
``--grad-threshold`` are skipped, like the reference ``FineTuner``.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch


def main(argv=None) -> int:
    from ..models.lora import apply_lora, save_adapters
    from ..oil.model_io import load_model, save_model
    from ..train.bpe import BPETokenizer
    from ..train.data import TokenDataset
    from ..train.trainer import TrainConfig, Trainer
    from .common import pick_device, runtime_setup

    ap = argparse.ArgumentParser(prog="oil-finetune", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--output", "-o", required=True)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--max-steps", type=int, default=1000)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-length", type=int, default=256)
    ap.add_argument("--method", default="full", choices=["full", "lora", "qlora", "dora"])
    ap.add_argument("--lora-rank", type=int, default=8)
    ap.add_argument("--lora-alpha", type=float, default=16.0)
    ap.add_argument("--target-modules", default="q,v")
    ap.add_argument("--merge", action="store_true", help="fold adapters into the base before saving")
    ap.add_argument("--grad-threshold", type=float, default=0.0)
    ap.add_argument("--freeze-base", action="store_true",
                    help="full method: keep every linear weight fixed (norms and embeddings still train); "
                         "adapter methods always freeze the base")
    ap.add_argument("--save-interval", type=int, default=0, help="also save every N steps")
    ap.add_argument("--log-interval", type=int, default=10)
    ap.add_argument("--gpu", "--device", dest="device", default="auto")
    ap.add_argument("--seed", type=int, default=None, help="default: OIL_SEED, else 42")
    a = ap.parse_args(argv)
    rt = runtime_setup(seed_default=42)
    if a.seed is None:
        a.seed = rt.seed
    device = pick_device(a.device)
    torch.manual_seed(a.seed)
    model, _ = load_model(a.model, device=device)
    vocab_path = (a.model[:-4] if a.model.endswith(".oil") else a.model) + ".vocab"
    tok = BPETokenizer.load(vocab_path) if os.path.exists(vocab_path) else BPETokenizer()
    ids = np.minimum(np.asarray(tok.encode(open(a.data, "rb").read()), dtype=np.int32), model.cfg.vocab_size - 1)
    if a.method != "full":
        apply_lora(model, a.lora_rank, a.lora_alpha, tuple(a.target_modules.split(",")), dora=(a.method == "dora"))
    elif a.freeze_base:
        from ..models.layers import OILLinear

        for m in model.modules():
            if isinstance(m, OILLinear):
                m.weight.requires_grad_(False)
    seq = min(a.seq_length, model.cfg.max_seq_len)
    tcfg = TrainConfig(batch_size=a.batch_size, seq_length=seq, epochs=a.epochs, max_steps=a.max_steps, lr=a.lr,
                       weight_decay=0.0, warmup_steps=max(1, a.max_steps // 20), log_interval=a.log_interval,
                       save_interval=a.save_interval if a.method == "full" else 0,
                       output_path=a.output if (a.method == "full" and a.save_interval) else "")
    tr = Trainer(model, tcfg, device=device)
    tr.log_callbacks.append(lambda m: print(f"step {m.step} loss {m.loss:.4f} gnorm {m.grad_norm:.3f}", flush=True))
    loader = TokenDataset(ids, a.batch_size, seq, seed=a.seed, pin=device.type == "cuda")
    tr.fit(loader)
    if a.method != "full" and not a.merge:
        save_adapters(model, a.output)
    else:
        if a.method != "full":
            from ..models.lora import merge_all

            merge_all(model)
            for blk in model.layers:  # unwrap for export
                for holder, names in ((blk.attention, ("qkv_proj", "o_proj")), (blk.ffn, ("up_proj", "down_proj"))):
                    for n in names:
                        m = getattr(holder, n, None)
                        if m is not None and hasattr(m, "base"):
                            setattr(holder, n, m.base)
        save_model(model, a.output)
    print(f"saved {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
