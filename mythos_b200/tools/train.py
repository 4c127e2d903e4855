"""oil-train: train a dense (or MoE) decoder from scratch on a text file or a synthetic stream.

Implemented flags of the reference tool keep their spelling (tools/train.cpp:30-74: ``--model``
is the OUTPUT path, ``--data --config --batch-size --seq-length --epochs --lr --vocab-size
--hidden-size --num-layers --num-heads --log-interval --save-interval``); the documented-only
flags are accepted too (``--output/-o --learning-rate --optimizer --weight-decay --warmup-steps
--gpu --resume --seed --verbose --dim --n-layers``). ``--config`` is honoured (the reference
parses and ignores it).

    oil-train --data corpus.txt --model out.oil --hidden-size 256 --num-layers 4 --num-heads 4
    oil-train --synthetic zipf --preset tiny-byte --max-steps 200 --model tiny.oil
"""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np
import torch


def build_parser():
    ap = argparse.ArgumentParser(prog="oil-train", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", "--output", "-o", dest="model", default="model.oil", help="output .oil path")
    ap.add_argument("--data", default=None, help="UTF-8 text corpus")
    ap.add_argument("--synthetic", default=None, choices=[None, "zipf"], help="seeded Zipf(1.1) token stream")
    ap.add_argument("--config", "-c", default=None)
    ap.add_argument("--preset", default=None)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--micro-batch-size", type=int, default=0)
    ap.add_argument("--seq-length", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--max-steps", type=int, default=0)
    ap.add_argument("--lr", "--learning-rate", dest="lr", type=float, default=3e-4)
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "adam", "sgd"])
    ap.add_argument("--weight-decay", type=float, default=1e-2)
    ap.add_argument("--warmup-steps", type=int, default=100)
    ap.add_argument("--vocab-size", type=int, default=0)
    ap.add_argument("--hidden-size", "--dim", dest="hidden_size", type=int, default=0)
    ap.add_argument("--num-layers", "--n-layers", dest="num_layers", type=int, default=0)
    ap.add_argument("--num-heads", "--n-heads", dest="num_heads", type=int, default=0)
    ap.add_argument("--ffn-hidden-size", type=int, default=0)
    ap.add_argument("--weight-format", default=None, choices=[None, "oil8", "oil4", "i2s", "fp32"])
    ap.add_argument("--block-size", type=int, default=0)
    ap.add_argument("--log-interval", type=int, default=10)
    ap.add_argument("--save-interval", type=int, default=0)
    ap.add_argument("--gpu", "--device", dest="device", default="auto")
    ap.add_argument("--resume", default=None)
    ap.add_argument("--seed", type=int, default=None, help="default: OIL_SEED, else 42")
    ap.add_argument("--python-loader", action="store_true", help="use the Python data loader instead of the C++ one")
    ap.add_argument("--streaming", action="store_true",
                    help="read and tokenise --data in 4 MB chunks while training (the tokenizer is trained on the first chunk)")
    ap.add_argument("--mask-prob", type=float, default=0.0, help="augmentation: input ids replaced by id 0")
    ap.add_argument("--replace-prob", type=float, default=0.0, help="augmentation: input ids replaced by random ids")
    ap.add_argument("--curriculum-epochs", type=int, default=0,
                    help="grow the sequence length from a quarter to full over this many epochs")
    ap.add_argument("--logdir", default=None, help="write TensorBoard events + JSONL here")
    ap.add_argument("--verbose", action="store_true")
    return ap


def main(argv=None) -> int:
    from ..models import DenseModel
    from ..oil.container import file_sha256
    from ..train.bpe import BPETokenizer
    from ..train.data import TokenDataset, ZipfStream
    from ..train.trainer import TrainConfig, Trainer
    from .common import load_json_config, model_config_from, pick_device, runtime_setup

    args = build_parser().parse_args(argv)
    rt = runtime_setup(seed_default=42)
    if args.seed is None:
        args.seed = rt.seed
    cfgj = load_json_config(args.config)
    tj = cfgj.get("training", {})
    device = pick_device(args.device)
    torch.manual_seed(args.seed)
    tokenizer, tokens = None, None
    vocab = args.vocab_size
    if args.data:
        with open(args.data, "rb") as fh:
            text = fh.read(4 << 20) if args.streaming else fh.read()
        tokenizer = BPETokenizer()
        tokenizer.train(text, max(256, vocab or 512))
        tokens = None if args.streaming else np.asarray(tokenizer.encode(text), dtype=np.int32)
        vocab = tokenizer.vocab_size
    cfg = model_config_from(args, cfgj, vocab or None)
    seq = args.seq_length or tj.get("seq_length") or min(cfg.max_seq_len, 512)
    cfg.max_seq_len = max(cfg.max_seq_len, seq)
    if cfg.num_experts > 0:
        from ..models.moe import MoEModel as Model
    else:
        Model = DenseModel
    with torch.device(device):
        model = Model(cfg)
    batch = tj.get("batch_size", args.batch_size)
    tcfg = TrainConfig(batch_size=batch, micro_batch_size=args.micro_batch_size, seq_length=seq, epochs=args.epochs,
                       max_steps=args.max_steps or tj.get("max_steps", 10000), lr=tj.get("learning_rate", args.lr),
                       weight_decay=tj.get("weight_decay", args.weight_decay),
                       warmup_steps=tj.get("warmup_steps", args.warmup_steps), log_interval=args.log_interval,
                       save_interval=args.save_interval, output_path=args.model, seed=args.seed)
    trainer = Trainer(model, tcfg, device=device)
    if args.resume:
        trainer.load_checkpoint(args.resume)
    writers = []
    if args.logdir:
        from ..train.metrics import EventWriter, JsonlLogger

        ew, jl = EventWriter(args.logdir), JsonlLogger("oil-train", str(int(time.time())), args.logdir)
        writers = [ew, jl]
        trainer.log_callbacks.append(lambda m: (ew.write_metrics(m), jl.log(m)))
    trainer.log_callbacks.append(lambda m: print(
        f"step {m.step:6d} epoch {m.epoch} loss {m.loss:.4f} ppl {m.perplexity:9.2f} lr {m.lr:.2e} "
        f"gnorm {m.grad_norm:.3f} tok/s {m.tokens_per_sec:,.0f}", flush=True))
    print(f"model: {model.param_count():,} parameters, format {cfg.weight_format}, device {device}")
    if tokens is not None:
        from ..oil import native_io

        if native_io.available() and not args.python_loader:
            # C++ loader: batches are assembled by a worker thread into a ring, copied into pinned tensors
            loader = native_io.NativeTokenLoader(tokens, batch, seq, shuffle=True, seed=args.seed,
                                                 pin=device.type == "cuda")
        else:
            loader = TokenDataset(tokens, batch, seq, shuffle=True, seed=args.seed, pin=device.type == "cuda")
        if len(loader) == 0:
            print("corpus is shorter than one batch; lower --batch-size / --seq-length", file=sys.stderr)
            return 2
    elif args.streaming and args.data:
        from ..train.data import StreamingTokenDataset

        loader = StreamingTokenDataset(args.data, tokenizer, batch, seq, vocab_limit=cfg.vocab_size)
    else:
        stream = ZipfStream(cfg.vocab_size, batch, seq, seed=args.seed)

        class _Synthetic:
            def __iter__(self):
                for _ in range(tcfg.max_steps):
                    yield stream.next_batch()

        loader = _Synthetic()
        tcfg.epochs = 1
    if args.mask_prob or args.replace_prob or args.curriculum_epochs:
        from ..train.data import AugmentedLoader, Curriculum

        cur = Curriculum(seq, args.curriculum_epochs) if args.curriculum_epochs else None
        loader = AugmentedLoader(loader, cfg.vocab_size, args.mask_prob, args.replace_prob, curriculum=cur,
                                 seed=args.seed)
    metrics = trainer.fit(loader)
    if tokenizer is not None:
        tokenizer.save(args.model[:-4] + ".vocab" if args.model.endswith(".oil") else args.model + ".vocab")
    for w in writers:
        w.close()
    print(f"saved {args.model} sha256 {file_sha256(args.model)} final loss {metrics.loss:.4f}")
    if rt.verbose:      # OIL_VERBOSE=1: device time per phase, from CUDA events recorded around the ranges
        from ..utils import trace

        print(trace.format_summary(trace.summary()))
    return 0


if __name__ == "__main__":
    sys.exit(main())
