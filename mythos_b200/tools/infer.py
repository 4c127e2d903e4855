"""oil-infer: generate text from a ``.oil`` model.

Reference spelling (tools/infer.cpp): ``oil-infer <model.oil> [prompt]`` with temperature 0.7,
top-k 40, top-p 0.9, 512 tokens, a sibling ``.vocab`` tokenizer (byte tokens without it) and tok/s
on stderr. Documented flags are accepted too: ``--model/-m --prompt/-p --max-tokens/-t
--temperature --top-k --top-p --seed --batch-size --output/-o --gpu --precision``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch


def build_parser():
    ap = argparse.ArgumentParser(prog="oil-infer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_pos", nargs="?", default=None)
    ap.add_argument("prompt_pos", nargs="?", default=None)
    ap.add_argument("--model", "-m", default=None)
    ap.add_argument("--prompt", "-p", default=None)
    ap.add_argument("--max-tokens", "-t", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None, help="default: OIL_SEED, else 0")
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--output", "-o", default=None)
    ap.add_argument("--gpu", "--device", dest="device", default="auto")
    ap.add_argument("--precision", default="auto", choices=["auto", "fp32", "fp16", "bf16", "int8"],
                    help="int8: int8 KV pages on the GPU engine, int8 activations on the CPU path; the other "
                         "values keep the engine's bf16 compute (GPU) / fp32 reference ops (CPU)")
    ap.add_argument("--verbose", action="store_true")
    return ap


def generate_text(model, tokenizer, prompt: str, max_tokens: int, sampler, device, precision: str = "auto"):
    """Returns (text, stats dict). CUDA: paged-KV engine; CPU: full-recompute loop on the reference ops."""
    from ..infer.sampler import sample

    ids = tokenizer.encode(prompt) if tokenizer is not None else list(prompt.encode("utf-8"))
    ids = [min(i, model.cfg.vocab_size - 1) for i in ids] or [0]
    t0 = time.perf_counter()
    if device.type == "cuda":
        from ..infer.engine import InferenceEngine

        S = len(ids)
        eng = InferenceEngine.from_model(model, device=device, max_batch=1,
                                         max_seq_len=min(model.cfg.max_seq_len, S + max_tokens) + 16,
                                         kv_dtype="int8" if precision == "int8" else "bf16")
        room = eng.max_seq_len - S
        res = eng.generate([ids], max_new_tokens=max(1, min(max_tokens, room)), sampler=sampler,
                           use_graph=sampler.greedy)
        new = res.tokens[0]
        stats = {"tokens_per_s": res.stats.tokens_per_s, "ttft_s": res.stats.ttft_s}
    else:
        seq = torch.tensor([ids], dtype=torch.int32)
        new = []
        ttft = None
        run = model
        if precision == "int8":
            from ..infer.extras import INT8Inference

            run = INT8Inference(model)
        with torch.no_grad():
            for step in range(max_tokens):
                window = seq[:, -model.cfg.max_seq_len:]
                logits = run(window)[:, -1].float()
                hist = seq[:, -64:].to(torch.int32)
                tok = sample(logits, sampler, history=hist, step=step)
                if ttft is None:
                    ttft = time.perf_counter() - t0
                new.append(int(tok[0]))
                seq = torch.cat([seq, tok.view(1, 1).to(torch.int32)], dim=1)
                if tokenizer is not None and int(tok[0]) == tokenizer.eos_id():
                    break
        dt = time.perf_counter() - t0
        stats = {"tokens_per_s": len(new) / max(dt, 1e-9), "ttft_s": ttft or 0.0}
    text = tokenizer.decode(new) if tokenizer is not None else bytes(t & 0xFF for t in new).decode("utf-8", "replace")
    return text, stats


def main(argv=None) -> int:
    from ..infer.sampler import SamplerConfig
    from ..oil.model_io import load_model
    from ..train.bpe import BPETokenizer
    from .common import pick_device, runtime_setup

    args = build_parser().parse_args(argv)
    rt = runtime_setup(seed_default=0)
    if args.seed is None:
        args.seed = rt.seed
    path = args.model or args.model_pos
    if not path:
        print("usage: oil-infer <model.oil> [prompt]", file=sys.stderr)
        return 2
    prompt = args.prompt if args.prompt is not None else (args.prompt_pos or "Once upon a time")
    device = pick_device(args.device)
    model, _ = load_model(path, device=device)
    model.eval()
    vocab = (path[:-4] if path.endswith(".oil") else path) + ".vocab"
    tokenizer = None
    if os.path.exists(vocab):
        tokenizer = BPETokenizer.load(vocab)
    else:
        print(f"warning: {vocab} not found, using byte tokens", file=sys.stderr)
    sampler = SamplerConfig(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            repetition_penalty=args.repetition_penalty, seed=args.seed)
    text, stats = generate_text(model, tokenizer, prompt, args.max_tokens, sampler, device, args.precision)
    out = prompt + text
    if args.output:
        with open(args.output, "w") as f:
            f.write(out)
    else:
        print(out)
    print(f"{stats['tokens_per_s']:.1f} tok/s, first token after {stats['ttft_s'] * 1e3:.1f} ms", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
