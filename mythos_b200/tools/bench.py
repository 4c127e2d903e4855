"""oil-bench: kernel micro-benchmarks and end-to-end generation speed.

Reference flags (tools/bench.cpp:24-44): ``--kernel {matmul,all} --size N``, ``--inference --model
--prompt``; documented extras ``--iterations --warmup --batch-size --max-tokens --csv --output``.
Kernel mode forwards to :mod:`mythos_b200.tools.kernel_bench`; inference mode loads a ``.oil``
model and reports prefill time (TTFT), decode tokens/s and ms/token.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="oil-bench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", default=None, help="matmul | attn_fwd | attn_bwd | rmsnorm | ... | all")
    ap.add_argument("--size", type=int, default=4096)
    ap.add_argument("--inference", action="store_true")
    ap.add_argument("--model", default=None)
    ap.add_argument("--prompt", default="The quick brown fox")
    ap.add_argument("--prompts", default=None, help="file with one prompt per line (each is timed; means are reported)")
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--iterations", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--csv", action="store_true")
    ap.add_argument("--output", default=None)
    ap.add_argument("--gpu", "--device", dest="device", default="auto")
    a = ap.parse_args(argv)
    if a.inference or a.model:
        import torch

        from ..infer.sampler import SamplerConfig
        from ..oil.model_io import load_model
        from .common import pick_device
        from .infer import generate_text

        device = pick_device(a.device)
        model, _ = load_model(a.model, device=device)
        model.eval()
        prompts = [a.prompt]
        if a.prompts:
            prompts = [ln.rstrip("\n") for ln in open(a.prompts, encoding="utf-8") if ln.strip()] or prompts
        runs = [generate_text(model, None, p, a.max_tokens, SamplerConfig(temperature=0.0), device)[1] for p in prompts]
        stats = {k: sum(r[k] for r in runs) / len(runs) for k in ("tokens_per_s", "ttft_s")}
        row = {"model": a.model, "prompts": len(prompts), "tokens_per_s": stats["tokens_per_s"],
               "ttft_ms": stats["ttft_s"] * 1e3, "ms_per_token": 1e3 / max(stats["tokens_per_s"], 1e-9),
               "memory_mb": torch.cuda.max_memory_allocated() / 2 ** 20 if device.type == "cuda" else 0.0}
        line = ",".join(f"{v}" for v in row.values()) if a.csv else json.dumps(row)
        print(line)
        if a.output:
            open(a.output, "w").write(line + "\n")
        return 0
    from . import kernel_bench

    kernel = {"matmul": "gemm", None: "all"}.get(a.kernel, a.kernel)
    argv2 = ["--kernel", kernel, "--iters", str(a.iterations), "--warmup", str(a.warmup)]
    if kernel == "gemm":
        argv2 += ["--m", str(a.size), "--n", str(a.size), "--k", str(a.size)]
    sys.argv = ["kernel_bench"] + argv2
    kernel_bench.main()
    return 0


if __name__ == "__main__":
    sys.exit(main())
