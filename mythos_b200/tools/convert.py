"""oil-convert: raw fp32 / GGUF / safetensors -> ``.oil``, optionally quantised to a target bpw.

Reference flags (tools/convert.cpp:25-48): ``--input --output --format {rawfp32,gguf} --bpw
--verbose``; documented extras: ``--input-format {auto,safetensors,gguf,pytorch} --target-bpw
--format-planner --codebook-size``. ``rawfp32`` reproduces the reference's output byte for byte
(one FP32 block named ``weights``, empty config). With ``--bpw`` every tensor is planned and
quantised block by block on its own (the reference quantises the concatenation of all tensors
with one global codebook and writes that blob into every tensor, tools/convert.cpp:498-509).
"""
from __future__ import annotations

import argparse
import sys

import numpy as np
import torch


def build_parser():
    ap = argparse.ArgumentParser(prog="oil-convert", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", "-i", required=True)
    ap.add_argument("--output", "-o", required=True)
    ap.add_argument("--format", "--input-format", dest="format", default="auto",
                    choices=["auto", "rawfp32", "gguf", "safetensors", "pytorch"])
    ap.add_argument("--bpw", "--target-bpw", dest="bpw", type=float, default=0.0)
    ap.add_argument("--weight-format", default=None, choices=[None, "oil8", "oil4", "i2s", "fp16", "fp32"],
                    help="quantise every 2-D tensor to this single format")
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--format-planner", default="magnitude", choices=["magnitude", "uniform", "awq", "custom"])
    ap.add_argument("--codebook-size", type=int, default=256)
    ap.add_argument("--verbose", action="store_true")
    return ap


def main(argv=None) -> int:
    from ..oil import importers, planner
    from ..oil.container import BlockData, file_sha256, write_oil
    from ..oil.formats import Format
    from ..oil.model_io import _fp32_blocks

    a = build_parser().parse_args(argv)
    fmt = a.format
    if fmt == "auto":
        fmt = "gguf" if a.input.endswith(".gguf") else "safetensors" if a.input.endswith(".safetensors") else \
            "pytorch" if a.input.endswith((".pt", ".pth", ".bin")) else "rawfp32"
    if fmt == "rawfp32":
        tensors = importers.read_raw_fp32(a.input)
    elif fmt == "gguf":
        tensors, _ = importers.read_gguf(a.input)
    elif fmt == "safetensors":
        tensors = importers.read_safetensors(a.input)
    else:
        sd = torch.load(a.input, map_location="cpu", weights_only=True)
        tensors = {k: v.float().numpy() for k, v in sd.items() if torch.is_tensor(v) and v.is_floating_point()}
    out, shapes, total_bits, total_w = [], {}, 0.0, 0
    for name, arr in tensors.items():
        arr = np.asarray(arr, dtype=np.float32)
        shapes[name] = list(arr.shape)
        quantisable = arr.ndim >= 2 and arr.size >= a.block_size
        if a.bpw > 0 and quantisable:
            t = torch.from_numpy(arr)
            fmts, achieved = planner.plan(t, a.bpw, a.block_size)
            _, blocks = planner.quantize_mixed(t, fmts, a.block_size)
            total_bits += achieved * arr.size
        elif a.weight_format and a.weight_format != "fp32" and quantisable:
            code = {"oil8": Format.OIL8, "oil4": Format.OIL4, "i2s": Format.TERNARY, "fp16": Format.FP16}[a.weight_format]
            nb = (arr.size + a.block_size - 1) // a.block_size
            _, blocks = planner.quantize_mixed(torch.from_numpy(arr), np.full(nb, int(code), dtype=np.uint8),
                                               a.block_size)
            total_bits += {"oil8": 8, "oil4": 4, "i2s": 1.58, "fp16": 16}[a.weight_format] * arr.size
        else:
            blocks = _fp32_blocks(arr) if fmt != "rawfp32" else [BlockData(Format.FP32, arr.size, b"", arr.tobytes())]
            total_bits += 32.0 * arr.size
        total_w += arr.size
        out.append((name, blocks))
        if a.verbose:
            print(f"  {name:60s} {str(list(arr.shape)):20s} {len(blocks)} blocks")
    write_oil(a.output, out, config=b"", write_idx=(fmt != "rawfp32"), shapes=shapes)
    print(f"wrote {a.output}: {len(out)} tensors, {total_w:,} weights, {total_bits / max(1, total_w):.2f} bpw, "
          f"sha256 {file_sha256(a.output)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
