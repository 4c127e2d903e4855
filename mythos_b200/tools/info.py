"""oil-info: describe a ``.oil`` file (header, architecture, tensors with formats, average bits per
weight, per-format share, codebook bytes). ``oil-info <model.oil>`` as in the reference
(tools/info.cpp); ``--json`` and ``--verify`` (check the sidecar digests) are additions."""
from __future__ import annotations

import argparse
import json
import sys
from collections import Counter


def describe(path: str) -> dict:
    from ..models.config import TransformerConfig
    from ..oil.container import OILReader
    from ..oil.formats import FORMAT_BPW, FORMAT_TO_NAME, Format

    rd = OILReader(path)
    info = {"path": path, "version": rd.version, "flags": rd.flags, "config_size": rd.config_size,
            "num_blocks": rd.num_blocks, "num_tensors": len(rd.tensor_order)}
    shapes = {}
    if rd.config_size >= 88:
        cfg = TransformerConfig.from_bytes(rd.config)
        info["architecture"] = {k: getattr(cfg, k) for k in (
            "vocab_size", "hidden_size", "num_layers", "num_heads", "head_dim", "ffn_hidden_size", "num_kv_heads",
            "max_seq_len", "activation", "weight_format", "oil_block_size", "num_experts")}
        shapes = (cfg.extras or {}).get("shapes", {})
    by_fmt, bits, weights, cb_bytes = Counter(), 0.0, 0, int(rd.block_cb_bytes.sum())
    tensors = []
    for name in rd.tensor_order:
        e = rd.tensors[name]
        n = int(rd.block_weights[e.block_start:e.block_start + e.num_blocks].sum())
        fmts = Counter(int(f) for f in rd.block_formats[e.block_start:e.block_start + e.num_blocks])
        for b in range(e.block_start, e.block_start + e.num_blocks):
            f = Format(int(rd.block_formats[b])) if rd.block_formats[b] <= 5 else Format.FP32
            by_fmt[FORMAT_TO_NAME[f]] += int(rd.block_weights[b])
            bits += FORMAT_BPW[f] * int(rd.block_weights[b])
        weights += n
        tensors.append({"name": name, "params": n, "shape": shapes.get(name),
                        "formats": {FORMAT_TO_NAME[Format(k)] if k <= 5 else "fp32": v for k, v in fmts.items()},
                        "blocks": e.num_blocks})
    info.update({"params": weights, "avg_bpw": bits / max(1, weights), "codebook_bytes": cb_bytes,
                 "format_share": {k: v / max(1, weights) for k, v in by_fmt.items()}, "tensors": tensors,
                 "file_bytes": int(rd.block_offsets[-1])})
    return info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="oil-info", description=__doc__)
    ap.add_argument("model_pos", nargs="?")
    ap.add_argument("--model", "-m", default=None)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    path = a.model or a.model_pos
    if not path:
        ap.print_usage(sys.stderr)
        return 2
    info = describe(path)
    if a.verify:
        from ..oil.container import verify

        info["verified_tensors"] = len(verify(path))
    if a.json:
        print(json.dumps(info, indent=2))
        return 0
    print(f"{path}: OIL1 v{info['version']} flags {info['flags']} config {info['config_size']} B, "
          f"{info['num_tensors']} tensors, {info['num_blocks']} blocks, {info['params']:,} weights")
    if "architecture" in info:
        print("architecture:", ", ".join(f"{k}={v}" for k, v in info["architecture"].items()))
    print(f"average {info['avg_bpw']:.2f} bits/weight; codebooks {info['codebook_bytes']:,} B; share: " +
          ", ".join(f"{k} {100 * v:.1f}%" for k, v in sorted(info["format_share"].items())))
    for t in info["tensors"]:
        print(f"  {t['name']:56s} {t['params']:>12,} {str(t['shape'] or ''):18s} "
              + ",".join(f"{k}x{v}" for k, v in t["formats"].items()))
    if a.verify:
        print(f"sidecar digests verified for {info['verified_tensors']} tensors")
    return 0


if __name__ == "__main__":
    sys.exit(main())
