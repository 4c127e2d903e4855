"""Shared helpers of the command-line tools: JSON config files with the documented sections
(``model``, ``training``, ``format``, ``quantization``), dotted overrides, device choice."""
from __future__ import annotations

import json

import torch

from ..models.config import NAMED_CONFIGS, TransformerConfig


def pick_device(arg: str | None) -> torch.device:
    """``auto`` -> the CUDA device named by ``OIL_GPU_DEVICE`` (default 0) when there is one, else
    the CPU; a number -> that CUDA device; anything else is passed to ``torch.device``."""
    if arg in (None, "", "auto"):
        from ..utils import env

        return env.current().default_device()
    if arg.isdigit():
        return torch.device("cuda", int(arg))
    return torch.device(arg)


def runtime_setup(seed_default: int | None = None):
    """Read the documented ``OIL_*`` variables and make them take effect (threads, log level,
    verbose range timing, seed). Returns the settings; ``seed_default`` is the tool's own default
    seed, which ``OIL_SEED`` replaces when it is set."""
    import os

    from ..utils import env

    env.reset()
    rt = env.current()
    if seed_default is not None and "OIL_SEED" not in os.environ:
        rt.seed = seed_default
    return rt.apply()


def load_json_config(path: str | None) -> dict:
    if not path:
        return {}
    with open(path) as f:
        return json.load(f)


def model_config_from(args, cfg_json: dict, vocab_size: int | None = None) -> TransformerConfig:
    preset = getattr(args, "preset", None)
    if preset:
        cfg = NAMED_CONFIGS[preset]()
    else:
        m = dict(cfg_json.get("model", {}))
        cfg = TransformerConfig.from_dict(m) if m else TransformerConfig()
    for attr, field in (("hidden_size", "hidden_size"), ("dim", "hidden_size"), ("num_layers", "num_layers"),
                        ("n_layers", "num_layers"), ("num_heads", "num_heads"), ("ffn_hidden_size", "ffn_hidden_size"),
                        ("seq_length", "max_seq_len"), ("weight_format", "weight_format"),
                        ("block_size", "oil_block_size")):
        v = getattr(args, attr, None)
        if v:
            setattr(cfg, field, v)
    if getattr(args, "hidden_size", None) or getattr(args, "dim", None) or getattr(args, "num_heads", None):
        cfg.head_dim = cfg.hidden_size // cfg.num_heads
        if not getattr(args, "ffn_hidden_size", None):
            cfg.ffn_hidden_size = 4 * cfg.hidden_size
    if vocab_size:
        cfg.vocab_size = vocab_size
    fmt = cfg_json.get("format", {})
    if fmt.get("weight_format"):
        cfg.weight_format = fmt["weight_format"]
    return cfg
