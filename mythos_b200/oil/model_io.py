"""Saving and loading models as ``.oil`` files.

Unlike the reference's ``DenseModel::save`` (always FP32 blocks, src/model.cpp:106-163), a model
is written *in its formats*: an ``OILLinear`` in OIL8/OIL4 becomes codebook + index blocks, I2_S
becomes {-s, 0, +s} + 2-bit codes, everything else FP32 blocks of at most 32768 weights (the
reference's chunking). One file block holds the weights that share one codebook
(``block_size * codebook_group`` weights) or, for I2_S, one scale.

Tensor names are the reference's where a one-to-one tensor exists (``tok_embeddings.weight``,
``layers.N.attention_norm.weight``, ``norm.weight``, ``lm_head.weight``, ...). Fused projections
are stored under ``attention.qkv_proj.weight`` / ``ffn.up_proj.weight`` (q|k|v and gate|up rows
concatenated); files written by the reference with separate ``q_proj``/``k_proj``/``v_proj`` and
``gate_proj``/``up_proj`` tensors are fused on load. Shapes and the quantisation layout travel in
the JSON tail of the config area and in the version-2 sidecar.

A save -> load -> save cycle reproduces the file byte for byte (and therefore its SHA-256):
loading restores weights to exact centroid values and the codebooks themselves, and the
quantisers are idempotent on already-quantised data.
"""
from __future__ import annotations

import struct

import numpy as np
import torch

from ..models.config import TransformerConfig
from . import codebook as cbk
from .container import BlockData, OILReader, file_sha256, write_oil
from .formats import Format, pack_nibbles, pack_trits

FP32_CHUNK = 32768


def _fp32_blocks(arr: np.ndarray) -> list[BlockData]:
    flat = np.ascontiguousarray(arr, dtype="<f4").reshape(-1)
    return [BlockData(Format.FP32, int(min(FP32_CHUNK, flat.size - o)), b"", flat[o:o + FP32_CHUNK].tobytes())
            for o in range(0, max(flat.size, 1), FP32_CHUNK) if flat.size]


def _i2s_quantize_idempotent(w: np.ndarray, bs: int):
    """Per-block (codes, scale). A block whose values already are {-s, 0, +s} keeps s."""
    n = w.size
    nb = (n + bs - 1) // bs
    pad = nb * bs - n
    wf = np.pad(w.astype(np.float32), (0, pad)).reshape(nb, bs)
    cnt = np.full(nb, bs, dtype=np.float32)
    if pad:
        cnt[-1] = bs - pad
    a = np.abs(wf)
    amax = a.max(axis=1)
    exact = np.all((a == 0) | (a == amax[:, None]), axis=1)
    scale = np.where(exact, amax, a.sum(axis=1) / cnt).astype(np.float32)
    inv = np.where(scale > 0, 1.0 / np.where(scale > 0, scale, 1), 0).astype(np.float32)
    t = np.clip(np.rint(wf * inv[:, None]), -1, 1).astype(np.int8)
    return (t + 1).astype(np.uint8), scale, cnt.astype(np.int64)


def linear_blocks(mod) -> list[BlockData]:
    """File blocks of one ``OILLinear`` in its own format."""
    w = mod.weight.detach().float().cpu()
    flat = w.reshape(-1)
    n = flat.numel()
    if mod.fmt == "i2s":
        codes, scale, cnt = _i2s_quantize_idempotent(flat.numpy(), mod.block_size)
        out = []
        for b in range(codes.shape[0]):
            k = int(cnt[b])
            s = np.float32(scale[b])
            out.append(BlockData(Format.TERNARY, k, np.array([-s, 0.0, s], dtype="<f4").tobytes(),
                                 pack_trits(codes[b, :k])))
        return out
    if mod.fmt == "mixed":
        from ..ops import reference as ref

        bs = mod.block_size
        cmap = mod.cb_map.detach().cpu()
        cb8, cb4 = mod.codebooks.detach().float().cpu(), mod.codebooks4.detach().float().cpu()
        idx8, _ = ref.nearest_centroid(flat, cb8, cmap, bs)
        idx4, _ = ref.nearest_centroid(flat, cb4, cmap, bs)
        codes, scale, cnt = _i2s_quantize_idempotent(flat.numpy(), bs)
        idx8, idx4 = idx8.numpy(), idx4.numpy()
        fm = mod.block_formats.detach().cpu().numpy()
        out = []
        for b, o in enumerate(range(0, n, bs)):
            k = min(bs, n - o)
            u = int(cmap[b])
            if fm[b] == int(Format.OIL8):
                out.append(BlockData(Format.OIL8, k, cbk.serialize_oil8(cb8[u]), idx8[o:o + k].tobytes()))
            elif fm[b] == int(Format.OIL4):
                out.append(BlockData(Format.OIL4, k, cbk.serialize_oil4(cb4[u]), pack_nibbles(idx4[o:o + k])))
            elif fm[b] == int(Format.BINARY):
                seg = flat[o:o + k].numpy()
                a = np.abs(seg)
                # a block that already holds {-s, +s} keeps s (the mean of |w| is then s itself)
                sc = np.float32(0) if not k else (a.max() if np.all(a == a.max()) else np.float32(a.mean()))
                bits = (seg > 0).astype(np.uint8)
                out.append(BlockData(Format.BINARY, k, np.array([-sc, sc], dtype="<f4").tobytes(),
                                     np.packbits(bits, bitorder="little").tobytes()))
            else:
                sc = np.float32(scale[b])
                out.append(BlockData(Format.TERNARY, k, np.array([-sc, 0.0, sc], dtype="<f4").tobytes(),
                                     pack_trits(codes[b, :k])))
        return out
    if mod.fmt in ("oil8", "oil4"):
        from ..ops import reference as ref

        cbs = mod.codebooks.detach().float().cpu()
        cmap = None if mod.cb_map is None else mod.cb_map.detach().cpu()
        idx, _ = ref.nearest_centroid(flat, cbs, cmap, mod.block_size)
        idx = idx.numpy()
        unit = mod.block_size * mod.codebook_group
        out = []
        for u, o in enumerate(range(0, n, unit)):
            k = min(unit, n - o)
            cb = cbs[u]
            if mod.fmt == "oil8":
                out.append(BlockData(Format.OIL8, k, cbk.serialize_oil8(cb), idx[o:o + k].tobytes()))
            else:
                out.append(BlockData(Format.OIL4, k, cbk.serialize_oil4(cb), pack_nibbles(idx[o:o + k])))
        return out
    if mod.fmt == "fp16":
        arr = flat.numpy().astype("<f2")
        return [BlockData(Format.FP16, int(min(FP32_CHUNK, arr.size - o)), b"", arr[o:o + FP32_CHUNK].tobytes())
                for o in range(0, arr.size, FP32_CHUNK)]
    return _fp32_blocks(flat.numpy())


def save_model(model, path: str, write_idx: bool = True) -> str:
    """Writes ``path`` (and its ``.oilidx`` sidecar). Returns the file's SHA-256 hex digest."""
    cfg: TransformerConfig = model.cfg
    tensors, shapes = [], {}
    for name, p, mod in model.export_named_tensors():
        shapes[name] = list(p.shape)
        if mod is not None:
            tensors.append((name, linear_blocks(mod)))
        else:
            tensors.append((name, _fp32_blocks(p.detach().float().cpu().numpy())))
    cfg.extras = dict(cfg.extras or {})
    cfg.extras["shapes"] = shapes
    cfg.extras["fused"] = True
    write_oil(path, tensors, config=cfg.to_bytes(extended=True), version=1, flags=0, write_idx=write_idx,
              idx_version=2, shapes=shapes)
    return file_sha256(path)


def _assign_linear(mod, rd: OILReader, name: str, reference_layout: bool = False) -> None:
    blocks = rd.read_tensor_blocks(name)
    vals = torch.from_numpy(rd.read_tensor(name).copy())
    if reference_layout:
        # the reference multiplies activations by the stored bytes read as [in, out] row-major
        # (src/autograd.cpp:27-30): transpose into this framework's [out, in]
        vals = vals.view(mod.in_features, mod.out_features).t().contiguous()
    mod.weight.data.copy_(vals.view(mod.weight.shape))
    if mod.fmt == "mixed" and len(blocks) == mod.n_blocks:
        # the file decides the format of every block; codebooks of the OIL8 / OIL4 blocks come with it
        fm = torch.tensor([int(b.format) for b in blocks], dtype=torch.uint8)
        mod.block_formats.copy_(fm)
        for u, b in enumerate(blocks):
            if not b.codebook or b.format not in (Format.OIL8, Format.OIL4):
                continue
            _, c = cbk.deserialize(b.codebook)
            row = int(mod.cb_map[u])
            (mod.codebooks if b.format == Format.OIL8 else mod.codebooks4)[row].copy_(torch.from_numpy(c.copy()))
        return
    if mod.fmt in ("oil8", "oil4") and mod.codebooks is not None:
        for u, b in enumerate(blocks):
            if u < mod.codebooks.shape[0] and b.format in (Format.OIL8, Format.OIL4) and b.codebook:
                _, c = cbk.deserialize(b.codebook)
                mod.codebooks[u].copy_(torch.from_numpy(c.copy()))


def load_model(path: str, device="cpu", model_cls=None):
    """Returns ``(model, reader)``. Accepts files written by :func:`save_model` and files written by
    the reference's ``DenseModel::save`` (FP32 blocks, separate q/k/v and gate/up tensors)."""
    from ..models.dense import DenseModel
    from ..models.layers import OILLinear

    rd = OILReader(path)
    if len(rd.config) < 88:
        raise ValueError(f"{path}: no model configuration in the header (config_size={len(rd.config)})")
    cfg = TransformerConfig.from_bytes(rd.config)
    cls = model_cls or DenseModel
    if cfg.num_experts > 0 and model_cls is None:
        from ..models.moe import MoEModel

        cls = MoEModel
    model = cls(cfg)
    names = set(rd.tensor_names())
    reference_layout = "fused" not in (cfg.extras or {})  # no JSON tail: written by the reference
    with torch.no_grad():
        for name, p, mod in model.export_named_tensors():
            if name in names:
                if isinstance(mod, OILLinear):
                    _assign_linear(mod, rd, name, reference_layout)
                else:
                    v = rd.read_tensor(name)
                    if v.size == p.numel():
                        p.data.copy_(torch.from_numpy(v.copy()).view(p.shape))
                continue
            # reference layout: separate projections -> fused rows
            parts = None
            if name.endswith("attention.qkv_proj.weight"):
                base = name[: -len("qkv_proj.weight")]
                parts = [base + "q_proj.weight", base + "k_proj.weight", base + "v_proj.weight"]
            elif name.endswith("ffn.up_proj.weight") and cfg.gated_ffn:
                base = name[: -len("up_proj.weight")]
                parts = [base + "gate_proj.weight", base + "up_proj.weight"]
            if parts and all(q in names for q in parts):
                # the reference multiplies activations by the stored bytes read as [in, out]
                # (src/autograd.cpp:27-30), so each stored tensor is transposed into [out, in]
                rows = []
                K = p.shape[1]
                for q in parts:
                    v = rd.read_tensor(q)
                    rows.append(torch.from_numpy(v.copy()).view(K, -1).t())
                fused = torch.cat(rows, dim=0)
                if fused.shape == p.shape:
                    p.data.copy_(fused)
    return model.to(device), rd
