"""Training add-ons: weight EMA over the flat master buffer, label-smoothing and R-Drop losses,
the fine-tuner's block selection and in-format update, and the second ("dense") trainer with its
own checkpoint container.

Reference counterparts: ``Trainer`` EMA init/step/apply/swap, ``label_smoothing_loss``,
``rdrop_loss`` (src/trainer.cpp:403-855, include/oil/trainer.h:20-295); ``FineTuner``
``find_trainable_blocks`` (256-weight blocks ranked by RMS gradient) and ``apply_oil_update``
(dequantise -> SGD -> re-quantise) (src/finetune.cpp); ``dense::DenseTrainer`` with chunk-level
shuffling and "CHPK" checkpoints (magic 0x4B504843, v2: step, lr, parameters, then Adam m / v, each
tensor as i32 rank, i64 dims, u8 dtype, raw data; engines/trainer/dense/checkpoint.cpp:53-171).
The reference fine-tuner computes its loss outside the autograd tape, so no gradient ever reaches
its weights (src/finetune.cpp:71-75); here the loss is the model's own fused cross-entropy.
"""
from __future__ import annotations

import struct

import numpy as np
import torch
import torch.nn.functional as tF

from ..ops import reference as ref


class WeightEMA:
    """Exponential moving average of all trainable weights, kept as one flat fp32 buffer next to
    the trainer's master buffer. ``swap`` exchanges live and averaged weights (evaluate with the
    average, swap back to continue training)."""

    def __init__(self, trainer, decay: float = 0.999):
        self.trainer, self.decay = trainer, decay
        self.shadow = trainer.store.master.detach().clone()
        self.steps = 0

    @torch.no_grad()
    def step(self) -> None:
        self.steps += 1
        d = min(self.decay, (1.0 + self.steps) / (10.0 + self.steps))     # warm-up of the average
        self.shadow.mul_(d).add_(self.trainer.store.master, alpha=1.0 - d)

    @torch.no_grad()
    def apply(self) -> None:
        self.trainer.store.master.copy_(self.shadow)
        self.trainer._stale = True

    @torch.no_grad()
    def swap(self) -> None:
        m = self.trainer.store.master
        tmp = m.clone()
        m.copy_(self.shadow)
        self.shadow.copy_(tmp)
        self.trainer._stale = True


def label_smoothing_loss(logits: torch.Tensor, targets: torch.Tensor, smoothing: float = 0.1) -> torch.Tensor:
    """``(1 - eps) * NLL + eps * mean over the vocabulary of -log p``."""
    logp = torch.log_softmax(logits.float(), dim=-1).reshape(-1, logits.shape[-1])
    nll = -logp.gather(1, targets.reshape(-1, 1).long()).squeeze(1)
    return ((1.0 - smoothing) * nll - smoothing * logp.mean(dim=-1)).mean()


def rdrop_loss(logits_a: torch.Tensor, logits_b: torch.Tensor, targets: torch.Tensor, alpha: float = 1.0):
    """Mean CE of two stochastic passes plus ``alpha`` times their symmetric KL."""
    V = logits_a.shape[-1]
    a, b = logits_a.float().reshape(-1, V), logits_b.float().reshape(-1, V)
    t = targets.reshape(-1).long()
    ce = 0.5 * (tF.cross_entropy(a, t) + tF.cross_entropy(b, t))
    la, lb = torch.log_softmax(a, -1), torch.log_softmax(b, -1)
    kl = 0.5 * (tF.kl_div(la, lb, log_target=True, reduction="batchmean")
                + tF.kl_div(lb, la, log_target=True, reduction="batchmean"))
    return ce + alpha * kl


# --------------------------------------------------------------------------- fine-tuner helpers


def find_trainable_blocks(grad: torch.Tensor, block_size: int = 256, fraction: float = 0.1) -> torch.Tensor:
    """Indices of the blocks (``block_size`` consecutive weights) with the largest RMS gradient."""
    g = grad.detach().float().reshape(-1)
    n = g.numel() // block_size
    rms = g[: n * block_size].view(n, block_size).pow(2).mean(dim=1).sqrt()
    k = max(1, int(round(n * fraction)))
    return torch.topk(rms, k).indices.sort().values


@torch.no_grad()
def apply_oil_update(module, grad: torch.Tensor, lr: float, blocks: torch.Tensor | None = None) -> None:
    """One in-format SGD step on an ``OILLinear``: the stored weight is what dequantisation yields,
    the step is applied in fp32 (to the selected blocks only, if given) and the result is snapped
    back onto the module's codebooks / ternary grid, so the model stays exactly representable."""
    w = module.weight
    flat = w.data.reshape(-1)
    upd = grad.reshape(-1).to(flat.dtype) * lr
    if blocks is not None:
        mask = torch.zeros(flat.numel() // module.block_size, dtype=torch.bool, device=flat.device)
        mask[blocks.to(flat.device)] = True
        upd = upd * mask.repeat_interleave(module.block_size)[: upd.numel()]
    flat.sub_(upd)
    if module.fmt in ("oil8", "oil4") and module.codebooks is not None:
        _, deq = ref.nearest_centroid(flat.float(), module.codebooks.float(), module.cb_map, module.block_size)
        flat.copy_(deq.to(flat.dtype))
    elif module.fmt == "i2s":
        _, _, deq = ref.i2s_quant(flat.float(), module.block_size)
        flat.copy_(deq.to(flat.dtype))


# --------------------------------------------------------------------------- CHPK checkpoints

CHPK_MAGIC, CHPK_VERSION = 0x4B504843, 2


def _write_record(f, name: str, t: torch.Tensor) -> None:
    """``u32 name_len, name, u32 size, Tensor::serialize bytes`` (checkpoint.cpp:14-29)."""
    from ..core import serialize_tensor

    if t.dtype in (torch.int32, torch.int16, torch.int8):
        t = t.long()
    body = serialize_tensor(t)
    if len(body) > 0xFFFFFFFF:
        raise ValueError("tensor too large for the checkpoint format (> 4 GB)")
    raw = name.encode()
    f.write(struct.pack("<I", len(raw)) + raw + struct.pack("<I", len(body)) + body)


def _read_record(f, expected: str) -> torch.Tensor:
    from ..core import OilError, deserialize_tensor

    head = f.read(4)
    if len(head) != 4:
        raise ValueError("corrupt checkpoint: name length")
    (n,) = struct.unpack("<I", head)
    name = f.read(n)
    size = f.read(4)
    if len(name) != n or len(size) != 4:
        raise ValueError("corrupt checkpoint: tensor size")
    if name.decode(errors="replace") != expected:
        raise ValueError(f"checkpoint record {name!r} where {expected!r} was expected")
    (nbytes,) = struct.unpack("<I", size)
    body = f.read(nbytes)
    if len(body) != nbytes:
        raise ValueError("corrupt checkpoint: tensor data")
    try:
        return deserialize_tensor(body)[0]
    except OilError as e:
        raise ValueError(f"corrupt checkpoint: {e}") from None


def save_chpk(path: str, step: int, lr: float, params, m=None, v=None) -> None:
    """The reference's dense-trainer checkpoint, byte for byte (engines/trainer/dense/
    checkpoint.cpp:53-103): u32 magic "CHPK", u32 version 2, u32 step, f32 lr, u32 count, records
    ``param_i``; u32 count, then per index the records ``m_i`` and ``v_i`` (zeros when the optimizer
    has no state yet)."""
    params = list(params)
    if not 0 <= step <= 0xFFFFFFFF:
        raise ValueError("checkpoint: step exceeds the uint32 range")
    m = list(m) if m is not None else [torch.zeros_like(p, dtype=torch.float32) for p in params]
    v = list(v) if v is not None else [torch.zeros_like(p, dtype=torch.float32) for p in params]
    with open(path, "wb") as f:
        f.write(struct.pack("<IIIfI", CHPK_MAGIC, CHPK_VERSION, step, lr, len(params)))
        for i, p in enumerate(params):
            _write_record(f, f"param_{i}", p)
        f.write(struct.pack("<I", len(params)))
        for i in range(len(params)):
            _write_record(f, f"m_{i}", m[i])
            _write_record(f, f"v_{i}", v[i])


def load_chpk(path: str):
    with open(path, "rb") as f:
        head = f.read(20)
        if len(head) != 20:
            raise ValueError(f"{path}: truncated checkpoint header")
        magic, version, step, lr, n = struct.unpack("<IIIfI", head)
        if magic != CHPK_MAGIC:
            raise ValueError(f"{path}: not a CHPK checkpoint")
        if version > CHPK_VERSION:
            raise ValueError(f"{path}: checkpoint version {version} is newer than {CHPK_VERSION}")
        params = [_read_record(f, f"param_{i}") for i in range(n)]
        m = v = None
        if version >= 2:
            cnt = f.read(4)
            if len(cnt) == 4:
                (num_opt,) = struct.unpack("<I", cnt)
                m, v = [], []
                for i in range(num_opt):
                    m.append(_read_record(f, f"m_{i}"))
                    v.append(_read_record(f, f"v_{i}"))
    return {"step": step, "lr": lr, "params": params, "m": m, "v": v}


class ChunkLoader:
    """Contiguous [B, S] windows with next-token targets; ``shuffle`` permutes whole windows
    (chunk-level, unlike the other loader of the reference, which shuffles single tokens)."""

    def __init__(self, tokens, batch_size: int, seq_length: int, seed: int = 42):
        self.tokens = np.asarray(tokens, dtype=np.int32)
        self.B, self.S, self.seed = batch_size, seq_length, seed
        self.n_chunks = (len(self.tokens) - 1) // seq_length
        self.order = np.arange(self.n_chunks)

    def shuffle(self, epoch: int) -> None:
        self.order = np.random.default_rng(self.seed + epoch).permutation(self.n_chunks)

    def __len__(self):
        return self.n_chunks // self.B

    def __iter__(self):
        for b in range(len(self)):
            idx = self.order[b * self.B:(b + 1) * self.B]
            x = np.stack([self.tokens[i * self.S:(i + 1) * self.S] for i in idx])
            y = np.stack([self.tokens[i * self.S + 1:(i + 1) * self.S + 1] for i in idx])
            yield torch.from_numpy(x), torch.from_numpy(y)


class DenseTrainer:
    """The simpler second trainer: own loader, ``train_step``, ``fit`` with ``<path>.step<N>``
    checkpoints in the CHPK container. It drives the same fused step as :class:`Trainer`."""

    def __init__(self, model, lr: float = 3e-4, batch_size: int = 8, seq_length: int = 128, max_grad_norm: float = 1.0,
                 weight_decay: float = 0.01, device=None, save_interval: int = 0, save_path: str = "dense.chpk"):
        from .trainer import TrainConfig, Trainer

        cfg = TrainConfig(batch_size=batch_size, seq_length=seq_length, lr=lr, max_grad_norm=max_grad_norm,
                          weight_decay=weight_decay, schedule="constant", warmup_steps=0, codebook_ema_interval=0)
        self.inner = Trainer(model, cfg, device=device)
        self.model, self.lr = model, lr
        self.save_interval, self.save_path = save_interval, save_path

    @property
    def step(self) -> int:
        return self.inner.step

    def train_step(self, ids, targets) -> float:
        return float(self.inner.train_step(ids, targets))

    def fit(self, loader: ChunkLoader, epochs: int = 1, max_steps: int | None = None) -> list[float]:
        losses = []
        for ep in range(epochs):
            loader.shuffle(ep)
            for x, y in loader:
                losses.append(self.train_step(x, y))
                if self.save_interval and self.step % self.save_interval == 0:
                    self.save_checkpoint(f"{self.save_path}.step{self.step}")
                if max_steps is not None and self.step >= max_steps:
                    return losses
        return losses

    def _slots(self):
        st = self.inner.store
        return [(s, st.master[s.offset:s.offset + s.numel].view(s.param.shape)) for s in st.slots]

    def save_checkpoint(self, path: str) -> None:
        st, tr = self.inner.store, self.inner
        params = [p for _, p in self._slots()]
        m = [tr.m[s.offset:s.offset + s.numel].view(s.param.shape) for s in st.slots]
        v = [tr.v[s.offset:s.offset + s.numel].view(s.param.shape) for s in st.slots]
        save_chpk(path, tr.step, self.lr, params, m, v)

    def load_checkpoint(self, path: str) -> None:
        ck = load_chpk(path)
        st, tr = self.inner.store, self.inner
        if len(ck["params"]) != len(st.slots):
            raise ValueError("checkpoint does not match the model (parameter count)")
        with torch.no_grad():
            for i, s in enumerate(st.slots):
                st.master[s.offset:s.offset + s.numel].copy_(ck["params"][i].reshape(-1).to(st.master.device))
                if ck["m"] is not None:
                    tr.m[s.offset:s.offset + s.numel].copy_(ck["m"][i].reshape(-1).to(tr.m.device))
                    tr.v[s.offset:s.offset + s.numel].copy_(ck["v"][i].reshape(-1).to(tr.v.device))
        tr.step, self.lr = int(ck["step"]), float(ck["lr"])
        tr._stale = True
