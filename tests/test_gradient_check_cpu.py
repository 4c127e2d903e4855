"""Finite-difference gradient checks of the CPU (reference-op) training path: parameters of every
kind in a tiny dense model, and the cross-entropy gradient against its closed form."""
import pytest
import torch

from mythos_b200.models import DenseModel, TransformerConfig
from mythos_b200.ops import reference as ref


def _tiny(fmt="fp32"):
    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=48, hidden_size=32, num_layers=2, num_heads=2, head_dim=16, num_kv_heads=1,
                            ffn_hidden_size=64, max_seq_len=16, weight_format=fmt, oil_block_size=32)
    return cfg, DenseModel(cfg)


def test_finite_differences_match_autograd_on_every_parameter_kind():
    cfg, model = _tiny()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (2, 12), generator=g, dtype=torch.int32)
    tgt = torch.randint(0, cfg.vocab_size, (2, 12), generator=g, dtype=torch.int32)
    loss = model(ids, tgt)
    loss.backward()
    probes = 0
    for name, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
        if not any(k in name for k in ("lm_head", "tok_embeddings", "qkv_proj", "o_proj", "up_proj", "down_proj", "norm")):
            continue
        flat, gflat = p.data.view(-1), p.grad.view(-1)
        idx = [int(gflat.abs().argmax())] + torch.randint(0, flat.numel(), (2,), generator=g).tolist()
        for i in idx:
            keep = float(flat[i])
            eps = 4e-3                  # the reference ops accumulate in fp32: the loss carries ~1e-6 of noise
            with torch.no_grad():
                flat[i] = keep + eps
                up = float(model(ids, tgt))
                flat[i] = keep - eps
                dn = float(model(ids, tgt))
                flat[i] = keep
            fd = (up - dn) / (2 * eps)
            an = float(gflat[i])
            assert abs(fd - an) <= 1e-3 + 3e-2 * max(abs(fd), abs(an)), (name, i, fd, an)
            probes += 1
    assert probes >= 3 * 8


def test_cross_entropy_gradient_closed_form():
    torch.manual_seed(2)
    rows, V = 7, 19
    logits = torch.randn(rows, V, requires_grad=True)
    tg = torch.randint(-2, V + 2, (rows,), dtype=torch.int32)          # out-of-range targets are clamped
    loss = ref.cross_entropy(logits, tg).sum() / rows
    loss.backward()
    p = torch.softmax(logits.detach(), dim=-1)
    onehot = torch.zeros_like(p)
    onehot[torch.arange(rows), tg.long().clamp(0, V - 1)] = 1.0
    assert torch.allclose(logits.grad, (p - onehot) / rows, atol=1e-6)
    assert torch.allclose(ref.cross_entropy_grad(logits.detach(), tg, 1.0 / rows), (p - onehot) / rows, atol=1e-6)


def test_ste_passes_gradients_straight_through():
    """With OIL8 fake-quantisation in the forward pass the weight gradient equals the gradient with
    respect to the quantised weight (identity backward), so it is finite and non-zero everywhere the
    fp32 model's is."""
    cfg, model = _tiny("oil8")
    ids = torch.randint(0, cfg.vocab_size, (2, 12), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    model(ids, ids).backward()
    for name, p in model.named_parameters():
        if name.endswith("proj.weight"):
            assert torch.isfinite(p.grad).all() and float(p.grad.abs().sum()) > 0, name


def test_activation_checkpointing_gives_the_same_gradients():
    """Blocks recomputed in the backward pass produce the gradients of the stored-activation run."""
    from mythos_b200.models import DenseModel, TransformerConfig

    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=3, num_heads=2, head_dim=16, ffn_hidden_size=64,
                            max_seq_len=16, oil_block_size=32)
    torch.manual_seed(0)
    model = DenseModel(cfg).train()
    ids = torch.randint(0, 64, (2, 16), dtype=torch.int32)
    tg = torch.randint(0, 64, (2, 16), dtype=torch.int32)
    grads = []
    for ckpt in (False, True):
        model.activation_checkpointing = ckpt
        model.zero_grad()
        loss = model(ids, tg)
        loss.backward()
        grads.append((float(loss), [p.grad.clone() for p in model.parameters()]))
    assert grads[0][0] == grads[1][0]
    for a, b in zip(grads[0][1], grads[1][1]):
        assert torch.allclose(a, b, atol=1e-7)
