"""All mixture-of-experts variants: shapes, finite outputs, gradients reach the experts, and the
routing invariants that define each variant."""
import pytest
import torch

from mythos_b200.models import moe_variants as mv


def _cfg(**kw):
    base = dict(num_experts=4, top_k=2, expert_hidden_size=32, num_groups=2, experts_per_group=2, top_groups=1,
                num_routed_experts=4, num_shared_layers=2, num_tasks=2,
                modality_experts={"text": 2, "vision": 1, "image_gen": 1, "video_gen": 0, "audio": 1, "ocr": 0,
                                  "cross_modal": 1})
    base.update(kw)
    return mv.MoEAllConfig(**base)


@pytest.mark.parametrize("variant", sorted(mv.VARIANTS))
def test_variant_forward_backward(variant):
    torch.manual_seed(0)
    m = mv.create_moe(variant, 16, _cfg())
    x = torch.randn(2, 6, 16, requires_grad=True)
    if variant == "hash":
        out = m(x, torch.arange(12).view(2, 6))
    else:
        out = m(x)
    assert out.output.shape == x.shape and torch.isfinite(out.output).all()
    loss = out.output.pow(2).mean() + out.load_balance_loss + out.z_loss
    loss.backward()
    grads = [p.grad for p in m.parameters() if p.grad is not None]
    assert grads and all(torch.isfinite(g).all() for g in grads)
    assert x.grad is not None


def test_dispatch_matches_per_token_loop_and_capacity():
    torch.manual_seed(1)
    experts = mv.create_experts(3, 8, 16)
    x = torch.randn(10, 8)
    logits = torch.randn(10, 3)
    idx, w = mv.softmax_with_topk(logits, 2)
    assert torch.allclose(w.sum(1), torch.softmax(logits, -1).topk(2).values.sum(1))   # not renormalised
    y, dropped = mv.moe_dispatch_batched(x, experts, idx, w)
    ref = torch.zeros_like(x)
    for t in range(10):
        for k in range(2):
            ref[t] += w[t, k] * experts[int(idx[t, k])](x[t:t + 1])[0]
    assert dropped == 0 and torch.allclose(y, ref, atol=1e-5)
    _, dropped = mv.moe_dispatch_batched(x, experts, idx, w, capacity=2)
    counts = torch.bincount(idx.reshape(-1), minlength=3)
    assert dropped == int((counts - 2).clamp_min(0).sum())


def test_load_balance_loss_uniform_is_one():
    logits = torch.zeros(8, 4)
    idx = torch.arange(8).view(8, 1) % 4
    assert abs(float(mv.compute_load_balance_loss(logits, idx, 4)) - 1.0) < 1e-6


def test_expert_choice_fills_capacity_and_base_layer_balances():
    torch.manual_seed(2)
    cfg = _cfg(capacity_factor=2.0)
    ec = mv.ExpertChoiceMoE(16, cfg)
    out = ec(torch.randn(1, 8, 16))
    assert out.expert_indices.shape == (4, 4)          # cap = 2 * 8 / 4 tokens per expert
    bl = mv.BaseLayerMoE(16, cfg)
    out = bl(torch.randn(1, 8, 16), training=True)
    assert torch.bincount(out.expert_indices.view(-1), minlength=4).tolist() == [2, 2, 2, 2]


def test_multimodal_hint_selects_modality_experts_and_deepseek_bias_moves():
    torch.manual_seed(3)
    mm = mv.MultiModalMoE(16, _cfg(top_k=1))
    hints = torch.full((1, 5), 1)                      # "vision" owns expert 2
    out = mm(torch.randn(1, 5, 16), hints)
    assert out.expert_indices.view(-1).tolist() == [2] * 5
    ds = mv.DeepSeekMoE(16, _cfg())
    before = ds.route_bias.clone()
    ds(torch.randn(2, 16, 16), training=True)
    assert not torch.equal(before, ds.route_bias)
    ds(torch.randn(2, 16, 16), training=False)


def test_quantised_variants_use_quantised_weights():
    torch.manual_seed(4)
    m = mv.create_moe("ternary", 16, _cfg())
    w = m.experts[0].up
    q = m.experts[0]._w(w)
    assert q.unique().numel() <= 3 * (w.numel() // min(256, w.numel())) + 3
    b = mv.create_moe("binary", 16, _cfg())
    qb = b.experts[0]._w(b.experts[0].down)
    assert all(r.abs().unique().numel() == 1 for r in qb)
