"""Mixture-of-modalities block, modality encoders and MoE utilities on CPU."""
import torch

from mythos_b200.models import encoders as enc
from mythos_b200.models import moe_enhance as me
from mythos_b200.models.config import TransformerConfig
from mythos_b200.models.mom import MODALITY_NAMES, MoMBlock, MoMConfig, MoMRouter


def test_router_modality_bias_and_losses():
    torch.manual_seed(0)
    cfg = MoMConfig(num_experts=16, top_k=3)
    r = MoMRouter(32, cfg)
    x = torch.randn(2, 5, 32)
    hints = torch.full((2, 5), MODALITY_NAMES.index("AUDIO"))
    out = r(x, hints)
    audio_experts = (r.expert_modality == MODALITY_NAMES.index("AUDIO")).nonzero().view(-1).tolist()
    assert out.indices.shape == (10, 3)
    # the +10 bias puts both audio experts into every token's top-3
    assert all(set(audio_experts) <= set(row) for row in out.indices.tolist())
    assert out.dominant_modality == MODALITY_NAMES.index("AUDIO")
    assert float(out.load_balance_loss.detach()) > 0 and float(out.z_loss.detach()) > 0
    free = r(x)
    assert torch.allclose(free.gates.sum(-1), torch.ones(10), atol=1e-5)


def test_mom_block_forward_backward_with_context():
    torch.manual_seed(1)
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, head_dim=16, ffn_hidden_size=48,
                            weight_format="fp32")
    blk = MoMBlock(cfg, MoMConfig(num_experts=16, top_k=3, expert_hidden_size=24))
    x = torch.randn(2, 6, 32, requires_grad=True)
    ctx = torch.randn(2, 4, 32)
    y = blk(x, context=ctx)
    assert y.shape == x.shape and torch.isfinite(y).all()
    (y.pow(2).mean() + blk.aux_loss()).backward()
    assert x.grad is not None and blk.router.gate.weight.grad is not None
    assert any(e.up.grad is not None for e in blk.moe.experts)


def test_encoders_shapes_and_gradients():
    torch.manual_seed(2)
    vit = enc.VisionEncoder(img_size=32, patch_size=8, hidden=32, layers=2, heads=2)
    img = torch.randn(2, 3, 32, 32)
    f = vit(img)
    assert f.shape == (2, 17, 32)
    assert vit.forward_video(torch.randn(1, 3, 3, 32, 32)).shape == (1, 3, 17, 32)
    det = enc.ObjectDetector(hidden=32, heads=2, num_queries=5, num_classes=7, layers=1)(f)
    assert det["logits"].shape == (2, 5, 8) and det["boxes"].min() >= 0 and det["boxes"].max() <= 1
    sg = enc.SceneGraphEncoder(hidden=32, num_relations=6)(det["features"])
    assert sg.shape == (2, 5, 5, 6)
    assert enc.AudioEncoder(n_mels=16, hidden=32, layers=1, heads=2, max_pos=8)(torch.randn(2, 16, 12)).shape == (2, 12, 32)
    assert enc.OCREncoder(hidden=32, layers=1, heads=2, patch_size=16)(torch.randn(1, 3, 32, 48)).shape == (1, 6, 32)
    assert enc.VideoEncoder(tube_size=2, img_size=16, patch_size=8, hidden=32, layers=1, heads=2)(
        torch.randn(1, 4, 3, 16, 16)).shape == (1, 8, 32)
    te = enc.TextEncoder(vocab=50, hidden=32, layers=1, heads=2)
    t = te(torch.randint(0, 50, (2, 7)))
    emb = enc.SentenceEmbedder(32, 8)(t)
    assert emb.shape == (2, 8) and torch.allclose(emb.norm(dim=-1), torch.ones(2), atol=1e-5)
    emb.sum().backward()
    assert te.embed.weight.grad is not None


def test_patchify_layout_and_sinusoids():
    img = torch.arange(2 * 3 * 4 * 4, dtype=torch.float32).view(2, 3, 4, 4)
    p = enc.patchify(img, 2)
    assert p.shape == (2, 4, 12)
    # patch 1 (row 0, col 1), channel 2, pixel (1, 0)
    assert float(p[0, 1, 2 * 4 + 1 * 2 + 0]) == float(img[0, 2, 1, 2])
    pe = enc.sinusoidal_positions(5, 8)
    assert torch.allclose(pe[0, 0::2], torch.zeros(4)) and torch.allclose(pe[0, 1::2], torch.ones(4))


def test_moe_utilities(tmp_path):
    caps = me.adaptive_capacity(4, 100, [1, 1, 2, 0])
    assert caps[2] > caps[0] and caps[3] == 1 and sum(caps) >= 100
    g, u, d = torch.randn(12, 8), torch.randn(12, 8), torch.randn(8, 12)
    ex = me.DenseToMoEPruner(8, 3, sparsity=0.25).prune_ffn(g, u, d)
    units = torch.cat([e["units"] for e in ex])
    assert len(ex) == 3 and units.numel() == 9 and units.unique().numel() == 9
    ts = [torch.randn(3, 4), torch.arange(6, dtype=torch.int32).view(2, 3), torch.randn(5).half()]
    path = str(tmp_path / "experts.bin")
    me.save_experts(ts, path)
    back = me.load_experts(path)
    assert back[0].dtype == torch.float32 and back[2].dtype == torch.float16 and back[1].dtype == torch.int64
    assert all(torch.equal(a.to(b.dtype), b) for a, b in zip(ts, back))
    raw = open(path, "rb").read()
    assert raw[4 + 4 + 16] == 6          # float32 carries the reference's DType number
    drop = me.ExpertDropout(0.25)
    assert drop.get_active_count(8) == 6 and sum(drop.get_mask(8)) == 6
    bal = me.compute_balance([0, 1, 2, 3, 0, 1, 2, 3], 4)
    assert bal.token_counts == [2, 2, 2, 2] and abs(bal.load_balance_loss - 1.0) < 1e-6 and bal.stddev == 0.0
    logits = torch.zeros(8, 2)
    logits[:, 0] = 1.0
    idx, gate = me.SwitchV2Router(2, capacity_factor=1.0)(logits)
    assert idx.tolist() == [0, 0, 0, 0, -1, -1, -1, -1] and float(gate[4]) == 0.0
    keep, w = me.ExpertChoiceV2(4, top_k=2)(torch.randn(6, 8), torch.randn(6, 4))
    assert keep.shape == (6, 4) and (keep.sum(1) <= 2).all() and torch.equal(w > 0, keep)
    a = torch.randn(4, 4)
    merged = me.ExpertMerger(0.95).merge([a, a * 1.01, -a])
    assert len(merged) == 2
    pool = me.DynamicExpertPool(max_experts=2)
    assert pool.add_expert(a) == 0 and pool.add_expert(a) == 1 and pool.add_expert(a) == -1
    assert pool.remove_expert(0) and not pool.remove_expert(0) and pool.count() == 1
