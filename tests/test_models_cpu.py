"""CPU tests of the model layer: config blob, reference operators, dense / MoE / LoRA behaviour,
trainer mechanics, schedules, codebooks."""
import math
import struct

import pytest
import torch

from mythos_b200.models import DenseModel, TransformerConfig
from mythos_b200.models.config import NAMED_CONFIGS


def _tiny(**kw):
    base = dict(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, head_dim=16, ffn_hidden_size=64,
                max_seq_len=32, oil_block_size=32)
    base.update(kw)
    return TransformerConfig(**base)


def test_config_blob_matches_reference_struct_layout():
    cfg = TransformerConfig(vocab_size=32000, hidden_size=768, num_layers=12, num_heads=12, head_dim=64,
                            ffn_hidden_size=3072, norm_eps=1e-5, rope_theta=10000.0, max_seq_len=2048,
                            activation="silu", num_kv_heads=4, use_parallel_residual=True)
    blob = cfg.to_bytes(extended=False)
    assert len(blob) == 88
    assert struct.unpack_from("<q", blob, 0)[0] == 32000 and struct.unpack_from("<q", blob, 8)[0] == 768
    assert struct.unpack_from("<q", blob, 40)[0] == 3072
    assert abs(struct.unpack_from("<f", blob, 48)[0] - 1e-5) < 1e-12 and struct.unpack_from("<f", blob, 52)[0] == 10000.0
    assert struct.unpack_from("<q", blob, 56)[0] == 2048 and struct.unpack_from("<i", blob, 64)[0] == 2
    assert struct.unpack_from("<q", blob, 72)[0] == 4 and blob[80] == 1
    assert blob[68:72] == b"\0\0\0\0" and blob[81:88] == b"\0" * 7
    back = TransformerConfig.from_bytes(blob)
    assert back.weight_format == "fp32" and back.num_kv_heads == 4 and back.hidden_size == 768
    ext = TransformerConfig.from_bytes(cfg.to_bytes())
    assert ext.weight_format == cfg.weight_format and ext.oil_block_size == cfg.oil_block_size
    for name, fn in NAMED_CONFIGS.items():
        c = fn()
        assert c.hidden_size % 8 == 0 and c.param_count() > 0, name
    assert 1.2e9 < NAMED_CONFIGS["llama-1.3b"]().param_count() < 1.5e9


def test_reference_attention_is_causal_and_gqa_grouped():
    from mythos_b200.ops import reference as ref

    torch.manual_seed(0)
    q = torch.randn(1, 6, 4, 8)
    k = torch.randn(1, 6, 2, 8)
    v = torch.randn(1, 6, 2, 8)
    o, lse = ref.attention(q, k, v, True)
    k2, v2 = k.clone(), v.clone()
    k2[:, 4:] += 5
    v2[:, 4:] -= 3
    o2, _ = ref.attention(q, k2, v2, True)
    assert torch.allclose(o[:, :4], o2[:, :4])          # the future does not leak
    o3, _ = ref.attention(q[:, :, :2], k[:, :, :1], v[:, :, :1], True)
    assert torch.allclose(o[:, :, :2], o3, atol=1e-6)   # heads 0,1 read kv head 0
    assert lse.shape == (1, 4, 6)


def test_rope_is_a_rotation_and_inverts():
    from mythos_b200.ops import reference as ref

    x = torch.randn(5, 3, 16)
    pos = torch.tensor([0, 1, 7, 100, 2047], dtype=torch.int32)
    y = ref.rope(x, pos, 10000.0)
    assert torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.allclose(ref.rope(y, pos, 10000.0, inverse=True), x, atol=1e-5)
    j, d, p = 3, 16, 7.0
    ang = p * 10000.0 ** (-2.0 * j / d)
    want = x[2, 0, j] * math.cos(ang) - x[2, 0, j + 8] * math.sin(ang)
    assert abs(float(y[2, 0, j]) - float(want)) < 1e-5


def test_dense_model_trains_on_cpu_and_ste_quantises():
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(0)
    m = DenseModel(_tiny())
    tr = Trainer(m, TrainConfig(batch_size=8, micro_batch_size=4, seq_length=16, lr=5e-3, warmup_steps=2,
                                max_steps=50, codebook_ema_interval=5), device="cpu")
    ds = ZipfStream(64, 8, 16, seed=1)
    losses = [float(tr.train_step(*ds.next_batch())) for _ in range(20)]
    assert losses[-1] < losses[0] - 0.2
    lin = m.layers[0].attention.qkv_proj
    wq = lin.compute_weight().detach()
    assert len(torch.unique(wq.reshape(-1, lin.block_size)[0])) <= 256
    assert not torch.equal(wq, lin.weight.detach())
    cb = lin.codebooks
    assert bool((cb[:, 1:] >= cb[:, :-1]).all())  # codebooks stay sorted after EMA updates


def test_grad_accumulation_equals_one_big_batch():
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(1)
    a, b = DenseModel(_tiny(weight_format="fp32")), DenseModel(_tiny(weight_format="fp32"))
    b.load_state_dict(a.state_dict())
    ta = Trainer(a, TrainConfig(batch_size=4, micro_batch_size=4, lr=1e-3, warmup_steps=0), device="cpu")
    tb = Trainer(b, TrainConfig(batch_size=4, micro_batch_size=1, lr=1e-3, warmup_steps=0), device="cpu")
    ids = torch.randint(0, 64, (4, 16), dtype=torch.int32)
    tg = torch.randint(0, 64, (4, 16), dtype=torch.int32)
    la, lb = ta.train_step(ids, tg), tb.train_step(ids, tg)
    assert abs(float(la) - float(lb)) < 1e-5
    assert torch.allclose(ta.store.master, tb.store.master, atol=1e-6)


def test_moe_reference_matches_per_token_loop_and_aux_loss():
    from mythos_b200.models.moe import MoEFFN, MoEModel
    from mythos_b200.ops import reference as ref

    torch.manual_seed(2)
    cfg = _tiny(num_experts=4, moe_top_k=2, moe_ffn_hidden_size=48, weight_format="fp32", moe_aux_coef=0.01)
    moe = MoEFFN(cfg)
    x = torch.randn(10, 32)
    out = moe(x)
    probs = torch.softmax(moe.router(x)[:, :4].float(), -1)
    w, idx = torch.topk(probs, 2, dim=-1)
    want = torch.zeros_like(x)
    for t in range(10):
        for j in range(2):
            want[t] += w[t, j] * moe._expert(int(idx[t, j]), x[t:t + 1])[0]   # weights are not renormalised
    assert torch.allclose(out, want, atol=1e-5)
    f = torch.bincount(idx.reshape(-1), minlength=4).float() / 10
    P = torch.stack([(probs[:, e] * (idx == e).any(1)).sum() / 10 for e in range(4)])
    assert abs(float(moe.last_aux) - 0.01 * 4 * float((f * P).sum())) < 1e-6
    assert abs(float(ref.z_loss(torch.zeros(3, 4), 0.5)) - 0.5 * math.log(4) ** 2) < 1e-6
    model = MoEModel(cfg)
    ids = torch.randint(0, 64, (2, 8), dtype=torch.int32)
    loss = model(ids, ids)
    loss.backward()
    assert model.layers[0].ffn.router.weight.grad is not None
    assert any(e.weight.grad is not None for e in model.layers[0].ffn.experts_up)
    # capacity factor drops overflow tokens; shared experts always run
    capped = MoEFFN(_tiny(num_experts=4, moe_top_k=1, weight_format="fp32", moe_shared_experts=1),
                    capacity_factor=0.5, drop_policy="drop")
    capped(torch.randn(16, 32))
    assert capped.last_stats["tokens_dropped"] > 0
    for routing in ("hash", "expert_choice", "dense"):
        assert MoEFFN(cfg, routing=routing)(x).shape == x.shape


def test_lora_adapters_train_while_base_stays_frozen():
    from mythos_b200.models.lora import LoRALinear, apply_lora, merge_all, nf4_codebook

    torch.manual_seed(3)
    m = DenseModel(_tiny(weight_format="oil4"))
    ids = torch.randint(0, 64, (2, 12), dtype=torch.int32)
    with torch.no_grad():
        before = m(ids)
    wrapped = apply_lora(m, rank=4, alpha=8.0, targets=("q", "v"))
    assert len(wrapped) == 2 and all(isinstance(w, LoRALinear) for w in wrapped)
    with torch.no_grad():
        assert torch.allclose(m(ids), before, atol=1e-6)   # B = 0: adapters start as identity
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    base_w = m.layers[0].attention.qkv_proj.base.weight.clone()
    opt = torch.optim.SGD([p for p in m.parameters() if p.requires_grad], lr=0.5)
    for _ in range(3):
        loss = m(ids, ids)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert torch.equal(m.layers[0].attention.qkv_proj.base.weight, base_w)
    assert float(m.layers[0].attention.qkv_proj.lora_B[0].abs().sum()) > 0
    lin = LoRALinear(DenseModel(_tiny(weight_format="fp32")).layers[0].attention.o_proj, rank=2)
    with torch.no_grad():
        lin.lora_B[0].normal_()
    x = torch.randn(3, 32)
    y = lin(x)
    lin.merge()
    assert torch.allclose(lin(x), y, atol=1e-5)
    lin.unmerge()
    assert torch.allclose(lin(x), y, atol=1e-5)
    assert nf4_codebook().numel() == 16 and float(nf4_codebook(2.0).max()) == 2.0
    merge_all(m)


def test_schedules_match_reference_formulas():
    from mythos_b200.train import sched

    assert sched.builtin_lr("warmup_cosine", 3e-4, 50, 100, 10000) == pytest.approx(1.5e-4)
    assert sched.builtin_lr("warmup_cosine", 3e-4, 100, 100, 10000) == pytest.approx(3e-4)
    mid = sched.builtin_lr("warmup_cosine", 3e-4, 5050, 100, 10000)
    assert mid == pytest.approx(3e-4 * 0.5 * (1 + math.cos(math.pi * 0.5)), abs=1e-9)
    assert sched.builtin_lr("warmup_cosine", 3e-4, 10000, 100, 10000) == pytest.approx(1e-8)
    assert sched.builtin_lr("constant", 1.0, 7) == 1.0
    assert sched.LinearDecay(1.0, 10).lr(5) == pytest.approx(0.5)
    assert sched.StepDecay(1.0, 10, 0.1).lr(25) == pytest.approx(0.01)
    assert sched.ExponentialDecay(1.0, 0.5).lr(3) == pytest.approx(0.125)
    assert sched.Warmup(sched.Constant(2.0), 4).lr(1) == pytest.approx(1.0)
    assert sched.Sequential([sched.Constant(1.0), sched.Constant(0.1)], [5]).lr(7) == pytest.approx(0.1)
    assert sched.Lambda(2.0, lambda s: 1.0 / (1 + s)).lr(1) == pytest.approx(1.0)
    oc = sched.OneCycle(1.0, 100)
    assert oc.lr(30) == pytest.approx(1.0) and oc.lr(0) < 0.1
    rp = sched.ReduceLROnPlateau(1.0, factor=0.5, patience=1)
    for v in (1.0, 1.0, 1.0):
        rp.observe(v)
    assert rp.lr(0) == pytest.approx(0.5)


def test_codebook_kmeans_ema_and_serialisation():
    from mythos_b200.oil import codebook as cbk

    torch.manual_seed(4)
    data = torch.cat([torch.randn(500) * 0.01 - 1, torch.randn(500) * 0.01 + 1])
    cb = cbk.kmeans_codebook(data, 16)
    assert bool((cb[1:] >= cb[:-1]).all()) and cb.min() < -0.9 and cb.max() > 0.9
    idx, cnt, sums = cbk.quantize(data, cb)
    assert int(cnt.sum()) == 1000 and idx.dtype == torch.uint8
    q = cbk.quantile_codebook(256, 0.02)
    assert abs(float(q.mean())) < 1e-6 and bool((q[1:] > q[:-1]).all())
    kind, back = cbk.deserialize(cbk.serialize_oil8(q))
    assert kind == "oil8" and torch.equal(torch.from_numpy(back.copy()), q)
    kind4, back4 = cbk.deserialize(cbk.serialize_oil4(cbk.quantile_codebook(16, fp16=True)))
    assert kind4 == "oil4" and back4.shape == (16,)
    books = q[None].clone()
    ema = cbk.EMAState(books, decay=0.5)
    ema.update(books, torch.ones(1, 256), books * 2)
    assert torch.allclose(books, torch.sort(q * 2).values[None])


def test_qlora_nf4_base_is_frozen_and_adapter_trains():
    from mythos_b200.models.lora import NF4_LEVELS, QLoRALinear, nf4_dequantize, nf4_quantize

    torch.manual_seed(0)
    w = torch.randn(48, 128) * 0.05
    packed, lo, hi = nf4_quantize(w, 64)
    assert packed.dtype == torch.uint8 and packed.numel() == w.numel() // 2 and lo.numel() == w.numel() // 64
    deq = nf4_dequantize(packed, lo, hi, w.numel(), 64).view_as(w)
    # every block reproduces its extremes exactly (levels -1 and +1 map onto min and max)
    blocks, dblocks = w.view(-1, 64), deq.view(-1, 64)
    assert torch.allclose(dblocks.amax(1), blocks.amax(1)) and torch.allclose(dblocks.amin(1), blocks.amin(1))
    # nearest-level error is at most half the widest gap between levels, scaled to the block range
    gaps = torch.tensor(NF4_LEVELS).diff().max() / 2
    assert float(((deq - w).abs().view(-1, 64) / ((hi - lo)[:, None] / 2)).max()) <= float(gaps) + 1e-6
    q = QLoRALinear(w, rank=4, alpha=8.0)
    assert q.base_bytes() < w.numel() * 4 / 6
    x = torch.randn(5, 128)
    assert torch.allclose(q(x), x @ q.base_weight().T, atol=1e-5)          # B = 0 at the start
    before = q.packed.clone()
    tgt = torch.randn(5, 48)
    opt = torch.optim.Adam([p for p in q.parameters() if p.requires_grad], lr=1e-2)
    first = None
    for _ in range(40):
        loss = ((q(x) - tgt) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.5 * first and torch.equal(q.packed, before)
    assert torch.allclose(x @ q.merged_weight().T, q(x), atol=1e-4)
    other = QLoRALinear(torch.zeros_like(w), rank=4, alpha=8.0)
    other.load_adapter_state(q.adapter_state("m."), "m.")
    assert torch.allclose(other(x), q(x), atol=1e-6)


def test_mixed_per_block_formats_train_save_and_reload(tmp_path):
    """A layer whose blocks carry different formats (OIL8 / OIL4 / ternary / binary planned for 1.5
    bits per weight): the fake-quantised image is the per-block application of each format, the
    model trains through the straight-through estimator, the .oil file holds every block in its own
    format and a save -> load -> save cycle reproduces the file byte for byte."""
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.models.layers import OILLinear
    from mythos_b200.oil import container as oc
    from mythos_b200.oil.formats import Format
    from mythos_b200.oil.model_io import load_model, save_model
    from mythos_b200.ops import functional as Fn
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(0)
    lin = OILLinear(256, 64, "mixed", 256, target_bpw=2.5)
    kinds = set(lin.block_formats.tolist())
    assert len(kinds) >= 3 and kinds <= {0, 1, 2, 3}
    bpw = sum({0: 1, 1: 2, 2: 4, 3: 8}[int(c)] for c in lin.block_formats) / lin.n_blocks
    assert abs(bpw - 2.5) < 0.3
    q = lin.quantize_now(lin.weight.detach())
    flat = lin.weight.detach().reshape(-1)
    q8, _ = Fn.oil_fake_quant(flat, lin.codebooks, lin.cb_map, 256)
    q4, _ = Fn.oil_fake_quant(flat, lin.codebooks4, lin.cb_map, 256)
    q2, _, _ = Fn.i2s_fake_quant(flat, 256)
    for b, code in enumerate(lin.block_formats.tolist()):
        seg = slice(b * 256, (b + 1) * 256)
        got = q.reshape(-1)[seg]
        if code == 3:
            assert torch.equal(got, q8.reshape(-1)[seg])
        elif code == 2:
            assert torch.equal(got, q4.reshape(-1)[seg])
        elif code == 1:
            assert torch.equal(got, q2.reshape(-1)[seg])
        else:
            s = flat[seg].abs().mean()
            assert torch.allclose(got.abs(), s.expand(256)) and torch.equal(got > 0, flat[seg] > 0)
    # a whole model in mixed format trains and round-trips
    cfg = TransformerConfig(vocab_size=64, hidden_size=64, num_layers=1, num_heads=2, head_dim=32, ffn_hidden_size=128,
                            max_seq_len=16, oil_block_size=256, weight_format="mixed")
    model = DenseModel(cfg)
    tr = Trainer(model, TrainConfig(batch_size=4, seq_length=16, lr=5e-3, warmup_steps=0), device="cpu")
    data = ZipfStream(64, 4, 16, seed=0)
    losses = [float(tr.train_step(*data.next_batch())) for _ in range(12)]
    assert losses[-1] < losses[0]
    p1, p2 = str(tmp_path / "a.oil"), str(tmp_path / "b.oil")
    save_model(model, p1)
    rd = oc.OILReader(p1)
    fmts = {b.format for b in rd.read_tensor_blocks("layers.0.ffn.up_proj.weight")}
    assert len(fmts) >= 2 and fmts <= {Format.OIL8, Format.OIL4, Format.TERNARY, Format.BINARY}
    loaded, _ = load_model(p1)
    assert torch.equal(loaded.layers[0].ffn.up_proj.block_formats, model.layers[0].ffn.up_proj.block_formats)
    save_model(loaded, p2)
    assert open(p1, "rb").read() == open(p2, "rb").read()


def test_converter_style_mixed_file_loads_into_a_mixed_model(tmp_path):
    """Blocks quantised by the format planner (what ``oil-convert --target-bpw 1.5`` writes) load into a
    ``weight_format="mixed"`` model: the file decides every block's format and codebook, the weights
    are the planner's dequantised values, and saving the model again reproduces the file."""
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.models.layers import OILLinear
    from mythos_b200.oil import container as oc, planner
    from mythos_b200.oil.model_io import _fp32_blocks, load_model, save_model

    torch.manual_seed(1)
    cfg = TransformerConfig(vocab_size=64, hidden_size=64, num_layers=1, num_heads=2, head_dim=32, ffn_hidden_size=128,
                            max_seq_len=16, oil_block_size=256, weight_format="mixed")
    src = DenseModel(cfg)
    tensors, shapes, want = [], {}, {}
    for name, p, mod in src.export_named_tensors():
        shapes[name] = list(p.shape)
        if isinstance(mod, OILLinear):
            fmts, _ = planner.plan(p.detach(), 1.5, 256)
            deq, blocks = planner.quantize_mixed(p.detach(), fmts, 256)
            tensors.append((name, blocks))
            want[name] = (fmts, deq)
        else:
            tensors.append((name, _fp32_blocks(p.detach().float().numpy())))
    cfg.extras = {"shapes": shapes, "fused": True}
    path = str(tmp_path / "planned.oil")
    oc.write_oil(path, tensors, config=cfg.to_bytes(extended=True), version=1, flags=0, write_idx=True, idx_version=2,
                 shapes=shapes)
    model, _ = load_model(path)
    for name, p, mod in model.export_named_tensors():
        if name in want:
            fmts, deq = want[name]
            assert mod.fmt == "mixed" and mod.block_formats.tolist() == [int(f) for f in fmts], name
            assert torch.equal(p.detach(), deq.view(p.shape)), name
            # the stored values are fixed points of the layer's quantiser
            assert torch.allclose(mod.quantize_now(p.detach()), p.detach(), atol=1e-6), name
    again = str(tmp_path / "again.oil")
    save_model(model, again)
    assert open(path, "rb").read() == open(again, "rb").read()
