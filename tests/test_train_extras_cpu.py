"""Weight EMA, smoothing / R-Drop losses, fine-tuner helpers, CHPK checkpoints, dense trainer."""
import numpy as np
import torch

from mythos_b200.models import DenseModel
from mythos_b200.models.config import tiny_byte_config
from mythos_b200.models.layers import OILLinear
from mythos_b200.train import extras as ex


def test_losses():
    torch.manual_seed(0)
    lg, t = torch.randn(4, 6, 11), torch.randint(0, 11, (4, 6))
    ce = torch.nn.functional.cross_entropy(lg.view(-1, 11), t.view(-1))
    assert torch.allclose(ex.label_smoothing_loss(lg, t, 0.0), ce, atol=1e-6)
    want = torch.nn.functional.cross_entropy(lg.view(-1, 11), t.view(-1), label_smoothing=0.1)
    assert torch.allclose(ex.label_smoothing_loss(lg, t, 0.1), want, atol=1e-5)
    assert torch.allclose(ex.rdrop_loss(lg, lg, t), ce, atol=1e-6)
    assert float(ex.rdrop_loss(lg, lg + torch.randn_like(lg), t)) > float(ce) - 1.0


def test_block_selection_and_in_format_update():
    g = torch.zeros(4 * 256)
    g[256:512] = 1.0
    g[768:] = 0.5
    assert ex.find_trainable_blocks(g, 256, 0.5).tolist() == [1, 3]
    torch.manual_seed(1)
    lin = OILLinear(64, 32, "oil8", block_size=64, codebook_group=4)
    before = lin.weight.detach().clone()
    grad = torch.randn_like(before)
    ex.apply_oil_update(lin, grad, lr=0.05, blocks=torch.tensor([0, 1]))
    after = lin.weight.detach()
    assert not torch.equal(after.view(-1)[:128], before.view(-1)[:128])
    # every updated weight sits exactly on a centroid of its codebook
    cb = lin.codebooks[lin.cb_map[0]] if lin.cb_map is not None else lin.codebooks[0]
    assert all(bool((cb == x).any()) for x in after.view(-1)[:64])
    tern = OILLinear(64, 8, "i2s", block_size=64)
    ex.apply_oil_update(tern, torch.randn(8, 64), lr=0.01)
    blk = tern.weight.detach().view(-1)[:64]
    assert blk.abs().unique().numel() <= 2


def test_chpk_round_trip(tmp_path):
    ps = [torch.randn(3, 4), torch.randn(5)]
    m, v = [torch.zeros_like(p) + 1 for p in ps], [torch.zeros_like(p) + 2 for p in ps]
    path = str(tmp_path / "a.chpk")
    ex.save_chpk(path, 17, 1e-3, ps, m, v)
    ck = ex.load_chpk(path)
    assert ck["step"] == 17 and abs(ck["lr"] - 1e-3) < 1e-9
    assert all(torch.equal(a, b) for a, b in zip(ps, ck["params"])) and torch.equal(ck["v"][1], v[1])
    # byte layout of the reference writer: 20-byte header with a u32 step, then named records
    import struct
    raw = open(path, "rb").read()
    assert struct.unpack_from("<IIIfI", raw, 0)[:3] == (0x4B504843, 2, 17) and struct.unpack_from("<I", raw, 16)[0] == 2
    assert raw[20:24] == struct.pack("<I", 7) and raw[24:31] == b"param_0"
    body = struct.unpack_from("<I", raw, 31)[0]
    assert body == 4 + 2 * 8 + 1 + 12 * 4 and raw[35:39] == struct.pack("<i", 2) and raw[35 + 4 + 16] == 6
    pos = [raw.index(struct.pack("<I", 3) + tag) for tag in (b"m_0", b"v_0", b"m_1", b"v_1")]
    assert pos == sorted(pos) and pos[0] > raw.index(b"param_1")        # moments interleaved per parameter
    ex.save_chpk(path, 3, 1e-2, ps)                      # no optimizer state yet: zeros are written
    ck0 = ex.load_chpk(path)
    assert ck0["step"] == 3 and all(float(t.abs().sum()) == 0 for t in ck0["m"] + ck0["v"])
    ex.save_chpk(path, 17, 1e-3, ps, m, v)
    with open(path, "r+b") as f:
        f.write(b"XXXX")
    try:
        ex.load_chpk(path)
        assert False
    except ValueError:
        pass


def test_dense_trainer_ema_and_resume(tmp_path):
    torch.manual_seed(2)
    cfg = tiny_byte_config()
    cfg.num_layers, cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden_size, cfg.max_seq_len = 1, 64, 1, 128, 32
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, 16, size=4000).astype(np.int32)
    loader = ex.ChunkLoader(tokens, 4, 32)
    loader.shuffle(0)
    first = loader.order.copy()
    loader.shuffle(1)
    assert not np.array_equal(first, loader.order) and sorted(loader.order) == sorted(first)
    tr = ex.DenseTrainer(DenseModel(cfg), lr=3e-3, batch_size=4, seq_length=32, device="cpu")
    ema = ex.WeightEMA(tr.inner, 0.9)
    losses = []
    for x, y in loader:
        losses.append(tr.train_step(x, y))
        ema.step()
        if len(losses) == 12:
            break
    assert losses[-1] < losses[0]
    live = tr.inner.store.master.clone()
    ema.swap()
    assert not torch.equal(tr.inner.store.master, live)
    ema.swap()
    assert torch.equal(tr.inner.store.master, live)
    path = str(tmp_path / "d.chpk")
    tr.save_checkpoint(path)
    x, y = next(iter(loader))
    ref_loss = tr.train_step(x, y)
    tr2 = ex.DenseTrainer(DenseModel(cfg), lr=1.0, batch_size=4, seq_length=32, device="cpu")
    tr2.load_checkpoint(path)
    assert tr2.step == 12 and abs(tr2.lr - 3e-3) < 1e-9
    assert abs(tr2.train_step(x, y) - ref_loss) < 1e-5


def test_streaming_loader_augmentation_and_curriculum(tmp_path):
    from mythos_b200.train.data import Curriculum, StreamingTokenDataset, TokenDataset, augment_batch

    text = bytes(range(32, 127)) * 400                         # 38,000 bytes, byte-level ids
    p = tmp_path / "corpus.bin"
    p.write_bytes(text)
    for use_mmap in (False, True):
        ds = StreamingTokenDataset(str(p), None, batch=4, seq=64, chunk_bytes=5000, prefetch=2, mmap=use_mmap)
        batches = list(ds)
        assert ds.chunks_read == 8 and len(batches) == (len(text) - 1) // 256
        flat = torch.cat([b[0].reshape(-1) for b in batches])
        assert torch.equal(flat, torch.tensor(list(text[: flat.numel()]), dtype=torch.int32))   # nothing lost at chunk seams
        assert all(torch.equal(i.reshape(-1)[1:], t.reshape(-1)[:-1]) for i, t in batches)
    whole = TokenDataset(list(text), 4, 64, shuffle=False, prefetch=0)
    assert torch.equal(next(iter(whole))[0], batches[0][0])
    g = torch.Generator().manual_seed(0)
    ids, tgt = batches[0]
    a_ids, a_tgt = augment_batch(ids, tgt, vocab=300, mask_prob=0.2, replace_prob=0.1, label_mask_prob=0.3, generator=g)
    changed = (a_ids != ids).float().mean().item()
    assert 0.15 < changed < 0.4 and 0.15 < (a_tgt == 0).float().mean().item() < 0.45 and int(a_ids.max()) < 300
    assert torch.equal(augment_batch(ids, tgt, 300)[0], ids)
    cur = Curriculum(64, total_epochs=4, min_fraction=0.25)
    lens = []
    for e in range(5):
        cur.step(e)
        lens.append(cur.length())
    assert lens == [16, 32, 48, 64, 64] and cur.apply(ids, tgt)[0].shape == (4, 64)
    cur.step(0)
    assert cur.apply(ids, tgt)[1].shape == (4, 16)
