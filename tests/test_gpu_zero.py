"""Peer-memory data-parallel kernels, checked on one GPU by emulating the ranks: every "rank"
gets its own buffers on the same device and the kernels (which never wait on one another) are
launched rank by rank. The flag barrier is exercised with a single rank and with a flag that
nothing sets (the bounded wait must expire and report, not hang)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_reduce_scatter_adamw_ste_allgather_emulated_ranks():
    from mythos_b200.oil.codebook import quantile_codebook
    from mythos_b200.ops import native, reference as ref

    C = native.require()
    torch.manual_seed(0)
    world, seg = 2, 256
    n_seg = 64
    total = n_seg * seg
    shard = total // world
    master = torch.randn(total, device="cuda") * 0.02
    grads = [torch.randn(total, device="cuda") * 0.01 for _ in range(world)]
    compute = [torch.zeros(total, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    # segments: first quarter cast, then OIL8 (two codebooks), OIL4, I2_S
    seg_fmt = torch.zeros(n_seg, dtype=torch.uint8)
    seg_cb = torch.zeros(n_seg, dtype=torch.int32)
    seg_fmt[16:32] = 1
    seg_cb[24:32] = 1
    seg_fmt[32:48] = 2
    seg_fmt[48:] = 3
    cb8 = torch.stack([quantile_codebook(256, 0.02), quantile_codebook(256, 0.03)]).cuda()
    cb4 = quantile_codebook(16, 0.02, fp16=True)[None].cuda()
    seg_fmt, seg_cb = seg_fmt.cuda(), seg_cb.cuda()
    ms = [torch.zeros(shard, device="cuda") for _ in range(world)]
    vs = [torch.zeros(shard, device="cuda") for _ in range(world)]
    masters = [master.clone() for _ in range(world)]
    gsh = [torch.empty(shard, device="cuda") for _ in range(world)]
    parts = torch.zeros(world, device="cuda")
    for r in range(world):
        p = torch.zeros(1, device="cuda")
        C.zero_reduce_scatter([g.data_ptr() for g in grads], gsh[r], r * shard, p)
        parts[r] = p[0]
    gsum = grads[0] + grads[1]
    for r in range(world):
        assert torch.allclose(gsh[r], gsum[r * shard:(r + 1) * shard], atol=1e-7)
    assert abs(parts.sum().item() - gsum.double().pow(2).sum().item()) < 1e-4
    gn = torch.zeros(1, device="cuda")
    max_norm = 0.5 * gsum.norm().item()  # force clipping
    for r in range(world):
        C.zero_adamw_ste_allgather(masters[r][r * shard:(r + 1) * shard], ms[r], vs[r], gsh[r],
                                   [c.data_ptr() for c in compute], r * shard, seg_fmt, seg_cb, cb8, cb4, parts, gn,
                                   max_norm, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, r, 0)
    torch.cuda.synchronize()
    assert abs(gn.item() - gsum.norm().item()) < 1e-3 * gsum.norm().item()
    # reference: AdamW on the clipped summed gradient, then per-segment quantisation
    pr, mr, vr = master.clone(), torch.zeros(total, device="cuda"), torch.zeros(total, device="cuda")
    clip = max_norm / (gsum.norm().item() + 1e-8)
    ref.adamw_step(pr, mr, vr, gsum, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, clip)
    new_master = torch.cat([masters[r][r * shard:(r + 1) * shard] for r in range(world)])
    assert torch.allclose(new_master, pr, rtol=1e-5, atol=1e-7)
    want = torch.empty(total, device="cuda")
    want[:16 * seg] = pr[:16 * seg]
    _, d = ref.nearest_centroid(pr[16 * seg:24 * seg], cb8[0:1], torch.zeros(8, dtype=torch.int32, device="cuda"), seg)
    want[16 * seg:24 * seg] = d
    _, d = ref.nearest_centroid(pr[24 * seg:32 * seg], cb8[1:2], torch.zeros(8, dtype=torch.int32, device="cuda"), seg)
    want[24 * seg:32 * seg] = d
    _, d = ref.nearest_centroid(pr[32 * seg:48 * seg], cb4, torch.zeros(16, dtype=torch.int32, device="cuda"), seg)
    want[32 * seg:48 * seg] = d
    _, _, d = ref.i2s_quant(pr[48 * seg:], seg)
    want[48 * seg:] = d
    for r in range(world):
        got = compute[r].float()
        mism = (got != want.to(torch.bfloat16).float()).float().mean().item()
        assert mism < 2e-3, f"rank {r}: {mism} of the compute image differs"  # ulp-level AdamW differences may flip a centroid
        assert torch.equal(compute[0], compute[r])


def test_flag_barrier_single_rank_and_timeout():
    from mythos_b200.ops import native
    from mythos_b200.parallel import symm

    C = native.require()
    bar = symm.FlagBarrier("cuda")
    val = torch.tensor([3.5], device="cuda")
    bar.sync(val)
    bar.sync()
    torch.cuda.synchronize()
    native.check_status("cuda")
    assert bar.slots[0].item() == 3.5
    # two "ranks" whose second flag array nobody signals: rank 0 must give up after the limit
    fa = torch.zeros(64, dtype=torch.int32, device="cuda")
    fb = torch.zeros(64, dtype=torch.int32, device="cuda")
    sl = torch.zeros(64, device="cuda")
    C.symm_barrier([fa.data_ptr(), fb.data_ptr()], [sl.data_ptr(), sl.data_ptr()], None, 0, 1, 2_000_000,
                   native.status_word("cuda"), None)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 1"):
        native.check_status("cuda")
    native.check_status("cuda")  # cleared
    assert fb[0].item() == 1  # the signal to the peer was still delivered


def test_timeout_stops_the_consuming_kernels_and_the_next_step():
    """A flag nobody sets makes the bounded barrier wait expire (status word set). The kernels that
    would consume the guarded data then return without writing, and the trainer raises at the
    start of the next step instead of training on."""
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.ops import native
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    C = native.require()
    st = native.status_word("cuda")
    fa = torch.zeros(64, dtype=torch.int32, device="cuda")
    fb = torch.zeros(64, dtype=torch.int32, device="cuda")
    sl = torch.zeros(64, device="cuda")
    C.symm_barrier([fa.data_ptr(), fb.data_ptr()], [sl.data_ptr(), sl.data_ptr()], None, 0, 1, 2_000_000, st, None)
    torch.cuda.synchronize()
    assert int(st.item()) != 0
    # reduce-scatter and pull all-reduce after the expired wait: outputs stay as they were
    g = torch.ones(1024, device="cuda")
    out = torch.full((1024,), 7.0, device="cuda")
    ss = torch.zeros(1, device="cuda")
    C.zero_reduce_scatter([g.data_ptr()], out, 0, ss)
    part = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    res = torch.full((1024,), 5.0, device="cuda", dtype=torch.bfloat16)
    C.tp_allreduce_pull([part.data_ptr()], [res.data_ptr()], 0, 1024)
    torch.cuda.synchronize()
    assert torch.all(out == 7.0) and float(ss) == 0.0 and torch.all(res == 5.0)
    with pytest.raises(RuntimeError, match="status 1"):
        native.check_status("cuda")
    C.zero_reduce_scatter([g.data_ptr()], out, 0, ss)                  # cleared: the kernels work again
    torch.cuda.synchronize()
    assert torch.all(out == 1.0)

    cfg = TransformerConfig(vocab_size=256, hidden_size=256, num_layers=1, num_heads=2, head_dim=128,
                            ffn_hidden_size=256, max_seq_len=128, oil_block_size=64)
    with torch.device("cuda"):
        model = DenseModel(cfg)
    tr = Trainer(model, TrainConfig(batch_size=2, seq_length=128, lr=1e-3, warmup_steps=0), device="cuda")
    data = ZipfStream(cfg.vocab_size, 2, 128, seed=0)
    tr.train_step(*data.next_batch())
    st.fill_(1 | (40 << 16))                                           # as an expired barrier wait would leave it
    tr.train_step(*data.next_batch())                                   # posts the word to the host
    with pytest.raises(RuntimeError, match="bounded wait expired"):
        tr.train_step(*data.next_batch())
    tr.train_step(*data.next_batch())                                   # cleared; training continues
    torch.cuda.synchronize()
    native.check_status("cuda")
