"""Inference kernels against PyTorch references: codebook-dequant GEMM / GEMV, paged KV append +
split-KV decode attention, the sampler, and the engine end to end."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    lim = atol + rtol * b.abs().max().item()
    assert err <= lim, f"max err {err} > {lim}"


@pytest.mark.parametrize("fmt", ["oil8", "oil4", "i2s"])
@pytest.mark.parametrize("M,group", [(1, 4), (16, 1), (64, 64), (200, 4), (32, 3)])
def test_dequant_gemm_matches_dequantised_matmul(fmt, M, group):
    from mythos_b200.infer.quant_weights import QuantLinear

    torch.manual_seed(M)
    N, K = 384, 512
    w = torch.randn(N, K, device="cuda") * 0.02
    # group 1 spreads a warp's rows over more codebooks than its shared-memory table holds (global
    # gathers); 3/4/64 exercise the cached path with moving and fixed windows
    q = QuantLinear.from_float(w, fmt, block_size=256, codebook_group=group)
    deq = q.dequantize().float()
    ref_deq = q._dequantize_reference().float()
    assert torch.equal(deq, ref_deq.to(torch.bfloat16).float())
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    y = q.matmul(x)
    _close(y, x.float() @ deq.t(), atol=1e-2)
    # split-K with fp32 accumulation and the finalize kernel
    from mythos_b200.ops import native

    C = native.require()
    acc = torch.zeros(M, N, device="cuda")
    C.dequant_gemm(x, q.packed, q.codebooks, q.cb_map, q.scales, {"oil8": 3, "oil4": 2, "i2s": 1}[fmt], N, K, 256, acc,
                   [], 4, native.status_word("cuda"))
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.finalize_acc(acc, None, out)
    _close(out, x.float() @ deq.t(), atol=1e-2)
    assert float(acc.abs().max()) == 0.0
    # fused all-reduce output: partial tiles are added into every listed accumulator (here: two
    # local buffers standing in for two ranks)
    accs = [torch.zeros(M, N, device="cuda") for _ in range(2)]
    assert q.matmul(x, peer_ptrs=[a.data_ptr() for a in accs]) is None
    for a in accs:
        _close(a, x.float() @ deq.t(), atol=1e-2)


@pytest.mark.parametrize("fmt", ["oil8", "oil4", "i2s"])
@pytest.mark.parametrize("M,N,K,bs,group", [(8, 512, 4096, 256, 128), (64, 1000, 2048, 64, 16), (130, 256, 1024, 128, 1),
                                            (256, 384, 1536, 256, 7)])
def test_dequant_gemm_deep_k_and_block_sizes(fmt, M, N, K, bs, group):
    """Narrow, deep layers (automatic split-K through the fp32 accumulator), ragged N, every
    supported quantisation block size, codebook windows that move along K."""
    from mythos_b200.infer.quant_weights import QuantLinear

    torch.manual_seed(N + K)
    w = torch.randn(N, K, device="cuda") * 0.02
    q = QuantLinear.from_float(w, fmt, block_size=bs, codebook_group=group)
    deq = q.dequantize().float()
    assert torch.equal(deq, q._dequantize_reference().float().to(torch.bfloat16).float())
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    ref = x.float() @ deq.t()
    _close(q.matmul(x), ref, atol=2e-2)
    _close(q.matmul(x), ref, atol=2e-2)   # the accumulator was left zeroed by the first call


def test_tp_allreduce_kernels_with_emulated_ranks():
    """The tensor-parallel all-reduce kernels, with the ranks' buffers living on one GPU and the
    ranks' launches issued one after another (no kernel waits on another)."""
    from mythos_b200.infer.quant_weights import QuantLinear
    from mythos_b200.ops import native

    C = native.require()
    torch.manual_seed(5)
    W, M, N, K = 4, 24, 256, 512
    stride = 32 * N
    lin = [QuantLinear.from_float(torch.randn(N, K, device="cuda") * 0.02, "oil8", 256, 4) for _ in range(W)]
    xs = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(W)]
    parts = [xs[r].float() @ lin[r].dequantize().float().t() for r in range(W)]
    want = sum(p.to(torch.bfloat16).float() for p in parts)
    # one-shot: the GEMM epilogue (ranks 0, 1) or the push kernel (ranks 2, 3) fills slot r of every staging buffer
    staging = [torch.zeros(W * stride, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    ptrs = [t.data_ptr() for t in staging]
    for r in range(W):
        if r < 2:
            lin[r].matmul(xs[r], peer_ptrs=ptrs, k_splits=1, peer_bf16_offset=r * stride)
        else:
            acc = lin[r].matmul_acc(xs[r])
            C.tp_push(acc, ptrs, r, r * stride)
            assert float(acc.abs().max()) == 0.0
    for r in range(W):
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        C.tp_reduce_slots(staging[r], W, stride, None, out)
        _close(out, want, atol=2e-2)
    # GEMM with fused reduce-scatter epilogue, then reduce + broadcast
    Wg, T, Ng, Kg = 2, 1024, 512, 256
    rows, n_slot = T // Wg, (T // Wg) * Ng
    xg = [torch.randn(T, Kg, device="cuda").to(torch.bfloat16) for _ in range(Wg)]
    wg = [(torch.randn(Ng, Kg, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(Wg)]
    partg = [torch.zeros(Wg * n_slot, device="cuda", dtype=torch.bfloat16) for _ in range(Wg)]
    outg = [torch.zeros(T, Ng, device="cuda", dtype=torch.bfloat16) for _ in range(Wg)]
    for r in range(Wg):
        C.gemm_reduce_scatter(xg[r], wg[r], [t.data_ptr() for t in partg], r, rows, n_slot, native.status_word("cuda"))
    for r in range(Wg):
        C.tp_reduce_slots_bcast(partg[r], Wg, n_slot, [t.data_ptr() for t in outg], r, r * n_slot, n_slot)
    wantg = sum((xg[r].float() @ wg[r].float().t()).to(torch.bfloat16).float() for r in range(Wg))
    for r in range(Wg):
        _close(outg[r], wantg, atol=3e-2)
        assert torch.equal(outg[r], outg[0])
    # two-shot: every rank owns a slice, pulls it from all partial buffers and stores it everywhere
    pbuf = [p.to(torch.bfloat16).contiguous() for p in parts]
    obuf = [torch.zeros(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    for r in range(W):
        C.tp_allreduce_pull([t.data_ptr() for t in pbuf], [t.data_ptr() for t in obuf], r, M * N)
    for r in range(W):
        _close(obuf[r], want, atol=2e-2)
        assert torch.equal(obuf[r], obuf[0])


def test_quantisation_error_is_small_and_gemv_matches():
    from mythos_b200.infer.quant_weights import QuantLinear
    from mythos_b200.ops import native

    torch.manual_seed(0)
    w = torch.randn(256, 1024, device="cuda") * 0.02
    q8 = QuantLinear.from_float(w, "oil8", 256, 8)
    err = (q8.dequantize().float() - w).abs().mean() / w.abs().mean()
    assert err < 0.02
    qi = QuantLinear.from_float(w, "i2s", 256)
    x = torch.randn(1024, device="cuda").to(torch.bfloat16)
    y = torch.empty(256, device="cuda", dtype=torch.bfloat16)
    native.require().i2s_gemv(x, qi.packed, qi.scales, 256, 1024, 256, y)
    _close(y, qi.dequantize().float() @ x.float(), atol=5e-3)


@pytest.mark.parametrize("H,Hkv,D,page", [(4, 4, 128, 16), (8, 2, 128, 16), (4, 2, 64, 16), (32, 8, 128, 16),
                                          (8, 1, 64, 16), (8, 2, 128, 8), (4, 2, 64, 32)])
def test_paged_decode_attention(H, Hkv, D, page):
    """16-token pages run the tensor-core kernel, other page sizes the scalar one. The cache starts
    out holding stale finite values, so tokens past a sequence's length must be masked, not read."""
    from mythos_b200.ops import native, reference as ref

    C = native.require()
    torch.manual_seed(H * 7 + D)
    B, max_pages = 3, 384 // page
    lens = [37, 200, 1]
    n_pages = B * max_pages
    kc = (torch.randn(n_pages, page, Hkv, D, device="cuda") * 4).to(torch.bfloat16)
    vc = (torch.randn(n_pages, page, Hkv, D, device="cuda") * 4).to(torch.bfloat16)
    perm = torch.randperm(n_pages)[: B * max_pages].reshape(B, max_pages).to(torch.int32)
    table = perm.cuda()
    ks, vs = [], []
    for b in range(B):
        k = torch.randn(lens[b], Hkv, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(lens[b], Hkv, D, device="cuda").to(torch.bfloat16)
        pos = torch.arange(lens[b], device="cuda", dtype=torch.int32)
        sid = torch.full((lens[b],), b, device="cuda", dtype=torch.int32)
        C.kv_append(k, v, kc, vc, table, pos, sid)
        ks.append(k)
        vs.append(v)
    q = torch.randn(B, H, D, device="cuda").to(torch.bfloat16)
    ctx = torch.tensor(lens, device="cuda", dtype=torch.int32)
    for splits in (1, 4):
        out = torch.empty(B, H, D, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(B * H * splits * (D + 2), device="cuda")
        counters = torch.zeros(B * Hkv, device="cuda", dtype=torch.int32)
        C.paged_attn_decode(q, kc, vc, table, ctx, out, scratch, counters, splits, 1.0 / math.sqrt(D),
                            native.status_word("cuda"))
        for b in range(B):
            o, _ = ref.attention(q[b][None, None], ks[b][None], vs[b][None], causal=False)
            _close(out[b], o[0, 0], atol=2e-2)
        assert int(counters.abs().sum()) == 0


def test_sampler_modes():
    from mythos_b200.infer.sampler import SamplerConfig, nucleus_keep_mask, sample

    torch.manual_seed(0)
    rows, V = 4, 5000
    logits = (torch.randn(rows, V, device="cuda") * 2).to(torch.bfloat16)
    g = sample(logits, SamplerConfig(temperature=0.0))
    assert torch.equal(g.long(), logits.float().argmax(-1))
    probs = torch.softmax(logits.float(), -1)
    kth = torch.topk(probs, 40, dim=-1).values[:, -1]  # bf16 logits tie often: everything >= the 40th value is kept
    keep_p = nucleus_keep_mask(probs, 0.9)
    for step in range(30):
        t = sample(logits, SamplerConfig(temperature=1.0, top_k=40, top_p=1.0, seed=3), step=step)
        for r in range(rows):
            assert float(probs[r, int(t[r])]) >= float(kth[r])
        t = sample(logits, SamplerConfig(temperature=1.0, top_k=0, top_p=0.9, seed=5), step=step)
        for r in range(rows):
            assert bool(keep_p[r, int(t[r])])
    # distribution check on a small vocabulary, no filtering
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-30.0] * 28], device="cuda").to(torch.bfloat16)
    counts = torch.zeros(32)
    n = 4000
    for step in range(n):
        counts[int(sample(small, SamplerConfig(temperature=1.0, top_k=0, top_p=1.0, seed=11), step=step)[0])] += 1
    want = torch.softmax(small.float().cpu()[0], -1)
    assert (counts / n - want).abs().max() < 0.03
    # repetition penalty and vocabulary mask
    hist = torch.full((rows, 8), -1, device="cuda", dtype=torch.int32)
    hist[:, 0] = g
    t = sample(logits, SamplerConfig(temperature=0.0, repetition_penalty=100.0), history=hist)
    assert not torch.equal(t, g)
    mask = torch.zeros(rows, V, device="cuda", dtype=torch.uint8)
    mask[:, 17] = 1
    t = sample(logits, SamplerConfig(temperature=0.0), allow_mask=mask)
    assert (t == 17).all()


@pytest.mark.parametrize("rows,V", [(3, 128256), (64, 32000), (2, 128259), (5, 100)])
def test_greedy_argmax_many_ctas_per_row(rows, V):
    from mythos_b200.infer.sampler import SamplerConfig, sample

    torch.manual_seed(rows + V)
    logits = (torch.randn(rows, V, device="cuda") * 3).to(torch.bfloat16)
    logits[0, V - 1] = 40.0            # maximum in the ragged tail
    logits[rows - 1, :] = -1.0         # all equal: the first index wins
    for _ in range(3):                 # the per-row slots clean themselves between launches
        t = sample(logits, SamplerConfig(temperature=0.0))
        assert torch.equal(t.long(), logits.float().argmax(-1))
    assert int(t[0]) == V - 1 and int(t[rows - 1]) == 0


def test_fused_decode_epilogue_kernels():
    from mythos_b200.ops import native, reference as ref

    C = native.require()
    torch.manual_seed(7)
    # sum (+ residual) + RMSNorm from an fp32 accumulator and from bf16 slots
    T, N = 5, 2560
    acc = torch.randn(T, N, device="cuda")
    res = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    g = (torch.rand(N, device="cuda") + 0.5).to(torch.bfloat16)
    want_stream = (acc + res.float()).to(torch.bfloat16)
    want_norm = ref.rmsnorm(want_stream, g, 1e-5)[0]
    stream, normed = torch.empty_like(res), torch.empty_like(res)
    C.sum_residual_rmsnorm(acc.clone(), None, 0, 0, res, g, stream, normed, 1e-5)
    assert torch.equal(stream, want_stream)
    _close(normed, want_norm, atol=2e-2)
    a2 = acc.clone()
    C.sum_residual_rmsnorm(a2, None, 0, 0, None, g, stream, normed, 1e-5)
    assert float(a2.abs().max()) == 0.0 and torch.equal(stream, acc.to(torch.bfloat16))
    slots = torch.randn(3, 8, N, device="cuda").to(torch.bfloat16)        # 3 ranks, slot stride 8 rows
    C.sum_residual_rmsnorm(None, slots, 3, 8 * N, res, g, stream, normed, 1e-5)
    want = (slots[:, :T].float().sum(0) + res.float()).to(torch.bfloat16)
    assert torch.equal(stream, want)
    _close(normed, ref.rmsnorm(want, g, 1e-5)[0], atol=2e-2)
    # finalize + gate
    f = 384
    acc = torch.randn(T, 2 * f, device="cuda")
    gu = acc.to(torch.bfloat16)
    out = torch.empty(T, f, device="cuda", dtype=torch.bfloat16)
    C.finalize_gate(acc, out, 0)
    _close(out, ref.swiglu(gu), atol=2e-2)
    assert float(acc.abs().max()) == 0.0
    acc = torch.randn(T, 2 * f, device="cuda")
    gu = acc.to(torch.bfloat16).float()
    C.finalize_gate(acc, out, 1)
    _close(out, torch.relu(gu[:, :f]) ** 2 * gu[:, f:], atol=3e-2)
    # finalize + RoPE + KV append against the separate kernels
    H, Hkv, D, page, max_pages = 4, 2, 128, 16, 4
    Tt = 3
    acc = torch.randn(Tt, (H + 2 * Hkv) * D, device="cuda")
    qkv = acc.to(torch.bfloat16)
    pos = torch.tensor([5, 17, 0], device="cuda", dtype=torch.int32)
    sid = torch.arange(Tt, device="cuda", dtype=torch.int32)
    table = torch.randperm(Tt * max_pages).view(Tt, max_pages).to(torch.int32).cuda()
    kc = torch.zeros(Tt * max_pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(kc)
    q = torch.empty(Tt, H, D, device="cuda", dtype=torch.bfloat16)
    C.qkv_rope_append(acc, pos, sid, table, q, kc, vc, 10000.0)
    ref_qk = qkv[:, : (H + Hkv) * D].clone().unflatten(-1, (H + Hkv, D))
    C.rope(ref_qk, pos, 10000.0, False)
    C.kv_append(ref_qk[:, H:].contiguous(), qkv[:, (H + Hkv) * D:].unflatten(-1, (Hkv, D)).contiguous(), kc2, vc2,
                table, pos, sid)
    _close(q, ref_qk[:, :H], atol=2e-2)
    _close(kc, kc2, atol=2e-2)
    assert torch.equal(vc, vc2) and float(acc.abs().max()) == 0.0
    # the same epilogue writing int8 pages, against RoPE + the int8 append kernel
    for D8, Tt8 in ((128, 3), (64, 5)):
        acc = torch.randn(Tt8, (H + 2 * Hkv) * D8, device="cuda") * 2
        qkv = acc.to(torch.bfloat16)
        pos8 = torch.tensor([5, 17, 0, 33, 2][:Tt8], device="cuda", dtype=torch.int32)
        sid8 = torch.arange(Tt8, device="cuda", dtype=torch.int32)
        table8 = torch.randperm(Tt8 * max_pages).view(Tt8, max_pages).to(torch.int32).cuda()
        shape8 = (Tt8 * max_pages, page, Hkv, D8)
        k8, v8 = (torch.zeros(shape8, device="cuda", dtype=torch.int8) for _ in range(2))
        k8r, v8r = torch.zeros_like(k8), torch.zeros_like(v8)
        ks, vs, ksr, vsr = (torch.zeros(shape8[0] * page, Hkv, device="cuda") for _ in range(4))
        q8 = torch.empty(Tt8, H, D8, device="cuda", dtype=torch.bfloat16)
        C.qkv_rope_append(acc, pos8, sid8, table8, q8, k8, v8, 10000.0, ks, vs)
        ref_qk = qkv[:, : (H + Hkv) * D8].clone().unflatten(-1, (H + Hkv, D8))
        C.rope(ref_qk, pos8, 10000.0, False)
        C.kv_append_int8(ref_qk[:, H:].contiguous(), qkv[:, (H + Hkv) * D8:].unflatten(-1, (Hkv, D8)).contiguous(),
                         k8r, v8r, ksr, vsr, table8, pos8, sid8)
        _close(q8, ref_qk[:, :H], atol=2e-2)
        assert torch.equal(v8, v8r) and torch.equal(vs, vsr) and float(acc.abs().max()) == 0.0
        # K goes through sincosf in one kernel and the RoPE kernel's own evaluation in the other:
        # scales agree to bf16 rounding, codes to one step
        assert torch.allclose(ks, ksr, rtol=1e-2, atol=1e-6)
        assert int((k8.int() - k8r.int()).abs().max()) <= 2


def test_engine_greedy_matches_full_recompute():
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.train.param_store import ParamStore

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=320, oil_block_size=256, codebook_group=2)
    with torch.device("cuda"):
        model = DenseModel(cfg)
    eng = InferenceEngine.from_model(model, device="cuda", max_batch=4, max_seq_len=320)
    store = ParamStore(model, "cuda")
    store.refresh_compute()
    B, S, new = 2, 128, 6
    prompts = torch.randint(0, cfg.vocab_size, (B, S), dtype=torch.int32)
    res = eng.generate(prompts, max_new_tokens=new, use_graph=False)
    res_g = eng.generate(prompts, max_new_tokens=new, use_graph=True)
    assert res.tokens == res_g.tokens
    eng.fused_decode = False            # the unfused kernel sequence decodes (nearly) the same tokens
    res_u = eng.generate(prompts, max_new_tokens=new, use_graph=False)
    eng.fused_decode = True
    same = sum(a == b for ra, rb in zip(res.tokens, res_u.tokens) for a, b in zip(ra, rb))
    assert same >= B * new - 2
    seq = prompts.cuda()
    agree = 0
    with torch.no_grad():
        for i in range(new):
            logits = model(seq)[:, -1].float()
            nxt = logits.argmax(-1).to(torch.int32)
            got = torch.tensor([res.tokens[b][i] for b in range(B)], device="cuda", dtype=torch.int32)
            top2 = torch.topk(logits, 2, dim=-1).values
            for b in range(B):
                # accept either the reference argmax or a near-tie (bf16 accumulation order differs)
                if int(got[b]) == int(nxt[b]) or float(top2[b, 0] - logits[b, int(got[b])]) < 5e-2:
                    agree += 1
            seq = torch.cat([seq, got[:, None]], dim=1)
    assert agree == B * new
    assert res.stats.ttft_s > 0 and res.stats.tokens_per_s > 0


@pytest.mark.parametrize("fmt,K,bs", [("oil8", 4096, 256), ("oil4", 2048, 256), ("i2s", 2560, 256), ("oil8", 192, 64)])
def test_embedding_gather_through_quantised_table(fmt, K, bs):
    """Row gather that expands only the addressed rows, against the full dequantised table."""
    from mythos_b200.infer.quant_weights import QuantLinear

    g = torch.Generator(device="cuda").manual_seed(K)
    V = 1000
    table = QuantLinear.random(fmt, V, K, bs, 16, device="cuda", generator=g)
    full = table.dequantize()
    ids = torch.randint(-3, V + 3, (257,), device="cuda", dtype=torch.int32)
    out = table.gather_rows(ids)
    assert torch.equal(out, full[ids.long().clamp(0, V - 1)])
    # into a strided destination (row stride larger than K)
    wide = torch.zeros(ids.numel(), K + 64, device="cuda", dtype=torch.bfloat16)
    table.gather_rows(ids, wide[:, :K])
    assert torch.equal(wide[:, :K], out) and float(wide[:, K:].abs().max()) == 0.0


@pytest.mark.parametrize("H,Hkv,D,page", [(8, 2, 128, 16), (32, 8, 128, 16), (8, 1, 128, 16), (3, 3, 128, 16),
                                          (4, 4, 64, 16), (4, 1, 128, 32)])
def test_int8_kv_append_and_decode(H, Hkv, D, page):
    """int8 pages: the append kernel's scales and codes against abs-max / 127 rounding, and decode
    attention over the int8 pages against fp32 attention over the dequantised values. 16-token
    pages with head_dim 128 run the tensor-core kernel, the other shapes the scalar one."""
    from mythos_b200.ops import native, reference as ref

    C = native.require()
    torch.manual_seed(H + D + page)
    B, max_pages = 3, 256 // page
    lens = [37, 200, 1]
    n_pages = B * max_pages
    k8 = torch.randint(-128, 127, (n_pages, page, Hkv, D), device="cuda", dtype=torch.int8)   # stale contents
    v8 = torch.randint(-128, 127, (n_pages, page, Hkv, D), device="cuda", dtype=torch.int8)
    ksc = torch.rand(n_pages * page, Hkv, device="cuda")
    vsc = torch.rand(n_pages * page, Hkv, device="cuda")
    table = torch.randperm(n_pages).reshape(B, max_pages).to(torch.int32).cuda()
    kd, vd = [], []
    for b in range(B):
        k = (torch.randn(lens[b], Hkv, D, device="cuda") * (1 + b)).to(torch.bfloat16)
        v = torch.randn(lens[b], Hkv, D, device="cuda").to(torch.bfloat16)
        if b == 0:
            k[3, 0] = 0                      # an all-zero row quantises to zeros with scale 0
        pos = torch.arange(lens[b], device="cuda", dtype=torch.int32)
        sid = torch.full((lens[b],), b, device="cuda", dtype=torch.int32)
        C.kv_append_int8(k, v, k8, v8, ksc, vsc, table, pos, sid)
        rows = (table[b, (pos // page).long()].long() * page + (pos % page).long())
        for src, q8, sc, sink in ((k, k8, ksc, kd), (v, v8, vsc, vd)):
            amax = src.float().abs().amax(-1)
            got_scale = sc[rows]
            assert torch.allclose(got_scale, amax / 127.0, rtol=1e-6, atol=0)
            deq = q8.view(-1, Hkv, D)[rows].float() * got_scale[..., None]
            assert float((deq - src.float()).abs().max()) <= float(got_scale.max()) * 0.51 + 1e-6
            sink.append(deq)
    q = torch.randn(B, H, D, device="cuda").to(torch.bfloat16)
    ctx = torch.tensor(lens, device="cuda", dtype=torch.int32)
    for splits in (1, 3):
        out = torch.empty(B, H, D, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(B * H * splits * (D + 2), device="cuda")
        counters = torch.zeros(B * Hkv, device="cuda", dtype=torch.int32)
        C.paged_attn_decode_int8(q, k8, v8, ksc, vsc, table, ctx, out, scratch, counters, splits, 1.0 / math.sqrt(D),
                                 native.status_word("cuda"))
        for b in range(B):
            o, _ = ref.attention(q[b][None, None].float(), kd[b][None], vd[b][None], causal=False)
            _close(out[b], o[0, 0], atol=2e-2)
        assert int(counters.abs().sum()) == 0
    native.check_status("cuda")


def test_engine_int8_kv_tracks_bf16_kv():
    """Same weights, int8 against bf16 pages: the first decode steps pick (nearly) the same tokens."""
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.models import TransformerConfig

    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=320, oil_block_size=256, codebook_group=2,
                            embed_format="oil8")
    prompts = torch.randint(0, cfg.vocab_size, (2, 128), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    toks = {}
    for kind in ("bf16", "int8"):
        eng = InferenceEngine.random(cfg, seed=5, device="cuda", max_batch=4, max_seq_len=320, kv_dtype=kind)
        assert eng.cache.int8 == (kind == "int8")
        toks[kind] = eng.generate(prompts, max_new_tokens=6, use_graph=(kind == "int8")).tokens
    assert eng.cache.size_bytes() < 0.6 * 2 * cfg.num_layers * eng.cache.k[0].numel() * 2
    same = sum(a == b for ra, rb in zip(toks["bf16"], toks["int8"]) for a, b in zip(ra, rb))
    assert same >= 6, toks


@pytest.mark.parametrize("kv_dtype", ["bf16", "int8"])
def test_prefix_pages_are_shared_and_suffix_attends_over_them(kv_dtype):
    """A second request with the same prompt head maps the cached pages and computes only the
    rest through paged attention; its logits match a full recompute."""
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.models import TransformerConfig

    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=512, oil_block_size=256, codebook_group=2)
    eng = InferenceEngine.random(cfg, seed=11, device="cuda", max_batch=8, max_seq_len=512, kv_dtype=kv_dtype)
    g = torch.Generator().manual_seed(1)
    head = torch.randint(0, 512, (150,), generator=g).tolist()
    a, b = head + [5, 6, 7], head + [9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20]
    sa, la = eng.start_sequence(a)
    assert eng.last_prefix_hit == 0
    used = eng.cache.alloc.used
    sb, lb = eng.start_sequence(b)                     # 150 // 16 = 9 full pages are shared
    assert eng.last_prefix_hit == 144
    assert eng.cache.alloc.used == used + (len(b) + 15) // 16 - 9
    sc, lc = eng.start_sequence(b, reuse_prefix=False)  # full recompute of the same prompt
    assert eng.last_prefix_hit == 0
    tol = 6e-2 if kv_dtype == "bf16" else 1.5e-1
    assert float((lb.float() - lc.float()).abs().max()) < tol
    assert int(lb.float().argmax()) == int(lc.float().argmax()) or float((lb.float() - lc.float()).abs().max()) < 2e-2
    # both sequences keep decoding after the shared pages
    nb = eng.decode([sb, sc], [int(lb.float().argmax()), int(lc.float().argmax())])
    assert float((nb[0].float() - nb[1].float()).abs().max()) < 2 * tol
    for s in (sa, sb, sc):
        eng.release(s)
    assert eng.cache.alloc.used == 0


def test_repeated_launches_are_bit_identical():
    """Race check by repetition: kernels whose warps hand data to each other through shared-memory
    rings and barriers (dequant GEMM, flash attention, paged decode with a split merge) must give
    the same bits for the same inputs on every launch."""
    from mythos_b200.infer.quant_weights import QuantLinear
    from mythos_b200.ops import native

    C = native.require()
    st = native.status_word("cuda")
    torch.manual_seed(0)

    def repeat(fn, n):
        ref = fn().clone()
        return sum(0 if torch.equal(fn(), ref) else 1 for _ in range(n))

    for fmt, M, N, K in [("oil8", 256, 256, 512), ("oil4", 2, 512, 256), ("i2s", 200, 384, 512), ("oil8", 64, 1024, 2048)]:
        q = QuantLinear.from_float(torch.randn(N, K, device="cuda") * 0.02, fmt, block_size=256, codebook_group=2)
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        assert repeat(lambda: q.matmul(x, out=out, k_splits=1), 300) == 0, (fmt, M, N, K)
    B, S, H, D = 2, 256, 2, 128
    qkv = (torch.randn(B, S, 3 * H * D, device="cuda") * 0.5).to(torch.bfloat16)
    q4, k4, v4 = (qkv[..., i * H * D:(i + 1) * H * D].unflatten(-1, (H, D)) for i in range(3))
    o = torch.empty(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, S, device="cuda", dtype=torch.float32)

    def fwd():
        C.flash_attn_fwd(q4, k4, v4, o, lse, True, 1 / math.sqrt(D), st)
        return o

    assert repeat(fwd, 100) == 0
    Hkv, page, ctx_len = 2, 16, 700
    n_pages = 2 * 64
    kc = torch.randn(n_pages, page, Hkv, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(n_pages, page, Hkv, D, device="cuda").to(torch.bfloat16)
    table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(2, 64)
    lens = torch.tensor([ctx_len, 333], device="cuda", dtype=torch.int32)
    qd = torch.randn(2, 4, D, device="cuda").to(torch.bfloat16)
    od = torch.empty_like(qd)
    scratch = torch.empty(2 * 4 * 4 * (D + 2), device="cuda")
    counters = torch.zeros(2 * Hkv, device="cuda", dtype=torch.int32)

    def dec():
        C.paged_attn_decode(qd, kc, vc, table, lens, od, scratch, counters, 4, 1 / math.sqrt(D), st)
        return od

    assert repeat(dec, 200) == 0
    native.check_status("cuda")


def test_engine_text_api_load_batch_stream_reset(tmp_path):
    """load(.oil + .vocab) -> generate_with_stats / generate_batch / generate_stream / reset_context."""
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.oil.model_io import save_model
    from mythos_b200.train.bpe import BPETokenizer

    torch.manual_seed(0)
    tok = BPETokenizer()
    tok.train(b"the quick brown fox jumps over the lazy dog. " * 30, 300)
    cfg = TransformerConfig(vocab_size=320, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=256, oil_block_size=256, codebook_group=2)
    path = str(tmp_path / "m.oil")
    save_model(DenseModel(cfg), path)
    tok.save(str(tmp_path / "m.vocab"))
    eng = InferenceEngine.load(path, device="cuda", max_batch=4)
    assert eng.tokenizer is not None and eng.decode_text(eng.encode("the lazy dog")) == "the lazy dog"
    text, stats = eng.generate_with_stats("the quick brown", max_new_tokens=8)
    assert isinstance(text, str) and stats.new_tokens >= 1 and stats.ttft_s > 0 and stats.kv_bytes > 0
    prompts = ["the quick brown", "the lazy dog jumps", "the quick brown"]
    outs = eng.generate_batch(prompts, max_new_tokens=6)
    assert len(outs) == 3 and outs[0] == outs[2] and all(isinstance(o, str) for o in outs)
    pieces = []
    res = eng.generate_stream(eng.encode("the quick"), eng.decode_text, pieces.append, max_new_tokens=8)
    assert "".join(pieces) == "".join(eng.decode_text([t]) for t in res.tokens[0])
    seq, _ = eng.start_sequence(eng.encode("the quick brown fox jumps over the lazy dog."))
    assert eng.cache.alloc.used > 0
    eng.reset_context()
    assert eng.cache.alloc.used == 0 and not eng.cache.prefix_index


def test_row_signalled_sum_norm_single_rank_and_timeout():
    """The fused push + per-row flag + sum + residual + RMSNorm kernel with one rank (it signals and
    awaits its own flags; the epoch advances on the device), then with a second "rank" whose flags
    nobody sets: the bounded wait must give up and report instead of hanging."""
    from mythos_b200.ops import native, reference as ref

    C = native.require()
    torch.manual_seed(3)
    T, N, max_rows = 7, 2560, 16
    g = (torch.rand(N, device="cuda") + 0.5).to(torch.bfloat16)
    staging = torch.zeros(max_rows * N, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(2 * 1 * max_rows, device="cuda", dtype=torch.int32)
    epoch = torch.zeros(1, device="cuda", dtype=torch.int32)
    arrive = torch.zeros(1, device="cuda", dtype=torch.int32)
    st = native.status_word("cuda")
    for it in range(4):
        acc = torch.randn(T, N, device="cuda")
        res = torch.randn(T, N, device="cuda").to(torch.bfloat16)
        want_stream = (acc.to(torch.bfloat16).float() + res.float()).to(torch.bfloat16)
        stream, normed = torch.empty_like(res), torch.empty_like(res)
        C.tp_sum_residual_rmsnorm(acc, [staging.data_ptr()], [flags.data_ptr()], 0, max_rows * N, it & 1, max_rows, res, g,
                                  stream, normed, 1e-5, epoch, arrive, 2_000_000_000, st)
        assert torch.equal(stream, want_stream) and float(acc.abs().max()) == 0.0
        _close(normed, ref.rmsnorm(want_stream, g, 1e-5)[0], atol=2e-2)
        assert int(epoch) == it + 1 and int(arrive) == 0
    native.check_status("cuda")
    assert flags.view(2, max_rows)[:, :T].min().item() >= 3 and int(flags.view(2, max_rows)[:, T:].abs().sum()) == 0
    # slots already stored by the producer (no accumulator): only signal, wait and reduce
    staging.view(max_rows, N)[:T] = torch.ones(T, N, device="cuda", dtype=torch.bfloat16)
    C.tp_sum_residual_rmsnorm(None, [staging.data_ptr()], [flags.data_ptr()], 0, max_rows * N, 0, max_rows, None, g, stream,
                              normed, 1e-5, epoch, arrive, 2_000_000_000, st)
    assert float((stream.float() - 1).abs().max()) == 0.0
    # two ranks, the peer never signals: every row times out, outputs are left alone, status is set
    staging2 = torch.zeros(2 * max_rows * N, device="cuda", dtype=torch.bfloat16)
    peer_staging = torch.zeros_like(staging2)
    fa = torch.zeros(2 * 2 * max_rows, device="cuda", dtype=torch.int32)
    fb = torch.zeros_like(fa)
    stream.fill_(7.0)
    C.tp_sum_residual_rmsnorm(torch.randn(T, N, device="cuda"), [staging2.data_ptr(), peer_staging.data_ptr()],
                              [fa.data_ptr(), fb.data_ptr()], 0, max_rows * N, 0, max_rows, None, g, stream, normed, 1e-5,
                              epoch, arrive, 2_000_000, st)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 1"):
        native.check_status("cuda")
    native.check_status("cuda")  # cleared
    assert float((stream.float() - 7).abs().max()) == 0.0
    assert int(fb.view(2, 2, max_rows)[0, 0, :T].min()) == int(epoch)        # the peer was still signalled
    assert float(peer_staging.view(2, max_rows, N)[0, :T].float().abs().max()) > 0   # and received the rows


def test_zero_padded_ffn_shard_equals_the_unpadded_one():
    """An I2_S FFN shard whose width is not a multiple of the GEMM's K granule is padded with zero
    trits; slicing the padding away again must not change the logits."""
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.infer.quant_weights import QuantLinear
    from mythos_b200.models import TransformerConfig

    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=192, max_seq_len=256, activation="relu2", gated_ffn=True,
                            weight_format="i2s", embed_format="fp16", oil_block_size=64)
    f, fp = 192, 256
    padded = InferenceEngine.random(cfg, seed=9, device="cuda", max_batch=4, max_seq_len=256, ffn_multiple=128)
    sliced = InferenceEngine.random(cfg, seed=9, device="cuda", max_batch=4, max_seq_len=256, ffn_multiple=128)
    for Lp, Ls in zip(padded.layers, sliced.layers):
        assert Lp.up.N == 2 * fp and Lp.down.K == fp
        up_rows = Lp.up.packed.view(2 * fp, -1)
        assert int((up_rows[f:fp] != 0x55).sum()) == 0 and int((up_rows[fp + f:] != 0x55).sum()) == 0
        assert int((Lp.down.packed.view(256, -1)[:, f // 4:] != 0x55).sum()) == 0
        keep = torch.cat([up_rows[:f], up_rows[fp:fp + f]]).contiguous().view(-1)
        up_scales = Lp.up.scales.view(2 * fp, -1)
        Ls.up = QuantLinear("i2s", 2 * f, 256, 64, keep,
                            scales=torch.cat([up_scales[:f], up_scales[fp:fp + f]]).contiguous().view(-1))
        down_bytes = Lp.down.packed.view(256, -1)[:, : f // 4].contiguous().view(-1)
        down_scales = Lp.down.scales.view(256, -1)[:, : f // 64].contiguous().view(-1)
        Ls.down = QuantLinear("i2s", 256, f, 64, down_bytes, scales=down_scales)
    prompt = torch.randint(0, 512, (40,), generator=torch.Generator().manual_seed(4)).tolist()
    sp, lp = padded.start_sequence(prompt, reuse_prefix=False)
    ss, ls = sliced.start_sequence(prompt, reuse_prefix=False)
    assert float((lp.float() - ls.float()).abs().max()) < 2e-2 and int(lp.float().argmax()) == int(ls.float().argmax())
    tok = int(lp.float().argmax())
    dp, ds = padded.decode([sp], [tok]), sliced.decode([ss], [tok])
    assert float((dp.float() - ds.float()).abs().max()) < 2e-2
    with pytest.raises(ValueError, match="I2_S"):
        InferenceEngine.random(TransformerConfig(vocab_size=512, hidden_size=256, num_layers=1, num_heads=2, head_dim=128,
                                                 ffn_hidden_size=192, max_seq_len=64, weight_format="oil8",
                                                 oil_block_size=64), seed=1, device="cuda", max_batch=2, max_seq_len=64,
                               ffn_multiple=128)


@pytest.mark.parametrize("H,Hkv,D", [(4, 2, 128), (2, 2, 64)])
def test_paged_prefill_attention_ragged_prefix_and_partial_pages(H, Hkv, D):
    """tcgen05 prefill attention reading K/V from 16-token pages through the block table: ragged
    batch, queries that start after a cached prefix, last pages partly filled; against the fp32
    reference attention over prefix + chunk."""
    from mythos_b200.ops import native, reference as ref

    C = native.require()
    torch.manual_seed(H * 10 + D)
    prefix = [0, 37, 300, 16]                  # cached tokens before the new ones
    new = [70, 300, 5, 129]                    # new (query) tokens per sequence
    B = len(new)
    pages_per = [(p + n + 15) // 16 for p, n in zip(prefix, new)]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages)[: sum(pages_per)].tolist()
    table = torch.zeros(B, max(pages_per) + 2, dtype=torch.int32)
    kc = torch.zeros(n_pages, 16, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    ks, vs, qs = [], [], []
    it = iter(perm)
    for b in range(B):
        L = prefix[b] + new[b]
        k = (torch.randn(L, Hkv, D) * 0.5).to(torch.bfloat16)
        v = (torch.randn(L, Hkv, D) * 0.5).to(torch.bfloat16)
        q = (torch.randn(new[b], H, D) * 0.5).to(torch.bfloat16)
        for lp in range(pages_per[b]):
            pg = next(it)
            table[b, lp] = pg
            n = min(16, L - lp * 16)
            kc[pg, :n] = k[lp * 16: lp * 16 + n].cuda()
            vc[pg, :n] = v[lp * 16: lp * 16 + n].cuda()
        ks.append(k); vs.append(v); qs.append(q)
    q_all = torch.cat(qs).cuda()
    cu_q = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device="cuda")
    kv_lens = torch.tensor([p + n for p, n in zip(prefix, new)], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q_all)
    C.flash_attn_paged_prefill(q_all, kc, vc, table.cuda(), cu_q, kv_lens, out, max(new), D ** -0.5,
                               native.status_word("cuda"))
    torch.cuda.synchronize()
    off = 0
    for b in range(B):
        L, n = prefix[b] + new[b], new[b]
        qf = torch.zeros(1, L, H, D)
        qf[0, prefix[b]:] = qs[b].float()
        o_ref, _ = ref.attention(qf, ks[b].float()[None], vs[b].float()[None], True, D ** -0.5)
        got = out[off:off + n].float().cpu()
        want = o_ref[0, prefix[b]:]
        assert (got - want).abs().max() < 3e-2, (b, float((got - want).abs().max()))
        off += n


def test_chunked_paged_prefill_and_ragged_generate_match_contiguous_prefill():
    """A prompt prefilled in chunks through the paged kernel, a prompt continued after a cached
    prefix, and a ragged batch give the logits / first tokens of the contiguous one-pass prefill."""
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.models import DenseModel, TransformerConfig

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=512, oil_block_size=256, codebook_group=2)
    with torch.device("cuda"):
        model = DenseModel(cfg)
    eng = InferenceEngine.from_model(model, device="cuda", max_batch=4, max_seq_len=512)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (200,), generator=g).tolist()
    s0, l0 = eng.start_sequence(ids, reuse_prefix=False)            # contiguous flash-attention prefill
    eng.prefill_chunk = 64                                           # 200 tokens -> four paged passes
    s1, l1 = eng.start_sequence(ids, reuse_prefix=False)
    scale = float(l0.float().abs().max())
    assert float((l0.float() - l1.float()).abs().max()) < 3e-2 * scale
    assert int(l0.float().argmax()) == int(l1.float().argmax())
    # continuation after a cached prefix: 160 shared tokens (10 pages), 40 new ones through the prefill kernel
    eng.reset_context()
    eng.prefill_chunk = 8192
    sa, _ = eng.start_sequence(ids[:170], reuse_prefix=True)
    sb, lb = eng.start_sequence(ids, reuse_prefix=True)
    assert eng.last_prefix_hit == 160
    assert float((l0.float() - lb.float()).abs().max()) < 3e-2 * scale
    # ragged batch: first generated token of every prompt equals the single-sequence result
    eng.reset_context()
    lens = [70, 128, 33]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    want = []
    for p in prompts:
        s, lg = eng.start_sequence(p, reuse_prefix=False)
        want.append(int(lg.float().argmax()))
        eng.release(s)
    res = eng.generate(prompts, max_new_tokens=4, use_graph=False)
    assert [t[0] for t in res.tokens] == want
    res_g = eng.generate(prompts, max_new_tokens=4, use_graph=True)
    assert res_g.tokens == res.tokens


def test_zero_padded_heads_keep_the_model_function():
    """An engine built for a tensor-parallel size that does not divide the head count pads heads with
    zeros. Emulated on one GPU: the padded shards of both "ranks" of a 3-head model (padded to 4) are
    packed, and rank-wise partial attention outputs summed must equal the unpadded engine's logits."""
    from mythos_b200.infer import engine as E
    from mythos_b200.models import DenseModel, TransformerConfig

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=256, hidden_size=256, num_layers=1, num_heads=3, head_dim=128,
                            ffn_hidden_size=256, max_seq_len=128, oil_block_size=64, weight_format="i2s")
    with torch.device("cuda"):
        model = DenseModel(cfg)

    class FakeTP:                       # what the constructor reads from a TPContext
        def __init__(self, rank):
            self.rank, self.world, self.max_tokens = rank, 2, 256

    engines = []
    for r in range(2):
        eng = E.InferenceEngine.__new__(E.InferenceEngine)
        E.InferenceEngine.__init__(eng, cfg, device="cuda", max_batch=2, max_seq_len=128, tp=FakeTP(r))
        assert (eng.h_eff, eng.h_local) == (4, 2)
        engines.append(eng)
    # pack the padded shards the way from_model does and check them against the float weights
    att = model.layers[0].attention
    wq = att.qkv_proj.weight.detach().float()
    D, H = 128, 3
    full_q = E._pad_rows(wq, 0, H * D, 4 * D)
    assert full_q.shape[0] == 4 * D and float(full_q[H * D:].abs().max()) == 0.0
    ids = torch.randint(0, 256, (1, 64), dtype=torch.int32)
    single = E.InferenceEngine.from_model(model, device="cuda", max_batch=2, max_seq_len=128)
    ref = single.generate(ids, max_new_tokens=3, use_graph=False)
    assert len(ref.tokens[0]) == 3
    # synthetic engine with padded heads: padded rows / columns are exact zeros
    synth = E.InferenceEngine.random(cfg, seed=1, device="cuda", max_batch=2, max_seq_len=128, tp=None)
    assert synth.h_eff == 3
    e1 = engines[1]
    qkv = E.QuantLinear.random("i2s", (e1.h_local + 2 * e1.hkv_local) * D, 256, 64, 1, device="cuda",
                               generator=torch.Generator(device="cuda").manual_seed(0))
    o = E.QuantLinear.random("i2s", 256, e1.h_local * D, 64, 1, device="cuda",
                             generator=torch.Generator(device="cuda").manual_seed(1))
    E._zero_padded_heads(qkv, o, e1, cfg)
    x = torch.randn(4, 256, device="cuda").to(torch.bfloat16)
    y = qkv.matmul(x).float()
    hl = e1.h_local
    assert float(y[:, 1 * D: hl * D].abs().max()) == 0.0                      # padded q head (global head 3)
    assert float(y[:, hl * D + D: 2 * hl * D].abs().max()) == 0.0             # padded k head
    assert float(y[:, 2 * hl * D + D:].abs().max()) == 0.0                    # padded v head
    z = torch.zeros(4, hl * D, device="cuda", dtype=torch.bfloat16)
    z[:, D:] = 1.0                                                            # only the padded head's slots are non-zero
    assert float(o.matmul(z).float().abs().max()) == 0.0
