"""Memory-bound kernels and flash attention against fp32 PyTorch references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    lim = atol + rtol * b.abs().max().item()
    assert err <= lim, f"max err {err} > {lim}"


@pytest.mark.parametrize("rows,dim", [(7, 256), (1024, 2048), (33, 4096), (5, 14336)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(rows, dim, with_res):
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(rows + dim)
    x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    r = torch.randn(rows, dim, device="cuda").to(torch.bfloat16) if with_res else None
    g = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
    xg = x.clone().requires_grad_()
    gg = g.clone().requires_grad_()
    y, h = F.rmsnorm(xg, gg, 1e-5, r)
    yr, hr = ref.rmsnorm(x, g, 1e-5, r)
    _close(y, yr)
    _close(h, hr)
    dy = torch.randn_like(y)
    y.backward(dy)
    hf = hr.float().requires_grad_()
    gf = g.float().requires_grad_()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5)
    (hf * rstd * gf).backward(dy.float())
    _close(xg.grad, hf.grad, atol=3e-2)
    _close(gg.grad, gf.grad, rtol=3e-2, atol=0.15)


@pytest.mark.parametrize("D", [64, 128])
def test_rope_matches_formula(D):
    from mythos_b200.ops import native, reference as ref

    torch.manual_seed(D)
    T, H = 50, 3
    buf = torch.randn(T, H * D + 32, device="cuda").to(torch.bfloat16)
    x = buf[:, : H * D].unflatten(-1, (H, D))
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    want = ref.rope(x.clone(), pos, 10000.0)
    orig = x.clone()
    native.require().rope(x, pos, 10000.0, False)
    _close(x, want, atol=2e-2)
    native.require().rope(x, pos, 10000.0, True)
    _close(x, orig, atol=3e-2)


def test_swiglu_relu2_and_activations():
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(3)
    gu = torch.randn(37, 2 * 5504, device="cuda").to(torch.bfloat16).requires_grad_()
    out = F.swiglu(gu)
    _close(out, ref.swiglu(gu.detach()))
    d = torch.randn_like(out)
    out.backward(d)
    gr = gu.detach().float().requires_grad_()
    f = gr.shape[-1] // 2
    (gr[:, :f] * torch.sigmoid(gr[:, :f]) * gr[:, f:]).backward(d.float())
    _close(gu.grad, gr.grad, atol=4e-2)
    x = torch.randn(64, 1024, device="cuda").to(torch.bfloat16).requires_grad_()
    y = F.relu2(x)
    _close(y, ref.relu2(x.detach()))
    y.backward(torch.ones_like(y))
    _close(x.grad, 2 * torch.relu(x.detach().float()))
    with torch.no_grad():
        for kind, fn in [("gelu", ref.gelu_erf), ("gelu_tanh", ref.gelu_tanh), ("sigmoid", torch.sigmoid),
                         ("tanh", torch.tanh), ("relu", torch.relu)]:
            _close(F.activation(x.detach(), kind), fn(x.detach().float()))
        _close(F.layernorm(x.detach(), torch.ones(1024, device="cuda", dtype=torch.bfloat16)),
               ref.layernorm(x.detach(), torch.ones(1024, device="cuda")))


def test_embedding_fwd_bwd():
    from mythos_b200.ops import functional as F

    torch.manual_seed(4)
    V, D = 1000, 256
    table = torch.randn(V, D, device="cuda").to(torch.bfloat16).requires_grad_()
    ids = torch.randint(0, V, (3, 77), device="cuda", dtype=torch.int32)
    gt = torch.zeros(V, D, device="cuda")
    out = F.embedding(ids, table, gt)
    assert torch.equal(out, table.detach()[ids.long()])
    d = torch.randn_like(out)
    out.backward(d)
    want = torch.zeros(V, D, device="cuda").index_add_(0, ids.reshape(-1).long(), d.reshape(-1, D).float())
    _close(gt, want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("rows,V", [(64, 32000), (9, 1003), (16, 128256)])
def test_cross_entropy_fused(rows, V):
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(V)
    logits = (torch.randn(rows, V, device="cuda") * 3).to(torch.bfloat16)
    pad = (8 - V % 8) % 8
    buf = torch.zeros(rows, V + pad, device="cuda", dtype=torch.bfloat16)
    buf[:, :V] = logits
    lg = buf[:, :V].requires_grad_()
    tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    want = ref.cross_entropy(logits, tg).sum() / rows
    wgrad = ref.cross_entropy_grad(logits, tg, 1.0 / rows)
    loss = F.cross_entropy(lg, tg)
    loss.backward()
    assert abs(loss.item() - want.item()) < 2e-3 * max(1.0, abs(want.item()))
    _close(lg.grad, wgrad, atol=2e-3 / rows + 1e-4)


@pytest.mark.parametrize("rows,V,W", [(32, 32000, 4), (9, 2006, 2), (16, 128256, 8)])
def test_cross_entropy_vocab_shards(rows, V, W):
    """Sharded cross-entropy: W column shards on one GPU, records merged on the host side of the
    op, against the fp32 closed form over full rows."""
    from mythos_b200.ops import reference as ref
    from mythos_b200.parallel import vocab_ce

    torch.manual_seed(V + W)
    logits = (torch.randn(rows, V, device="cuda") * 3).to(torch.bfloat16)
    tg = torch.randint(-1, V + 2, (rows,), device="cuda", dtype=torch.int32)
    tg_c = tg.clamp(0, V - 1)
    want = ref.cross_entropy(logits, tg_c)
    wgrad = ref.cross_entropy_grad(logits, tg_c, 1.0 / rows)
    v = V // W
    shards = []
    for r in range(W):                       # row stride padded to a multiple of 8 elements
        buf = torch.zeros(rows, (v + 7) // 8 * 8, device="cuda", dtype=torch.bfloat16)
        buf[:, :v] = logits[:, r * v:(r + 1) * v]
        shards.append(buf[:, :v])
    stats = torch.stack([vocab_ce.shard_stats(sh, tg, r * v, V) for r, sh in enumerate(shards)])
    lse, tgt = vocab_ce.merge_stats(stats)
    _close(lse - tgt, want, atol=2e-3, rtol=2e-3)
    for r, sh in enumerate(shards):
        vocab_ce.shard_grad_(sh, tg, lse, r * v, V, 1.0 / rows)
        _close(sh, wgrad[:, r * v:(r + 1) * v], atol=2e-3 / rows + 1e-4)
    # single-rank autograd path
    buf = torch.zeros(rows, (V + 7) // 8 * 8, device="cuda", dtype=torch.bfloat16)
    buf[:, :V] = logits
    lg = buf[:, :V].requires_grad_()
    loss = vocab_ce.vocab_parallel_cross_entropy(lg, tg_c)
    loss.backward()
    assert abs(loss.item() - want.mean().item()) < 2e-3 * max(1.0, want.mean().item())
    _close(lg.grad, wgrad, atol=2e-3 / rows + 1e-4)


def test_adamw_and_sumsq():
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(5)
    n = 100003
    p = torch.randn(n, device="cuda")
    m = torch.randn(n, device="cuda") * 0.01
    v = torch.rand(n, device="cuda") * 0.01
    g = torch.randn(n, device="cuda")
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    ref.adamw_step(pr, mr, vr, g, 3e-4, 0.9, 0.999, 1e-8, 0.01, 7, 0.5)
    clip = torch.tensor([0.5], device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    F.adamw_step(p, m, v, g, lr=3e-4, step=7, clip_coef=clip, p_bf16=pb)
    assert torch.allclose(p, pr, rtol=1e-5, atol=1e-6)
    assert torch.allclose(m, mr, rtol=1e-5, atol=1e-7)
    assert torch.allclose(v, vr, rtol=1e-5, atol=1e-7)
    assert torch.equal(pb, p.to(torch.bfloat16))
    ss = F.sumsq(g)
    assert abs(ss.item() - g.double().pow(2).sum().item()) < 1e-3 * n


@pytest.mark.parametrize("fmt,bs,group", [("oil8", 64, 1), ("oil8", 256, 16), ("oil4", 256, 4)])
def test_fake_quant_matches_bruteforce(fmt, bs, group):
    from mythos_b200.oil import codebook as cbk
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(bs + group)
    n = bs * 37 + 11
    w = torch.randn(n, device="cuda") * 0.02
    size = 256 if fmt == "oil8" else 16
    nb = (n + bs - 1) // bs
    ncb = (nb + group - 1) // group
    cb = cbk.quantile_codebook(size, 0.02, fp16=(fmt == "oil4")).cuda()[None].repeat(ncb, 1)
    cb = (cb * (1 + 0.1 * torch.rand(ncb, 1, device="cuda"))).contiguous()
    cmap = (torch.arange(nb, device="cuda") // group).to(torch.int32) if group > 1 else None
    wq, idx = F.oil_fake_quant(w, cb, cmap, bs, want_idx=True)
    ridx, rdeq = ref.nearest_centroid(w, cb, cmap, bs)
    assert torch.equal(idx, ridx)
    assert torch.equal(wq, rdeq.to(torch.bfloat16))


def test_i2s_fake_quant():
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(6)
    w = torch.randn(256 * 9 + 5, device="cuda") * 0.02
    wq, codes, scales = F.i2s_fake_quant(w, 256, want_codes=True)
    rc, rs, rd = ref.i2s_quant(w, 256)
    assert torch.allclose(scales, rs, rtol=1e-5)
    assert (codes != rc).float().mean().item() < 1e-3  # round-half ties may differ by one ulp of w/scale
    _close(wq, rd, atol=1e-3)


@pytest.mark.parametrize("B,S,H,Hkv,D,causal", [
    (1, 256, 2, 2, 128, True), (2, 512, 4, 2, 128, True), (1, 300, 2, 1, 128, True), (1, 384, 2, 2, 128, False),
    (2, 256, 4, 4, 64, True), (1, 2048, 2, 2, 128, True), (3, 1000, 5, 5, 128, True)])
@pytest.mark.parametrize("mode", [0, 1])
def test_flash_attention_forward(B, S, H, Hkv, D, causal, mode):
    """mode 0: the first forward kernel; mode 1: the persistent 128 x 128 kernel with P in tensor memory
    (head_dim 128; other shapes fall back to the first kernel)."""
    from mythos_b200.ops import functional as F, native, reference as ref

    torch.manual_seed(S + H)
    q = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16)
    C = native.require()
    before = C.get_attn_fwd_mode()
    C.set_attn_fwd_mode(mode)
    try:
        o, lse = F.flash_attention(q, k, v, causal)
        torch.cuda.synchronize()
    finally:
        C.set_attn_fwd_mode(before)
    orf, lser = ref.attention(q, k, v, causal)
    _close(o, orf, atol=2e-2)
    assert torch.allclose(lse, lser, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("B,S,H,Hkv,D", [(1, 256, 2, 2, 128), (2, 384, 4, 2, 128), (1, 200, 2, 1, 128),
                                        (1, 1024, 2, 2, 128), (2, 256, 4, 2, 64), (1, 200, 3, 3, 64)])
def test_attention_qkv_forward_backward(B, S, H, Hkv, D):
    """RoPE + flash attention over a fused projection, gradients against autograd of the naive form.
    Head dimension 64 runs the backward kernel on zero-padded heads."""
    from mythos_b200.ops import functional as F, reference as ref

    torch.manual_seed(S)
    W = (H + 2 * Hkv) * D
    qkv = (torch.randn(B, S, W, device="cuda") * 0.5).to(torch.bfloat16)
    pos = torch.arange(S, device="cuda", dtype=torch.int32).repeat(B)
    x = qkv.clone().requires_grad_()
    o = F.attention_qkv(x, pos, H, Hkv, D, 10000.0, True)
    do = torch.randn_like(o)
    o.backward(do)

    xr = qkv.float().requires_grad_()
    qf = xr[..., : H * D].reshape(B * S, H, D)
    kf = xr[..., H * D:(H + Hkv) * D].reshape(B * S, Hkv, D)
    vf = xr[..., (H + Hkv) * D:].reshape(B, S, Hkv, D)
    qf, kf = ref.rope(qf, pos, 10000.0), ref.rope(kf, pos, 10000.0)
    orf, _ = ref.attention(qf.reshape(B, S, H, D), kf.reshape(B, S, Hkv, D), vf, True)
    orf = orf.reshape(B, S, H * D)
    orf.backward(do.float())
    _close(o, orf, atol=2e-2)
    _close(x.grad, xr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("B,S,H,Hkv", [(2, 320, 4, 2), (1, 200, 2, 2)])
def test_attention_backward_undoes_rope_in_kernel(B, S, H, Hkv):
    """With a position bound the backward kernel rotates dq (in the fp32 -> bf16 conversion) and dk (in
    its epilogue) back itself; the gradients must match autograd of the naive fp32 form."""
    from mythos_b200.ops import functional as F, reference as ref

    D = 128
    torch.manual_seed(S + 1)
    W = (H + 2 * Hkv) * D
    qkv = (torch.randn(B, S, W, device="cuda") * 0.5).to(torch.bfloat16)
    pos = torch.arange(S, device="cuda", dtype=torch.int32).repeat(B)
    x = qkv.clone().requires_grad_()
    o = F.attention_qkv(x, pos, H, Hkv, D, 10000.0, True, rope_max_pos=S)
    do = torch.randn_like(o)
    o.backward(do)

    xr = qkv.float().requires_grad_()
    qf = xr[..., : H * D].reshape(B * S, H, D)
    kf = xr[..., H * D:(H + Hkv) * D].reshape(B * S, Hkv, D)
    vf = xr[..., (H + Hkv) * D:].reshape(B, S, Hkv, D)
    qf, kf = ref.rope(qf, pos, 10000.0), ref.rope(kf, pos, 10000.0)
    orf, _ = ref.attention(qf.reshape(B, S, H, D), kf.reshape(B, S, Hkv, D), vf, True)
    orf.reshape(B, S, H * D).backward(do.float())
    _close(x.grad, xr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("rows,dim,with_beta", [(33, 256, True), (700, 2048, False), (5, 6144, True)])
def test_layernorm_forward_backward(rows, dim, with_beta):
    from mythos_b200.ops import functional as F

    torch.manual_seed(dim)
    x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    g = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
    b = (0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16) if with_beta else None
    xs, gs = x.clone().requires_grad_(), g.clone().requires_grad_()
    bs = b.clone().requires_grad_() if with_beta else None
    y = F.layernorm(xs, gs, bs, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, gr = x.float().requires_grad_(), g.float().requires_grad_()
    br = b.float().requires_grad_() if with_beta else None
    yr = torch.nn.functional.layer_norm(xr, (dim,), gr, br, 1e-5)
    yr.backward(dy.float())
    _close(y, yr, atol=3e-2)
    _close(xs.grad, xr.grad, rtol=3e-2, atol=3e-2)
    _close(gs.grad, gr.grad, rtol=3e-2, atol=0.02 * max(1.0, rows ** 0.5))
    if with_beta:
        _close(bs.grad, br.grad, rtol=3e-2, atol=0.02 * max(1.0, rows ** 0.5))


@pytest.mark.parametrize("kind", ["relu", "gelu", "gelu_tanh", "silu", "sigmoid", "tanh"])
def test_activation_backward(kind):
    from mythos_b200.ops import functional as F

    torch.manual_seed(3)
    x = (2 * torch.randn(64, 264, device="cuda")).to(torch.bfloat16)
    xs = x.clone().requires_grad_()
    y = F.activation(xs, kind)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.float().requires_grad_()
    ref = {"relu": torch.relu, "gelu": torch.nn.functional.gelu,
           "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
           "silu": torch.nn.functional.silu, "sigmoid": torch.sigmoid, "tanh": torch.tanh}[kind]
    yr = ref(xr)
    yr.backward(dy.float())
    _close(y, yr, atol=2e-2)
    _close(xs.grad, xr.grad, rtol=2e-2, atol=2e-2)


def test_softmax_forward_backward():
    from mythos_b200.ops import functional as F

    torch.manual_seed(4)
    x = torch.randn(37, 1000, device="cuda").to(torch.bfloat16)
    xs = x.clone().requires_grad_()
    y = F.softmax(xs)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.float().requires_grad_()
    yr = torch.softmax(xr, dim=-1)
    yr.backward(dy.float())
    _close(y, yr, atol=1e-3)
    _close(xs.grad, xr.grad, rtol=3e-2, atol=1e-3)


def test_b200_backend_surface_matches_host():
    from mythos_b200.utils import backend as bk

    dev, host = bk.B200Backend(), bk.HostBackend()
    assert dev.is_available() and isinstance(bk.select_optimal_backend(), bk.B200Backend)
    torch.manual_seed(0)
    A = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
    B = torch.randn(128, 96, device="cuda").to(torch.bfloat16)
    C = torch.zeros(64, 96, device="cuda")
    dev.gemm(1.0, A, B, 0.0, C)
    assert (C - A.float() @ B.float()).abs().max() < 0.5
    y = torch.zeros(64, device="cuda")
    dev.gemv(1.0, A, torch.ones(128, device="cuda", dtype=torch.bfloat16), 0.0, y)
    assert (y - A.float().sum(1)).abs().max() < 0.5
    x = torch.randn(32, 256, device="cuda").to(torch.bfloat16)
    g = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    for name, args in (("softmax", (x,)), ("rms_norm", (x, g)), ("relu", (x,)), ("gelu", (x,)), ("silu", (x,))):
        a = getattr(dev, name)(*args).float()
        b = getattr(host, name)(*[t.float() for t in args]).float()
        assert (a - b).abs().max() < 3e-2, name
    assert dev.memory_free() > 0 and dev.memory_total() >= dev.memory_free()
    r = bk.benchmark_operation(dev, "gemm", 1024, 3)
    assert r["gflops"] > 1000


def test_kernel_c_abi_through_ctypes():
    """libmythos_kernels.so: the launchers behind a plain C ABI, called with raw device pointers."""
    import ctypes
    import os

    import mythos_b200
    from mythos_b200.ops import reference as ref

    path = os.path.join(os.path.dirname(mythos_b200.__file__), "libmythos_kernels.so")
    if not os.path.exists(path):
        pytest.skip("libmythos_kernels.so not built")
    lib = ctypes.CDLL(path)
    lib.mythos_last_error.restype = ctypes.c_char_p
    vp, ll, i32, f32 = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    torch.manual_seed(0)
    x = torch.randn(64, 512, device="cuda").to(torch.bfloat16)
    g = (torch.rand(512, device="cuda") + 0.5).to(torch.bfloat16)
    y = torch.empty_like(x)
    stream = vp(torch.cuda.current_stream().cuda_stream)
    lib.mythos_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, f32, vp]
    rc = lib.mythos_rmsnorm_fwd(x.data_ptr(), None, g.data_ptr(), y.data_ptr(), None, None, 64, 512, 1e-5, stream)
    assert rc == 0, lib.mythos_last_error()
    torch.cuda.synchronize()
    want = ref.rmsnorm(x, g, 1e-5)[0]
    assert (y.float() - want.float()).abs().max() < 3e-2
    a = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    b = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    c = torch.empty(128, 64, device="cuda", dtype=torch.bfloat16)
    lib.mythos_gemm_bf16.argtypes = [vp, ll, i32, vp, ll, i32, vp, ll, i32, i32, i32, i32, f32, vp, vp]
    rc = lib.mythos_gemm_bf16(a.data_ptr(), 256, 0, b.data_ptr(), 256, 0, c.data_ptr(), 64, 128, 64, 256, 0, 1.0,
                              None, stream)
    assert rc == 0, lib.mythos_last_error()
    torch.cuda.synchronize()
    assert (c.float() - a.float() @ b.float().t()).abs().max() < 0.5
    rc = lib.mythos_gemm_bf16(a.data_ptr(), 255, 0, b.data_ptr(), 256, 0, c.data_ptr(), 64, 128, 64, 256, 0, 1.0,
                              None, stream)
    assert rc != 0 and len(lib.mythos_last_error()) > 0        # misaligned row stride is reported, not launched


@pytest.mark.parametrize("group", [2, 3])
def test_ternary_lut_gemm_kernels_match_integer_reference(group):
    """TL1 / TL2 table kernels: int8 activations, exact int32 accumulation, against the direct integer
    product and the CPU table formulation."""
    from mythos_b200.oil import ternary_kernels as tk

    torch.manual_seed(group)
    M, N, K = 5, 300, 2556 if group == 3 else 2560
    K = K // 12 * 12
    trits = torch.randint(-1, 2, (N, K))
    x = torch.randn(M, K)
    packed = tk.pack_trits(trits)
    fn = tk.tl1_gemm if group == 2 else tk.tl2_gemm
    want = tk.ternary_reference(trits, x)
    cpu = fn(packed, x, K)
    got = fn(packed.cuda(), x.cuda(), K).cpu()
    assert torch.allclose(cpu, want, rtol=1e-6, atol=1e-5)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-4)
