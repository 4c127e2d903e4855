"""tcgen05 GEMM against an fp32 PyTorch reference of the same product (all three operand
layouts, every epilogue, ragged M/N/K)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= 2e-2 * scale + 1e-3, f"max err {err} vs scale {scale} (K={K})"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 1000, 200), (4096, 2048, 2048),
                                   (136, 144, 72), (8192, 5504, 2048)])
@pytest.mark.parametrize("layout", ["kk", "kmn", "mnmn"])
def test_gemm_layouts(M, N, K, layout):
    from mythos_b200.ops import functional as F

    torch.manual_seed(M + N + K)
    a_mn, b_mn = {"kk": (False, False), "kmn": (False, True), "mnmn": (True, True)}[layout]
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
    out = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _check(out, _ref(a, b, a_mn, b_mn), K)


def test_gemm_epilogues():
    from mythos_b200.ops import functional as F

    torch.manual_seed(0)
    M, N, K = 512, 768, 4096
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    o32 = F.gemm(a, b, epi=F.EPI_F32)
    _check(o32, ref, K)
    acc = torch.ones(M, N, device="cuda")
    F.gemm(a, b, out=acc, epi=F.EPI_F32_ACC)
    _check(acc, ref + 1.0, K)
    at = torch.full((M, N), 2.0, device="cuda")
    F.gemm(a, b, out=at, epi=F.EPI_F32_ATOMIC)
    _check(at, ref + 2.0, K)
    half = F.gemm(a, b, alpha=0.5)
    _check(half, 0.5 * ref, K)


def test_gemm_strided_views():
    """Operands that are column slices of a wider buffer (fused projections)."""
    from mythos_b200.ops import functional as F

    torch.manual_seed(1)
    big = torch.randn(300, 1024, device="cuda").to(torch.bfloat16)
    a = big[:, 256:768]
    w = torch.randn(640, 512, device="cuda").to(torch.bfloat16)
    out = F.gemm(a, w)
    _check(out, a.float() @ w.float().t(), 512)


def test_linear_autograd_matches_reference():
    from mythos_b200.ops import functional as F

    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    gt = torch.zeros(384, 256, device="cuda")
    y = F.linear(x, w, gt)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    _check(y, yr.detach(), 256)
    _check(x.grad, xr.grad, 384)
    _check(gt, wr.grad, 4 * 96)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (1000, 1000, 200), (4096, 5504, 2048)])
@pytest.mark.parametrize("layout", ["kk", "kmn", "mnmn"])
def test_gemm_paired_sm_kernel(M, N, K, layout):
    """The cta_group::2 kernel forced on (mode 2), including ragged edges of the 256x256 tile."""
    from mythos_b200.ops import functional as F, native

    C = native.require()
    torch.manual_seed(M * 3 + N + K)
    a_mn, b_mn = {"kk": (False, False), "kmn": (False, True), "mnmn": (True, True)}[layout]
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
    C.set_gemm_mode(2)
    try:
        out = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        acc = torch.ones(M, N, device="cuda")
        F.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, epi=F.EPI_F32_ACC)
        torch.cuda.synchronize()
    finally:
        C.set_gemm_mode(0)
    ref = _ref(a, b, a_mn, b_mn)
    _check(out, ref, K)
    _check(acc, ref + 1.0, K)


@pytest.mark.parametrize("M,F,K", [(256, 256, 128), (512, 640, 256), (1000, 384, 200), (4096, 5504, 2048)])
def test_gemm_swiglu_forward_epilogue(M, F, K):
    """gate/up projection with silu(gate) * up computed in the GEMM epilogue, against fp32."""
    from mythos_b200.ops import native

    C = native.require()
    torch.manual_seed(M + F)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * F, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    gu = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    C.gemm_swiglu_fwd(x, w, gu, h, native.status_word(x.device))
    ref = x.float() @ w.float().t()
    _check(gu, ref, K)
    g, u = ref[:, :F], ref[:, F:]
    _check(h, g * torch.sigmoid(g) * u, K)
    h2 = torch.empty_like(h)
    C.gemm_swiglu_fwd(x, w, None, h2, native.status_word(x.device))      # without the pre-activation output
    assert torch.equal(h, h2)


@pytest.mark.parametrize("M,F,K", [(256, 256, 256), (520, 640, 320), (4096, 5504, 2048)])
def test_gemm_swiglu_backward_epilogue(M, F, K):
    """down-projection dgrad with the SwiGLU derivative in the epilogue, against fp32 autograd."""
    from mythos_b200.ops import native

    C = native.require()
    torch.manual_seed(M + F + 1)
    dy = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w_down = (torch.randn(K, F, device="cuda") / K ** 0.5).to(torch.bfloat16)
    gu = torch.randn(M, 2 * F, device="cuda").to(torch.bfloat16)
    dgu = torch.empty_like(gu)
    C.gemm_swiglu_bwd(dy, w_down, gu, dgu, native.status_word(dy.device))
    guf = gu.float().requires_grad_()
    hh = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    hh.backward(dy.float() @ w_down.float())
    _check(dgu, guf.grad, K)


@pytest.mark.parametrize("M,heads,kv_heads,K", [(256, 2, 2, 128), (600, 3, 1, 256), (4096, 16, 16, 2048)])
def test_gemm_rope_epilogue(M, heads, kv_heads, K):
    """QKV projection with the rotary embedding of the q and k heads in the epilogue; v untouched."""
    from mythos_b200.ops import functional as Fn, native, reference as ref

    C = native.require()
    torch.manual_seed(M + heads)
    D = 128
    N = (heads + 2 * kv_heads) * D
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    pos = torch.randint(0, 512, (M,), device="cuda", dtype=torch.int32)
    table = Fn.rope_table(10000.0, 512, x.device)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm_rope(x, w, out, pos, table, (heads + kv_heads) * D, native.status_word(x.device))
    y = x.float() @ w.float().t()
    nr = heads + kv_heads
    rot = ref.rope(y[:, : nr * D].reshape(M, nr, D), pos, 10000.0).reshape(M, nr * D)
    _check(out[:, : nr * D], rot, K)
    _check(out[:, nr * D:], y[:, nr * D:], K)


def test_fused_ffn_and_rope_layers_match_unfused_autograd():
    """The fused FFN / QKV+RoPE functions give the gradients of the unfused operator chain."""
    from mythos_b200.ops import functional as Fn

    torch.manual_seed(3)
    M, d, F = 512, 256, 384
    x = torch.randn(M, d, device="cuda").to(torch.bfloat16).requires_grad_()
    w_gu = (torch.randn(2 * F, d, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    w_dn = (torch.randn(d, F, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(M, d, device="cuda").to(torch.bfloat16)
    assert Fn.fused_ffn_ok(x, w_gu, w_dn)
    y = Fn.swiglu_ffn(x, w_gu, w_dn)
    y.backward(dy)
    got = (y.detach().float(), x.grad.float(), w_gu.grad.float(), w_dn.grad.float())
    xf, wg, wd = (t.detach().float().requires_grad_() for t in (x, w_gu, w_dn))
    u = xf @ wg.t()
    yr = (torch.nn.functional.silu(u[:, :F]) * u[:, F:]) @ wd.t()
    yr.backward(dy.float())
    for a, b in zip(got, (yr.detach(), xf.grad, wg.grad, wd.grad)):
        assert (a - b).abs().max().item() <= 3e-2 * b.abs().max().item() + 1e-3
    # residual-gradient add inside the RMSNorm backward
    hdn = torch.randn(M, d, device="cuda").to(torch.bfloat16).requires_grad_()
    res = torch.randn(M, d, device="cuda").to(torch.bfloat16).requires_grad_()
    gamma = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    yn, hs = Fn.rmsnorm(hdn, gamma, 1e-5, res)
    g1, g2 = torch.randn_like(yn), torch.randn_like(hs)
    torch.autograd.backward([yn, hs], [g1, g2])
    hf, rf, gf = (t.detach().float().requires_grad_() for t in (hdn, res, gamma))
    s = hf + rf
    ynr = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * gf
    torch.autograd.backward([ynr, s], [g1.float(), g2.float()])
    assert (hdn.grad.float() - hf.grad).abs().max().item() <= 5e-2
    assert torch.equal(hdn.grad, res.grad)
    assert (gamma.grad.float() - gf.grad).abs().max().item() <= 3e-2 * gf.grad.abs().max().item() + 1e-2


def test_grouped_gemms_over_ragged_segments():
    """Ragged-M and ragged-K grouped GEMMs (segments described by device arrays, 256-aligned starts,
    zero padding rows) against per-segment fp32 products."""
    from mythos_b200.ops import native

    C = native.require()
    torch.manual_seed(5)
    rows = [300, 0, 77, 512]
    K, N = 256, 384
    starts, off = [], 0
    for r in rows:
        starts.append(off)
        off += (r + 255) // 256 * 256
    cap = off + 256
    a = torch.zeros(cap, K, device="cuda", dtype=torch.bfloat16)
    for s0, r in zip(starts, rows):
        a[s0:s0 + r] = torch.randn(r, K, device="cuda").to(torch.bfloat16)
    ws = [(torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16) for _ in rows]
    seg_start = torch.tensor(starts, device="cuda", dtype=torch.int32)
    seg_rows = torch.tensor(rows, device="cuda", dtype=torch.int32)
    st = native.status_word(a.device)
    out = torch.full((cap, N), 7.0, device="cuda", dtype=torch.bfloat16)
    C.gemm_grouped_rows(a, ws, False, out, seg_start, seg_rows, 0, None, None, st)
    for s0, r, w in zip(starts, rows, ws):
        if r:
            _check(out[s0:s0 + r], a[s0:s0 + r].float() @ w.float().t(), K)
    # MN-major weights (the dgrad form): out = a @ w with w [K, N]
    wt = [w.t().contiguous() for w in ws]
    out2 = torch.empty(cap, N, device="cuda", dtype=torch.bfloat16)
    C.gemm_grouped_rows(a, wt, True, out2, seg_start, seg_rows, 0, None, None, st)
    for s0, r, w in zip(starts, rows, ws):
        if r:
            _check(out2[s0:s0 + r], a[s0:s0 + r].float() @ w.float().t(), K)
    # ragged K: grads[e] += a[rows of e]^T @ b[rows of e]
    b = torch.zeros(cap, N, device="cuda", dtype=torch.bfloat16)
    for s0, r in zip(starts, rows):
        b[s0:s0 + r] = torch.randn(r, N, device="cuda").to(torch.bfloat16)
    grads = [torch.ones(K, N, device="cuda") for _ in rows]
    C.gemm_grouped_k(a, b, grads, seg_start, seg_rows, st)
    for s0, r, g in zip(starts, rows, grads):
        ref = 1.0 + a[s0:s0 + r].float().t() @ b[s0:s0 + r].float()
        _check(g, ref, max(r, 1))
