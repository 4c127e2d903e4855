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
