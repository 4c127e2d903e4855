"""Operation surface, hardware probe and micro-benchmarks (host side)."""
import torch

from mythos_b200.utils import backend as bk


def test_host_backend_ops_and_probe():
    b = bk.HostBackend()
    A, B = torch.randn(4, 6), torch.randn(6, 5)
    C = torch.ones(4, 5)
    b.gemm(2.0, A, B, 0.5, C)
    assert torch.allclose(C, 2.0 * A @ B + 0.5, atol=1e-5)
    y = torch.zeros(4)
    b.gemv(1.0, A, torch.ones(6), 0.0, y)
    assert torch.allclose(y, A.sum(1), atol=1e-5)
    x = torch.randn(3, 8)
    assert torch.allclose(b.softmax(x).sum(-1), torch.ones(3), atol=1e-6)
    assert torch.allclose(b.rms_norm(x, torch.ones(8)), x / x.pow(2).mean(-1, keepdim=True).add(1e-5).sqrt(), atol=1e-5)
    assert torch.allclose(b.layer_norm(x, torch.ones(8), torch.zeros(8)).mean(-1), torch.zeros(3), atol=1e-5)
    assert float(b.silu(torch.tensor([0.0]))) == 0.0 and float(b.relu(torch.tensor([-1.0]))) == 0.0
    assert b.memory_total() > 0 and b.is_available()
    hp = bk.probe_hardware()
    assert hp.cpu_cores > 0 and hp.ram_total > 0
    sel = bk.select_optimal_backend(hp)
    assert sel.name in ("host-fp32", "b200-sm100a")
    r = bk.benchmark_operation(b, "gemm", 64, 2)
    assert r["gflops"] > 0 and bk.benchmark_operation(b, "add", 64, 2)["gbs"] > 0
