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


def test_runtime_environment_variables_take_effect():
    import logging

    from mythos_b200.utils import env, trace

    rt = env.RuntimeEnv.from_environ({"OIL_NUM_THREADS": "3", "OIL_SEED": "7", "OIL_LOG_LEVEL": "DEBUG",
                                      "OIL_VERBOSE": "1", "OIL_GPU_DEVICE": "5", "OIL_MEMORY_POOL_SIZE": "junk"})
    assert (rt.num_threads, rt.seed, rt.log_level, rt.verbose, rt.gpu_device) == (3, 7, "debug", True, 5)
    assert rt.memory_pool_size == 64 << 20                   # unparsable values fall back to the default
    before = torch.get_num_threads()
    try:
        rt.apply()
        assert torch.get_num_threads() == 3 and trace.timing_enabled()
        assert logging.getLogger("mythos_b200").level == logging.DEBUG
        a = torch.rand(4)
        rt.apply()
        assert torch.equal(a, torch.rand(4))                 # the seed is applied
        assert rt.default_device().type == ("cuda" if torch.cuda.is_available() else "cpu")
        with trace.span("outer"):
            with trace.span("inner"):
                torch.ones(10).sum()
        with trace.span("inner"):
            pass
        rows = trace.summary()
        assert rows["inner"]["calls"] == 2 and rows["outer"]["calls"] == 1 and rows["outer"]["ms"] >= 0
        assert "inner" in trace.format_summary(rows) and trace.summary() == {}
    finally:
        torch.set_num_threads(before)
        trace.enable_timing(False)
        logging.getLogger("mythos_b200").setLevel(logging.NOTSET)
    assert env.RuntimeEnv.from_environ({}).seed == 42
