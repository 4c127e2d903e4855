"""Device surface, hardware probe and operation micro-benchmarks.

The reference hides eight compute backends behind one virtual interface (CPU scalar / AVX2 /
"AVX512", iGPU shared memory, DirectX 12, RAM-swap, "distributed", stub CUDA; include/oil/backend.h:49-80,
src/backend.cpp:36-438) and picks one by probing the machine (:464-735). This framework targets one
device, so there is no dispatch layer on any hot path: models call the sm_100a kernels directly.
What remains useful is kept here: the same operation surface as two concrete classes (the B200
kernels, and the fp32 host oracle the tests compare against), the probe, and
``benchmark_operation`` (the reference's ``:737-829``), which reports GFLOP/s or GB/s per operation.
DirectX / Vulkan / Metal / iGPU / RAM-swap backends have no counterpart: they are graphics-API or
host-memory paths that do not exist on this platform.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field

import torch

from ..ops import reference as ref


class HostBackend:
    """fp32 reference implementation of the operation surface (the oracle)."""

    name = "host-fp32"

    def is_available(self) -> bool:
        return True

    def gemm(self, alpha, A, B, beta, C):
        C.copy_(alpha * (A.float() @ B.float()) + beta * C.float())
        return C

    def gemv(self, alpha, A, x, beta, y):
        y.copy_(alpha * (A.float() @ x.float()) + beta * y.float())
        return y

    def softmax(self, x, axis: int = -1):
        return torch.softmax(x.float(), dim=axis).to(x.dtype)

    def layer_norm(self, x, gamma, beta, eps: float = 1e-5):
        return ref.layernorm(x, gamma, beta, eps)

    def rms_norm(self, x, gamma, eps: float = 1e-5):
        return ref.rmsnorm(x, gamma, eps)[0]

    def relu(self, x):
        return torch.relu(x)

    def gelu(self, x):
        return ref.gelu_erf(x)

    def silu(self, x):
        return ref.silu(x.float()).to(x.dtype)

    def add(self, a, b):
        return a + b

    def mul(self, a, b):
        return a * b

    def scale(self, s, x):
        return x * s

    def copy(self, src, dst):
        return dst.copy_(src)

    def fill(self, t, val):
        return t.fill_(val)

    def zero(self, t):
        return t.zero_()

    def memory_total(self) -> int:
        return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")

    def memory_free(self) -> int:
        try:
            return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_AVPHYS_PAGES")
        except (ValueError, OSError):
            return 0

    def synchronize(self) -> None:
        pass


class B200Backend(HostBackend):
    """The same surface on the device kernels (bf16 tensors on a CUDA device)."""

    name = "b200-sm100a"

    def __init__(self, device="cuda"):
        self.device = torch.device(device)

    def is_available(self) -> bool:
        from ..ops import native

        return torch.cuda.is_available() and native.available()

    def gemm(self, alpha, A, B, beta, C):
        """C = alpha * A @ B + beta * C with A [M, K], B [K, N] (B is consumed K-major without a copy)."""
        from ..ops import functional as F

        out = F.gemm(A.contiguous(), B.contiguous(), b_mn=True, epi=F.EPI_F32, alpha=alpha)
        C.copy_(out if beta == 0 else out + beta * C.float())
        return C

    def gemv(self, alpha, A, x, beta, y):
        from ..ops import functional as F

        xb = torch.zeros(8, x.numel(), device=x.device, dtype=A.dtype)     # GEMM columns come in groups of 8
        xb[0] = x.reshape(-1)
        out = F.gemm(A.contiguous(), xb, epi=F.EPI_F32, alpha=alpha)[:, 0]
        y.copy_(out if beta == 0 else out + beta * y.float())
        return y

    def softmax(self, x, axis: int = -1):
        from ..ops import native

        if axis not in (-1, x.dim() - 1):
            return super().softmax(x, axis)
        y = torch.empty_like(x.contiguous())
        native.require().softmax_rows(x.contiguous(), y)
        return y

    def layer_norm(self, x, gamma, beta, eps: float = 1e-5):
        from ..ops import functional as F

        with torch.no_grad():
            return F.layernorm(x, gamma, beta, eps)

    def rms_norm(self, x, gamma, eps: float = 1e-5):
        from ..ops import functional as F

        return F.rmsnorm(x, gamma, eps, None)[0]

    def _act(self, x, kind):
        from ..ops import functional as F

        with torch.no_grad():
            return F.activation(x, kind)

    def relu(self, x):
        return self._act(x, "relu")

    def gelu(self, x):
        return self._act(x, "gelu")

    def silu(self, x):
        return self._act(x, "silu")

    def memory_total(self) -> int:
        return torch.cuda.mem_get_info(self.device)[1]

    def memory_free(self) -> int:
        return torch.cuda.mem_get_info(self.device)[0]

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)


@dataclass
class HardwareProfile:
    cpu_cores: int = 0
    cpu_flags: list = field(default_factory=list)
    ram_total: int = 0
    gpus: list = field(default_factory=list)          # dicts: name, sm, capability, memory, l2
    peer_access: list = field(default_factory=list)   # matrix of bools
    native_kernels: bool = False


def probe_hardware() -> HardwareProfile:
    hp = HardwareProfile(cpu_cores=os.cpu_count() or 0)
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    hp.cpu_flags = sorted(flags & {"avx2", "avx512f", "fma", "sse4_2", "amx_bf16"})
                    break
    except OSError:
        pass
    hp.ram_total = HostBackend().memory_total()
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            hp.gpus.append({"name": p.name, "sm": p.multi_processor_count, "capability": f"{p.major}.{p.minor}",
                            "memory": p.total_memory, "l2": getattr(p, "L2_cache_size", 0)})
        hp.peer_access = [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
        from ..ops import native

        hp.native_kernels = native.available()
    return hp


def select_optimal_backend(profile: HardwareProfile | None = None):
    """The device kernels when a B200-class GPU and the built extension are present, else the host oracle."""
    profile = profile or probe_hardware()
    if profile.gpus and profile.native_kernels and profile.gpus[0]["capability"].startswith("10."):
        return B200Backend()
    return HostBackend()


def benchmark_operation(backend, op: str, size: int = 1024, iters: int = 10) -> dict:
    """Time one operation; returns {"op", "ms", "gflops" or "gbs"}. Operations: gemm, relu, add,
    softmax, rms_norm (the set the reference measures)."""
    dev = getattr(backend, "device", torch.device("cpu"))
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    x = torch.randn(size, size, device=dev).to(dt)
    y = torch.randn(size, size, device=dev).to(dt)
    g = torch.ones(size, device=dev, dtype=dt)
    c = torch.zeros(size, size, device=dev, dtype=torch.float32)
    fns = {"gemm": lambda: backend.gemm(1.0, x, y, 0.0, c), "relu": lambda: backend.relu(x),
           "add": lambda: backend.add(x, y), "softmax": lambda: backend.softmax(x, -1),
           "rms_norm": lambda: backend.rms_norm(x, g, 1e-5)}
    fn = fns[op]
    fn()
    backend.synchronize()
    if dev.type == "cuda":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        backend.synchronize()
        ms = a.elapsed_time(b) / iters
    else:
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        ms = (time.perf_counter() - t0) * 1e3 / iters
    out = {"op": op, "size": size, "ms": ms, "backend": backend.name}
    if op == "gemm":
        out["gflops"] = 2.0 * size ** 3 / ms / 1e6
    else:
        nbytes = x.numel() * x.element_size() * (3 if op == "add" else 2)
        out["gbs"] = nbytes / ms / 1e6
    return out
