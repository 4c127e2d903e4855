"""The allocation-free C entry point (RMSNorm backward with its partial-sum scratch in a fixed
device array inside the library). It is for embedders that may not call the CUDA allocator — a
serving loop under a fixed memory budget, a host application that owns all device memory — so
the test calls it the way they would: through the exported C symbol, with raw device pointers,
and checks two consecutive calls against the regular entry point."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mythos_b200.ops import native

    ext = native.require()
    lib = ctypes.CDLL(ext.__file__)
    fn = lib.mythos_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.mythos_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _regular(dy, x, gamma, rstd, accumulate_into=None):
    from mythos_b200.ops import native

    C = native.require()
    rows, dim = x.shape
    dx = torch.empty_like(x)
    partial = torch.empty(min(rows, 296), dim, device="cuda", dtype=torch.float32)
    dg = torch.zeros(dim, device="cuda") if accumulate_into is None else accumulate_into.clone()
    C.rmsnorm_bwd(dy, x, gamma, rstd, dx, partial, dg, accumulate_into is not None)
    return dx, dg


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    prev_dg = None
    for call, (rows, dim) in enumerate([(300, 2048), (77, 4096)]):
        torch.manual_seed(call)
        x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
        dy = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
        gamma = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        want_dx, want_dg = _regular(dy, x, gamma, rstd)
        dx = torch.empty_like(x)
        dg = torch.full((dim,), 123.0, device="cuda")  # must be overwritten when accumulate == 0
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), rows,
                dim, 0, stream)
        assert rc == 0, lib.mythos_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(dx, want_dx)
        assert torch.allclose(dg, want_dg, rtol=2e-3, atol=2e-2)
        # accumulate variant on top of the previous result
        rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), rows,
                dim, 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(dg, 2 * want_dg, rtol=2e-3, atol=4e-2)
        prev_dg = dg
    assert prev_dg is not None


def test_noalloc_with_zero_rows_writes_zeros_or_leaves_the_accumulator():
    lib, fn = _lib()
    t = torch.zeros(64, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(1, device="cuda")
    dg = torch.full((64,), 5.0, device="cuda")
    args = (t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), dg.data_ptr(), 0, 64)
    assert fn(*args, 1, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(dg, torch.full((64,), 5.0, device="cuda"))       # accumulate: unchanged
    assert fn(*args, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(dg, torch.zeros(64, device="cuda"))              # overwrite: the gradient is zero


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib, fn = _lib()
    t = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), f.data_ptr(), 1, 16384, 0, None)
    assert rc == -2 and b"exceeds" in lib.mythos_noalloc_last_error()
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), f.data_ptr(), 1, 12, 0, None)
    assert rc == -1
    rc = fn(None, t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), f.data_ptr(), 1, 8, 0, None)
    assert rc == -1
