import torch

from mythos_b200.oil import ternary_kernels as tk


def test_lut_gemms_match_integer_matmul():
    g = torch.Generator().manual_seed(0)
    N, K, M = 10, 48, 5
    trits = torch.randint(-1, 2, (N, K), generator=g)
    x = torch.randn(M, K, generator=g) * 3
    packed = tk.pack_trits(trits)
    assert packed.shape == (N, K // 4) and torch.equal(tk.unpack_trits(packed, K), trits.int())
    want = tk.ternary_reference(trits, x)
    assert torch.equal(tk.tl1_gemm(packed, x, K), want)
    assert torch.equal(tk.tl2_gemm(packed, x, K), want)
    # int8 quantisation error of the activations only: close to the float product
    assert (want - x @ trits.float().t()).abs().max() < 0.05 * x.abs().max() * K ** 0.5
    q, s = tk.quantize_activations_int8(x)
    assert int(q.abs().max()) == 127 and torch.allclose(q.float().abs().amax(1) / s, x.abs().amax(1), rtol=1e-2)
    scales = torch.rand(N, K // 16, generator=g) + 0.5
    y = tk.i2s_gemm_int8(packed, scales, x, K, 16)
    deq = trits.float() * scales.repeat_interleave(16, dim=1)
    assert torch.allclose(y, (q.float() @ deq.t()) / s[:, None], atol=1e-4)
