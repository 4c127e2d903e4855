"""Quantisation engines (FP8, NF4, AWQ/GPTQ group INT4, ternary/binary packers, U8/INT8) against
closed-form expectations and round trips."""
import math

import pytest
import torch

from mythos_b200.oil import engines as E


def test_fp8_round_trip_and_known_codes():
    x = torch.tensor([0.0, 1.0, -1.0, 448.0, 1000.0, -1000.0, 0.015625, 2.0 ** -9, 1.75])
    q = E.fp8_e4m3_quantize(x)
    d = E.fp8_e4m3_dequantize(q)
    assert d.tolist() == [0.0, 1.0, -1.0, 448.0, 448.0, -448.0, 0.015625, 2.0 ** -9, 1.75]
    assert int(q[1]) == 0x38 and int(q[3]) == 0x7E
    # every finite code decodes and re-encodes to itself
    codes = torch.arange(256, dtype=torch.uint8)
    vals = E.fp8_e4m3_dequantize(codes)
    fin = torch.isfinite(vals)
    assert torch.equal(E.fp8_e4m3_quantize(vals[fin]) & 0x7F, codes[fin] & 0x7F)
    vals5 = E.fp8_e5m2_dequantize(codes)
    fin5 = torch.isfinite(vals5)
    assert torch.equal(E.fp8_e5m2_quantize(vals5[fin5]) & 0x7F, codes[fin5] & 0x7F)
    g = torch.Generator().manual_seed(0)
    w = torch.randn(4096, generator=g)
    rel = (E.fp8_e4m3_dequantize(E.fp8_e4m3_quantize(w)) - w).abs() / w.abs().clamp_min(2.0 ** -6)
    assert float(rel.max()) <= 1 / 16 + 1e-6          # 3 mantissa bits: half an ulp
    rel5 = (E.fp8_e5m2_dequantize(E.fp8_e5m2_quantize(w)) - w).abs() / w.abs().clamp_min(2.0 ** -14)
    assert float(rel5.max()) <= 1 / 8 + 1e-6


def test_nf4_levels_and_error():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(1000, generator=g) * 0.02
    idx, scales = E.nf4_quantize(w, 64)
    assert idx.max() < 16 and scales.numel() == 16
    d = E.nf4_dequantize(idx, scales, 64)
    # exact levels survive; the abs-max element of each block maps to +-1 * scale
    assert torch.allclose(d.view(-1)[:960].view(15, 64).abs().amax(1), scales[:15])
    assert float((d - w).abs().max()) < 0.16 * float(scales.max())


def test_awq_and_gptq_group_int4():
    g = torch.Generator().manual_seed(2)
    w = torch.randn(8, 256, generator=g) * 0.05
    act = torch.randn(256, generator=g)
    q = E.AWQQuantizer(group_size=64, alpha=0.5)
    s = q.compute_scales(w, act)
    exp = act.abs().max().sqrt() / (w.abs().amax(1) + 1e-10)
    assert torch.allclose(s, exp.clamp(1e-8, 1e4))
    fq = q.quantize(w)
    # at most 16 distinct values per (row, group), error below half a step
    for r in range(8):
        for g0 in range(0, 256, 64):
            blk = fq[r, g0:g0 + 64]
            assert blk.unique().numel() <= 16
            step = float(w[r, g0:g0 + 64].abs().max()) / 7
            assert float((blk - w[r, g0:g0 + 64]).abs().max()) <= step / 2 + 1e-7
    h = torch.ones_like(w)
    gq = E.GPTQQuantizer(64, 4).quantize(w, h)
    assert float((gq - w).abs().max()) <= float(w.abs().max()) / 7 / 2 + 1e-6


def test_i2s_and_block_packers():
    w = torch.tensor([0.5, -0.5, 0.1, 0.0, 1.0, -1.0, 0.34, -0.32] * 16)      # 128 values, one block
    packed, scales = E.i2s_quantize(w, 128)
    assert packed.numel() == 32 and float(scales[0]) == 1.0
    # first byte: codes 2,0,1,1 -> 2 | 0<<2 | 1<<4 | 1<<6
    assert int(packed[0]) == 2 | (1 << 4) | (1 << 6)
    d = E.i2s_dequantize(packed, scales, 128, 128)
    assert d[:8].tolist() == [1.0, -1.0, 0.0, 0.0, 1.0, -1.0, 1.0, 0.0]
    blk = torch.tensor([1.0, -0.9, 0.2, 0.6, -0.1, 0.0, 0.58, -0.57])
    p, s = E.ternary_block_quantize(blk)
    kept = [1.0, 0.9, 0.6, 0.58]
    assert math.isclose(s, sum(kept) / 4, rel_tol=1e-6)
    assert E.ternary_block_dequantize(p, s, 8).tolist() == [s, -s, 0.0, s, 0.0, 0.0, s, 0.0]
    p, s = E.binary_block_quantize(blk)
    assert math.isclose(s, float(blk.abs().mean()), rel_tol=1e-6)
    assert (E.binary_block_dequantize(p, s, 8) > 0).tolist() == (blk > 0).tolist()
    p, s = E.binary_tensor_quantize(blk)
    assert s == 1.0 and int(p[0]) & (1 << 5)          # zero counts as +1 in the tensor variant


def test_integer_quantisers():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(16, 64, generator=g)
    q, s, zp = E.affine_u8_quantize(x)
    assert float((E.affine_u8_dequantize(q, s, zp) - x).abs().max()) <= s * 0.5 + 1e-6
    q8, s8 = E.int8_quantize_per_tensor(x)
    assert float((E.int8_dequantize(q8, s8) - x).abs().max()) <= s8 * 0.5 + 1e-6
    qt, st = E.int8_quantize_per_token(x)
    assert st.shape == (16,) and int(qt.abs().amax(1).min()) == 127
    assert float((E.int8_dequantize(qt, st) - x).abs().max()) <= float(st.max()) * 0.5 + 1e-6


def test_codebook_engines_reduce_error():
    g = torch.Generator().manual_seed(4)
    w = torch.randn(4096, generator=g) * 0.02
    for make in (E.OIL8Engine, E.OIL4Engine):
        eng = make()
        before = float(((eng.dequantize(eng.quantize(w)) - w) ** 2).mean())
        eng.train_codebook(w)
        d = eng.dequantize(eng.quantize(w))
        after = float(((d - w) ** 2).mean())
        assert after < before                       # Lloyd iterations lower the squared error
        assert E.compute_quant_error(w, d) == float((d - w).abs().max())


def test_ffn_shard_padding_writes_exact_zero_trits():
    from mythos_b200.infer.engine import _zero_ffn_padding
    from mythos_b200.infer.quant_weights import QuantLinear

    up = QuantLinear.random("i2s", 2 * 256, 256, 64, device="cpu", generator=torch.Generator().manual_seed(0))
    down = QuantLinear.random("i2s", 256, 256, 64, device="cpu", generator=torch.Generator().manual_seed(1))
    before_up, before_down = up._dequantize_reference().clone(), down._dequantize_reference().clone()
    _zero_ffn_padding(up, down, 192, 256, True)
    w, wd = up._dequantize_reference(), down._dequantize_reference()
    assert float(w[192:256].abs().max()) == 0 and float(w[256 + 192:].abs().max()) == 0 and float(wd[:, 192:].abs().max()) == 0
    assert torch.equal(w[:192], before_up[:192]) and torch.equal(w[256:256 + 192], before_up[256:256 + 192])
    assert torch.equal(wd[:, :192], before_down[:, :192])
    oil = QuantLinear.random("oil8", 256, 256, 64, 1, device="cpu", generator=torch.Generator().manual_seed(2))
    with pytest.raises(ValueError, match="I2_S"):
        _zero_ffn_padding(oil, down, 192, 256, False)
