"""The C++ host runtime against its Python twins: container reader/writer, SHA-256, sidecar check,
BPE, RNG, page allocator."""
import hashlib

import numpy as np
import pytest
import torch

from mythos_b200.oil import native_io

pytestmark = pytest.mark.skipif(not native_io.available(), reason="liboil_host.so not built")


def test_sha256_matches_hashlib(tmp_path):
    for data in (b"", b"abc", bytes(range(256)) * 1000):
        assert native_io.sha256(data) == hashlib.sha256(data).digest()
    p = tmp_path / "f.bin"
    p.write_bytes(b"x" * 3_000_001)
    assert native_io.sha256_file(str(p)) == hashlib.sha256(b"x" * 3_000_001).hexdigest()


def test_native_reader_and_writer_agree_with_python(tmp_path):
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.oil import container as oc
    from mythos_b200.oil.model_io import save_model

    torch.manual_seed(0)
    for fmt in ("oil8", "oil4", "i2s", "fp16"):
        cfg = TransformerConfig(vocab_size=64, hidden_size=64, num_layers=1, num_heads=2, head_dim=32,
                                ffn_hidden_size=128, max_seq_len=16, weight_format=fmt, oil_block_size=64)
        p = str(tmp_path / f"{fmt}.oil")
        save_model(DenseModel(cfg), p)
        py, nat = oc.OILReader(p), native_io.NativeReader(p)
        assert nat.tensor_names() == py.tensor_names() and nat.num_blocks() == py.num_blocks
        assert nat.config == py.config
        for name in py.tensor_names():
            assert np.array_equal(nat.read_tensor(name), py.read_tensor(name)), (fmt, name)
            assert nat.tensor_sha256(name) == py.tensor_sha256(name)
        # the native writer reproduces the file byte for byte
        q = str(tmp_path / f"{fmt}_copy.oil")
        native_io.write_oil_native(q, [(n, py.read_tensor_blocks(n)) for n in py.tensor_names()], py.config)
        assert open(p, "rb").read() == open(q, "rb").read()
        assert native_io.idx_check(oc.idx_path_for(p)) == len(py.tensor_names())
    with pytest.raises(oc.OILError):
        native_io.NativeReader(str(tmp_path / "missing.oil"))
    bad = tmp_path / "bad.oil"
    bad.write_bytes(open(p, "rb").read()[:100])
    with pytest.raises(oc.OILError, match="truncated"):
        native_io.NativeReader(str(bad))


def test_native_idx_check_names_the_corrupt_tensor(tmp_path):
    from mythos_b200.oil import container as oc

    p = str(tmp_path / "m.oilidx")
    oc.write_idx_file(p, ["alpha.weight", "beta.weight"], version=1)
    raw = bytearray(open(p, "rb").read())
    raw[raw.find(b"beta") + 1] ^= 0x20
    open(p, "wb").write(bytes(raw))
    with pytest.raises(oc.OILError, match="index 1"):
        native_io.idx_check(p)


def test_native_bpe_matches_python(tmp_path):
    from mythos_b200.train.bpe import BPETokenizer

    text = ("she sells sea shells by the sea shore. the shells she sells are sea shells. " * 40).encode()
    py = BPETokenizer()
    py.train(text, 320)
    nat = native_io.NativeBPE.train(text, 320)
    assert nat.vocab_size == py.vocab_size
    sample = text[:200]
    ids = nat.encode(sample)
    assert nat.decode(ids) == sample and py.decode_bytes(py.encode(sample)) == sample
    assert len(ids) == len(py.encode(sample)) < len(sample)
    f = str(tmp_path / "t.vocab")
    nat.save(f)
    assert BPETokenizer.load(f).encode(sample) == ids  # the .vocab layout is shared


def test_native_rng_and_pages():
    a, b = native_io.NativeRNG(42), native_io.NativeRNG(42)
    assert [a.next_u64() for _ in range(5)] == [b.next_u64() for _ in range(5)]
    u = native_io.NativeRNG(7).fill_uniform(20000, -1.0, 1.0)
    assert -1.0 <= u.min() and u.max() < 1.0 and abs(float(u.mean())) < 0.03
    r = native_io.NativeRNG(3)
    z = np.array([r.normal() for _ in range(20000)])
    assert abs(z.mean()) < 0.03 and abs(z.std() - 1.0) < 0.03
    pages = native_io.NativePageAllocator(3)
    p0, p1 = pages.alloc(), pages.alloc()
    pages.retain(p0)
    pages.release(p0)
    assert pages.used == 2
    pages.release(p0)
    pages.release(p1)
    assert pages.used == 0
    got = {pages.alloc() for _ in range(3)}
    assert got == {0, 1, 2}
    with pytest.raises(MemoryError):
        pages.alloc()
