"""``.oil`` container and sidecar: byte layout against a golden written by the reference's own
``oil_convert`` (8 floats, rawfp32), round trips of every block format, the idx sidecar's
fail-fast behaviour (the cases of the reference's tests/test_sha256_corrupt.cpp), and the model
save -> load -> save digest check of the tiny byte-level configuration."""
import hashlib
import os
import struct

import numpy as np
import pytest
import torch

from mythos_b200.oil import container as oc
from mythos_b200.oil.formats import (Format, decode_block, encode_block, pack_nibbles, pack_trits, quantize_binary,
                                     quantize_ternary, unpack_nibbles, unpack_trits)

# bytes produced by `oil_convert --format rawfp32` of the reference for float32 1..8
GOLDEN_HEX = (
    "4f494c31" "01000000" "00000000" "00000000"
    "01000000" "00000000" "05" "00000000"
    "01000000" "0700" "77656967687473" "00000000" "01000000"
    "08000000" "00000000" "20000000"
    + np.arange(1, 9, dtype="<f4").tobytes().hex())
GOLDEN_SHA256 = "8a87641b625e603e3d4c4bfb2e33dbe364b23110287c374b09879a12fb5da1b9"


def test_writer_matches_reference_golden(tmp_path):
    p = str(tmp_path / "g.oil")
    vals = np.arange(1, 9, dtype="<f4")
    oc.write_oil(p, [("weights", [oc.BlockData(Format.FP32, 8, b"", vals.tobytes())])], write_idx=False)
    data = open(p, "rb").read()
    assert data.hex() == GOLDEN_HEX
    assert len(data) == 94
    assert hashlib.sha256(data).hexdigest() == GOLDEN_SHA256 == oc.file_sha256(p)
    rd = oc.OILReader(p)
    assert rd.tensor_names() == ["weights"] and rd.num_blocks == 1
    assert np.array_equal(rd.read_tensor("weights"), vals)
    assert rd.read_tensor("missing").size == 0


def test_all_block_formats_round_trip(tmp_path):
    from mythos_b200.oil.codebook import quantile_codebook

    rng = np.random.default_rng(0)
    w = (rng.standard_normal(300) * 0.02).astype(np.float32)
    cb8 = quantile_codebook(256).numpy()
    idx8 = np.abs(w[:, None] - cb8[None]).argmin(1).astype(np.uint8)
    cb4 = quantile_codebook(16, fp16=True).numpy()
    idx4 = np.abs(w[:, None] - cb4[None]).argmin(1).astype(np.uint8)
    tcodes, ts = quantize_ternary(w)
    bits, bs = quantize_binary(w)
    blocks = [
        ("fp32", oc.BlockData(Format.FP32, 300, *encode_block(Format.FP32, w))),
        ("fp16", oc.BlockData(Format.FP16, 300, *encode_block(Format.FP16, w))),
        ("oil8", oc.BlockData(Format.OIL8, 300, *encode_block(Format.OIL8, None, cb8, idx8))),
        ("oil4", oc.BlockData(Format.OIL4, 299, *encode_block(Format.OIL4, None, cb4, idx4[:299]))),
        ("i2s", oc.BlockData(Format.TERNARY, 300, *encode_block(Format.TERNARY, None, None, tcodes, ts))),
        ("bin", oc.BlockData(Format.BINARY, 300, *encode_block(Format.BINARY, None, None, bits, bs))),
    ]
    p = str(tmp_path / "f.oil")
    oc.write_oil(p, [(n, [b]) for n, b in blocks], config=b"cfg!")
    rd = oc.OILReader(p)
    assert rd.config == b"cfg!"
    assert np.array_equal(rd.read_tensor("fp32"), w)
    assert np.allclose(rd.read_tensor("fp16"), w, atol=1e-4)
    assert np.array_equal(rd.read_tensor("oil8"), cb8[idx8])
    assert np.array_equal(rd.read_tensor("oil4"), cb4[idx4[:299]])
    assert np.allclose(rd.read_tensor("i2s"), (tcodes.astype(np.float32) - 1) * np.float32(ts))
    assert np.allclose(rd.read_tensor("bin"), np.where(bits > 0, bs, -bs))
    assert [f.name for f in rd.tensor_formats("oil4")] == ["OIL4"]
    # OIL8 codebook blob: magic 0x4F494C38 + 256 floats; OIL4: magic + 16 halves
    assert len(blocks[2][1].codebook) == 1028 and struct.unpack("<I", blocks[2][1].codebook[:4])[0] == 0x4F494C38
    assert len(blocks[3][1].codebook) == 36 and struct.unpack("<I", blocks[3][1].codebook[:4])[0] == 0x4F494C34
    assert oc.verify(p) == [n for n, _ in blocks]
    assert np.array_equal(unpack_nibbles(pack_nibbles(idx4), 300), idx4)
    assert np.array_equal(unpack_trits(pack_trits(tcodes), 300), tcodes)
    assert pack_nibbles(np.array([1, 2], dtype=np.uint8)) == bytes([0x21])  # even index in the low nibble
    assert pack_trits(np.array([0, 1, 2, 1], dtype=np.uint8)) == bytes([0b01100100])  # first weight in bits 0-1


def test_idx_sidecar_detects_corruption_and_truncation(tmp_path):
    names = ["tok_embeddings.weight", "layers.0.attention.q_proj.weight", "norm.weight"]
    p = str(tmp_path / "m.oilidx")
    oc.write_idx_file(p, names, version=1)
    ver, recs = oc.read_idx_file(p)
    assert ver == 1 and [r.name for r in recs] == names
    raw = bytearray(open(p, "rb").read())
    assert raw[:10] == b"MYTHOSIDX\x00"
    # flip one byte inside the second tensor's name: the reader must name that tensor
    pos = raw.find(b"layers.0") + 3
    raw[pos] ^= 0x01
    bad = str(tmp_path / "bad.oilidx")
    open(bad, "wb").write(bytes(raw))
    with pytest.raises(oc.OILError) as e:
        oc.read_idx_file(bad)
    assert "hash mismatch" in str(e.value) and "at index 1" in str(e.value)
    trunc = str(tmp_path / "t.oilidx")
    open(trunc, "wb").write(bytes(open(p, "rb").read()[:40]))
    with pytest.raises(oc.OILError, match="truncated"):
        oc.read_idx_file(trunc)
    notidx = str(tmp_path / "n.oilidx")
    open(notidx, "wb").write(b"NOTANIDXFILE" * 4)
    with pytest.raises(oc.OILError, match="invalid idx"):
        oc.read_idx_file(notidx)


def test_truncated_container_and_content_hash(tmp_path):
    p = str(tmp_path / "c.oil")
    w = np.arange(100, dtype="<f4")
    oc.write_oil(p, [("a", [oc.BlockData(Format.FP32, 100, b"", w.tobytes())]),
                     ("b", [oc.BlockData(Format.FP32, 100, b"", (w * 2).tobytes())])])
    assert oc.verify(p) == ["a", "b"]
    data = bytearray(open(p, "rb").read())
    data[-5] ^= 0xFF
    open(p, "wb").write(bytes(data))
    with pytest.raises(oc.OILError, match='content hash mismatch for tensor "b"'):
        oc.verify(p)
    open(p, "wb").write(bytes(data[:60]))
    with pytest.raises(oc.OILError, match="truncated"):
        oc.OILReader(p)


def test_write_dedup_stores_identical_blobs_once(tmp_path):
    p = str(tmp_path / "d.oil")
    with oc.OILWriter(p) as w:
        w.write_header()
        a = w.write_dedup(b"x" * 100)
        b = w.write_dedup(b"y" * 50)
        c = w.write_dedup(b"x" * 100)
    assert a == c and b == a + 100
    assert os.path.getsize(p) == 16 + 150


@pytest.mark.parametrize("fmt", ["oil8", "oil4", "i2s", "fp32"])
def test_model_save_load_save_is_bit_exact(tmp_path, fmt):
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.oil.model_io import load_model, save_model

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=64, hidden_size=64, num_layers=2, num_heads=2, head_dim=32,
                            ffn_hidden_size=128, max_seq_len=32, weight_format=fmt, oil_block_size=64,
                            codebook_group=2)
    m = DenseModel(cfg)
    p1, p2 = str(tmp_path / "a.oil"), str(tmp_path / "b.oil")
    d1 = save_model(m, p1)
    m2, rd = load_model(p1)
    d2 = save_model(m2, p2)
    assert d1 == d2
    assert open(p1, "rb").read() == open(p2, "rb").read()
    assert oc.verify(p1)
    ids = torch.randint(0, 64, (2, 16), dtype=torch.int32)
    with torch.no_grad():
        assert torch.allclose(m(ids), m2(ids), atol=1e-5)
    fmts = rd.tensor_formats("layers.0.attention.qkv_proj.weight")
    want = {"oil8": Format.OIL8, "oil4": Format.OIL4, "i2s": Format.TERNARY, "fp32": Format.FP32}[fmt]
    assert set(fmts) == {want}
    assert m2.cfg.weight_format == fmt and m2.cfg.oil_block_size == 64


def test_reader_fuzz_only_raises_oil_errors(tmp_path):
    """Truncations and byte flips in the header / tables: the Python reader either reads the file or
    raises OILError, never an IndexError / struct.error / MemoryError from a wild size field."""
    import random

    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.oil.container import OILError, OILReader, read_idx_file
    from mythos_b200.oil.model_io import save_model

    random.seed(0)
    torch.manual_seed(0)
    rejected = 0
    for fmt in ("oil8", "i2s"):
        cfg = TransformerConfig(vocab_size=32, hidden_size=32, num_layers=1, num_heads=2, head_dim=16,
                                ffn_hidden_size=64, max_seq_len=16, weight_format=fmt, oil_block_size=32)
        p = str(tmp_path / f"{fmt}.oil")
        save_model(DenseModel(cfg), p)
        raw = open(p, "rb").read()
        trials = [raw[:c] for c in list(range(0, 160, 5)) + [len(raw) * i // 11 for i in range(11)]]
        for _ in range(80):
            b = bytearray(raw)
            pos = random.randrange(0, min(len(b), 400))
            b[pos] = random.choice([0x00, 0xFF, 0x7F, 0x80, b[pos] ^ (1 << random.randrange(8))])
            trials.append(bytes(b))
        q = str(tmp_path / "trial.oil")
        for t in trials:
            open(q, "wb").write(t)
            try:
                r = OILReader(q)
                for name in r.tensor_names():
                    try:
                        r.read_tensor(name)
                    except OILError:
                        rejected += 1
            except OILError:
                rejected += 1
        rawi = open(p + "idx", "rb").read()
        qi = str(tmp_path / "trial.oilidx")
        for c in range(0, len(rawi) - 1, 9):
            open(qi, "wb").write(rawi[:c])
            with pytest.raises(OILError):
                read_idx_file(qi)
    assert rejected > 50
