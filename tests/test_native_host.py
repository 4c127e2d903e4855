"""The C++ host runtime against its Python twins: container reader/writer, SHA-256, sidecar check,
BPE, RNG, page allocator."""
import hashlib
import os

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


def test_native_reader_rejects_corrupt_block_ranges_and_sizes(tmp_path):
    """A tensor entry that points past the block table, and a block whose weight count needs more
    index bytes than the file holds, are errors (they used to index out of range / read past the
    mapping)."""
    import struct

    from mythos_b200.oil import container as oc
    from mythos_b200.oil.formats import Format

    p = str(tmp_path / "g.oil")
    oc.write_oil(p, [("w", [oc.BlockData(Format.FP32, 8, b"", np.arange(8, dtype=np.float32).tobytes())])])
    raw = open(p, "rb").read()
    o = 16 + struct.unpack_from("<I", raw, 12)[0]
    nb = struct.unpack_from("<I", raw, o)[0]
    fmt_byte = o + 4 + 4
    t = o + 4 + 9 * nb + 4
    ln = struct.unpack_from("<H", raw, t)[0]
    start_off = t + 2 + ln
    block0 = start_off + 8
    for off in (start_off, start_off + 4):
        b = bytearray(raw)
        struct.pack_into("<I", b, off, 0x100000)
        q = tmp_path / "range.oil"
        q.write_bytes(bytes(b))
        with pytest.raises(oc.OILError, match="beyond the block table"):
            native_io.NativeReader(str(q))
    b = bytearray(raw)
    b[fmt_byte] = int(Format.FP16)
    struct.pack_into("<I", b, block0, 50_000_000)
    q = tmp_path / "size.oil"
    q.write_bytes(bytes(b))
    r = native_io.NativeReader(str(q))
    with pytest.raises(oc.OILError, match="index data shorter"):
        r.read_tensor("w")
    r.close()


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


ASAN_WORKER = r'''
import os, random, struct, sys
import numpy as np
sys.path.insert(0, os.environ["REPO_ROOT"])
from mythos_b200.oil import native_io
from mythos_b200.oil.container import OILError

work = sys.argv[1]
assert native_io.lib()._name.endswith("liboil_host_asan.so")     # the sanitizer build is the one in use
random.seed(0)
opened = rejected = 0

def try_read(path):
    global opened, rejected
    try:
        r = native_io.NativeReader(path)
    except OILError:
        rejected += 1
        return
    opened += 1
    try:
        for name in r.tensor_names():
            try:
                r.read_tensor(name)
                r.tensor_sha256(name)
            except OILError:
                pass
    finally:
        r.close()

for fname in sorted(os.listdir(work)):
    if not fname.endswith(".oil"):
        continue
    raw = open(os.path.join(work, fname), "rb").read()
    try_read(os.path.join(work, fname))
    cuts = sorted(set(list(range(0, min(len(raw), 160), 3)) + [len(raw) * i // 23 for i in range(23)] + [len(raw) - 1]))
    for cut in cuts:                                   # truncation anywhere must be an error, not a bad read
        p = os.path.join(work, "cut.bin")
        open(p, "wb").write(raw[:cut])
        try_read(p)
    for _ in range(150):                               # corrupt sizes / counts / offsets in the tables
        b = bytearray(raw)
        pos = random.randrange(0, min(len(b), 400))
        b[pos] = random.choice([0x00, 0xFF, 0x7F, 0x80, b[pos] ^ (1 << random.randrange(8))])
        p = os.path.join(work, "flip.bin")
        open(p, "wb").write(bytes(b))
        try_read(p)
    # structured corruption: the fields that size later reads, at their offsets in this file
    u32 = lambda o: struct.unpack_from("<I", raw, o)[0]
    o = 16 + u32(12)
    nb = u32(o); fmt_table = o + 4; o = fmt_table + 9 * nb
    nt = u32(o); o += 4
    fields = [(fmt_table + 9 * i + 4, 1) for i in range(min(nb, 6))]          # per-block format byte
    for _ in range(nt):
        ln = struct.unpack_from("<H", raw, o)[0]; o += 2 + ln
        fields += [(o, 4), (o + 4, 4)]; o += 8                                   # tensor start / count
    for _ in range(min(nb, 6)):                                                  # block headers
        cbn = u32(o + 4); ibn = u32(o + 8 + cbn)
        fields += [(o, 4), (o + 4, 4), (o + 8 + cbn, 4)]                         # num_weights / cb / idx bytes
        o += 12 + cbn + ibn
    for pos, width in fields:
        for val in (0, 1, 0x7F, 0xFF, 0x100000, 50_000_000, 0x7FFFFFFF, 0xFFFFFFFF):
            for fmt_byte in ((None,) if width == 4 else (0, 1, 2, 3, 4, 5, 9)):
                b = bytearray(raw)
                if width == 4:
                    struct.pack_into("<I", b, pos, val)
                else:
                    b[pos] = fmt_byte
                p = os.path.join(work, "field.bin")
                open(p, "wb").write(bytes(b))
                try_read(p)
            if width == 1:
                break
    idx = os.path.join(work, fname + "idx")
    if os.path.exists(idx):
        rawi = open(idx, "rb").read()
        for cut in range(0, len(rawi), 7):
            p = os.path.join(work, "cut.oilidx")
            open(p, "wb").write(rawi[:cut])
            try:
                native_io.idx_check(p)
            except OILError:
                pass
text = (b"the quick brown fox jumps over the lazy dog. " * 40) + bytes(range(256))
bpe = native_io.NativeBPE.train(text, 300)
assert bpe.decode(bpe.encode(text)) == text
assert bpe.decode(bpe.encode(b"")) == b""
rng = native_io.NativeRNG(7)
assert rng.fill_uniform(1000, -1.0, 1.0).shape == (1000,)
pool = native_io.NativePageAllocator(4)
pages = [pool.alloc() for _ in range(4)]
for p in pages:
    pool.release(p)
assert pool.used == 0
assert native_io.sha256(b"abc").hex().startswith("ba7816bf")
L = native_io.lib()
toks = np.arange(500, dtype=np.int32)
h = L.oil_loader_create(toks.ctypes.data, toks.size, 3, 8, 1, 5, 2)
ids, tgt = np.empty((3, 8), np.int32), np.empty((3, 8), np.int32)
for epoch in range(3):
    L.oil_loader_reset(h, epoch)
    n = 0
    while L.oil_loader_next(h, ids.ctypes.data, tgt.ctypes.data):
        assert (tgt[:, :-1] == ids[:, 1:]).all()
        n += 1
        if epoch == 2 and n == 5:
            break                                      # freed with batches still queued
    assert n == (L.oil_loader_num_batches(h) if epoch < 2 else 5)
L.oil_loader_free(h)
print("ASAN_OK", opened, rejected)
'''


def test_host_runtime_under_address_and_ub_sanitizers(tmp_path):
    """Truncated and bit-flipped containers, sidecars, BPE, RNG and the page pool through the host
    library built with -fsanitize=address,undefined: every malformed file must end in an OILError
    (or a clean read), never in an out-of-bounds access."""
    import subprocess
    import sys

    from mythos_b200 import build
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.oil.model_io import save_model

    asan = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("no AddressSanitizer runtime in this toolchain")
    lib = build.build_host_sanitized(tmp_path)
    torch.manual_seed(0)
    work = tmp_path / "files"
    work.mkdir()
    for fmt in ("oil8", "oil4", "i2s", "fp16"):
        cfg = TransformerConfig(vocab_size=32, hidden_size=32, num_layers=1, num_heads=2, head_dim=16,
                                ffn_hidden_size=64, max_seq_len=16, weight_format=fmt, oil_block_size=32)
        save_model(DenseModel(cfg), str(work / f"{fmt}.oil"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, REPO_ROOT=root, LD_PRELOAD=asan, MYTHOS_HOST_LIB=str(lib),
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=66", UBSAN_OPTIONS="halt_on_error=1:exitcode=67")
    res = subprocess.run([sys.executable, "-c", ASAN_WORKER, str(work)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "ASAN_OK" in res.stdout, res.stdout[-1500:] + res.stderr[-4000:]


def test_native_token_loader_matches_python_windows_and_shuffles_per_epoch():
    from mythos_b200.train.data import TokenDataset

    tokens = np.arange(1000, dtype=np.int32)
    nat = native_io.NativeTokenLoader(tokens, batch=4, seq=16, shuffle=False, prefetch=3)
    py = TokenDataset(tokens, 4, 16, shuffle=False, prefetch=0)
    assert len(nat) == len(py) == 15
    for _ in range(2):                                   # two passes give the same batches
        nat.reset(0)
        got = list(nat)
        assert len(got) == 15
        for (a, b), (c, d) in zip(got, py):
            assert torch.equal(a, c) and torch.equal(b, d)
    sh = native_io.NativeTokenLoader(tokens, 4, 16, shuffle=True, seed=7, prefetch=2)
    e0 = [b[0][:, 0].tolist() for b in sh]
    sh.reset(0)
    assert [b[0][:, 0].tolist() for b in sh] == e0       # deterministic in (seed, epoch)
    sh.reset(1)
    e1 = [b[0][:, 0].tolist() for b in sh]
    starts0, starts1 = sorted(sum(e0, [])), sorted(sum(e1, []))
    assert e1 != e0 and len(set(starts0)) == 60 and all(s % 16 == 0 for s in starts0) and len(set(starts1)) == 60
    for ids, tgt in sh:
        pass                                             # an exhausted epoch yields nothing more
    half = iter(native_io.NativeTokenLoader(tokens, 4, 16, prefetch=2))
    next(half)                                           # dropping a loader mid-epoch stops its worker
    del half
    with pytest.raises(ValueError):
        native_io.NativeTokenLoader(np.zeros(1, dtype=np.int32), 1, 1)
