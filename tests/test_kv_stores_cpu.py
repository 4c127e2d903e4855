import os

import torch

from mythos_b200.infer.kv_stores import KVCache, PagedKVCache1T


def test_contiguous_cache_fp_and_int8():
    torch.manual_seed(0)
    for int8 in (False, True):
        c = KVCache(2, 16, 2, 64, int8=int8)
        k1, v1 = torch.randn(1, 2, 5, 64), torch.randn(1, 2, 5, 64)
        for layer in range(2):
            c.append(layer, k1, v1)
        assert c.context_len() == 5
        k2 = torch.randn(1, 2, 1, 64)
        for layer in range(2):
            c.append(layer, k2, k2)
        ka, va = c.get_all(1)
        want = torch.cat([k1, k2], dim=2)
        tol = 0.0 if not int8 else float(want.abs().max()) / 127 * 0.51
        assert ka.shape == (1, 2, 6, 64) and (ka - want).abs().max() <= tol + 1e-7
        kr, _ = c.get_range(0, 2, 4)
        assert (kr - k1[:, :, 2:4]).abs().max() <= tol + 1e-7
        c.resize(32)
        assert c.max_seq == 32 and c.context_len() == 6 and (c.get_all(0)[0] - want).abs().max() <= tol + 1e-7
        c.clear()
        assert c.context_len() == 0
    assert KVCache(1, 8, 1, 64, int8=True).size_bytes() < KVCache(1, 8, 1, 64).size_bytes() / 3


def test_sparse_store_spills_and_reloads(tmp_path):
    torch.manual_seed(1)
    s = PagedKVCache1T(1, 2, 8, block_size=16, fanout=64, max_resident=2, spill_dir=str(tmp_path))
    assert s.capacity_tokens() == 64 ** 3 * 16
    pos = [0, 5, 17, 40, 1_000_000, 3_000_017]
    data = {p: (torch.randn(2, 8), torch.randn(2, 8)) for p in pos}
    for p in pos:
        s.append(0, p, *data[p])
    assert len(s.resident) == 2 and s.stats["evictions"] >= 3
    assert any(f.startswith("paged_kv_l0_b") for f in os.listdir(tmp_path))
    for p in pos:
        assert s.verify_retrieval(0, p, *data[p])
    assert s.stats["reloads"] >= 3
    k, v = s.get_range(0, 0, 20)
    assert torch.equal(k[5], data[5][0]) and torch.equal(k[17], data[17][0]) and float(k[1].abs().sum()) == 0.0
    assert s.flush_to_disk() == 2 and len(s.resident) == 0
    assert s.verify_retrieval(0, 1_000_000, *data[1_000_000])
    try:
        s.append(0, 64 ** 3 * 16, *data[0])
        assert False
    except ValueError:
        pass


def test_paged_cache_prefix_sharing_and_recycled_pages():
    from mythos_b200.infer.kv_paged import PagedKVCache

    c = PagedKVCache(num_layers=1, kv_heads=1, head_dim=8, num_pages=8, page_size=4, max_seqs=4, max_pages_per_seq=4,
                     device="cpu", dtype=torch.float32)
    toks = list(range(10))
    a = c.new_sequence()
    c.reserve(a, len(toks))
    c.advance(a, len(toks))
    c.publish_prefix(a, toks)                       # two full pages
    assert c.alloc.used == 3
    b = c.new_sequence()
    assert c.share_prefix(b, toks[:9]) == 8 and c.lens[b] == 8
    pages_a = [int(p) for p in c.block_table_host[a][:2]]
    assert [int(p) for p in c.block_table_host[b][:2]] == pages_a and all(c.alloc.refs[p] == 2 for p in pages_a)
    c.reserve(b, 2)
    assert c.alloc.used == 4
    c.free_sequence(a)
    assert all(c.alloc.refs[p] == 1 for p in pages_a)   # still held by b
    c.free_sequence(b)
    assert c.alloc.used == 0
    # the pages go to someone else: the published entry must not match them any more
    d = c.new_sequence()
    c.reserve(d, 16)
    e = c.new_sequence()
    assert c.share_prefix(e, toks[:9]) == 0
    # int8 pages carry scales and count them
    q = PagedKVCache(1, 2, 64, 4, 16, 2, 2, device="cpu", dtype=torch.int8)
    assert q.int8 and q.k_scale[0].shape == (64, 2) and q.size_bytes() == 2 * (4 * 16 * 2 * 64 + 64 * 2 * 4)
