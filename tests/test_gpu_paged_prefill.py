"""GPU parity: chunked prefill into a PAGED cache: mf_paged_kv_append for the chunk's rows (bit-exact
against the oracle's contiguous append after gathering the pages), then mf_paged_prefill, whose
attention must match the oracle on the gathered contiguous cache (max-abs 2e-3, f32 tiled softmax and
fp64 gold).  The paged layout is not in the reference; it is pinned by the identity paged == contiguous.
"""
import numpy as np
import pytest

import oracle
from kvcases import dev, dev_u32, host, max_abs, normal

pytestmark = pytest.mark.gpu
TOL = 2e-3

# (n_heads, n_kv_heads, head_dim, page_size, cached, m)
CASES = [
    (14, 2, 64, 16, 64, 26),
    (16, 2, 128, 16, 500, 33),
    (24, 8, 128, 64, 768, 256),
    (8, 8, 128, 32, 0, 70),
    (16, 2, 128, 128, 1000, 48),
    (8, 2, 64, 8, 2100, 17),     # long enough for the split-K route
    # chunks of 64 rows and more take the tcgen05 kernel, which gathers its 128-key tiles page by page
    (16, 2, 128, 16, 500, 333),  # ragged tail: 833 keys, the last page holds one row
    (14, 2, 64, 16, 300, 200),
    (8, 2, 128, 8, 130, 129),
    (16, 2, 128, 128, 1000, 148),
    (24, 8, 128, 64, 2048, 512),
    (16, 2, 128, 32, 700, 200),
    (14, 2, 64, 8, 200, 100),
]


@pytest.mark.parametrize("case", CASES)
def test_paged_chunked_prefill(mfk, foundry, case):
    import torch

    hq, hkv, d, P, cached, m = case
    L = cached + m
    n_seq_pages = (L + P - 1) // P
    n_pages = n_seq_pages + 5
    rng = np.random.default_rng(cached * 31 + m)
    pages = rng.permutation(n_pages)[:n_seq_pages].astype(np.uint32)
    k_pool = np.full((n_pages, hkv, P, d), 0x7E00, np.uint16)  # NaN wherever nothing is written
    v_pool = np.full((n_pages, hkv, P, d), 0x7E00, np.uint16)
    kc = np.full((hkv, L, d), 0x7E00, np.uint16)
    vc = np.full((hkv, L, d), 0x7E00, np.uint16)
    kc[:, :cached] = normal(10, hkv * cached * d).reshape(hkv, cached, d)
    vc[:, :cached] = normal(11, hkv * cached * d).reshape(hkv, cached, d)
    for t in range(cached):
        k_pool[pages[t // P], :, t % P] = kc[:, t]
        v_pool[pages[t // P], :, t % P] = vc[:, t]
    q = normal(1, m * hq * d).reshape(m, hq * d)
    k = normal(2, m * hkv * d).reshape(m, hkv * d)
    v = normal(3, m * hkv * d).reshape(m, hkv * d)
    cos, sin = oracle.rope_tables(1e6, d, L)
    # the oracle on the contiguous cache
    q_ref = oracle.kv_prep_fused(q.ravel(), k.ravel(), v.ravel(), kc.ravel(), vc.ravel(), cos, sin, n_heads=hq,
                                 n_kv_heads=hkv, head_dim=d, seq_len=m, position_offset=cached, max_seq_len=L, rope_mode=0)
    scale = np.float32(1.0) / np.sqrt(np.float32(d))
    args = dict(n_heads=hq, cache_heads=hkv, head_dim=d, capacity=L, q_len=m, kv_len=L, query_offset=cached, scale=scale)
    want = oracle.prefill_causal(q_ref, kc.ravel(), vc.ravel(), **args)
    gold = oracle.prefill_gold(q_ref, kc.ravel(), vc.ravel(), **args)

    dk, dv = dev(k_pool), dev(v_pool)
    # the sequence is one of three in the batch; the other rows of the table point past the pool
    seq = (cached + m) % 3
    table = np.full((3, n_seq_pages), 0x7FFFFFF0, np.uint32)
    table[seq] = pages
    lens = np.ones(3, np.uint32)
    lens[seq] = L
    d_table, d_lens = dev_u32(table), dev_u32(lens)  # the descriptor holds raw pointers: keep these alive
    desc = mfk.paged_kv(dk, dv, d_table, d_lens, n_kv_heads=hkv, page_size=P, head_dim=d)
    q_rot = torch.full((hq, m, d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.paged_kv_append(desc, dev(q), dev(k), dev(v), q_rot, dev(cos), dev(sin), n_heads=hq, rope_mode=0, seq=seq,
                            position_offset=cached, seq_len=m)
    out = torch.full((m, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.paged_prefill(desc, q_rot, out, seq=seq, q_len=m, kv_len=L, query_offset=cached, n_heads=hq, scale=float(scale))
    foundry.synchronize()
    assert np.array_equal(host(q_rot).ravel(), q_ref)
    for pool_dev, cache_ref in ((dk, kc), (dv, vc)):  # the chunk's rows landed in the right pages, bit-exact
        got = np.empty((hkv, L, d), np.uint16)
        oracle.lib().mfo_paged_gather(np.ascontiguousarray(host(pool_dev)), pages, L, hkv, P, d, got)
        assert np.array_equal(got, cache_ref.reshape(hkv, L, d))
    assert max_abs(host(out), want) <= TOL
    assert max_abs(host(out), gold) <= TOL
    if m >= 64 and mfk.prefill_split_k(L, m) == 1:
        # both kernels on the same pages: the tcgen05 one (or fail) and the mma.sync one
        outs = {}
        for impl in (2, 1):
            foundry.set_option(3, impl)
            o = torch.full((m, hq * d), float("nan"), dtype=torch.float16, device="cuda")
            foundry.paged_prefill(desc, q_rot, o, seq=seq, q_len=m, kv_len=L, query_offset=cached, n_heads=hq,
                                  scale=float(scale))
            foundry.synchronize()
            outs[impl] = host(o)
        foundry.set_option(3, 0)
        assert max_abs(outs[2], want) <= TOL and max_abs(outs[2], gold) <= TOL
        assert max_abs(outs[1], want) <= TOL


def test_paged_prefill_rejects_bad_arguments(mfk, foundry):
    import torch

    dk = torch.zeros((4, 2, 16, 64), dtype=torch.float16, device="cuda")
    dv, d_table, d_lens = dk.clone(), dev_u32(np.zeros((1, 2), np.uint32)), dev_u32(np.array([20], np.uint32))
    desc = mfk.paged_kv(dk, dv, d_table, d_lens, n_kv_heads=2, page_size=16, head_dim=64)
    q = torch.zeros((4, 8, 64), dtype=torch.float16, device="cuda")
    out = torch.zeros((8, 4 * 64), dtype=torch.float16, device="cuda")
    with pytest.raises(mfk.MetalError) as e:  # 40 keys need three pages, the table has two
        foundry.paged_prefill(desc, q, out, seq=0, q_len=8, kv_len=40, query_offset=32, n_heads=4)
    assert e.value.kind == "InvalidOperation"
    with pytest.raises(mfk.MetalError) as e:
        foundry.paged_prefill(desc, q, out, seq=3, q_len=8, kv_len=20, query_offset=12, n_heads=4)
    assert e.value.kind == "InvalidOperation"
    with pytest.raises(mfk.MetalError) as e:  # heads do not divide
        foundry.paged_prefill(desc, q, out, seq=0, q_len=8, kv_len=20, query_offset=12, n_heads=5)
    assert e.value.kind == "InvalidShape"
    foundry.synchronize()
