"""GPU parity: KV growth copy and contiguous -> paged migration, bit-exact against the oracle.

Growth follows ensure_kv_capacity / reallocate_kv_buffers of the reference
(src/model/executor.rs:2332-2619): capacity 2048 -> max(2x, required) aligned to 128, per-head copy
of the live rows, RoPE tables extended for the new positions; decode over the grown cache must give
the same bits as before the growth.
"""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, PagedCase, dev, dev_u32, host, max_abs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(8, 128, 300, 384, 768), (2, 64, 511, 512, 1024), (14, 64, 1, 128, 256),
                                   (8, 128, 2048, 2048, 4096)])
def test_growth_copy_bit_exact(mfk, foundry, shape):
    import torch

    heads, d, pos, old_cap, new_cap = shape
    assert mfk.grown_capacity(old_cap, old_cap + 1, 1 << 20) == new_cap
    old = oracle.normal_fill(9, 1, heads * old_cap * d).reshape(heads, old_cap, d)
    ref = np.full((heads, new_cap, d), 0x1234, np.uint16)
    oracle.lib().mfo_kv_cache_grow(old, ref, heads, d, old_cap, new_cap, pos)
    new = torch.from_numpy(np.full((heads, new_cap, d), 0x1234, np.uint16).view(np.float16)).cuda()
    foundry.kv_cache_grow(dev(old), new, pos)
    foundry.synchronize()
    assert np.array_equal(host(new), ref)


def test_decode_is_unchanged_by_growth(mfk, foundry):
    import torch

    case = ContigCase(n_heads=24, n_kv_heads=8, head_dim=128, cached=2047, capacity=2048, theta=5e5, rope_mode=1)
    q_rot, kc, vc = case.oracle_append()

    def decode(k, v, cap):
        out = torch.zeros(24 * 128, dtype=torch.float16, device="cuda")
        st = mfk.MfFlashDecodeStrides(24 * 128, 128, 8 * cap * 128, cap * 128, 8 * cap * 128, cap * 128, 24 * 128, 128)
        foundry.flash_decode(dev(q_rot), k, v, out, st, mfk.SdpaParams(2048, 128, float(case.scale), 128, 128), 24, 1, 0)
        foundry.synchronize()
        return host(out)

    before = decode(dev(kc), dev(vc), 2048)
    new_cap = mfk.grown_capacity(2048, 2049, 8192)
    assert new_cap == 4096
    k2 = torch.zeros((8, new_cap, 128), dtype=torch.float16, device="cuda")
    v2 = torch.zeros_like(k2)
    foundry.kv_cache_grow(dev(kc), k2, 2048)
    foundry.kv_cache_grow(dev(vc), v2, 2048)
    assert np.array_equal(decode(k2, v2, new_cap), before)
    # the RoPE tables continue where the old ones stopped
    cos_old, sin_old = mfk.rope_tables(5e5, 128, 2048)
    cos_ext, sin_ext = mfk.rope_tables(5e5, 128, new_cap - 2048, first_pos=2048)
    cos_all, sin_all = mfk.rope_tables(5e5, 128, new_cap)
    assert np.array_equal(np.concatenate([cos_old, cos_ext]), cos_all)
    assert np.array_equal(np.concatenate([sin_old, sin_ext]), sin_all)


def test_growth_rejects_bad_arguments(mfk, foundry):
    import torch

    a = torch.zeros((8, 128, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(mfk.MetalError) as e:
        foundry.kv_cache_grow(a, torch.zeros((4, 256, 64), dtype=torch.float16, device="cuda"), 10)
    assert e.value.kind == "InvalidShape"
    with pytest.raises(mfk.MetalError) as e:
        foundry.kv_cache_grow(a, torch.zeros((8, 256, 64), dtype=torch.float16, device="cuda"), 129)
    assert e.value.kind == "InvalidOperation"


def test_contiguous_to_pages_roundtrip(mfk, foundry):
    """Migration into the paged pool equals the oracle's scatter, and gathering it back is the identity."""
    import torch

    case = PagedCase(batch=3, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[70, 333, 15], poison=False)
    k_pool, v_pool = dev(case.k_pool), dev(case.v_pool)
    pt, lens = dev_u32(case.page_table), dev_u32(case.kv_lens)
    desc = mfk.paged_kv(k_pool, v_pool, pt, lens, n_kv_heads=2, page_size=16, head_dim=128)
    ref_k = case.k_pool.copy()
    for b in range(3):
        n, cap = int(case.cached[b]), int(case.cached[b]) + 5
        cache = oracle.normal_fill(21, b, 2 * cap * 128).reshape(2, cap, 128)
        oracle.lib().mfo_paged_scatter(cache, ref_k, case.page_table[b], n, 2, cap, 16, 128)
        d_cache = dev(cache)
        foundry.kv_cache_to_pages(d_cache, desc, False, b, n)
        back = torch.zeros((2, n, 128), dtype=torch.float16, device="cuda")
        foundry.paged_gather(desc, False, b, n, back)
        foundry.synchronize()
        assert np.array_equal(host(back), cache[:, :n])
    assert np.array_equal(host(k_pool), ref_k)
    assert np.array_equal(host(v_pool), case.v_pool)  # the V pool was not touched


def test_prefix_snapshot_and_restore(mfk, foundry):
    """KV prefix snapshots of the reference (src/model/executor.rs:1136-1350) are per-head copies of
    rows [0, prefix_len) into a private buffer and back: KvCacheRead saves, KvCacheWrite restores,
    also into a cache of another capacity.  A decode over the restored cache gives the same bits."""
    import torch

    hq, hkv, d, cap, prefix = 16, 2, 128, 640, 500
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=prefix - 1, capacity=cap)
    q_rot, kc, vc = case.oracle_append()
    k_dev, v_dev = dev(kc), dev(vc)
    snap_k = torch.empty((hkv, prefix, d), dtype=torch.float16, device="cuda")
    snap_v = torch.empty_like(snap_k)
    foundry.kv_cache_read(k_dev, snap_k, prefix)
    foundry.kv_cache_read(v_dev, snap_v, prefix)
    new_cap = 1024
    k2 = torch.zeros((hkv, new_cap, d), dtype=torch.float16, device="cuda")
    v2 = torch.zeros_like(k2)
    wp = mfk.KvCacheWriteParamsResolved(hkv, d, prefix, 0, new_cap, hkv * prefix * d, 0)
    foundry.kv_cache_write(snap_k, k2, wp)
    foundry.kv_cache_write(snap_v, v2, wp)
    foundry.synchronize()
    assert np.array_equal(host(k2)[:, :prefix], kc[:, :prefix]) and not host(k2)[:, prefix:].any()

    def decode(k, v, c):
        out = torch.zeros(hq * d, dtype=torch.float16, device="cuda")
        st = mfk.MfFlashDecodeStrides(hq * d, d, hkv * c * d, c * d, hkv * c * d, c * d, hq * d, d)
        foundry.flash_decode(dev(q_rot), k, v, out, st, mfk.SdpaParams(prefix, d, float(case.scale), d, d), hq, 1, 0)
        foundry.synchronize()
        return host(out)

    assert np.array_equal(decode(k2, v2, new_cap), decode(k_dev, v_dev, cap))
