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


def test_prefix_pages_shared_between_sequences(mfk, foundry):
    """A cached prefix is handed to a new sequence as shared pages; only the partly filled last page
    is copied before the new sequence appends into it.  The sharing sequence must produce the same
    bits as one that owns private copies of the same rows, and the cached pages must stay untouched."""
    import torch

    hq, hkv, d, P, n_prefix = 16, 2, 128, 16, 40
    n_pages = 12
    pool = mfk.PagePool(n_pages)
    cache = mfk.PrefixCache(pool, P)
    rng = np.random.default_rng(11)
    k_pool = np.full((n_pages, hkv, P, d), 0x7E00, np.uint16)  # NaN everywhere that is not written
    v_pool = np.full((n_pages, hkv, P, d), 0x7E00, np.uint16)
    rows_k = rng.standard_normal((hkv, n_prefix, d), dtype=np.float32).astype(np.float16).view(np.uint16)
    rows_v = rng.standard_normal((hkv, n_prefix, d), dtype=np.float32).astype(np.float16).view(np.uint16)

    def fill(pages):
        for t in range(n_prefix):
            k_pool[pages[t // P], :, t % P] = rows_k[:, t]
            v_pool[pages[t // P], :, t % P] = rows_v[:, t]

    tokens = rng.integers(1, 1000, size=n_prefix).astype(np.uint32)
    a_pages = pool.alloc(3)  # the sequence that computed the prefix
    fill(a_pages)
    cache.store(tokens, a_pages)
    pool.release(a_pages)  # it ends; the cache keeps the pages alive
    assert all(pool.refcount(int(p)) == 1 for p in a_pages)
    own_pages = pool.alloc(3)  # a sequence with private copies of the same rows
    fill(own_pages)

    dk, dv = dev(k_pool), dev(v_pool)
    prompt = np.concatenate([tokens, np.array([5, 6], np.uint32)])
    matched, shared = cache.lookup(prompt)
    assert matched == n_prefix and shared.tolist() == a_pages.tolist()
    # the new sequence will append at row 40, inside the last shared page: copy it first
    private = pool.alloc(1)
    t0, l0 = dev_u32(np.zeros((1, 1), np.uint32)), dev_u32(np.zeros(1, np.uint32))  # kept alive: the descriptor holds pointers
    desc0 = mfk.paged_kv(dk, dv, t0, l0, n_kv_heads=hkv, page_size=P, head_dim=d)
    foundry.paged_copy_pages(desc0, dev_u32(shared[-1:]), dev_u32(private), 1)
    pool.release(shared[-1:])
    b_pages = np.concatenate([shared[:-1], private])
    assert pool.refcount(int(a_pages[0])) == 2 and pool.refcount(int(a_pages[2])) == 1

    table = np.stack([b_pages, own_pages]).astype(np.uint32)
    kv_lens = np.array([n_prefix + 1, n_prefix + 1], np.uint32)
    d_table, d_lens = dev_u32(table), dev_u32(kv_lens)
    desc = mfk.paged_kv(dk, dv, d_table, d_lens, n_kv_heads=hkv, page_size=P, head_dim=d)
    q = rng.standard_normal((1, hq * d), dtype=np.float32).astype(np.float16).view(np.uint16).repeat(2, axis=0)
    k = rng.standard_normal((1, hkv * d), dtype=np.float32).astype(np.float16).view(np.uint16).repeat(2, axis=0)
    v = rng.standard_normal((1, hkv * d), dtype=np.float32).astype(np.float16).view(np.uint16).repeat(2, axis=0)
    cos, sin = oracle.rope_tables(1e6, d, n_prefix + 1)
    plan = foundry.decode_plan(kv_lens, n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P)
    out = torch.full((2, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.paged_decode(plan, desc, dev(q), out, n_heads=hq, k=dev(k), v=dev(v), cos=dev(cos), sin=dev(sin), rope=True,
                         rope_mode=0, append=True)
    foundry.synchronize()
    plan.close()
    got = host(out)
    assert np.isfinite(oracle.h2f(got)).all()
    assert np.array_equal(got[0], got[1])  # sharing changes nothing
    kp, vp = host(dk), host(dv)
    assert np.array_equal(kp[a_pages[2]], k_pool[a_pages[2]])  # the cached last page was not appended to
    assert np.array_equal(vp[a_pages[2]], v_pool[a_pages[2]])
    assert np.array_equal(kp[private[0], :, :n_prefix % P], k_pool[a_pages[2], :, :n_prefix % P])
    assert np.array_equal(kp[private[0], :, n_prefix % P], kp[own_pages[2], :, n_prefix % P])  # the appended row
    # the oracle on the private copy agrees within tolerance
    zero_row = np.zeros((hkv, 1, d), np.uint16)
    kc = np.ascontiguousarray(np.concatenate([rows_k, zero_row], axis=1))
    vc = np.ascontiguousarray(np.concatenate([rows_v, zero_row], axis=1))
    q_rot = oracle.kv_prep_fused(np.ascontiguousarray(q[0]), np.ascontiguousarray(k[0]), np.ascontiguousarray(v[0]), kc, vc,
                                 cos, sin, n_heads=hq, n_kv_heads=hkv, head_dim=d, seq_len=1, position_offset=n_prefix,
                                 max_seq_len=n_prefix + 1, rope_mode=0)
    assert np.array_equal(kc[:, n_prefix], kp[private[0], :, n_prefix % P])  # appended rows, bit-exact
    assert np.array_equal(vc[:, n_prefix], vp[private[0], :, n_prefix % P])
    ref = oracle.decode_online(q_rot, kc, vc, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=n_prefix + 1,
                               kv_len=n_prefix + 1, scale=np.float32(1.0 / np.sqrt(d)))
    assert max_abs(got[0], ref) <= 2e-3
    pool.release(b_pages)
    pool.release(own_pages)
    cache.close()
    assert pool.free_count == n_pages
    pool.close()
