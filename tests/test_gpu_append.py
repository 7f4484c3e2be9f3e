"""GPU parity: RoPE + K/V append kernels against the CPU oracle, through the C ABI.

Shapes follow the reference's own tests (crates/metallic-foundry/tests/kv_prep_fused.rs:249-267,
tests/rope.rs:160-253, tests/kv_cache.rs:55-179) plus the benchmark configurations.
Bar: bit-exact (slot addressing, V copy, and the roped f16 values: both f32 products are
exact, so the CUDA and the oracle arithmetic agree to the bit; the contract allows 1 ulp).
"""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, dev, host, lcg, ulp_distance

pytestmark = pytest.mark.gpu


def run_kv_prep(mfk, foundry, case, layer_idx=0, no_rope_layer_step=0):
    import torch

    q, k, v = dev(case.q), dev(case.k), dev(case.v)
    kc, vc = dev(case.k_cache), dev(case.v_cache)
    cos, sin = dev(case.cos), dev(case.sin)
    q_rot = torch.full((case.Hq * case.M * case.D,), float("nan"), dtype=torch.float16, device="cuda")
    p = mfk.KvPrepFusedParamsResolved(case.Hq * case.D, case.Hkv * case.D, case.D, case.Hq, case.Hkv, case.G, case.M,
                                      case.cached, case.cap, case.Hq * case.M * case.D, case.rope_mode, layer_idx,
                                      no_rope_layer_step)
    foundry.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, p)
    foundry.synchronize()
    return host(q_rot), host(kc), host(vc)


# (seq_len, position_offset, max_seq_len, n_heads, n_kv_heads, head_dim): tests/kv_prep_fused.rs:249-267
REF_SHAPES = [(1, 5, 16, 14, 2, 64), (4, 0, 16, 14, 2, 64), (2, 0, 64, 32, 8, 128)]
# decode step of the benchmark configurations + a prefill chunk
BENCH_SHAPES = [(1, 511, 512, 14, 2, 64), (1, 8191, 8192, 24, 8, 128), (1, 777, 1024, 16, 2, 128),
                (96, 160, 256, 24, 8, 128)]


@pytest.mark.parametrize("shape", REF_SHAPES + BENCH_SHAPES)
@pytest.mark.parametrize("rope_mode", [0, 1])
@pytest.mark.parametrize("expanded", [False, True])
def test_kv_prep_fused_bit_exact(mfk, foundry, shape, rope_mode, expanded):
    m, off, cap, hq, hkv, d = shape
    if expanded and cap > 1024:
        pytest.skip("expanded layout is covered at the small shapes")
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=off, m=m, capacity=cap, theta=1e4,
                      rope_mode=rope_mode, expanded=expanded)
    q_ref, k_ref, v_ref = case.oracle_append()
    q_got, k_got, v_got = run_kv_prep(mfk, foundry, case)
    assert ulp_distance(q_got, q_ref) == 0
    assert np.array_equal(k_got, k_ref)  # whole cache: the new rows and nothing else changed
    assert np.array_equal(v_got, v_ref)


def test_kv_prep_fused_equals_unfused_chain(mfk, foundry):
    """The reference pins the fused kernel against KvRearrange -> Rope -> KvCacheWrite
    (tests/kv_prep_fused.rs:233-244): K/V cache bit-exact."""
    import torch

    m, off, cap, hq, hkv, d = 4, 3, 32, 14, 2, 64
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=off, m=m, capacity=cap, theta=1e4, rope_mode=0)
    _, k_fused, v_fused = run_kv_prep(mfk, foundry, case)
    # the unfused chain on the GPU: KvRearrange, Rope, KvCacheWrite
    k_heads = np.empty((hkv, m, d), np.uint16)
    v_heads = np.empty((hkv, m, d), np.uint16)
    L = oracle.lib()
    L.mfo_kv_rearrange(case.k, k_heads, hkv * d, d, hkv, hkv, d, m)
    L.mfo_kv_rearrange(case.v, v_heads, hkv * d, d, hkv, hkv, d, m)
    rp = mfk.KvRearrangeParamsResolved(hkv * d, hkv * d, d, hkv, hkv, d, m, hkv * m * d)
    k_in = torch.empty((hkv, m, d), dtype=torch.float16, device="cuda")
    v_in = torch.empty((hkv, m, d), dtype=torch.float16, device="cuda")
    foundry.kv_rearrange(dev(case.k), k_in, rp)
    foundry.kv_rearrange(dev(case.v), v_in, rp)
    foundry.synchronize()
    assert np.array_equal(host(k_in), k_heads) and np.array_equal(host(v_in), v_heads)
    k_rot = torch.empty((hkv, m, d), dtype=torch.float16, device="cuda")
    foundry.rope(k_in, k_rot, dev(case.cos), dev(case.sin), mfk.RopeParamsResolved(d, m, off, hkv * m * d))
    kc, vc = dev(case.k_cache), dev(case.v_cache)
    wp = mfk.KvCacheWriteParamsResolved(hkv, d, m, off, cap, hkv * m * d, 0)
    foundry.kv_cache_write(k_rot, kc, wp)
    foundry.kv_cache_write(v_in, vc, wp)
    foundry.synchronize()
    assert np.array_equal(host(kc), k_fused)
    assert np.array_equal(host(vc), v_fused)


def test_kv_prep_no_rope_layer_step(mfk, foundry):
    """Every N-th layer skips RoPE (kv_prep_fused.metal:56-57; SmolLM3 uses N=4)."""
    case = ContigCase(n_heads=8, n_kv_heads=2, head_dim=64, cached=2, m=3, capacity=16, rope_mode=1)
    for layer in range(8):
        ref = case.oracle_append(layer_idx=layer, no_rope_layer_step=4)
        got = run_kv_prep(mfk, foundry, case, layer_idx=layer, no_rope_layer_step=4)
        for a, b in zip(got, ref):
            assert np.array_equal(a, b)
    # layer 3 must be a pure rearrangement
    q_rot, _, _ = run_kv_prep(mfk, foundry, case, layer_idx=3, no_rope_layer_step=4)
    expect = case.q.reshape(3, 8, 64).transpose(1, 0, 2).ravel()
    assert np.array_equal(q_rot, expect)


# (dim, seq_len, num_rows, position_offset): tests/rope.rs:160-253
ROPE_SHAPES = [(64, 8, 4, 0), (128, 16, 8, 0), (256, 32, 4, 0), (64, 1, 14, 0), (64, 1, 4, 10), (64, 8, 14, 0),
               (64, 127, 3, 0), (128, 1, 32, 1024)]


@pytest.mark.parametrize("shape", ROPE_SHAPES)
def test_rope_matches_cpu_rope(mfk, foundry, shape):
    import torch

    dim, seq_len, num_rows, off = shape
    total = num_rows * seq_len * dim
    x = lcg(7, total, 1.0)
    cos, sin = oracle.rope_tables(1e4, dim, off + seq_len)
    ref = np.empty(total, np.uint16)
    oracle.lib().mfo_rope_neox(x, ref, cos, sin, dim, seq_len, off, total)
    out = torch.empty(total, dtype=torch.float16, device="cuda")
    foundry.rope(dev(x), out, dev(cos), dev(sin), mfk.RopeParamsResolved(dim, seq_len, off, total))
    foundry.synchronize()
    assert np.array_equal(host(out), ref)


def test_kv_cache_write_read_roundtrip(mfk, foundry):
    """tests/kv_cache.rs: write at an offset, read the prefix back; expanded write repeats heads."""
    import torch

    hkv, d, cap = 2, 8, 16
    x0, x1 = lcg(1, hkv * 3 * d, 1.0).reshape(hkv, 3, d), lcg(2, hkv * 1 * d, 1.0).reshape(hkv, 1, d)
    cache = torch.zeros((hkv, cap, d), dtype=torch.float16, device="cuda")
    ref = np.zeros((hkv, cap, d), np.uint16)
    foundry.kv_cache_write(dev(x0), cache, mfk.KvCacheWriteParamsResolved(hkv, d, 3, 0, cap, hkv * 3 * d, 0))
    foundry.kv_cache_write(dev(x1), cache, mfk.KvCacheWriteParamsResolved(hkv, d, 1, 3, cap, hkv * d, 0))
    oracle.lib().mfo_kv_cache_write(ref, x0, hkv, d, 3, 0, cap)
    oracle.lib().mfo_kv_cache_write(ref, x1, hkv, d, 1, 3, cap)
    out = torch.empty((hkv, 4, d), dtype=torch.float16, device="cuda")
    foundry.kv_cache_read(cache, out, 4)
    foundry.synchronize()
    assert np.array_equal(host(cache), ref)
    ref_read = np.empty((hkv, 4, d), np.uint16)
    oracle.lib().mfo_kv_cache_read(ref, ref_read, hkv, d, 4, cap)
    assert np.array_equal(host(out), ref_read)
    # expanded
    g = 3
    big = torch.zeros((hkv * g, cap, d), dtype=torch.float16, device="cuda")
    ref_big = np.zeros((hkv * g, cap, d), np.uint16)
    foundry.kv_cache_write(dev(x0), big, mfk.KvCacheWriteRepeatKvHeadsParamsResolved(hkv, hkv * g, g, d, 3, 5, cap,
                                                                                      hkv * 3 * d, 0))
    oracle.lib().mfo_kv_cache_write_repeat(ref_big, x0, hkv, g, d, 3, 5, cap)
    foundry.synchronize()
    assert np.array_equal(host(big), ref_big)


def test_kv_prep_rejects_bad_arguments(mfk, foundry):
    """Contract violations are reported on the host with the reference's error kinds."""
    import torch

    case = ContigCase(n_heads=14, n_kv_heads=2, head_dim=64, cached=15, m=2, capacity=16)
    q, k, v = dev(case.q), dev(case.k), dev(case.v)
    kc, vc, cos, sin = dev(case.k_cache), dev(case.v_cache), dev(case.cos), dev(case.sin)
    q_rot = torch.empty(14 * 2 * 64, dtype=torch.float16, device="cuda")
    P = mfk.KvPrepFusedParamsResolved
    with pytest.raises(mfk.MetalError) as e:  # position_offset + seq_len > max_seq_len
        foundry.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, P(896, 128, 64, 14, 2, 7, 2, 15, 16, 1792, 0, 0, 0))
    assert e.value.kind == "InvalidOperation"
    with pytest.raises(mfk.MetalError) as e:  # group size inconsistent
        foundry.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, P(896, 128, 64, 14, 2, 5, 1, 0, 16, 896, 0, 0, 0))
    assert e.value.kind == "InvalidShape"
    with pytest.raises(mfk.MetalError) as e:  # cache heads neither compact nor expanded
        bad = torch.zeros((3, 16, 64), dtype=torch.float16, device="cuda")
        foundry.kv_prep_fused(q, k, v, q_rot, bad, bad, cos, sin, P(896, 128, 64, 14, 2, 7, 1, 0, 16, 896, 0, 0, 0))
    assert e.value.kind == "InvalidShape"
    with pytest.raises(mfk.MetalError) as e:  # wrong dtype
        foundry.kv_prep_fused(q.float(), k, v, q_rot, kc, vc, cos, sin, P(896, 128, 64, 14, 2, 7, 1, 0, 16, 896, 0, 0, 0))
    assert e.value.kind == "UnsupportedDtype"
    foundry.synchronize()
    assert np.array_equal(host(kc), case.k_cache)  # nothing was launched


def test_kv_rearrange_and_repeat_kv_heads(mfk, foundry):
    """KvRearrange with grouped heads and a padded row stride (kv_rearrange.metal:27-46), RepeatKvHeads out
    of a cache with capacity slack (repeat_kv_heads.metal:25-43): pure index maps, bit-exact."""
    import torch

    hq, hkv, d, seq, row_stride = 12, 4, 64, 7, 4 * 64 + 32
    rows = oracle.normal_fill(5, 1, seq * row_stride).reshape(seq, row_stride)
    want = np.empty((hq, seq, d), np.uint16)
    oracle.lib().mfo_kv_rearrange(rows, want, row_stride, d, hq, hkv, d, seq)
    got = torch.full((hq, seq, d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.kv_rearrange(dev(rows), got, mfk.KvRearrangeParamsResolved(hkv * d, row_stride, d, hq, hkv, d, seq, hq * seq * d))
    foundry.synchronize()
    assert np.array_equal(host(got), want)
    # kv_dim smaller than the heads ask for: the elements past it are left alone (kv_rearrange.metal:40)
    got2 = torch.zeros((hq, seq, d), dtype=torch.float16, device="cuda")
    foundry.kv_rearrange(dev(rows), got2, mfk.KvRearrangeParamsResolved(3 * d, row_stride, d, hq, hkv, d, seq, hq * seq * d))
    foundry.synchronize()
    g = hq // hkv
    assert np.array_equal(host(got2)[:3 * g], want[:3 * g]) and not host(got2)[3 * g:].any()

    cap, live = 32, 19
    cache = oracle.normal_fill(5, 2, hkv * cap * d).reshape(hkv, cap, d)
    rep_want = np.empty((hq, live, d), np.uint16)
    oracle.lib().mfo_repeat_kv_heads(np.ascontiguousarray(cache[:, :live]), rep_want, hkv, g, live, d)
    rep = torch.full((hq, live, d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.repeat_kv_heads(dev(cache), rep, mfk.RepeatKvHeadsParamsResolved(g, 1, hkv, hq, live, d, cap, hq * live * d))
    foundry.synchronize()
    assert np.array_equal(host(rep), rep_want)
    with pytest.raises(mfk.MetalError) as e:
        foundry.repeat_kv_heads(dev(cache), rep, mfk.RepeatKvHeadsParamsResolved(g, 1, hkv, hq + 1, live, d, cap, 1))
    assert e.value.kind == "InvalidShape"
