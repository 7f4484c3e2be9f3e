"""GPU parity: flash-decode over the contiguous cache against the CPU oracle, through the C ABI.

Tolerance: max-abs 2e-3 against the oracle's f32 online softmax and against the fp64
gold (the stated contract of this path; the reference's own tests allow 5e-2 / 6e-2:
tests/sdpa_v2_parity.rs:239, tests/flashattention_decode_parity.rs:190).
"""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, dev, host, lcg, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3


def decode_strides(mfk, case, batch_heads=None):
    hq, d, cap, ch = case.Hq, case.D, case.cap, case.cache_heads
    return mfk.MfFlashDecodeStrides(hq * d, d, ch * cap * d, cap * d, ch * cap * d, cap * d, hq * d, d)


def oracle_decode(case, q_rot, kc, vc):
    out = oracle.decode_online(q_rot, kc, vc, n_heads=case.Hq, cache_heads=case.cache_heads, head_dim=case.D,
                               capacity=case.cap, kv_len=case.L, scale=case.scale)
    gold = oracle.decode_gold(q_rot, kc, vc, n_heads=case.Hq, cache_heads=case.cache_heads, head_dim=case.D,
                              capacity=case.cap, kv_len=case.L, scale=case.scale)
    return out, gold


def gpu_decode(mfk, foundry, case, q_rot, kc, vc, n_splits=0):
    import torch

    out = torch.full((case.Hq * case.D,), float("nan"), dtype=torch.float16, device="cuda")
    sp = mfk.SdpaParams(case.L, case.D, float(case.scale), case.D, case.D)
    foundry.flash_decode(dev(q_rot), dev(kc), dev(vc), out, decode_strides(mfk, case), sp, case.Hq, 1, n_splits)
    foundry.synchronize()
    return host(out)


# (n_heads, n_kv_heads, head_dim, cached, capacity, expanded)
SHAPES = [
    (14, 2, 64, 511, 512, False),     # configuration 1: Qwen2.5-0.5B layer, 511 cached + 1
    (14, 14, 64, 127, 128, True),     # tests/flashattention_decode_parity.rs: Hq=14 D=64 L=128, expanded cache
    (14, 14, 64, 26, 64, True),       # L=27 in a capacity-64 buffer
    (8, 8, 128, 127, 128, True),      # Hq=8 D=128 L=128
    (24, 8, 128, 2047, 2048, False),  # Llama-3.2-3B heads, G=3
    (16, 2, 128, 999, 1024, False),   # Qwen2.5-3B heads, G=8
    (32, 2, 128, 300, 384, False),    # G=16: two 8-head tiles
    (4, 4, 128, 0, 128, False),       # a single key
    (14, 2, 64, 63, 64, False),       # exactly one tile
    (14, 2, 64, 64, 130, False),      # one key into the second tile, odd capacity
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("rope_mode", [0, 1])
def test_append_then_decode(mfk, foundry, shape, rope_mode):
    """KvPrepFused then FlashDecode, the reference's per-layer order (models/qwen25.json:529-566)."""
    hq, hkv, d, cached, cap, expanded = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, capacity=cap, rope_mode=rope_mode,
                      expanded=expanded, poison=True)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_decode(case, q_rot, kc, vc)
    got = gpu_decode(mfk, foundry, case, q_rot, kc, vc)
    assert max_abs(got, ref) <= TOL
    assert max_abs(got, gold.ravel()) <= TOL


@pytest.mark.parametrize("n_splits", [1, 2, 3, 7, 32])
def test_split_kv_equals_unsplit(mfk, foundry, n_splits):
    case = ContigCase(n_heads=24, n_kv_heads=8, head_dim=128, cached=1500, capacity=1536)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_decode(case, q_rot, kc, vc)
    got = gpu_decode(mfk, foundry, case, q_rot, kc, vc, n_splits=n_splits)
    assert max_abs(got, ref) <= TOL
    assert max_abs(got, gold.ravel()) <= TOL


def test_lcg_fixture_shapes(mfk, foundry):
    """Inputs from the reference's deterministic LCG (tests/flashattention_decode_parity.rs:15-30),
    scale 0.25, expanded cache."""
    for (hq, d, L, seed) in [(14, 64, 128, 1), (8, 128, 128, 7), (14, 64, 27, 42)]:
        case = ContigCase(n_heads=hq, n_kv_heads=hq, head_dim=d, cached=L - 1, capacity=max(L, 64), expanded=True,
                          gen="lcg", seed=seed, scale=0.25)
        q_rot, kc, vc = case.oracle_append()
        ref, gold = oracle_decode(case, q_rot, kc, vc)
        got = gpu_decode(mfk, foundry, case, q_rot, kc, vc)
        assert max_abs(got, ref) <= TOL and max_abs(got, gold.ravel()) <= TOL


def test_long_context_over_65536_keys(mfk, foundry):
    """The Metal kernels give up above 65536 keys (flash_decode.metal:168); this path does not."""
    case = ContigCase(n_heads=6, n_kv_heads=2, head_dim=128, cached=70000, capacity=70016)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_decode(case, q_rot, kc, vc)
    got = gpu_decode(mfk, foundry, case, q_rot, kc, vc)
    assert max_abs(got, ref) <= TOL and max_abs(got, gold.ravel()) <= TOL


@pytest.mark.parametrize("bh_l_d", [(1, 1, 128, 64), (2, 4, 32, 128)])
@pytest.mark.parametrize("identity", [True, False])
def test_rope_flash_decode_vs_cpu_sdpa_attention(mfk, foundry, bh_l_d, identity):
    """tests/sdpa_v2_parity.rs:135-239: fused RoPE->decode against the Rust CPU oracle restated
    in C (identity RoPE there; real tables as well here)."""
    import torch

    b, h, L, d = bh_l_d
    bh = b * h
    q = lcg(11, bh * d, 1.0)
    k = lcg(19, bh * L * d, 1.0)
    v = lcg(29, bh * L * d, 1.0)
    if identity:
        cos = np.full((L, d // 2), 0x3C00, np.uint16)
        sin = np.zeros((L, d // 2), np.uint16)
    else:
        cos, sin = oracle.rope_tables(1e4, d, L)
    ref = np.empty(bh * d, np.uint16)
    oracle.lib().mfo_cpu_sdpa_attention(q, k, v, cos, sin, bh, L, d, ref)
    # The CPU oracle ropes K itself; the kernel expects roped keys in the cache.
    k_roped = np.empty_like(k)
    oracle.lib().mfo_rope_neox(k, k_roped, cos, sin, d, L, 0, k.size)
    out = torch.full((bh * d,), float("nan"), dtype=torch.float16, device="cuda")
    # tensors are [B*H, L, D]: every (batch, head) has its own K/V ("expanded"), batch = B*H of 1 head
    strides = mfk.MfFlashDecodeStrides(d, d, L * d, L * d, L * d, L * d, d, d)
    foundry.rope_flash_decode(dev(q), dev(k_roped), dev(v), dev(cos), dev(sin), out,
                              mfk.RopeParamsResolved(d, L, L - 1, bh * d),
                              mfk.SdpaParams(L, d, 1.0 / np.sqrt(d), d, d), strides, 1, bh)
    foundry.synchronize()
    assert max_abs(host(out), ref) <= TOL


def test_flash_attention_dispatcher(mfk, foundry):
    """Routing and preconditions of FlashAttentionStep (src/metals/sdpa/step.rs:193-197, 271, 442-456)."""
    import torch

    case = ContigCase(n_heads=14, n_kv_heads=2, head_dim=64, cached=99, capacity=128)
    q_rot, kc, vc = case.oracle_append()
    ref, _ = oracle_decode(case, q_rot, kc, vc)
    q, k, v = dev(q_rot).view(1, 14 * 64), dev(kc), dev(vc)
    out = torch.zeros((1, 14 * 64), dtype=torch.float16, device="cuda")
    route = foundry.flash_attention(q, k, v, out, causal=True, query_offset=99, n_heads=14, head_dim=64,
                                    kv_seq_len=100, m=1)
    foundry.synchronize()
    assert route == mfk.ROUTE_DECODE
    assert max_abs(host(out).ravel(), ref) <= TOL
    # m = 0 is treated as 1
    assert foundry.flash_attention(q, k, v, out, causal=True, query_offset=99, n_heads=14, head_dim=64,
                                   kv_seq_len=100, m=0) == mfk.ROUTE_DECODE
    with pytest.raises(mfk.MetalError) as e:
        foundry.flash_attention(q, k, v, out, causal=True, query_offset=99, n_heads=14, head_dim=64, kv_seq_len=100,
                                kv_head_major=False)
    assert e.value.kind == "OperationNotSupported"
    # causal decode with a masked tail: the reference falls back to SdpaReference (sdpa/step.rs:271-303);
    # only keys 0..50 are visible
    route = foundry.flash_attention(q, k, v, out, causal=True, query_offset=50, n_heads=14, head_dim=64, kv_seq_len=100)
    foundry.synchronize()
    assert route == mfk.ROUTE_REFERENCE
    masked = oracle.decode_online(q_rot, kc, vc, n_heads=14, cache_heads=2, head_dim=64, capacity=128, kv_len=51,
                                  scale=case.scale)
    assert max_abs(host(out).ravel(), masked) <= TOL
    with pytest.raises(mfk.MetalError) as e:  # head_dim 96
        foundry.flash_attention(dev(q_rot[:96 * 14]).view(1, -1), k, v, out[:, :96 * 14].contiguous(), causal=True,
                                query_offset=99, n_heads=14, head_dim=96, kv_seq_len=100)
    assert e.value.kind == "OperationNotSupported"
    with pytest.raises(mfk.MetalError) as e:  # kv_len beyond the capacity of the cache tensor
        foundry.flash_attention(q, k, v, out, causal=True, query_offset=199, n_heads=14, head_dim=64, kv_seq_len=200)
    assert e.value.kind == "InvalidOperation"
    foundry.synchronize()


def test_kv_len_zero_writes_nothing(mfk, foundry):
    import torch

    case = ContigCase(n_heads=4, n_kv_heads=2, head_dim=64, cached=3, capacity=64)
    out = torch.full((4 * 64,), 7.0, dtype=torch.float16, device="cuda")
    sp = mfk.SdpaParams(0, 64, 0.125, 64, 64)
    foundry.flash_decode(dev(case.q.ravel()), dev(case.k_cache), dev(case.v_cache), out, decode_strides(mfk, case),
                         sp, 4, 1, 0)
    foundry.synchronize()
    assert bool((out == 7.0).all())


def test_repeated_launches_are_stable(mfk, foundry):
    """The merge counters reset themselves: many launches in a row give the same bits."""
    import torch

    case = ContigCase(n_heads=24, n_kv_heads=8, head_dim=128, cached=4000, capacity=4096)
    q_rot, kc, vc = case.oracle_append()
    q, k, v = dev(q_rot), dev(kc), dev(vc)
    sp = mfk.SdpaParams(case.L, case.D, float(case.scale), case.D, case.D)
    outs = []
    for _ in range(5):
        out = torch.zeros(case.Hq * case.D, dtype=torch.float16, device="cuda")
        foundry.flash_decode(q, k, v, out, decode_strides(mfk, case), sp, case.Hq, 1, 0)
        outs.append(out)
    foundry.synchronize()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    ref, _ = oracle_decode(case, q_rot, kc, vc)
    assert max_abs(host(outs[0]), ref) <= TOL


# shapes for which a short launch takes the cluster form: several CTAs per (sequence, kv head) unit, few tiles each
CLUSTER_SHAPES = [
    (24, 8, 128, 8191, 8192),   # configuration 2: 8 units x 16 CTAs, one cluster per unit
    (16, 2, 128, 8191, 8192),   # 2 units: several clusters per unit, their partials merged through memory
    (14, 2, 64, 511, 512),      # configuration 1: clusters of 8 with one tile each
    (32, 2, 128, 3000, 3072),   # G = 16 (two 8-head tiles)
    (24, 8, 128, 1100, 2048),   # uneven shares: 18 tiles over a cluster
    (8, 1, 128, 4097, 5000),    # a single unit
]


@pytest.mark.parametrize("shape", CLUSTER_SHAPES)
@pytest.mark.parametrize("clusters_off", [0, 1])
@pytest.mark.parametrize("overlap", [0, 1])
def test_decode_cluster_form_and_plain_form(mfk, foundry, shape, clusters_off, overlap):
    """The CTAs of a unit combined through distributed shared memory (cluster form) or through partials in
    global memory and a ticket (plain form): both within tolerance of the oracle and the fp64 gold, with the
    fused append (caches bit-exact) and without."""
    import torch

    hq, hkv, d, cached, cap = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, capacity=cap, poison=True)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_decode(case, q_rot, kc, vc)
    foundry.set_option(mfk.OPTION_DECODE_CLUSTERS, clusters_off)
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)
    try:
        got = gpu_decode(mfk, foundry, case, q_rot, kc, vc)
        # one launch: q rotated, the new row appended and attended over
        kc1, vc1 = dev(case.k_cache), dev(case.v_cache)
        out1 = torch.full((1, hq * d), float("nan"), dtype=torch.float16, device="cuda")
        q_rot1 = torch.full((1, hq * d), float("nan"), dtype=torch.float16, device="cuda")
        p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, 1, cached, cap, hq * d, 0, 0, 0)
        for _ in range(2):  # twice: the second launch follows a launch that wrote the same cache
            foundry.kv_prep_flash_decode(dev(case.q), dev(case.k), dev(case.v), q_rot1, kc1, vc1, dev(case.cos), dev(case.sin),
                                         out1, p)
        foundry.synchronize()
    finally:
        foundry.set_option(mfk.OPTION_DECODE_CLUSTERS, 0)
        foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    assert max_abs(got, ref) <= TOL and max_abs(got, gold.ravel()) <= TOL
    assert np.array_equal(host(kc1), kc) and np.array_equal(host(vc1), vc)
    assert np.array_equal(host(q_rot1).ravel(), q_rot)
    assert max_abs(host(out1).ravel(), ref) <= TOL and max_abs(host(out1).ravel(), gold.ravel()) <= TOL
    assert np.array_equal(host(out1).ravel(), got)  # same kernel, same cut: the fused form gives the same bits
