"""GPU parity: causal chunked prefill (append M rows, then attend) through the C ABI.

Shapes follow tests/flashattention_prefill_parity.rs:143-538 of the reference (M in
{2,7,16,17,26,31,32,33}, with and without a 64-token prefix, forced split-K at kv 256 / 1024,
D 64 and 128) plus GQA with a compact cache, which the reference never pins at kernel level.
Tolerance: max-abs 2e-3 against the oracle's tiled f32 softmax and the fp64 gold (the
reference's own bar against its materialised GPU path is 8e-2).
"""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, dev, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3


def oracle_prefill(case, q_rot, kc, vc):
    args = dict(n_heads=case.Hq, cache_heads=case.cache_heads, head_dim=case.D, capacity=case.cap, q_len=case.M,
                kv_len=case.L, query_offset=case.cached, scale=case.scale)
    return oracle.prefill_causal(q_rot, kc, vc, **args), oracle.prefill_gold(q_rot, kc, vc, **args)


def gpu_prefill(mfk, foundry, case, q_rot, kc, vc, split_k=1):
    import torch

    hq, d, m, cap = case.Hq, case.D, case.M, case.cap
    out = torch.full((m, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    base = mfk.SdpaPrefillParams(case.L, d, float(case.scale), d, d, case.cached,
                                 hq * m * d, m * d,      # q_stride_b, q_stride_h  (head-major packed over M)
                                 0, cap * d, 0, cap * d,  # k/v stride_b, stride_h
                                 0, d,                    # out_stride_b, out_stride_h
                                 d, hq * d,               # q_stride_m, out_stride_m
                                 hq // case.cache_heads, m)
    foundry.flash_prefill(dev(q_rot), dev(kc), dev(vc), out, mfk.SdpaPrefillSplitKParams(base, hq, split_k))
    foundry.synchronize()
    return host(out)


M_VALUES = [2, 7, 16, 17, 26, 31, 32, 33]


@pytest.mark.parametrize("m", M_VALUES)
@pytest.mark.parametrize("prefix", [0, 64])
@pytest.mark.parametrize("hd", [(14, 14, 64), (8, 8, 128), (14, 2, 64), (24, 8, 128)])
def test_prefill_various_m(mfk, foundry, m, prefix, hd):
    hq, hkv, d = hd
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=prefix, m=m, capacity=128, poison=True)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_prefill(case, q_rot, kc, vc)
    got = gpu_prefill(mfk, foundry, case, q_rot, kc, vc)
    assert max_abs(got, ref) <= TOL
    assert max_abs(got, gold) <= TOL


@pytest.mark.parametrize("shape", [(14, 64, 32, 256), (14, 64, 17, 256), (14, 64, 32, 1024), (8, 128, 32, 256),
                                   (8, 128, 17, 256), (8, 128, 32, 1024)])
@pytest.mark.parametrize("split_k", [1, 4, 8])
def test_prefill_split_k(mfk, foundry, shape, split_k):
    hq, d, m, kv = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hq, head_dim=d, cached=kv - m, m=m, capacity=kv)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_prefill(case, q_rot, kc, vc)
    got = gpu_prefill(mfk, foundry, case, q_rot, kc, vc, split_k=split_k)
    assert max_abs(got, ref) <= TOL
    assert max_abs(got, gold) <= TOL


def test_prefill_chunk_after_long_prefix_gqa(mfk, foundry):
    """A scaled-down configuration 4: 256 new tokens after 768 cached, 24 q / 8 kv heads, D 128."""
    case = ContigCase(n_heads=24, n_kv_heads=8, head_dim=128, cached=768, m=256, capacity=1024, theta=5e5,
                      rope_mode=1)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_prefill(case, q_rot, kc, vc)
    got = gpu_prefill(mfk, foundry, case, q_rot, kc, vc)
    assert max_abs(got, ref) <= TOL
    assert max_abs(got, gold) <= TOL


def test_prefill_through_kv_prep_and_dispatcher(mfk, foundry):
    """KvPrepFused -> FlashAttention with m > 1, the reference's chunked-prefill order, with the
    q tensor described by token-major metadata [1, M_cap, d_model] while holding head-major
    contents (tests/flashattention_prefill_parity.rs:413-505)."""
    import torch

    hq, hkv, d, m, cached, cap, m_cap = 14, 2, 64, 26, 64, 128, 32
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=cap)
    q_ref, kc_ref, vc_ref = case.oracle_append()
    ref, gold = oracle_prefill(case, q_ref, kc_ref, vc_ref)
    q, k, v = dev(case.q), dev(case.k), dev(case.v)
    kc, vc, cos, sin = dev(case.k_cache), dev(case.v_cache), dev(case.cos), dev(case.sin)
    q_rot = torch.zeros((1, m_cap, hq * d), dtype=torch.float16, device="cuda")
    p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, m, cached, cap, hq * m * d, 0, 0, 0)
    foundry.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, p)
    out = torch.zeros((1, m_cap, hq * d), dtype=torch.float16, device="cuda")
    route = foundry.flash_attention(q_rot, kc, vc, out, causal=True, query_offset=cached, n_heads=hq, head_dim=d,
                                    kv_seq_len=cached + m, m=m)
    foundry.synchronize()
    assert route == mfk.ROUTE_PREFILL
    got = host(out)[0, :m]
    assert max_abs(got, ref) <= TOL and max_abs(got, gold) <= TOL
    assert not host(out)[0, m:].any()  # rows past q_len are not written
    # causal invariant broken, or non-causal: the reference falls back to SdpaReference (sdpa/step.rs:442-470)
    for causal, offset in ((True, cached + 1), (True, cached - 3), (False, cached)):
        out.zero_()
        route = foundry.flash_attention(q_rot, kc, vc, out, causal=causal, query_offset=offset, n_heads=hq, head_dim=d,
                                        kv_seq_len=cached + m, m=m)
        foundry.synchronize()
        assert route == mfk.ROUTE_REFERENCE
        args = dict(n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap, q_len=m, kv_len=cached + m,
                    query_offset=offset if causal else cached + m, scale=case.scale)
        want = oracle.prefill_causal(q_ref, kc_ref, vc_ref, **args)
        gold_g = oracle.prefill_gold(q_ref, kc_ref, vc_ref, **args)
        got = host(out)[0, :m]
        assert max_abs(got, want) <= TOL and max_abs(got, gold_g) <= TOL


def test_prefill_split_k_heuristic_route(mfk, foundry):
    """kv >= 2048 and m >= 16 selects split-K 4 (src/metals/flashattention/step.rs:849-866)."""
    import torch

    hq, hkv, d, m, cached = 8, 2, 128, 64, 2048 - 64
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=2048)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_prefill(case, q_rot, kc, vc)
    q3 = dev(q_rot).view(hq, m, d)
    out = torch.zeros((m, hq * d), dtype=torch.float16, device="cuda")
    route = foundry.flash_attention(q3, dev(kc), dev(vc), out, causal=True, query_offset=cached, n_heads=hq,
                                    head_dim=d, kv_seq_len=2048, m=m)
    foundry.synchronize()
    assert route == mfk.ROUTE_PREFILL_SPLITK
    assert max_abs(host(out), ref) <= TOL and max_abs(host(out), gold) <= TOL


# (n_heads, n_kv_heads, cached, m, capacity[, head_dim = 128])
TC_SHAPES = [(8, 8, 0, 128, 128), (8, 8, 0, 64, 64), (24, 8, 768, 256, 1024), (6, 2, 100, 200, 333),
             (4, 4, 1, 130, 131), (16, 2, 500, 64, 600), (3, 1, 0, 385, 400),
             (14, 2, 64, 130, 256, 64), (14, 14, 0, 64, 64, 64), (8, 2, 500, 200, 768, 64), (2, 1, 3, 513, 520, 64)]


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_prefill_tcgen05_kernel(mfk, foundry, shape):
    """The tcgen05 / TMEM kernel alone (MF_OPTION_PREFILL_IMPL = 2), head_dim 128 and 64: whole and
    ragged tiles, prefixes that are not multiples of the tile, GQA, poisoned rows past kv_len."""
    hq, hkv, cached, m, cap = shape[:5]
    d = shape[5] if len(shape) > 5 else 128
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=cap, poison=True)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_prefill(case, q_rot, kc, vc)
    foundry.set_option(3, 2)
    try:
        got = gpu_prefill(mfk, foundry, case, q_rot, kc, vc)
    finally:
        foundry.set_option(3, 0)
    assert max_abs(got, ref) <= TOL
    assert max_abs(got, gold) <= TOL


def test_prefill_kernels_agree(mfk, foundry):
    """mma.sync and tcgen05 kernels on the same inputs (token-major q this time)."""
    import torch

    hq, hkv, d, m, cached, cap = 12, 4, 128, 192, 320, 512
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=cap)
    q_rot, kc, vc = case.oracle_append()
    ref, gold = oracle_prefill(case, q_rot, kc, vc)
    q_tok = dev(np.ascontiguousarray(q_rot.reshape(hq, m, d).transpose(1, 0, 2)))  # [M, Hq, D]
    k, v = dev(kc), dev(vc)
    outs = []
    for impl in (1, 2):
        foundry.set_option(3, impl)
        out = torch.zeros((m, hq * d), dtype=torch.float16, device="cuda")
        foundry.run_flash_decode(q_tok, k, v, out, hq, d, cached + m, q_seq_len=m)
        foundry.synchronize()
        outs.append(host(out))
    foundry.set_option(3, 0)
    for o in outs:
        assert max_abs(o, ref) <= TOL and max_abs(o, gold) <= TOL
