"""The reference's own assertions for this path, replayed with the CUDA kernels on the flash side.

Same fixtures and bounds as test_reference_assertions.py (the LCG seeds, draw order and shapes of
tests/flashattention_decode_parity.rs and tests/flashattention_prefill_parity.rs of the reference;
6e-2 for decode, 8e-2 for prefill, against the materialised path with f16 S and P), through the
operator entry points the reference's tests call: FlashAttention / run_flash_decode for the flash
side.  On top of the reference's bound every case is also held to this repository's own bar
(2e-3 against the fp64 gold), and mf_sdpa_reference is compared with the reference's CPU functions
on the two shapes the reference checks its materialised path on.
"""
import numpy as np
import pytest

import oracle
import refcases
from kvcases import dev, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.mark.parametrize("case", refcases.decode_cases(), ids=lambda c: c.name)
def test_flash_decode_vs_materialized(mfk, foundry, case):
    import torch

    mat = refcases.materialized(case)
    q, k, v = dev(case.q), dev(case.k), dev(case.v)
    out = torch.full((1, case.n_heads * case.head_dim), float("nan"), dtype=torch.float16, device="cuda")
    route = foundry.flash_attention(q, k, v, out, causal=True, query_offset=case.kv_len - 1, n_heads=case.n_heads,
                                    head_dim=case.head_dim, kv_seq_len=case.kv_len, m=1)
    foundry.synchronize()
    assert route == mfk.ROUTE_DECODE
    assert max_abs(host(out), mat) < refcases.DECODE_TOL
    gold = oracle.decode_gold(case.q.ravel(), case.k, case.v, n_heads=case.n_heads, cache_heads=case.n_heads,
                              head_dim=case.head_dim, capacity=case.capacity, kv_len=case.kv_len, scale=case.scale)
    assert max_abs(host(out), gold.ravel()) <= TOL


@pytest.mark.parametrize("case", refcases.prefill_cases(), ids=lambda c: c.name)
def test_flash_prefill_vs_materialized(mfk, foundry, case):
    import torch

    h, d, m = case.n_heads, case.head_dim, case.m
    mat = refcases.materialized(case)
    k, v = dev(case.k), dev(case.v)
    rows = case.m_cap or m
    out = torch.zeros((rows, h * d), dtype=torch.float16, device="cuda")
    if case.split_k > 1:
        # the reference forces split-K through an environment variable; here the explicit-parameter entry point
        base = mfk.SdpaPrefillParams(case.kv_len, d, float(case.scale), d, d, case.query_offset,
                                     0, d,                                   # q token-major: head stride D
                                     0, case.capacity * d, 0, case.capacity * d,
                                     0, d, h * d, h * d,                      # q_stride_m, out_stride_m
                                     1, m)
        foundry.flash_prefill(dev(case.q), k, v, out, mfk.SdpaPrefillSplitKParams(base, h, case.split_k))
    elif case.m_cap:
        # [1, M_cap, d_model] metadata over head-major packed contents (flashattention_prefill_parity.rs:413-505)
        q_buf = torch.zeros((1, case.m_cap, h * d), dtype=torch.float16, device="cuda")
        q_buf.view(-1)[: h * m * d] = dev(case.q).view(-1)
        foundry.run_flash_decode(q_buf, k, v, out, h, d, case.kv_len, m)
    elif m == 1:
        # one query row: the reference's run_flash_decode takes its decode branch
        foundry.run_flash_decode(dev(case.q), k, v, out, h, d, case.kv_len, 1)
    else:
        route = foundry.flash_attention(dev(case.q), k, v, out, causal=True, query_offset=case.query_offset, n_heads=h,
                                        head_dim=d, kv_seq_len=case.kv_len, m=m)
        assert route in (mfk.ROUTE_PREFILL, mfk.ROUTE_PREFILL_SPLITK)
    foundry.synchronize()
    got = host(out)[:m]
    assert max_abs(got, mat) < refcases.PREFILL_TOL
    gold = oracle.prefill_gold(refcases.q_head_major(case), case.k, case.v, n_heads=h, cache_heads=h, head_dim=d,
                               capacity=case.capacity, q_len=m, kv_len=case.kv_len, query_offset=case.query_offset,
                               scale=case.scale)
    assert max_abs(got, gold) <= TOL
    if case.m_cap:
        assert not host(out)[m:].any()  # rows past the true M stay untouched


@pytest.mark.parametrize("which", ["misaligned", "m4"])
def test_sdpa_reference_vs_the_cpu_functions_of_the_reference_tests(mfk, foundry, which):
    """tests/sdpa_head_stride_misaligned.rs (bound 0.05) and tests/sdpa_materialized_prefill_parity.rs
    (bound 0.15): head-major Q [H, m, D] in, token-major [m, H*D] out, non-causal."""
    import torch

    c = refcases.misaligned_case() if which == "misaligned" else refcases.materialized_m4_case()
    bound = 0.05 if which == "misaligned" else 0.15
    h, d, m, L = c["n_heads"], c["head_dim"], c["m"], c["seq_k"]
    out = torch.full((m, h * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.sdpa_reference(dev(c["q"]), dev(c["k"]), dev(c["v"]), out, causal=False, query_offset=0, n_heads=h, head_dim=d,
                           kv_seq_len=L, m=m)
    foundry.synchronize()
    got = oracle.h2f(host(out)).astype(np.float32)
    assert np.max(np.abs(got - c["expected"])) < bound
    # and the restated materialised path agrees with the kernel far inside that bound
    mat = oracle.sdpa_materialized(c["q"], c["k"], c["v"], n_heads=h, head_dim=d, m=m, kv_len=L, causal=False,
                                   query_offset=0, scale=c["scale"], q_head_major=True)
    assert max_abs(host(out), mat) < 5e-3
