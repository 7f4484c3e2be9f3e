"""The reference's own assertions for this path, replayed on its own fixtures (CPU part).

The reference project stores no expected outputs: its attention tests assert that its flash
kernels stay within a bound of its materialised path (S and P rounded to f16) on inputs drawn
from a fixed LCG, and two tests compare the materialised path with a CPU function written in
the test.  Here the materialised path is restated with its rounding points
(oracle.sdpa_materialized), the fixtures are regenerated from the same seeds, and the same
bounds are asserted with the oracle's flash restatements on the flash side.  The GPU part
(test_gpu_reference_assertions.py) puts the CUDA kernels on the flash side.
"""
import numpy as np
import pytest

import oracle
import refcases
from kvcases import max_abs


@pytest.mark.parametrize("case", refcases.decode_cases(), ids=lambda c: c.name)
def test_flash_decode_vs_materialized(case):
    """tests/flashattention_decode_parity.rs:117-346: |flash - materialised| < 6e-2."""
    mat = refcases.materialized(case)
    q = case.q.ravel()
    flash = oracle.decode_online(q, case.k, case.v, n_heads=case.n_heads, cache_heads=case.n_heads, head_dim=case.head_dim,
                                 capacity=case.capacity, kv_len=case.kv_len, scale=case.scale)
    assert max_abs(flash, mat.ravel()) < refcases.DECODE_TOL
    # the kernel's block order for every (warps x keys_per_warp) of the reference's variant table (:32-114)
    for block in (16 * 32, 8 * 32, 8 * 16, 16 * 16, 8 * 8, 16 * 8):
        blocked = oracle.decode_blocked(q, case.k, case.v, n_heads=case.n_heads, cache_heads=case.n_heads,
                                        head_dim=case.head_dim, capacity=case.capacity, kv_len=case.kv_len, scale=case.scale,
                                        block_keys=block)
        assert max_abs(blocked, mat.ravel()) < refcases.DECODE_TOL
    # and the materialised path is itself close to the fp64 gold (its f16 S and P cost about 1e-3 here)
    gold = oracle.decode_gold(q, case.k, case.v, n_heads=case.n_heads, cache_heads=case.n_heads, head_dim=case.head_dim,
                              capacity=case.capacity, kv_len=case.kv_len, scale=case.scale)
    assert max_abs(mat.ravel(), gold.ravel()) < 5e-3


@pytest.mark.parametrize("case", refcases.prefill_cases(), ids=lambda c: c.name)
def test_flash_prefill_vs_materialized(case):
    """tests/flashattention_prefill_parity.rs:143-538: |flash - materialised| < 8e-2, incl. forced split-K = 4."""
    mat = refcases.materialized(case)
    q = refcases.q_head_major(case)
    kw = dict(n_heads=case.n_heads, cache_heads=case.n_heads, head_dim=case.head_dim, capacity=case.capacity,
              q_len=case.m, kv_len=case.kv_len, query_offset=case.query_offset, scale=case.scale)
    if case.split_k == 1:
        flash = oracle.prefill_causal(q, case.k, case.v, **kw)
    else:
        accs, ms, ls = [], [], []
        L = oracle.lib()
        import ctypes as C

        for s in range(case.split_k):
            tb, te = C.c_uint32(), C.c_uint32()
            L.mfo_splitk_tile_range(case.kv_len, case.split_k, s, C.byref(tb), C.byref(te))
            _, acc, m_, l_ = oracle.prefill_causal(q, case.k, case.v, tile_begin=tb.value, tile_end=te.value, partials=True, **kw)
            accs.append(acc.reshape(-1, case.head_dim))
            ms.append(m_.ravel())
            ls.append(l_.ravel())
        merged = oracle.merge_partials(np.stack(accs), np.stack(ms), np.stack(ls))  # rows ordered [H, M]
        flash = merged.reshape(case.n_heads, case.m, case.head_dim).transpose(1, 0, 2).reshape(case.m, -1)
    assert max_abs(np.ascontiguousarray(flash), mat) < refcases.PREFILL_TOL
    gold = oracle.prefill_gold(q, case.k, case.v, **kw)
    assert max_abs(mat, gold) < 5e-3


def test_materialized_vs_the_cpu_function_of_the_misaligned_test():
    """tests/sdpa_head_stride_misaligned.rs: closed-form inputs, the test's own CPU function, bound 0.05."""
    c = refcases.misaligned_case()
    got = oracle.sdpa_materialized(c["q"], c["k"], c["v"], n_heads=c["n_heads"], head_dim=c["head_dim"], m=c["m"],
                                   kv_len=c["seq_k"], causal=False, query_offset=0, scale=c["scale"], q_head_major=True)
    assert np.max(np.abs(oracle.h2f(got).astype(np.float32) - c["expected"])) < 0.05


def test_materialized_vs_the_cpu_function_of_the_m4_test():
    """tests/sdpa_materialized_prefill_parity.rs: m=4, L=8, H=2, D=64, non-causal, bound 0.15."""
    c = refcases.materialized_m4_case()
    got = oracle.sdpa_materialized(c["q"], c["k"], c["v"], n_heads=c["n_heads"], head_dim=c["head_dim"], m=c["m"],
                                   kv_len=c["seq_k"], causal=False, query_offset=0, scale=c["scale"], q_head_major=True)
    assert np.max(np.abs(oracle.h2f(got).astype(np.float32) - c["expected"])) < 0.15


def test_materialized_mask_rule():
    """softmax_sdpa_batched.metal:25-37: causal hides key i from row r iff i > r + query_offset; a key
    made visible must change the output, a hidden one must not."""
    case = refcases.prefill_cases()[0]
    base = refcases.materialized(case)
    k2 = case.k.copy()
    k2[:, case.kv_len - 1] ^= 0x0400  # perturb the last key: only the last row sees it
    changed = oracle.sdpa_materialized(case.q, k2, case.v, n_heads=case.n_heads, head_dim=case.head_dim, m=case.m,
                                       kv_len=case.kv_len, causal=True, query_offset=case.query_offset, scale=case.scale,
                                       q_head_major=False)
    assert np.array_equal(changed[:-1], base[:-1]) and not np.array_equal(changed[-1], base[-1])
