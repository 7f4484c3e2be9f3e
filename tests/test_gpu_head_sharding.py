"""GPU parity: a batch-1 decode step and a prefill chunk with the KV heads split over ranks.

Each "rank" (run one after the other on one GPU) gets the caches of its KV heads and the matching
columns of q / k / v, runs the reference's two ops on them, and the outputs put side by side must be
the unsplit oracle result: caches bit-exact, attention within 2e-3.  No data crosses ranks.
"""
import importlib

import numpy as np
import pytest

import oracle
from kvcases import ContigCase, dev, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m", [1, 96])
def test_kv_heads_over_ranks(mfk, foundry, world, m):
    import torch

    sharding = importlib.import_module("test-burn_b200.sharding")
    hq, hkv, d, cached, cap = 24, 8, 128, 300, 512
    g = hq // hkv
    full = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=cap, theta=5e5, rope_mode=1)
    q_ref, k_ref, v_ref = full.oracle_append()
    if m == 1:
        want = oracle.decode_online(q_ref, k_ref, v_ref, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap,
                                    kv_len=cached + 1, scale=full.scale).reshape(1, hq, d)
    else:
        want = oracle.prefill_causal(q_ref, k_ref.ravel(), v_ref.ravel(), n_heads=hq, cache_heads=hkv, head_dim=d,
                                     capacity=cap, q_len=m, kv_len=cached + m, query_offset=cached,
                                     scale=full.scale).reshape(m, hq, d)
    cos, sin = dev(full.cos), dev(full.sin)
    outs, covered = [], 0
    for rank in range(world):
        h0, h1 = sharding.shard_kv_heads(hkv, world, rank)
        assert h0 == covered
        covered = h1
        n_kv, n_q = h1 - h0, (h1 - h0) * g
        q = dev(np.ascontiguousarray(full.q.reshape(m, hq, d)[:, h0 * g:h1 * g]).reshape(m, n_q * d))
        k = dev(np.ascontiguousarray(full.k.reshape(m, hkv, d)[:, h0:h1]).reshape(m, n_kv * d))
        v = dev(np.ascontiguousarray(full.v.reshape(m, hkv, d)[:, h0:h1]).reshape(m, n_kv * d))
        kc, vc = dev(full.k_cache[h0:h1]), dev(full.v_cache[h0:h1])
        q_rot = torch.full((n_q, m, d), float("nan"), dtype=torch.float16, device="cuda")
        p = mfk.KvPrepFusedParamsResolved(n_q * d, n_kv * d, d, n_q, n_kv, g, m, cached, cap, n_q * m * d, 1, 0, 0)
        foundry.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, p)
        out = torch.full((m, n_q * d), float("nan"), dtype=torch.float16, device="cuda")
        # the decode route wants q as rows of d_model; [Hq, 1, D] packed is the same memory
        foundry.flash_attention(q_rot.view(1, n_q * d) if m == 1 else q_rot, kc, vc, out, causal=True, query_offset=cached, n_heads=n_q, head_dim=d,
                                kv_seq_len=cached + m, m=m)
        foundry.synchronize()
        assert np.array_equal(host(kc), k_ref.reshape(hkv, cap, d)[h0:h1])
        assert np.array_equal(host(vc), v_ref.reshape(hkv, cap, d)[h0:h1])
        assert np.array_equal(host(q_rot), q_ref.reshape(hq, m, d)[h0 * g:h1 * g])
        outs.append(host(out).reshape(m, n_q, d))
    assert covered == hkv
    got = np.concatenate(outs, axis=1)
    assert max_abs(np.ascontiguousarray(got), np.ascontiguousarray(want)) <= TOL
