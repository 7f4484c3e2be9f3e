"""GPU parity: KvPrepFused and the decode route of FlashAttention in ONE launch on a contiguous cache
(mf_kv_prep_flash_decode), against the oracle and against the reference's two-step order on the GPU:
q_rot and the whole caches bit for bit, the attention output bit for bit with the two launches and
within 2e-3 of the oracle.
"""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, dev, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3

# (position_offset, max_seq_len, n_heads, n_kv_heads, head_dim)
SHAPES = [(5, 16, 14, 2, 64), (511, 512, 14, 2, 64), (777, 1024, 16, 2, 128), (8191, 8192, 24, 8, 128), (0, 8, 8, 8, 128),
          (64, 200, 32, 8, 128)]


def _params(mfk, case, layer_idx=0, step=0):
    return mfk.KvPrepFusedParamsResolved(case.Hq * case.D, case.Hkv * case.D, case.D, case.Hq, case.Hkv, case.G, 1,
                                         case.cached, case.cap, case.Hq * case.D, case.rope_mode, layer_idx, step)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("rope_mode", [0, 1])
@pytest.mark.parametrize("overlap", [0, 1])
def test_append_and_decode_in_one_launch(mfk, foundry, shape, rope_mode, overlap):
    import torch

    off, cap, hq, hkv, d = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=off, m=1, capacity=cap, theta=1e4,
                      rope_mode=rope_mode, poison=True)
    q_ref, k_ref, v_ref = case.oracle_append()
    want = oracle.decode_online(q_ref, k_ref, v_ref, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap,
                                kv_len=off + 1, scale=case.scale)
    q, k, v, cos, sin = dev(case.q), dev(case.k), dev(case.v), dev(case.cos), dev(case.sin)
    p = _params(mfk, case)
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)
    # two launches, the reference's order
    kc2, vc2 = dev(case.k_cache), dev(case.v_cache)
    q_rot2 = torch.full((1, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    out2 = torch.full((1, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.kv_prep_fused(q, k, v, q_rot2, kc2, vc2, cos, sin, p)
    foundry.flash_attention(q_rot2, kc2, vc2, out2, causal=True, query_offset=off, n_heads=hq, head_dim=d,
                            kv_seq_len=off + 1, m=1)
    # one launch, with and without the copy of the rotated q
    res = []
    for with_q_rot in (True, False):
        kc1, vc1 = dev(case.k_cache), dev(case.v_cache)
        q_rot1 = torch.full((1, hq * d), float("nan"), dtype=torch.float16, device="cuda") if with_q_rot else None
        out1 = torch.full((1, hq * d), float("nan"), dtype=torch.float16, device="cuda")
        foundry.kv_prep_flash_decode(q, k, v, q_rot1, kc1, vc1, cos, sin, out1, p)
        foundry.synchronize()
        res.append((q_rot1, kc1, vc1, out1))
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    for q_rot1, kc1, vc1, out1 in res:
        assert np.array_equal(host(kc1), k_ref) and np.array_equal(host(vc1), v_ref)
        assert np.array_equal(host(kc1), host(kc2)) and np.array_equal(host(vc1), host(vc2))
        assert np.array_equal(host(out1), host(out2))
        assert max_abs(host(out1).ravel(), want) <= TOL
    assert np.array_equal(host(res[0][0]).ravel(), q_ref)


def test_one_launch_respects_the_no_rope_layers(mfk, foundry):
    import torch

    case = ContigCase(n_heads=8, n_kv_heads=2, head_dim=64, cached=9, m=1, capacity=16, rope_mode=1)
    q, k, v, cos, sin = dev(case.q), dev(case.k), dev(case.v), dev(case.cos), dev(case.sin)
    for layer in range(4):
        q_ref, k_ref, v_ref = case.oracle_append(layer_idx=layer, no_rope_layer_step=4)
        kc, vc = dev(case.k_cache), dev(case.v_cache)
        q_rot = torch.zeros((1, 8 * 64), dtype=torch.float16, device="cuda")
        out = torch.zeros((1, 8 * 64), dtype=torch.float16, device="cuda")
        foundry.kv_prep_flash_decode(q, k, v, q_rot, kc, vc, cos, sin, out, _params(mfk, case, layer, 4))
        foundry.synchronize()
        assert np.array_equal(host(q_rot).ravel(), q_ref)
        assert np.array_equal(host(kc), k_ref) and np.array_equal(host(vc), v_ref)
    assert np.array_equal(q_ref, case.q.ravel())  # layer 3 skipped the rotation


def test_one_launch_refuses_what_the_two_calls_are_for(mfk, foundry):
    import torch

    case = ContigCase(n_heads=8, n_kv_heads=2, head_dim=64, cached=3, m=1, capacity=16, expanded=True)
    q, k, v, cos, sin = dev(case.q), dev(case.k), dev(case.v), dev(case.cos), dev(case.sin)
    kc, vc = dev(case.k_cache), dev(case.v_cache)
    out = torch.zeros((1, 8 * 64), dtype=torch.float16, device="cuda")
    with pytest.raises(mfk.MetalError) as e:  # expanded cache: G rows per new key
        foundry.kv_prep_flash_decode(q, k, v, None, kc, vc, cos, sin, out, _params(mfk, case))
    assert e.value.kind == "OperationNotSupported"
    compact = ContigCase(n_heads=8, n_kv_heads=2, head_dim=64, cached=3, m=2, capacity=16)
    p = mfk.KvPrepFusedParamsResolved(8 * 64, 2 * 64, 64, 8, 2, 4, 2, 3, 16, 8 * 2 * 64, 0, 0, 0)
    with pytest.raises(mfk.MetalError) as e:  # two new tokens are a prefill chunk
        foundry.kv_prep_flash_decode(dev(compact.q), dev(compact.k), dev(compact.v), None, dev(compact.k_cache),
                                     dev(compact.v_cache), cos, sin, out, p)
    assert e.value.kind == "OperationNotSupported"
    foundry.synchronize()


@pytest.mark.parametrize("overlap", [0, 1])
def test_steps_in_a_row_on_one_cache(mfk, foundry, overlap):
    """A one-layer model: every launch appends to the cache the next one reads, positions advancing.
    With overlapped launches the library must not let a launch stream the cache ahead of the row the
    launch before it is still writing."""
    import torch

    hq, hkv, d, cap, start, steps = 16, 2, 128, 512, 300, 48
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=start, m=steps, capacity=cap, theta=1e4, rope_mode=0)
    cos, sin = dev(case.cos), dev(case.sin)
    kc, vc = dev(case.k_cache), dev(case.v_cache)
    q_all, k_all, v_all = dev(case.q), dev(case.k), dev(case.v)  # [steps, ...]: row t is step t's token
    outs = torch.full((steps, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)
    for t in range(steps):
        p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, 1, start + t, cap, hq * d, 0, 0, 0)
        foundry.kv_prep_flash_decode(q_all[t:t + 1], k_all[t:t + 1], v_all[t:t + 1], None, kc, vc, cos, sin, outs[t:t + 1], p)
    foundry.synchronize()
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    # the oracle: all rows appended at once, then each step attends over its prefix
    q_ref, k_ref, v_ref = case.oracle_append()
    assert np.array_equal(host(kc), k_ref) and np.array_equal(host(vc), v_ref)
    q_rows = q_ref.reshape(hq, steps, d)
    got = host(outs)
    for t in range(steps):
        q_t = np.ascontiguousarray(q_rows[:, t]).ravel()
        want = oracle.decode_online(q_t, k_ref, v_ref, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap,
                                    kv_len=start + t + 1, scale=case.scale)
        assert max_abs(got[t], want) <= TOL, t
