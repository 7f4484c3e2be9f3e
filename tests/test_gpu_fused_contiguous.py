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


@pytest.mark.parametrize("n_caches", [4, 5, 8])
@pytest.mark.parametrize("overlap", [0, 1, 2])
def test_steps_in_a_row_on_rotating_caches(mfk, foundry, n_caches, overlap):
    """A model of 4, 5 or 8 layers, each with a cache of its own, short context (a handful of CTAs per
    launch, so that many launches would fit on the GPU at once): launch after launch appends to the
    cache that the launch `n_caches` later reads.  Under overlapped launches no launch may stream a
    cache ahead of a row that an earlier launch is still writing; the reference puts a barrier after
    every dispatch (src/types/mod.rs:577-595).  Every step of every layer is checked."""
    import torch

    hq, hkv, d, cap, start, steps = 14, 2, 64, 384, 300, 48
    cases = [ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=start, m=steps, capacity=cap, theta=1e6,
                        rope_mode=0, seed=0x5EED + 17 * layer) for layer in range(n_caches)]
    cos, sin = dev(cases[0].cos), dev(cases[0].sin)
    caches = [(dev(c.k_cache), dev(c.v_cache)) for c in cases]
    inputs = [(dev(c.q), dev(c.k), dev(c.v)) for c in cases]  # [steps, ...]: row t is step t's token
    outs = torch.full((n_caches, steps, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)
    for t in range(steps):
        p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, 1, start + t, cap, hq * d, 0, 0, 0)
        for layer in range(n_caches):
            q_all, k_all, v_all = inputs[layer]
            kc, vc = caches[layer]
            foundry.kv_prep_flash_decode(q_all[t:t + 1], k_all[t:t + 1], v_all[t:t + 1], None, kc, vc, cos, sin,
                                         outs[layer, t:t + 1], p)
    foundry.synchronize()
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    got = host(outs)
    for layer, case in enumerate(cases):
        q_ref, k_ref, v_ref = case.oracle_append()
        kc, vc = caches[layer]
        assert np.array_equal(host(kc), k_ref) and np.array_equal(host(vc), v_ref), layer
        q_rows = q_ref.reshape(hq, steps, d)
        for t in range(steps):
            q_t = np.ascontiguousarray(q_rows[:, t]).ravel()
            want = oracle.decode_online(q_t, k_ref, v_ref, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap,
                                        kv_len=start + t + 1, scale=case.scale)
            assert max_abs(got[layer, t], want) <= TOL, (layer, t)


def test_rotating_caches_replayed_from_a_cuda_graph(mfk):
    """The same rotation with the launches of one step captured into a CUDA graph and replayed: the
    early-stream decision is frozen at capture time, replays follow one another in stream order."""
    import torch

    hq, hkv, d, cap, start, steps, n_caches = 14, 2, 64, 384, 300, 24, 4
    cases = [ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=start, m=steps, capacity=cap, theta=1e6,
                        rope_mode=0, seed=0xABC + layer) for layer in range(n_caches)]
    stream = torch.cuda.Stream()
    f = mfk.Foundry(0, stream.cuda_stream)
    f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 1)
    cos, sin = dev(cases[0].cos), dev(cases[0].sin)
    caches = [(dev(c.k_cache), dev(c.v_cache)) for c in cases]
    inputs = [(dev(c.q), dev(c.k), dev(c.v)) for c in cases]
    # a graph replays fixed addresses: the step's rows are copied into these before each replay
    q_in = [torch.zeros((1, hq * d), dtype=torch.float16, device="cuda") for _ in range(n_caches)]
    k_in = [torch.zeros((1, hkv * d), dtype=torch.float16, device="cuda") for _ in range(n_caches)]
    v_in = [torch.zeros((1, hkv * d), dtype=torch.float16, device="cuda") for _ in range(n_caches)]
    out_s = [torch.zeros((1, hq * d), dtype=torch.float16, device="cuda") for _ in range(n_caches)]
    outs = torch.full((n_caches, steps, hq * d), float("nan"), dtype=torch.float16, device="cuda")

    def params(t):
        return mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, 1, start + t, cap, hq * d, 0, 0, 0)

    # one eager call on a scratch copy does what does not belong inside a capture (attributes, arena)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        f.kv_prep_flash_decode(q_in[0], k_in[0], v_in[0], None, dev(cases[0].k_cache), dev(cases[0].v_cache), cos, sin,
                               out_s[0], params(0))
    f.synchronize()
    for t in range(steps):
        with torch.cuda.stream(stream):
            for layer in range(n_caches):
                q_in[layer].copy_(inputs[layer][0][t:t + 1])
                k_in[layer].copy_(inputs[layer][1][t:t + 1])
                v_in[layer].copy_(inputs[layer][2][t:t + 1])
        stream.synchronize()
        g = torch.cuda.CUDAGraph()  # the position is a launch argument: one graph per step
        with torch.cuda.graph(g, stream=stream):
            for layer in range(n_caches):
                kc, vc = caches[layer]
                f.kv_prep_flash_decode(q_in[layer], k_in[layer], v_in[layer], None, kc, vc, cos, sin, out_s[layer], params(t))
        with torch.cuda.stream(stream):
            g.replay()
            for layer in range(n_caches):
                outs[layer, t:t + 1].copy_(out_s[layer])
        stream.synchronize()
    f.synchronize()
    got = host(outs)
    for layer, case in enumerate(cases):
        q_ref, k_ref, v_ref = case.oracle_append()
        kc, vc = caches[layer]
        assert np.array_equal(host(kc), k_ref) and np.array_equal(host(vc), v_ref), layer
        q_rows = q_ref.reshape(hq, steps, d)
        for t in range(steps):
            q_t = np.ascontiguousarray(q_rows[:, t]).ravel()
            want = oracle.decode_online(q_t, k_ref, v_ref, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap,
                                        kv_len=start + t + 1, scale=case.scale)
            assert max_abs(got[layer, t], want) <= TOL, (layer, t)
    f.close()
