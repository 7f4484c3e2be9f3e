"""mf_flash_decode_static_scratch: the decode entry point for callers that must not allocate.

Some hosts cannot call cudaMalloc at decode time: their own memory pool owns the whole GPU and
forbids plug-ins to allocate, or the loop cannot take the device-wide synchronisation an
allocation implies.  This entry point keeps the kernel's split-KV partials and tickets in an
array compiled into the library instead.  The test calls it through the C ABI twice in a row
(the array is shared and keeps the previous call's contents) and checks the result against the CPU
oracle and the fp64 gold, and against mf_flash_decode, the allocating entry point, on the same
inputs.  It must pass both alone in a fresh process and
after every other test, so it builds its own inputs and relies on no state left by others.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from kvcases import ContigCase, dev, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3  # the tolerance of the decode parity tests


def strides_of(mfk, case):
    hq, d, cap, ch = case.Hq, case.D, case.cap, case.cache_heads
    return mfk.MfFlashDecodeStrides(hq * d, d, ch * cap * d, cap * d, ch * cap * d, cap * d, hq * d, d)


@pytest.mark.parametrize("shape", [(24, 8, 128, 8191, 8192), (14, 2, 64, 511, 512), (32, 2, 128, 1000, 1024)])
def test_static_scratch_decode_matches_allocating_decode(mfk, foundry, shape):
    import torch

    hq, hkv, d, cached, cap = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, capacity=cap)
    q_rot, kc, vc = case.oracle_append()
    q, k, v = dev(q_rot), dev(kc), dev(vc)
    sp = mfk.SdpaParams(case.L, d, float(case.scale), d, d)
    st = strides_of(mfk, case)
    ref = torch.zeros(hq * d, dtype=torch.float16, device="cuda")
    # the allocating entry point in its plain form (every span writes a partial, the last one merges): that is
    # the form this entry point always takes
    foundry.set_option(mfk.OPTION_DECODE_CLUSTERS, 1)
    foundry.flash_decode(q, k, v, ref, st, sp, hq, 1, 0)
    foundry.synchronize()
    foundry.set_option(mfk.OPTION_DECODE_CLUSTERS, 0)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):  # two calls in a row share the built-in array
        out = torch.full((hq * d,), float("nan"), dtype=torch.float16, device="cuda")
        err = C.create_string_buffer(256)
        rc = mfk.lib.mf_flash_decode_static_scratch(stream if stream else None, q.data_ptr(), k.data_ptr(),
                                                    v.data_ptr(), out.data_ptr(), C.byref(st), C.byref(sp), hq, 1,
                                                    err, 256)
        assert rc == 0, err.value.decode()
        outs.append(out)
    status = C.c_uint32(0xFFFFFFFF)
    assert mfk.lib.mf_static_scratch_status(stream if stream else None, C.byref(status)) == 0
    torch.cuda.synchronize()
    assert status.value == 0  # no device-side wait ran out
    want = oracle.decode_online(q_rot, kc, vc, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap, kv_len=case.L,
                                scale=case.scale)
    gold = oracle.decode_gold(q_rot, kc, vc, n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap, kv_len=case.L,
                              scale=case.scale)
    for out in outs:
        assert max_abs(host(out), want) <= TOL
        assert max_abs(host(out), gold.ravel()) <= TOL
        # and the allocating entry point, in the same form, cuts the work the same way: the bits agree too
        assert torch.equal(out, ref)
    assert torch.equal(outs[0], outs[1])


def test_static_scratch_rejects_what_does_not_fit(mfk):
    """Beyond the built-in array the call is refused with a message and launches nothing."""
    import torch

    hq, hkv, d, cap, batch = 16, 16, 128, 64, 512  # 8192 (batch x kv head) units > 4096
    q = torch.zeros((batch, hq * d), dtype=torch.float16, device="cuda")
    kv = torch.zeros((batch * hkv * cap, d), dtype=torch.float16, device="cuda")
    out = torch.full((batch, hq * d), 3.0, dtype=torch.float16, device="cuda")
    st = mfk.MfFlashDecodeStrides(hq * d, d, hkv * cap * d, cap * d, hkv * cap * d, cap * d, hq * d, d)
    sp = mfk.SdpaParams(cap, d, 0.088, d, d)
    with pytest.raises(mfk.MetalError) as e:
        mfk.flash_decode_static_scratch(torch.cuda.current_stream().cuda_stream, q, kv, kv, out, st, sp, hq, batch)
    assert e.value.kind == "OutOfMemory" and "built-in array" in str(e.value)
    torch.cuda.synchronize()
    assert bool((out == 3.0).all())
