"""GPU parity: SdpaReference, the route the reference takes when the flash kernels do not apply
(src/metals/sdpa/step.rs:89-158, 558-779; softmax_sdpa_batched.metal:14-115).

Shapes follow the reference's CPU-checked tests: non-causal m=4, L=8, H=2, D=64
(tests/sdpa_materialized_prefill_parity.rs:70-106) and m=17 with a head-major Q
(tests/sdpa_head_stride_misaligned.rs:73-112), both with one cache head per query head; then causal
offsets that break the flash routes' invariant, grouped-query caches and a single masked row.
The oracle is the tiled f32 softmax with the general mask (key i hidden iff causal and
i > row + query_offset) and its fp64 gold; tolerance max-abs 2e-3 (the reference allows 0.05-0.15
against its f16-intermediate path).
"""
import numpy as np
import pytest

import oracle
from kvcases import dev, host, max_abs, normal

pytestmark = pytest.mark.gpu
TOL = 2e-3

# (n_heads, n_kv_heads, head_dim, m, kv_len, capacity, causal, query_offset)
CASES = [
    (2, 2, 64, 4, 8, 8, False, 0),
    (2, 2, 64, 17, 40, 40, False, 0),
    (14, 14, 64, 17, 64, 64, False, 5),
    (8, 8, 128, 32, 96, 128, True, 10),     # offset + m < kv_len: the tail of the cache stays hidden
    (8, 8, 128, 32, 96, 128, True, 90),     # offset + m > kv_len: clipped at kv_len
    (14, 2, 64, 9, 200, 256, True, 100),    # grouped-query cache
    (24, 8, 128, 130, 300, 384, False, 0),  # large enough for the tcgen05 kernel
    (24, 8, 128, 130, 300, 384, True, 7),
    (16, 2, 128, 1, 77, 128, True, 20),     # one row, masked tail
    (16, 2, 128, 1, 77, 128, False, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_sdpa_reference(mfk, foundry, case):
    import torch

    hq, hkv, d, m, kv_len, cap, causal, offset = case
    q = normal(1, hq * m * d).reshape(hq, m, d)           # head-major, as KvPrepFused leaves it
    kc = normal(2, hkv * cap * d).reshape(hkv, cap, d)
    vc = normal(3, hkv * cap * d).reshape(hkv, cap, d)
    kc[:, kv_len:] = 0x7E00                               # rows past kv_len are NaN and must not matter
    vc[:, kv_len:] = 0x7E00
    scale = np.float32(1.0) / np.sqrt(np.float32(d))
    args = dict(n_heads=hq, cache_heads=hkv, head_dim=d, capacity=cap, q_len=m, kv_len=kv_len,
                query_offset=offset if causal else kv_len, scale=scale)
    want = oracle.prefill_causal(q.ravel(), kc.ravel(), vc.ravel(), **args)
    gold = oracle.prefill_gold(q.ravel(), kc.ravel(), vc.ravel(), **args)
    out = torch.full((m, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    foundry.sdpa_reference(dev(q), dev(kc), dev(vc), out, causal=causal, query_offset=offset, n_heads=hq, head_dim=d,
                           kv_seq_len=kv_len, m=m)
    foundry.synchronize()
    got = host(out)
    assert max_abs(got, want) <= TOL
    assert max_abs(got, gold) <= TOL
    # the dispatcher reaches the same route with the same bits
    out2 = torch.full_like(out, float("nan"))
    flash_ok = (causal and offset + m == kv_len) or (m == 1 and not causal)  # one unmasked row is plain decode
    # one row: the decode route wants the token-major row view (sdpa/step.rs:305-349); same memory
    q_disp = dev(q).view(1, hq * d) if m == 1 else dev(q)
    route = foundry.flash_attention(q_disp, dev(kc), dev(vc), out2, causal=causal, query_offset=offset, n_heads=hq,
                                    head_dim=d, kv_seq_len=kv_len, m=m)
    foundry.synchronize()
    assert (route != mfk.ROUTE_REFERENCE) == flash_ok
    if flash_ok:
        assert max_abs(host(out2), want) <= TOL
    else:
        assert np.array_equal(host(out2), got)
