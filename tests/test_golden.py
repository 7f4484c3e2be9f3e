"""Golden vectors (tests/golden/kv_path_golden.npz, made by tests/golden/make_golden.py).

CPU: the oracle reproduces the committed vectors bit for bit (they are oracle outputs on the
reference's test shapes and LCG inputs; the reference itself stores no expected outputs).
GPU: the CUDA path against the same vectors - appended rows and q_rot bit-exact, attention
within max-abs 2e-3.
"""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from kvcases import ContigCase, dev, host, max_abs

GOLD = Path(__file__).resolve().parent / "golden" / "kv_path_golden.npz"
spec = importlib.util.spec_from_file_location("make_golden", GOLD.with_name("make_golden.py"))
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def test_oracle_reproduces_golden(orc, gold):
    fresh = {}
    for c in make_golden.CASES:
        fresh.update(make_golden.build(*c))
    for c in make_golden.QKV_CASES:
        fresh.update(make_golden.build_qkv(*c))
    for k, v in fresh.items():
        assert np.array_equal(v, gold[k]), k
    assert np.array_equal(orc.lcg_fill(1, 256, 0.25)[0], gold["lcg_seed1_scale025"])
    assert np.array_equal(orc.normal_fill(0x5EED, 1, 256), gold["normal_seed5EED_t1"])
    cos, sin = orc.rope_tables(1e6, 64, 512)
    assert np.array_equal(cos[[0, 1, 2, 255, 511]], gold["rope_1e6_d64/cos_rows"])
    assert np.array_equal(sin[[0, 1, 2, 255, 511]], gold["rope_1e6_d64/sin_rows"])


def test_product_rope_tables_match_golden(mfk, gold):
    cos, sin = mfk.rope_tables(5e5, 128, 8192)
    assert np.array_equal(cos[[1, 4095, 8191]], gold["rope_5e5_d128/cos_rows"])
    assert np.array_equal(sin[[1, 4095, 8191]], gold["rope_5e5_d128/sin_rows"])


@pytest.mark.gpu
@pytest.mark.parametrize("case_def", make_golden.CASES, ids=[c[0] for c in make_golden.CASES])
def test_cuda_against_golden(mfk, foundry, gold, case_def):
    import torch

    name, hq, hkv, d, cached, m, cap, mode, seed, scale = case_def
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=cached, m=m, capacity=cap, theta=1e4,
                      rope_mode=mode, gen="lcg", seed=seed, scale=scale)
    q, k, v = dev(case.q), dev(case.k), dev(case.v)
    kc, vc, cos, sin = dev(case.k_cache), dev(case.v_cache), dev(case.cos), dev(case.sin)
    q_rot = torch.zeros(hq * m * d, dtype=torch.float16, device="cuda")
    p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, m, cached, cap, hq * m * d, mode, 0, 0)
    foundry.kv_prep_fused(q, k, v, q_rot, kc, vc, cos, sin, p)
    out = torch.zeros((m, hq * d), dtype=torch.float16, device="cuda")
    if not name.startswith("append"):
        route = foundry.flash_attention(q_rot.view(hq, m, d) if m > 1 else q_rot.view(1, hq * d), kc, vc, out,
                                        causal=True, query_offset=cached, n_heads=hq, head_dim=d,
                                        kv_seq_len=cached + m, m=m)
        assert route == (mfk.ROUTE_DECODE if m == 1 else mfk.ROUTE_PREFILL)
    foundry.synchronize()
    assert np.array_equal(host(q_rot), gold[f"{name}/q_rot"])
    assert np.array_equal(host(kc)[:, cached:cached + m], gold[f"{name}/k_rows"])
    assert np.array_equal(host(vc)[:, cached:cached + m], gold[f"{name}/v_rows"])
    if not name.startswith("append"):
        assert max_abs(host(out).reshape(gold[f"{name}/out"].shape), gold[f"{name}/out"]) <= 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("case_def", make_golden.QKV_CASES, ids=[c[0] for c in make_golden.QKV_CASES])
def test_cuda_fused_qkv_against_golden(mfk, foundry, gold, case_def):
    """The projection in front of the append: one f16 ulp of the value plus 1e-3 (f32 sums in another order)."""
    import torch

    name, m, k_dim, n_dim, n_kv, gamma, bias, wpb, seed = case_def
    x, ws, g, bs = make_golden.qkv_inputs(m, k_dim, n_dim, n_kv, gamma, bias, wpb, seed)
    if wpb:
        ws = [np.ascontiguousarray(w.reshape(n, k_dim // wpb, wpb).transpose(1, 0, 2)).ravel()
              for w, n in zip(ws, (n_dim, n_kv, n_kv))]
    out = tuple(torch.zeros(m * n, dtype=torch.float16, device="cuda") for n in (n_dim, n_kv, n_kv))
    args = foundry.fused_qkv_args(dev(x), *[dev(w) for w in ws], k_dim=k_dim, n_dim=n_dim, n_kv=n_kv, m=m,
                                  gamma=None if g is None else dev(g),
                                  bias=None if bs[0] is None else tuple(dev(b) for b in bs), out=out,
                                  weights_per_block=wpb)
    foundry.fused_qkv(args)
    foundry.synchronize()
    for o, key in zip(out, ("q", "k", "v")):
        got = host(o).view(np.float16).astype(np.float32)
        ref = gold[f"{name}/{key}"].view(np.float16).astype(np.float32)
        assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -10 + 1e-3)
