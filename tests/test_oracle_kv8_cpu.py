"""CPU checks of the oracle's 8-bit cache functions (the checker of tests/test_gpu_kv8.py).

The reference has no quantised cache (docs/FLASH.md:121-186 is a roadmap), so these pin the oracle to independent
restatements: the E4M3 codec against torch.float8_e4m3fn over all 256 bytes and a sweep of floats, the row quantiser
against its definition, the V pool's byte order against the package's layout helper, and attention over a quantised
cache against numpy in float64 on the dequantised rows.
"""
import ctypes as C
import importlib

import numpy as np
import pytest

import oracle


def test_e4m3_codec_against_torch():
    torch = pytest.importorskip("torch")
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("torch without float8_e4m3fn")
    L = oracle.lib()
    L.mfo_e4m3_to_f32.restype = C.c_float
    L.mfo_e4m3_to_f32.argtypes = [C.c_uint8]
    L.mfo_f32_to_e4m3.restype = C.c_uint8
    L.mfo_f32_to_e4m3.argtypes = [C.c_float]
    table = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    for b in range(256):
        got = L.mfo_e4m3_to_f32(b)
        if np.isnan(table[b]):
            assert np.isnan(got)
        else:
            assert got == table[b], b
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 200, 4000), rng.uniform(-2 ** -6, 2 ** -6, 2000),
                         np.array([0.0, -0.0, 448.0, -448.0, 1e6, -1e6, 2 ** -9, 2 ** -10, 464.0, 465.0])]).astype(np.float32)
    want = torch.from_numpy(xs).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).numpy()  # saturating
    got = np.array([L.mfo_f32_to_e4m3(float(x)) for x in xs], np.uint8)
    assert np.array_equal(got, want)


def test_row_quantiser_definition():
    L = oracle.lib()
    rng = np.random.default_rng(6)
    for amp in (1.0, 1e-3, 300.0, 0.0):
        row = (rng.normal(0, 1, 128) * amp).astype(np.float16)
        q = np.zeros(128, np.uint8)
        s = C.c_float()
        L.mfo_quantize_row_e4m3(row.view(np.uint16), 128, q, C.byref(s))
        amax = np.abs(row.astype(np.float32)).max()
        want_scale = np.float32(amax) / np.float32(448.0) if amax > 0 else np.float32(1.0)
        assert np.float32(s.value) == want_scale
        deq = np.array([L.mfo_e4m3_to_f32(int(b)) for b in q], np.float32) * s.value
        # three mantissa bits: half an ulp is 2^-4 relative for normal values, scale * 2^-10 for the smallest
        assert np.all(np.abs(deq - row.astype(np.float32)) <= np.abs(row.astype(np.float32)) * 2.0 ** -4 + s.value * 2.0 ** -10 + 1e-12)


def test_v_pool_byte_order_matches_the_layout_helper():
    mfk = importlib.import_module("test-burn_b200") if _has_lib() else None
    L = oracle.lib()
    for P in (16, 32, 64):
        n_pages, hkv, D = 3, 2, 128
        rows = np.arange(n_pages * hkv * P * D, dtype=np.uint32).reshape(n_pages, hkv, P, D)
        flat = np.zeros(rows.size, np.uint32)
        for r in range(n_pages * hkv * P):
            for d in range(0, D, 7):
                flat[L.mfo_kv8_v_index(r, d, D, P)] = rows.reshape(-1, D)[r, d]
        # every byte index is inside the row's own (page, kv head) run and distinct
        idx = np.array([[L.mfo_kv8_v_index(r, d, D, P) for d in range(D)] for r in range(2 * P)])
        assert len(np.unique(idx)) == idx.size
        assert idx[:P].min() == 0 and idx[:P].max() == P * D - 1 and idx[P:].min() == P * D
        if mfk is not None:
            pool = mfk.kv8_v_pool_from_rows(rows.astype(np.uint8))
            assert np.array_equal(mfk.kv8_v_rows_from_pool(pool), rows.astype(np.uint8))
            r, d = 1 * P + 5, 77
            assert pool.reshape(-1)[L.mfo_kv8_v_index(r, d, D, P)] == rows.astype(np.uint8).reshape(-1, D)[r, d]


def _has_lib():
    try:
        importlib.import_module("test-burn_b200")
        return True
    except Exception:
        return False


def test_decode_over_a_quantised_cache_against_numpy():
    L = oracle.lib()
    rng = np.random.default_rng(7)
    Hq, Hkv, D, P, n = 4, 2, 128, 16, 75
    n_pages = 6
    table = rng.permutation(n_pages).astype(np.uint32)
    k_rows = rng.normal(0, 1, (n_pages, Hkv, P, D)).astype(np.float16)
    v_rows = (rng.normal(0, 1, (n_pages, Hkv, P, D)) * rng.uniform(0.1, 10, (n_pages, Hkv, P, 1))).astype(np.float16)
    k8 = np.zeros((n_pages * Hkv * P, D), np.uint8)
    v8 = np.zeros(n_pages * Hkv * P * D, np.uint8)
    ks = np.zeros(n_pages * Hkv * P, np.float32)
    vs = np.zeros(n_pages * Hkv * P, np.float32)
    lut = np.array([L.mfo_e4m3_to_f32(b) for b in range(256)], np.float64)
    vq = np.zeros(D, np.uint8)
    vdeq = np.zeros((n_pages * Hkv * P, D))
    for r in range(n_pages * Hkv * P):
        s = C.c_float()
        L.mfo_quantize_row_e4m3(np.ascontiguousarray(k_rows.reshape(-1, D)[r]).view(np.uint16), D, k8[r], C.byref(s))
        ks[r] = s.value
        L.mfo_quantize_row_e4m3(np.ascontiguousarray(v_rows.reshape(-1, D)[r]).view(np.uint16), D, vq, C.byref(s))
        vs[r] = s.value
        for d in range(D):
            v8[L.mfo_kv8_v_index(r, d, D, P)] = vq[d]
        vdeq[r] = lut[vq] * float(s.value)
    q = rng.normal(0, 1, (Hq, D)).astype(np.float16)
    out = np.zeros((Hq, D), np.uint16)
    gold = np.zeros((Hq, D), np.float64)
    scale = 1.0 / np.sqrt(D)
    L.mfo_decode_kv8(q.view(np.uint16), k8.reshape(-1), v8, ks, vs, table, n, Hq, Hkv, D, P, C.c_float(scale), out,
                     gold.ctypes.data)
    for h in range(Hq):
        kh = h // (Hq // Hkv)
        rows = [(int(table[t // P]) * Hkv + kh) * P + t % P for t in range(n)]
        kd = lut[k8[rows]] * ks[rows, None].astype(np.float64)
        sc = kd @ q[h].astype(np.float64) * np.float64(np.float32(scale))
        w = np.exp(sc - sc.max())
        want = (w[:, None] * vdeq[rows]).sum(0) / w.sum()
        assert np.abs(gold[h] - want).max() <= 1e-9
        assert np.abs(out[h].view(np.float16).astype(np.float64) - want).max() <= 2e-3
