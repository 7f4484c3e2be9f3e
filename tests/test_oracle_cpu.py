"""CPU tests of the oracle itself (no GPU): conversions, generators, the identities the
reference's tests assert, and agreement with an independent numpy restatement."""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, PagedCase, lcg, max_abs, ulp_distance


def test_f16_conversions_exhaustive(orc):
    L = orc.lib()
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([L.mfo_f16_to_f32(int(b)) for b in bits], np.float32)
    finite = ~np.isnan(ref)
    assert np.array_equal(got.view(np.uint32)[finite], ref.view(np.uint32)[finite])
    assert np.isnan(got[~finite]).all()
    back = np.array([L.mfo_f32_to_f16(float(x)) for x in ref[finite]], np.uint16)
    assert np.array_equal(back, bits[finite])


def test_f32_to_f16_round_to_nearest_even(orc):
    L = orc.lib()
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s
                         for s in (1.0, 1e-3, 6e-5, 1e-7, 3e-8, 300.0, 60000.0)])
    # exact ties between neighbouring f16 values
    h = np.arange(0, 0x7BFF, 37, dtype=np.uint16)
    lo = h.view(np.float16).astype(np.float32)
    hi = (h + 1).astype(np.uint16).view(np.float16).astype(np.float32)
    xs = np.concatenate([xs, (lo + hi) / 2, -(lo + hi) / 2, np.float32([65504, 65519.9, 65520, 1e9, 0.0, -0.0])])
    with np.errstate(over="ignore"):
        ref = xs.astype(np.float16).view(np.uint16)
    got = np.array([L.mfo_f32_to_f16(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, ref)


def test_lcg_generator_known_values(orc):
    """tests/flashattention_decode_parity.rs:15-30 restated in numpy uint32 arithmetic."""
    state = np.uint32(1)
    vals = []
    for _ in range(64):
        state = np.uint32((int(state) * 1664525 + 1013904223) & 0xFFFFFFFF)
        r01 = np.float32(int(state) >> 9) * np.float32(1.0 / (1 << 23))
        vals.append(np.float16((r01 * np.float32(2.0) - np.float32(1.0)) * np.float32(0.25)))
    got, end_state = orc.lcg_fill(1, 64, 0.25)
    assert np.array_equal(got, np.array(vals, np.float16).view(np.uint16))
    assert end_state == int(state)
    # the first LCG state after seed 1 is the classic Numerical Recipes value
    assert (1 * 1664525 + 1013904223) & 0xFFFFFFFF == 1015568748


def test_normal_generator_is_counter_based(orc):
    a = orc.normal_fill(0x5EED, 3, 1000)
    b = orc.normal_fill(0x5EED, 3, 400, first=600)
    assert np.array_equal(a[600:], b)
    x = orc.h2f(orc.normal_fill(0x5EED, 9, 200000))
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01
    assert not np.array_equal(a, orc.normal_fill(0x5EED, 4, 1000))


def numpy_rope_tables(theta, d, n):
    """Independent restatement of executor.rs:1980-2007 in numpy float32."""
    i = np.arange(d // 2, dtype=np.float32)
    inv = np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * i) / np.float32(d), dtype=np.float32)
    ang = np.arange(n, dtype=np.float32)[:, None] * inv[None, :]
    return np.cos(ang, dtype=np.float32).astype(np.float16), np.sin(ang, dtype=np.float32).astype(np.float16)


@pytest.mark.parametrize("theta,d,n", [(1e4, 64, 128), (1e6, 64, 512), (5e5, 128, 1024)])
def test_rope_tables_vs_numpy(orc, theta, d, n):
    cos, sin = orc.rope_tables(theta, d, n)
    rc, rs = numpy_rope_tables(theta, d, n)
    # libm and numpy pow/cos/sin may differ in the last f32 bit, which can move a value across
    # an f16 rounding boundary (and by several tiny ulps next to a zero crossing): compare in
    # absolute terms, one f16 ulp at 1.0, and require almost all entries to be identical.
    assert max_abs(cos, rc.view(np.uint16)) <= 2.0 ** -10
    assert max_abs(sin, rs.view(np.uint16)) <= 2.0 ** -10
    assert (cos != rc.view(np.uint16)).mean() < 0.01 and (sin != rs.view(np.uint16)).mean() < 0.01
    # row 0 is exactly cos 0 = 1, sin 0 = 0
    assert (cos[0] == 0x3C00).all() and (sin[0] == 0).all()
    # offset tables continue the same sequence
    c2, s2 = orc.rope_tables(theta, d, 16, first_pos=n - 16)
    assert np.array_equal(c2, cos[-16:]) and np.array_equal(s2, sin[-16:])


def test_rope_freq_factors(orc):
    ff = np.linspace(1.0, 8.0, 32).astype(np.float32)
    cos, _ = orc.rope_tables(5e5, 64, 64, freq_factors=ff)
    cos1, _ = orc.rope_tables(5e5, 64, 64)
    assert np.array_equal(cos[:, 0], cos1[:, 0])  # factor 1 leaves the first frequency alone
    assert not np.array_equal(cos, cos1)


def numpy_rope(x, cos, sin, pos, mode):
    """Independent restatement of the RoPE pair math on a [rows, D] block at positions pos."""
    x = x.view(np.float16).astype(np.float32)
    d = x.shape[-1]
    c = cos.view(np.float16).astype(np.float32)[pos]
    s = sin.view(np.float16).astype(np.float32)[pos]
    out = np.empty_like(x)
    if mode == 0:
        a, b = x[..., : d // 2], x[..., d // 2:]
        out[..., : d // 2] = a * c - b * s
        out[..., d // 2:] = b * c + a * s
    else:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = b * c + a * s
    return out.astype(np.float16).view(np.uint16)


# (seq_len, position_offset, max_seq_len, n_heads, n_kv_heads, head_dim): tests/kv_prep_fused.rs:249-267
REF_SHAPES = [(1, 5, 16, 14, 2, 64), (4, 0, 16, 14, 2, 64), (2, 0, 64, 32, 8, 128)]


@pytest.mark.parametrize("shape", REF_SHAPES)
@pytest.mark.parametrize("mode", [0, 1])
def test_fused_append_vs_numpy_and_unfused_chain(orc, shape, mode):
    m, off, cap, hq, hkv, d = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=off, m=m, capacity=cap, theta=1e4,
                      rope_mode=mode, gen="lcg", seed=3, scale=1.0)
    q_rot, kc, vc = case.oracle_append()
    pos = np.arange(off, off + m)
    # numpy restatement
    q_np = numpy_rope(case.q.reshape(m, hq, d), case.cos, case.sin, pos[:, None], mode)  # [m, hq, d]
    k_np = numpy_rope(case.k.reshape(m, hkv, d), case.cos, case.sin, pos[:, None], mode)
    assert np.array_equal(q_rot.reshape(hq, m, d), q_np.transpose(1, 0, 2))
    assert np.array_equal(kc[:, off:off + m], k_np.transpose(1, 0, 2))
    assert np.array_equal(vc[:, off:off + m], case.v.reshape(m, hkv, d).transpose(1, 0, 2))
    assert not kc[:, off + m:].any() and not vc[:, off + m:].any()
    if mode == 0:
        # the reference's seven-kernel chain: KvRearrange -> Rope -> KvCacheWrite (bit-exact pin)
        L = orc.lib()
        kh = np.empty((hkv, m, d), np.uint16)
        vh = np.empty((hkv, m, d), np.uint16)
        qh = np.empty((hq, m, d), np.uint16)
        L.mfo_kv_rearrange(case.k, kh, hkv * d, d, hkv, hkv, d, m)
        L.mfo_kv_rearrange(case.v, vh, hkv * d, d, hkv, hkv, d, m)
        L.mfo_kv_rearrange(case.q, qh, hq * d, d, hq, hq, d, m)
        kr, qr = np.empty_like(kh), np.empty_like(qh)
        L.mfo_rope_neox(kh, kr, case.cos, case.sin, d, m, off, kh.size)
        L.mfo_rope_neox(qh, qr, case.cos, case.sin, d, m, off, qh.size)
        kc2, vc2 = case.k_cache.copy(), case.v_cache.copy()
        L.mfo_kv_cache_write(kc2, kr, hkv, d, m, off, cap)
        L.mfo_kv_cache_write(vc2, vh, hkv, d, m, off, cap)
        assert np.array_equal(kc2, kc) and np.array_equal(vc2, vc) and np.array_equal(qr.ravel(), q_rot)


def test_expanded_layout_repeats_heads(orc):
    case = ContigCase(n_heads=6, n_kv_heads=2, head_dim=64, cached=2, m=2, capacity=8, expanded=True)
    _, kc, vc = case.oracle_append()
    comp = ContigCase(n_heads=6, n_kv_heads=2, head_dim=64, cached=2, m=2, capacity=8, expanded=False)
    _, kc2, vc2 = comp.oracle_append()
    assert np.array_equal(kc, np.repeat(kc2, 3, axis=0)) and np.array_equal(vc, np.repeat(vc2, 3, axis=0))
    rep = np.empty_like(kc)
    orc.lib().mfo_repeat_kv_heads(kc2, rep, 2, 3, 8, 64)
    assert np.array_equal(rep, kc)


def numpy_attention(q, k, v, scale, kvh_of):
    """fp64 softmax(q k^T) v with a GQA map, independent of the C code."""
    q = q.view(np.float16).astype(np.float64)
    k = k.view(np.float16).astype(np.float64)
    v = v.view(np.float16).astype(np.float64)
    out = np.empty_like(q)
    for h in range(q.shape[0]):
        s = (k[kvh_of(h)] @ q[h]) * float(scale)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v[kvh_of(h)]
    return out


@pytest.mark.parametrize("hq,hkv,d,L", [(14, 2, 64, 512), (24, 8, 128, 300), (8, 8, 128, 128), (14, 14, 64, 27)])
def test_decode_orders_agree_with_gold_and_numpy(orc, hq, hkv, d, L):
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=L - 1, capacity=L + 5)
    q_rot, kc, vc = case.oracle_append()
    kw = dict(n_heads=hq, cache_heads=hkv, head_dim=d, capacity=case.cap, kv_len=L, scale=case.scale)
    online = orc.decode_online(q_rot, kc, vc, **kw)
    gold = orc.decode_gold(q_rot, kc, vc, **kw)
    ref = numpy_attention(q_rot.reshape(hq, d), kc[:, :L], vc[:, :L], case.scale, lambda h: h // (hq // hkv))
    assert np.max(np.abs(gold - ref)) < 1e-12
    assert max_abs(online, gold.ravel()) <= 1e-3
    for block in (128, 256, 512):  # the reference kernel's block sizes (variants.rs:184-236)
        blocked = orc.decode_blocked(q_rot, kc, vc, block_keys=block, **kw)
        assert max_abs(blocked, gold.ravel()) <= 1e-3
        assert ulp_distance(blocked, online) <= 2


@pytest.mark.parametrize("b,h,L,d", [(1, 1, 128, 64), (2, 4, 32, 128)])
def test_cpu_sdpa_attention_identity_rope(orc, b, h, L, d):
    """tests/sdpa_v2_parity.rs: identity RoPE isolates the attention math; the restated Rust
    oracle must equal the per-key online decode on an expanded cache."""
    bh = b * h
    q, k, v = lcg(5, bh * d, 1.0), lcg(6, bh * L * d, 1.0), lcg(7, bh * L * d, 1.0)
    cos = np.full((L, d // 2), 0x3C00, np.uint16)
    sin = np.zeros((L, d // 2), np.uint16)
    out = np.empty(bh * d, np.uint16)
    orc.lib().mfo_cpu_sdpa_attention(q, k, v, cos, sin, bh, L, d, out)
    ref = orc.decode_online(q, k.reshape(bh, L, d), v.reshape(bh, L, d), n_heads=bh, cache_heads=bh, head_dim=d,
                            capacity=L, kv_len=L, scale=np.float32(1.0) / np.sqrt(np.float32(d)))
    assert np.array_equal(out, ref)


def test_split_partials_merge_to_unsplit(orc):
    case = ContigCase(n_heads=24, n_kv_heads=8, head_dim=128, cached=999, capacity=1000)
    q_rot, kc, vc = case.oracle_append()
    kw = dict(n_heads=24, cache_heads=8, head_dim=128, capacity=1000, scale=case.scale)
    full = orc.decode_online(q_rot, kc, vc, kv_len=1000, **kw)
    cuts = [0, 100, 101, 640, 1000]
    accs, ms, ls = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        _, acc, m, l = orc.decode_online(q_rot, kc, vc, kv_len=b, key_begin=a, partials=True, **kw)
        accs.append(acc), ms.append(m), ls.append(l)
    merged = orc.merge_partials(np.stack(accs), np.stack(ms), np.stack(ls))
    assert ulp_distance(merged.ravel(), full) <= 2
    # an empty split (l = 0, m = -1e30) is skipped
    accs.append(np.zeros_like(accs[0])), ms.append(np.full_like(ms[0], -1e30)), ls.append(np.zeros_like(ls[0]))
    merged2 = orc.merge_partials(np.stack(accs), np.stack(ms), np.stack(ls))
    assert np.array_equal(merged2, merged)


def test_paged_equals_contiguous(orc):
    case = PagedCase(batch=3, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[33, 500, 16])
    q_rot, kp, vp, out, gold = case.oracle_step()
    L = orc.lib()
    for b in range(case.B):
        c = int(case.cached[b])
        # the same sequence in a contiguous cache, appended with the contiguous kernel math
        cont = ContigCase(n_heads=16, n_kv_heads=2, head_dim=128, cached=c, capacity=c + 1)
        kc0 = np.empty((2, c, 128), np.uint16)
        vc0 = np.empty((2, c, 128), np.uint16)
        L.mfo_paged_gather(case.k_pool, case.page_table[b], c, 2, 16, 128, kc0)
        L.mfo_paged_gather(case.v_pool, case.page_table[b], c, 2, 16, 128, vc0)
        cont.k_cache[:, :c], cont.v_cache[:, :c] = kc0, vc0
        cont.q, cont.k, cont.v = case.q[b:b + 1], case.k[b:b + 1], case.v[b:b + 1]
        cont.cos, cont.sin = case.cos, case.sin
        q2, kc, vc = cont.oracle_append()
        got_k = np.empty((2, c + 1, 128), np.uint16)
        got_v = np.empty((2, c + 1, 128), np.uint16)
        L.mfo_paged_gather(kp, case.page_table[b], c + 1, 2, 16, 128, got_k)
        L.mfo_paged_gather(vp, case.page_table[b], c + 1, 2, 16, 128, got_v)
        assert np.array_equal(got_k, kc) and np.array_equal(got_v, vc) and np.array_equal(q2, q_rot[b])
        ref = orc.decode_online(q2, kc, vc, n_heads=16, cache_heads=2, head_dim=128, capacity=c + 1, kv_len=c + 1,
                                scale=case.scale)
        assert np.array_equal(ref, out[b])
    # the threaded baseline routine computes the same step
    kp2, vp2 = case.k_pool.copy(), case.v_pool.copy()
    out2 = np.empty_like(out)
    L.mfo_paged_decode_layer(case.q, case.k, case.v, kp2, vp2, case.cos, case.sin, case.page_table, case.pt_stride,
                             case.kv_lens, case.B, 16, 2, 128, 16, 0, float(case.scale), out2)
    assert np.array_equal(kp2, kp) and np.array_equal(vp2, vp) and np.array_equal(out2, out)


@pytest.mark.parametrize("m,prefix,hq,hkv,d", [(7, 0, 14, 14, 64), (17, 64, 8, 8, 128), (33, 64, 14, 2, 64),
                                                (32, 224, 24, 8, 128)])
def test_prefill_causal_vs_gold_and_numpy(orc, m, prefix, hq, hkv, d):
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=prefix, m=m, capacity=prefix + m + 3)
    q_rot, kc, vc = case.oracle_append()
    kw = dict(n_heads=hq, cache_heads=hkv, head_dim=d, capacity=case.cap, q_len=m, kv_len=prefix + m,
              query_offset=prefix, scale=case.scale)
    out = orc.prefill_causal(q_rot, kc, vc, **kw)
    gold = orc.prefill_gold(q_rot, kc, vc, **kw)
    assert max_abs(out, gold) <= 1e-3
    # numpy causal attention: row r sees keys 0..r+prefix
    q3 = q_rot.reshape(hq, m, d)
    for r in (0, m // 2, m - 1):
        ref = numpy_attention(np.ascontiguousarray(q3[:, r]), kc[:, :prefix + r + 1], vc[:, :prefix + r + 1],
                              case.scale, lambda h: h // (hq // hkv))
        assert np.max(np.abs(gold[r].reshape(hq, d) - ref)) < 1e-12
    # the last row of a prefill chunk is a decode step over the same cache
    dec = orc.decode_online(np.ascontiguousarray(q3[:, m - 1]).ravel(), kc, vc, n_heads=hq, cache_heads=hkv,
                            head_dim=d, capacity=case.cap, kv_len=prefix + m, scale=case.scale)
    assert ulp_distance(dec, out[m - 1]) <= 2


def test_prefill_split_k_partials(orc):
    """Split ranges follow splitk_tile_range; part + reduce equals the single pass."""
    hq, d, m, kv = 14, 64, 32, 1024
    case = ContigCase(n_heads=hq, n_kv_heads=hq, head_dim=d, cached=kv - m, m=m, capacity=kv)
    q_rot, kc, vc = case.oracle_append()
    kw = dict(n_heads=hq, cache_heads=hq, head_dim=d, capacity=kv, q_len=m, kv_len=kv, query_offset=kv - m,
              scale=case.scale)
    single = orc.prefill_causal(q_rot, kc, vc, **kw)
    L = orc.lib()
    import ctypes as C

    accs, ms, ls, covered = [], [], [], 0
    for s in range(4):
        tb, te = C.c_uint32(), C.c_uint32()
        L.mfo_splitk_tile_range(kv, 4, s, C.byref(tb), C.byref(te))
        assert tb.value == covered
        covered = te.value
        _, acc, mm, ll = orc.prefill_causal(q_rot, kc, vc, tile_begin=tb.value, tile_end=te.value, partials=True, **kw)
        accs.append(acc.reshape(-1, d)), ms.append(mm.ravel()), ls.append(ll.ravel())
    assert covered == kv // 32
    merged = orc.merge_partials(np.stack(accs), np.stack(ms), np.stack(ls)).reshape(hq, m, d).transpose(1, 0, 2)
    assert ulp_distance(merged.reshape(m, hq * d), single) <= 2


@pytest.mark.parametrize("shape", [(2, 128, 128, 64, False, True), (1, 1024, 1024, 128, True, False)])
def test_fused_qkv_restatement(orc, shape):
    """The projection in front of the append, on the two shapes the reference checks on its CPU
    (tests/fused_qkv_batched_rmsnorm_parity.rs:23-56,58-66: f32 RMSNorm then x @ W^T, blocked weights;
    tests/qkv_parity_f16.rs:18-69,87-89: f16-rounded norm, row-major weights, bias): the restatement
    follows the second (the kernel's own rounding points) and is compared with a float64 version of
    the same steps; the blocked and the row-major layouts must give the same bits."""
    m, k_dim, n_dim, n_kv, bias, blocked = shape
    rng = np.random.default_rng(7)
    f16 = lambda lo, hi, n: rng.uniform(lo, hi, n).astype(np.float32).astype(np.float16)
    x, gamma = f16(-1, 1, (m, k_dim)), f16(0.5, 1.5, k_dim)
    ws = [f16(-0.1, 0.1, (n, k_dim)) for n in (n_dim, n_kv, n_kv)]
    bs = [f16(-0.1, 0.1, n) for n in (n_dim, n_kv, n_kv)] if bias else [None] * 3
    bits = lambda a: None if a is None else np.ascontiguousarray(a).view(np.uint16).ravel()
    kw = dict(m=m, k_dim=k_dim, n_dim=n_dim, n_kv=n_kv, gamma=bits(gamma), b_q=bits(bs[0]), b_k=bits(bs[1]),
              b_v=bits(bs[2]))
    row_major = orc.fused_qkv(bits(x), *[bits(w) for w in ws], weights_per_block=0, **kw)
    packed = [np.ascontiguousarray(w.reshape(w.shape[0], k_dim // 32, 32).transpose(1, 0, 2)) for w in ws]
    blocked_out = orc.fused_qkv(bits(x), *[bits(w) for w in packed], weights_per_block=32, **kw)
    for a, b in zip(row_major, blocked_out):
        assert np.array_equal(a, b)
    xf = x.astype(np.float64)
    inv = 1.0 / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-6)
    xn = (xf * inv * gamma.astype(np.float64)).astype(np.float16).astype(np.float64)
    for got, w, b in zip(blocked_out if blocked else row_major, ws, bs):
        ref = xn @ w.astype(np.float64).T + (0.0 if b is None else b.astype(np.float64))
        got = got.view(np.float16).astype(np.float64).reshape(ref.shape)
        assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -10 + 1e-3)
    # no gamma: the input goes into the projection as it is
    plain = orc.fused_qkv(bits(x), *[bits(w) for w in ws], m=m, k_dim=k_dim, n_dim=n_dim, n_kv=n_kv)
    ref = x.astype(np.float64) @ ws[0].astype(np.float64).T
    assert np.all(np.abs(plain[0].view(np.float16).astype(np.float64).reshape(ref.shape) - ref) <= np.abs(ref) * 2.0 ** -10 + 1e-3)


@pytest.mark.parametrize("cfg", [dict(batch=5, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[511, 1000, 2049, 3, 0]),
                                 dict(batch=3, n_heads=14, n_kv_heads=2, head_dim=64, page_size=16, cached=[511, 31, 32]),
                                 dict(batch=2, n_heads=24, n_kv_heads=8, head_dim=128, page_size=64, cached=[63, 700])])
@pytest.mark.parametrize("rope_mode", [0, 1])
def test_fast_cpu_arm_agrees_with_the_strict_oracle(cfg, rope_mode):
    """The timed CPU arm (mf_oracle_fast.c: F16C, FMA vectors, one K/V pass per KV head, blocked softmax,
    OpenMP) against the strict scalar oracle on the same layer: pools bit-exact, outputs within 2e-3."""
    from kvcases import PagedCase, max_abs

    case = PagedCase(rope_mode=rope_mode, **cfg)
    _, kp_ref, vp_ref, out_ref, gold = case.oracle_step()
    F = oracle.fast_lib()
    kp, vp = case.k_pool.copy(), case.v_pool.copy()
    out = np.zeros((case.B, case.Hq * case.D), np.uint16)
    rc = F.mfo_fast_paged_decode_layer(case.q, case.k, case.v, kp, vp, case.cos, case.sin, case.page_table, case.pt_stride,
                                       case.kv_lens, case.B, case.Hq, case.Hkv, case.D, case.P, rope_mode,
                                       float(case.scale), out)
    assert rc == 0
    assert np.array_equal(kp, kp_ref) and np.array_equal(vp, vp_ref)
    assert max_abs(out, out_ref) <= 2e-3
    assert max_abs(out, gold.ravel()) <= 2e-3
