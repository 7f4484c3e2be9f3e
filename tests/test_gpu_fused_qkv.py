"""GPU parity: the step in front of the append — RMSNorm -> fused Q/K/V projection (f16 weights) —
alone and fused with the RoPE + K/V append into one launch, through the C ABI.

  * the projection against the oracle's restatement of the reference's FusedQkv on the shapes of the
    reference's own tests (tests/fused_qkv_batched_rmsnorm_parity.rs:58-66: m=2, 128 -> 128/64, blocked
    weights, gamma = 1; tests/qkv_parity_f16.rs:87-89: 1024 -> 1024/128, row-major, gamma and bias) and
    on the model shapes of the benchmark configurations.  The reference allows 0.1 - 0.2 absolute; here
    one f16 ulp of the value plus 1e-3 (the f32 sums run in a different order);
  * projection + append in one launch against projection, then KvPrepFused / the paged append, as two
    launches: q_rot and the whole caches bit for bit;
  * the same bits for any number of input rows per CTA.
"""
import numpy as np
import pytest

import oracle
from kvcases import ContigCase, PagedCase, dev, dev_u32, host

pytestmark = pytest.mark.gpu
SEED = 20250


def _uniform_f16(rng, lo, hi, n):
    return rng.uniform(lo, hi, n).astype(np.float32).astype(np.float16).view(np.uint16)


def _blocked(w_bits, n, k, wpb=32):
    """Row-major [n, k] -> the reference's blocked layout (pack_canonical_f16 of its tests)."""
    return np.ascontiguousarray(w_bits.reshape(n, k // wpb, wpb).transpose(1, 0, 2)).ravel()


class Proj:
    def __init__(self, *, m, k_dim, n_dim, n_kv, gamma=True, bias=False, blocked=False, seed=SEED):
        rng = np.random.default_rng(seed)
        self.m, self.K, self.N, self.Nkv, self.blocked = m, k_dim, n_dim, n_kv, blocked
        self.x = _uniform_f16(rng, -1, 1, m * k_dim)
        self.gamma = _uniform_f16(rng, 0.5, 1.5, k_dim) if gamma else None
        self.w = [_uniform_f16(rng, -0.1, 0.1, n * k_dim) for n in (n_dim, n_kv, n_kv)]
        self.bias = [_uniform_f16(rng, -0.1, 0.1, n) for n in (n_dim, n_kv, n_kv)] if bias else None
        self.wpb = 32 if blocked else 0
        if blocked:
            self.w_dev_bits = [_blocked(w, n, k_dim) for w, n in zip(self.w, (n_dim, n_kv, n_kv))]
        else:
            self.w_dev_bits = self.w

    def oracle(self):
        b = self.bias or (None, None, None)
        return oracle.fused_qkv(self.x, *self.w_dev_bits, m=self.m, k_dim=self.K, n_dim=self.N, n_kv=self.Nkv,
                                gamma=self.gamma, b_q=b[0], b_k=b[1], b_v=b[2], weights_per_block=self.wpb)

    def args(self, foundry, out=None, m=None, x=None):
        if not hasattr(self, "_dev"):
            self._dev = dict(x=dev(self.x), w=[dev(w) for w in self.w_dev_bits],
                             gamma=None if self.gamma is None else dev(self.gamma),
                             bias=None if self.bias is None else tuple(dev(b) for b in self.bias))
        d = self._dev
        return foundry.fused_qkv_args(d["x"] if x is None else x, *d["w"], k_dim=self.K, n_dim=self.N, n_kv=self.Nkv,
                                      m=self.m if m is None else m, gamma=d["gamma"], bias=d["bias"], out=out,
                                      weights_per_block=self.wpb)


def _run_plain(foundry, pj, m=None, x=None):
    import torch

    m = pj.m if m is None else m
    out = tuple(torch.full((m * n,), float("nan"), dtype=torch.float16, device="cuda") for n in (pj.N, pj.Nkv, pj.Nkv))
    foundry.fused_qkv(pj.args(foundry, out=out, m=m, x=x))
    foundry.synchronize()
    return [host(o).ravel() for o in out]


def _close(got_bits, ref_bits):
    got = got_bits.view(np.float16).astype(np.float32)
    ref = ref_bits.view(np.float16).astype(np.float32)
    return bool(np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -10 + 1e-3))


# (m, k_dim, n_dim, n_kv, gamma, bias, blocked)
PROJ_SHAPES = [
    (2, 128, 128, 64, "ones", False, True),     # tests/fused_qkv_batched_rmsnorm_parity.rs:58-66
    (1, 1024, 1024, 128, True, True, False),    # tests/qkv_parity_f16.rs:87-89
    (1, 896, 896, 128, True, True, True),       # Qwen2.5-0.5B layer (14 q / 2 kv heads of 64)
    (1, 2048, 2048, 256, True, True, True),     # Qwen2.5-3B layer
    (1, 3072, 3072, 1024, True, False, True),   # Llama-3.2-3B layer
    (3, 3072, 3072, 1024, True, False, False),
    (5, 256, 64, 32, False, False, True),       # no norm, rows not a multiple of the rows per CTA
    (9, 160, 48, 16, True, True, False),        # k blocks (5) not a multiple of the eight warps
    (8, 8192, 128, 32, True, True, True),       # staged rows above 48 KB of shared memory (opt-in size)
    (8, 16384, 64, 16, True, False, False),     # rows per CTA cut to what fits: five, then three
]


@pytest.mark.parametrize("shape", PROJ_SHAPES)
def test_fused_qkv_against_oracle(mfk, foundry, shape):
    m, k_dim, n_dim, n_kv, gamma, bias, blocked = shape
    pj = Proj(m=m, k_dim=k_dim, n_dim=n_dim, n_kv=n_kv, gamma=bool(gamma), bias=bias, blocked=blocked)
    if gamma == "ones":
        pj.gamma = np.full(k_dim, 0x3C00, np.uint16)
    ref = pj.oracle()
    got = _run_plain(foundry, pj)
    for g, r in zip(got, ref):
        assert _close(g, r)


def test_fused_qkv_rows_per_cta_do_not_change_bits(mfk, foundry):
    """Seven rows share one pass over the weights; each row alone, and two of them together, give the same bits."""
    pj = Proj(m=7, k_dim=512, n_dim=256, n_kv=64, gamma=True, bias=True, blocked=True)
    all_rows = _run_plain(foundry, pj)
    x = dev(pj.x).reshape(7, 512)
    for row in (0, 3, 6):
        one = _run_plain(foundry, pj, m=1, x=x[row])
        for a, o, n in zip(all_rows, one, (256, 64, 64)):
            assert np.array_equal(a.reshape(7, n)[row], o)
    two = _run_plain(foundry, pj, m=2, x=x[4:6])
    assert np.array_equal(all_rows[0].reshape(7, 256)[4:6].ravel(), two[0])


@pytest.mark.parametrize("rope_mode", [0, 1])
@pytest.mark.parametrize("shape", [(1, 777, 1024, 16, 2, 128, 2048), (4, 3, 32, 14, 2, 64, 896),
                                   (6, 10, 64, 24, 8, 128, 512)])
@pytest.mark.parametrize("expanded", [False, True])
def test_projection_and_append_in_one_launch(mfk, foundry, shape, rope_mode, expanded):
    import torch

    m, off, cap, hq, hkv, d, k_dim = shape
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=off, m=m, capacity=cap, theta=1e4,
                      rope_mode=rope_mode, expanded=expanded)
    pj = Proj(m=m, k_dim=k_dim, n_dim=hq * d, n_kv=hkv * d, gamma=True, bias=True, blocked=True)
    q_bits, k_bits, v_bits = _run_plain(foundry, pj)
    p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, m, off, cap, hq * m * d, rope_mode, 0, 0)
    cos, sin = dev(case.cos), dev(case.sin)
    # two launches
    kc2, vc2 = dev(case.k_cache), dev(case.v_cache)
    q_rot2 = torch.full((hq * m * d,), float("nan"), dtype=torch.float16, device="cuda")
    foundry.kv_prep_fused(dev(q_bits.reshape(m, hq * d)), dev(k_bits.reshape(m, hkv * d)),
                          dev(v_bits.reshape(m, hkv * d)), q_rot2, kc2, vc2, cos, sin, p)
    # one launch; the plain outputs are asked for as well and must not change
    kc1, vc1 = dev(case.k_cache), dev(case.v_cache)
    q_rot1 = torch.full((hq * m * d,), float("nan"), dtype=torch.float16, device="cuda")
    out = tuple(torch.full((m * n,), float("nan"), dtype=torch.float16, device="cuda") for n in (hq * d, hkv * d, hkv * d))
    foundry.fused_qkv_kv_prep(pj.args(foundry, out=out), q_rot1, kc1, vc1, cos, sin, p)
    foundry.synchronize()
    assert np.array_equal(host(q_rot1), host(q_rot2))
    assert np.array_equal(host(kc1), host(kc2)) and np.array_equal(host(vc1), host(vc2))
    for o, bits in zip(out, (q_bits, k_bits, v_bits)):
        assert np.array_equal(host(o).ravel(), bits)
    # and the oracle chain end to end: projection restated on the CPU, its bits through the append oracle
    case.q, case.k, case.v = (q_bits.reshape(m, hq * d), k_bits.reshape(m, hkv * d), v_bits.reshape(m, hkv * d))
    q_ref, k_ref, v_ref = case.oracle_append()
    assert np.array_equal(host(q_rot1), q_ref)
    assert np.array_equal(host(kc1), k_ref) and np.array_equal(host(vc1), v_ref)


def test_projection_and_paged_append_in_one_launch(mfk, foundry):
    """One new token per sequence into a paged cache (the decode step), and a chunk of one sequence."""
    import torch

    hq, hkv, d, P, k_dim = 16, 2, 128, 16, 1024
    cached = [5, 16, 47, 130, 0, 31]
    case = PagedCase(batch=len(cached), n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P, cached=cached, poison=False)
    B = case.B
    pj = Proj(m=B, k_dim=k_dim, n_dim=hq * d, n_kv=hkv * d, gamma=True, bias=True, blocked=True)
    q_bits, k_bits, v_bits = _run_plain(foundry, pj)
    cos, sin = dev(case.cos), dev(case.sin)
    d_table, d_lens = dev_u32(case.page_table), dev_u32(case.kv_lens)
    res = []
    for fused in (False, True):
        kp, vp = dev(case.k_pool), dev(case.v_pool)
        desc = mfk.paged_kv(kp, vp, d_table, d_lens, n_kv_heads=hkv, page_size=P, head_dim=d)
        q_rot = torch.full((B, hq * d), float("nan"), dtype=torch.float16, device="cuda")
        if fused:
            foundry.fused_qkv_paged_append(pj.args(foundry), desc, q_rot, cos, sin, n_heads=hq)
        else:
            foundry.paged_kv_append(desc, dev(q_bits.reshape(B, hq * d)), dev(k_bits.reshape(B, hkv * d)),
                                    dev(v_bits.reshape(B, hkv * d)), q_rot, cos, sin, n_heads=hq)
        foundry.synchronize()
        res.append((host(q_rot), host(kp), host(vp)))
    for a, b in zip(*res):
        assert np.array_equal(a, b)
    # a chunk: rows 0..B of sequence 3 appended at position 130
    res = []
    for fused in (False, True):
        kp, vp = dev(case.k_pool), dev(case.v_pool)
        lens = case.kv_lens.copy()
        # sequence 3 owns ceil(131/16) = 9 pages: positions 130..135 stay inside them
        desc = mfk.paged_kv(kp, vp, d_table, dev_u32(lens), n_kv_heads=hkv, page_size=P, head_dim=d)
        q_rot = torch.full((hq, B, d), float("nan"), dtype=torch.float16, device="cuda")
        if fused:
            foundry.fused_qkv_paged_append(pj.args(foundry), desc, q_rot, cos, sin, n_heads=hq, seq=3, position_offset=130)
        else:
            foundry.paged_kv_append(desc, dev(q_bits.reshape(B, hq * d)), dev(k_bits.reshape(B, hkv * d)),
                                    dev(v_bits.reshape(B, hkv * d)), q_rot, cos, sin, n_heads=hq, seq=3,
                                    position_offset=130, seq_len=B)
        foundry.synchronize()
        res.append((host(q_rot), host(kp), host(vp)))
    for a, b in zip(*res):
        assert np.array_equal(a, b)


def test_fused_qkv_rejects_what_it_cannot_do(mfk, foundry):
    pj = Proj(m=1, k_dim=64, n_dim=32, n_kv=16)
    out = tuple(dev(np.zeros(n, np.uint16)) for n in (32, 16, 16))
    good = pj.args(foundry, out=out)
    foundry.fused_qkv(good)
    for field, value, kind in (("k_dim", 48, "InvalidShape"), ("n_dim", 24, "InvalidShape"),
                               ("weights_per_block", 64, "OperationNotSupported"), ("out_k", None, "InputNotFound"),
                               ("bias_q", 1 << 20, "InputNotFound")):
        bad = pj.args(foundry, out=out)
        setattr(bad, field, value)
        with pytest.raises(mfk.MetalError) as e:
            foundry.fused_qkv(bad)
        assert e.value.kind == kind, field
    foundry.synchronize()


def test_projection_and_paged_append_more_rows_than_one_pass(mfk, foundry):
    """Nineteen sequences: three passes of up to eight input rows, one new token per sequence."""
    import torch

    hq, hkv, d, P, k_dim = 14, 2, 64, 16, 896
    cached = [3 + 7 * i for i in range(19)]
    case = PagedCase(batch=len(cached), n_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=P, cached=cached, poison=False)
    B = case.B
    pj = Proj(m=B, k_dim=k_dim, n_dim=hq * d, n_kv=hkv * d, gamma=True, bias=True, blocked=True)
    q_bits, k_bits, v_bits = _run_plain(foundry, pj)
    cos, sin = dev(case.cos), dev(case.sin)
    d_table, d_lens = dev_u32(case.page_table), dev_u32(case.kv_lens)
    res = []
    for fused in (False, True):
        kp, vp = dev(case.k_pool), dev(case.v_pool)
        desc = mfk.paged_kv(kp, vp, d_table, d_lens, n_kv_heads=hkv, page_size=P, head_dim=d)
        q_rot = torch.full((B, hq * d), float("nan"), dtype=torch.float16, device="cuda")
        if fused:
            foundry.fused_qkv_paged_append(pj.args(foundry), desc, q_rot, cos, sin, n_heads=hq, rope_mode=1)
        else:
            foundry.paged_kv_append(desc, dev(q_bits.reshape(B, hq * d)), dev(k_bits.reshape(B, hkv * d)),
                                    dev(v_bits.reshape(B, hkv * d)), q_rot, cos, sin, n_heads=hq, rope_mode=1)
        foundry.synchronize()
        res.append((host(q_rot), host(kp), host(vp)))
    for a, b in zip(*res):
        assert np.array_equal(a, b)
    assert not np.array_equal(res[0][1], case.k_pool)  # rows were written


# ---- the tensor-core (tcgen05) projection: eight input rows or more (automatic choice) ----------------------------------------------
# (m, k_dim, n_dim, n_kv, gamma, bias, blocked)
TC_SHAPES = [
    (16, 2048, 2048, 256, True, True, True),     # Qwen2.5-3B layer, the smallest batch that takes this path
    (64, 3072, 3072, 1024, True, False, True),   # Llama-3.2-3B layer at C3's batch
    (70, 896, 896, 128, True, True, True),       # two row tiles, the second partial; 7 k stages over a cluster of 7
    (33, 1024, 1024, 128, True, True, False),    # row-major weights (128-byte swizzle)
    (64, 256, 128, 128, False, False, True),     # no norm; two k stages
    (130, 128, 128, 128, True, True, False),     # one k stage: no split, three row tiles
]


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_fused_qkv_tensor_core_kernel_against_oracle(mfk, foundry, shape):
    m, k_dim, n_dim, n_kv, gamma, bias, blocked = shape
    pj = Proj(m=m, k_dim=k_dim, n_dim=n_dim, n_kv=n_kv, gamma=bool(gamma), bias=bias, blocked=blocked)
    ref = pj.oracle()
    foundry.set_option(mfk.OPTION_QKV_IMPL, 2)  # fail rather than fall back
    try:
        got = _run_plain(foundry, pj)
    finally:
        foundry.set_option(mfk.OPTION_QKV_IMPL, 0)
    for g, r in zip(got, ref):
        assert _close(g, r)
    # the mma.sync kernel on the same rows: same contract, other order of the f32 sums
    foundry.set_option(mfk.OPTION_QKV_IMPL, 1)
    try:
        old = _run_plain(foundry, pj)
    finally:
        foundry.set_option(mfk.OPTION_QKV_IMPL, 0)
    for g, o in zip(got, old):
        assert _close(g, o)


def test_fused_qkv_tensor_core_rows_do_not_depend_on_their_company(mfk, foundry):
    """A row's bits are the same whether 16, 40 or 64 rows are projected with it (same tile columns or not)."""
    pj = Proj(m=64, k_dim=1024, n_dim=256, n_kv=128, gamma=True, bias=True, blocked=True)
    foundry.set_option(mfk.OPTION_QKV_IMPL, 2)
    try:
        full = _run_plain(foundry, pj)
        x = dev(pj.x).reshape(64, 1024)
        part = _run_plain(foundry, pj, m=16, x=x[24:40].contiguous())
        one = _run_plain(foundry, pj, m=1, x=x[63].contiguous())
    finally:
        foundry.set_option(mfk.OPTION_QKV_IMPL, 0)
    for a, b, c, n in zip(full, part, one, (256, 128, 128)):
        assert np.array_equal(a.reshape(64, n)[24:40].ravel(), b)
        assert np.array_equal(a.reshape(64, n)[63], c)


@pytest.mark.parametrize("rope_mode", [0, 1])
@pytest.mark.parametrize("shape", [(40, 100, 256, 16, 2, 128, 2048), (64, 0, 64, 14, 2, 64, 896)])
def test_tensor_core_projection_and_append_in_one_launch(mfk, foundry, shape, rope_mode):
    """Projection + RoPE + append by the tensor-core kernel against its own plain outputs pushed through KvPrepFused."""
    import torch

    m, off, cap, hq, hkv, d, k_dim = shape
    if (hq * d) % 128 or (hkv * d) % 128:
        pytest.skip("shape outside the tensor-core kernel's envelope")
    case = ContigCase(n_heads=hq, n_kv_heads=hkv, head_dim=d, cached=off, m=m, capacity=cap, theta=1e4, rope_mode=rope_mode)
    pj = Proj(m=m, k_dim=k_dim, n_dim=hq * d, n_kv=hkv * d, gamma=True, bias=True, blocked=True)
    p = mfk.KvPrepFusedParamsResolved(hq * d, hkv * d, d, hq, hkv, hq // hkv, m, off, cap, hq * m * d, rope_mode, 0, 0)
    cos, sin = dev(case.cos), dev(case.sin)
    foundry.set_option(mfk.OPTION_QKV_IMPL, 2)
    try:
        q_bits, k_bits, v_bits = _run_plain(foundry, pj)
        kc1, vc1 = dev(case.k_cache), dev(case.v_cache)
        q_rot1 = torch.full((hq * m * d,), float("nan"), dtype=torch.float16, device="cuda")
        out = tuple(torch.full((m * n,), float("nan"), dtype=torch.float16, device="cuda") for n in (hq * d, hkv * d, hkv * d))
        foundry.fused_qkv_kv_prep(pj.args(foundry, out=out), q_rot1, kc1, vc1, cos, sin, p)
    finally:
        foundry.set_option(mfk.OPTION_QKV_IMPL, 0)
    kc2, vc2 = dev(case.k_cache), dev(case.v_cache)
    q_rot2 = torch.full((hq * m * d,), float("nan"), dtype=torch.float16, device="cuda")
    foundry.kv_prep_fused(dev(q_bits.reshape(m, hq * d)), dev(k_bits.reshape(m, hkv * d)), dev(v_bits.reshape(m, hkv * d)),
                          q_rot2, kc2, vc2, cos, sin, p)
    foundry.synchronize()
    assert np.array_equal(host(q_rot1), host(q_rot2))
    assert np.array_equal(host(kc1), host(kc2)) and np.array_equal(host(vc1), host(vc2))
    for o, bits in zip(out, (q_bits, k_bits, v_bits)):
        assert np.array_equal(host(o).ravel(), bits)
    ref = pj.oracle()
    for g, r in zip((q_bits, k_bits, v_bits), ref):
        assert _close(g, r)


@pytest.mark.parametrize("m", [8, 9, 17, 31, 48, 63, 65, 127, 129])
def test_fused_qkv_tensor_core_kernel_row_counts(mfk, foundry, m):
    """Row counts around the tile edges (N of the MMA = 16, 32, 48, 64; one, two and three 64-row tiles; the last rank
    of the cluster owning fewer rows or none), automatic kernel choice."""
    pj = Proj(m=m, k_dim=512, n_dim=256, n_kv=128, gamma=True, bias=True, blocked=(m % 2 == 1))
    ref = pj.oracle()
    before = foundry.launch_count
    got = _run_plain(foundry, pj)
    assert foundry.launch_count - before == 2  # the normalisation and the tensor-core projection
    for g, r in zip(got, ref):
        assert _close(g, r)
