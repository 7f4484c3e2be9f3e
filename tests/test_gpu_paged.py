"""GPU parity: batched paged decode (fused RoPE + append + GQA flash-decode) through the C ABI.

The paged layout, batch > 1 and split-KV decode are not in the reference; they are pinned by
identities against the restated oracle: pool contents after the append are bit-exact, the
gathered pages equal the contiguous cache bit-exact, and attention matches the contiguous
oracle (f32 online softmax and fp64 gold) within max-abs 2e-3.
"""
import numpy as np
import pytest

import oracle
from kvcases import PagedCase, dev, dev_u32, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3


class DeviceCase:
    def __init__(self, mfk, case):
        self.k_pool, self.v_pool = dev(case.k_pool), dev(case.v_pool)
        self.page_table = dev_u32(case.page_table)
        self.kv_lens = dev_u32(case.kv_lens)
        self.q, self.k, self.v = dev(case.q), dev(case.k), dev(case.v)
        self.cos, self.sin = dev(case.cos), dev(case.sin)
        self.desc = mfk.paged_kv(self.k_pool, self.v_pool, self.page_table, self.kv_lens, n_kv_heads=case.Hkv,
                                 page_size=case.P, head_dim=case.D)


def run_fused(mfk, foundry, case, max_ctas=0, repeats=1):
    import torch

    dc = DeviceCase(mfk, case)
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D,
                               page_size=case.P, max_ctas=max_ctas)
    out = torch.full((case.B, case.Hq * case.D), float("nan"), dtype=torch.float16, device="cuda")
    q_rot = torch.full_like(out, float("nan"))
    for _ in range(repeats):
        foundry.paged_decode(plan, dc.desc, dc.q, out, n_heads=case.Hq, k=dc.k, v=dc.v, cos=dc.cos, sin=dc.sin,
                             rope=True, rope_mode=case.rope_mode, append=True, q_rot=q_rot, scale=float(case.scale))
    foundry.synchronize()
    res = host(out), host(q_rot), host(dc.k_pool), host(dc.v_pool)
    plan.close()
    return res


def check(case, got, ref):
    out, q_rot, kp, vp = got
    q_ref, kp_ref, vp_ref, out_ref, gold = ref
    assert np.array_equal(q_rot, q_ref)
    assert np.array_equal(kp, kp_ref)  # the appended rows, bit-exact, and nothing else touched
    assert np.array_equal(vp, vp_ref)
    assert max_abs(out, out_ref) <= TOL
    assert max_abs(out, gold.ravel()) <= TOL


CASES = [
    # batch, Hq, Hkv, D, P, cached lengths
    dict(batch=6, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[0, 14, 15, 16, 63, 64]),
    dict(batch=5, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[511, 1000, 2049, 3, 4095]),
    dict(batch=4, n_heads=24, n_kv_heads=8, head_dim=128, page_size=64, cached=[0, 63, 64, 1337]),
    dict(batch=3, n_heads=14, n_kv_heads=2, head_dim=64, page_size=16, cached=[511, 31, 32]),
    dict(batch=3, n_heads=32, n_kv_heads=2, head_dim=64, page_size=32, cached=[200, 7, 95]),
    dict(batch=2, n_heads=4, n_kv_heads=4, head_dim=128, page_size=8, cached=[77, 130]),
    dict(batch=2, n_heads=8, n_kv_heads=1, head_dim=128, page_size=128, cached=[300, 127]),
]


@pytest.mark.parametrize("cfg", CASES)
@pytest.mark.parametrize("rope_mode", [0, 1])
def test_fused_append_decode(mfk, foundry, cfg, rope_mode):
    case = PagedCase(rope_mode=rope_mode, **cfg)
    check(case, run_fused(mfk, foundry, case), case.oracle_step())


@pytest.mark.parametrize("max_ctas", [1, 3, 40, 1000])
def test_any_cta_count_gives_the_same_answer(mfk, foundry, max_ctas):
    """Span boundaries move with the CTA count; parity must not."""
    case = PagedCase(batch=5, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[511, 1000, 2049, 3, 4095])
    check(case, run_fused(mfk, foundry, case, max_ctas=max_ctas), case.oracle_step())


@pytest.mark.parametrize("item_cost", [1, 6, 64])
@pytest.mark.parametrize("max_ctas", [7, 40])
def test_any_item_cost_gives_the_same_answer(mfk, foundry, item_cost, max_ctas):
    """What the planner charges per piece of a unit moves the span boundaries (and leaves some CTAs without work);
    parity must not move."""
    case = PagedCase(batch=9, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16,
                     cached=[511, 40, 1000, 2049, 3, 4095, 70, 64, 900])
    foundry.set_option(mfk.OPTION_PLAN_ITEM_COST, item_cost)
    try:
        got = run_fused(mfk, foundry, case, max_ctas=max_ctas)
    finally:
        foundry.set_option(mfk.OPTION_PLAN_ITEM_COST, 0)
    check(case, got, case.oracle_step())


def test_fused_step_is_idempotent(mfk, foundry):
    """Running the same step again rewrites the same row and gives the same output."""
    case = PagedCase(batch=4, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[100, 2000, 17, 900])
    a = run_fused(mfk, foundry, case, repeats=1)
    b = run_fused(mfk, foundry, case, repeats=4)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_separate_append_then_decode(mfk, foundry):
    """mf_paged_kv_append + decode without fusion equals the fused launch bit for bit."""
    import torch

    case = PagedCase(batch=4, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[5, 700, 64, 2047])
    fused = run_fused(mfk, foundry, case)
    dc = DeviceCase(mfk, case)
    q_rot = torch.empty((case.B, case.Hq * case.D), dtype=torch.float16, device="cuda")
    foundry.paged_kv_append(dc.desc, dc.q, dc.k, dc.v, q_rot, dc.cos, dc.sin, n_heads=case.Hq,
                            rope_mode=case.rope_mode)
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
    out = torch.empty_like(q_rot)
    foundry.paged_decode(plan, dc.desc, q_rot, out, n_heads=case.Hq, scale=float(case.scale))
    foundry.synchronize()
    assert np.array_equal(host(q_rot), fused[1])
    assert np.array_equal(host(dc.k_pool), fused[2])
    assert np.array_equal(host(dc.v_pool), fused[3])
    assert np.array_equal(host(out), fused[0])
    plan.close()


def test_paged_gather_equals_contiguous(mfk, foundry):
    """Pages gathered in logical order are the contiguous [Hkv, L, D] cache, bit-exact."""
    import torch

    case = PagedCase(batch=3, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[33, 500, 16],
                     poison=False)
    dc = DeviceCase(mfk, case)
    for b in range(case.B):
        n = int(case.cached[b])
        for use_v, pool in ((False, case.k_pool), (True, case.v_pool)):
            out = torch.empty((case.Hkv, n, case.D), dtype=torch.float16, device="cuda")
            foundry.paged_gather(dc.desc, use_v, b, n, out)
            foundry.synchronize()
            ref = np.empty((case.Hkv, n, case.D), np.uint16)
            oracle.lib().mfo_paged_gather(pool, case.page_table[b], n, case.Hkv, case.P, case.D, ref)
            assert np.array_equal(host(out), ref)


def test_plan_update_follows_growing_sequences(mfk, foundry):
    """Three decode steps in a row: lengths grow by one, the plan is updated in place."""
    import torch

    cached = np.array([14, 62, 300], np.uint32)
    case = PagedCase(batch=3, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=cached + 3, poison=False)
    # start three tokens earlier and replay the appends with the oracle and the GPU side by side
    k_pool, v_pool = case.k_pool.copy(), case.v_pool.copy()
    dk, dv = dev(k_pool), dev(v_pool)
    pt = dev_u32(case.page_table)
    cos, sin = dev(case.cos), dev(case.sin)
    plan = None
    L = oracle.lib()
    for step in range(3):
        lens = cached + step + 1
        q = oracle.normal_fill(77, 10 + step, case.B * case.Hq * case.D).reshape(case.B, -1)
        k = oracle.normal_fill(77, 20 + step, case.B * case.Hkv * case.D).reshape(case.B, -1)
        v = oracle.normal_fill(77, 30 + step, case.B * case.Hkv * case.D).reshape(case.B, -1)
        q_rot = np.empty_like(q)
        L.mfo_paged_kv_append(q, k, v, q_rot, k_pool, v_pool, case.cos, case.sin, case.page_table, case.pt_stride,
                              (lens - 1).astype(np.uint32), case.B, case.Hq, case.Hkv, case.D, case.P, 0, 1)
        ref = np.empty((case.B, case.Hq * case.D), np.uint16)
        for b in range(case.B):
            n = int(lens[b])
            kc = np.empty((case.Hkv, n, case.D), np.uint16)
            vc = np.empty((case.Hkv, n, case.D), np.uint16)
            L.mfo_paged_gather(k_pool, case.page_table[b], n, case.Hkv, case.P, case.D, kc)
            L.mfo_paged_gather(v_pool, case.page_table[b], n, case.Hkv, case.P, case.D, vc)
            ref[b] = oracle.decode_online(q_rot[b], kc, vc, n_heads=case.Hq, cache_heads=case.Hkv, head_dim=case.D,
                                          capacity=n, kv_len=n, scale=case.scale)
        dl = dev_u32(lens)
        desc = mfk.paged_kv(dk, dv, pt, dl, n_kv_heads=case.Hkv, page_size=case.P, head_dim=case.D)
        if plan is None:
            plan = foundry.decode_plan(lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
        else:
            plan.update(lens)
        out = torch.empty((case.B, case.Hq * case.D), dtype=torch.float16, device="cuda")
        foundry.paged_decode(plan, desc, dev(q), out, n_heads=case.Hq, k=dev(k), v=dev(v), cos=cos, sin=sin,
                             rope=True, append=True, scale=float(case.scale))
        foundry.synchronize()
        assert max_abs(host(out), ref) <= TOL
        assert np.array_equal(host(dk), k_pool)
    plan.close()


def test_partials_and_merge_equal_full_decode(mfk, foundry):
    """Sequence-sharded decode on one GPU: two shards of one long sequence emit (acc, m, l);
    mf_merge_partials over the gathered partials equals the unsharded result."""
    import torch

    Hq, Hkv, D, P, L = 24, 8, 128, 64, 4096 + 17
    full = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False)
    q_ref, kp, vp, out_ref, gold = full.oracle_step()
    dk, dv = dev(kp), dev(vp)  # pools after the append
    q_rot = dev(q_ref)
    n_pages = full.page_table.shape[1]
    cut = (n_pages // 2)
    shards = [(0, cut), (cut, n_pages)]
    accs, ms, ls = [], [], []
    for (p0, p1) in shards:
        pt = np.ascontiguousarray(full.page_table[:, p0:p1])
        lens = np.array([min(L, p1 * P) - p0 * P], np.uint32)
        d_pt, d_len = dev_u32(pt), dev_u32(lens)
        desc = mfk.paged_kv(dk, dv, d_pt, d_len, n_kv_heads=Hkv, page_size=P, head_dim=D)
        plan = foundry.decode_plan(lens, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P)
        acc = torch.zeros((1, Hq, D), dtype=torch.float32, device="cuda")
        m = torch.full((1, Hq), -1e30, dtype=torch.float32, device="cuda")
        l = torch.zeros((1, Hq), dtype=torch.float32, device="cuda")
        foundry.paged_decode_partial(plan, desc, q_rot, acc, m, l, n_heads=Hq, scale=float(full.scale))
        foundry.synchronize()
        plan.close()
        accs.append(acc.view(Hq, D))
        ms.append(m.view(Hq))
        ls.append(l.view(Hq))
    acc = torch.stack(accs).contiguous()
    m = torch.stack(ms).contiguous()
    l = torch.stack(ls).contiguous()
    out = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
    foundry.merge_partials(acc, m, l, out)
    foundry.synchronize()
    assert max_abs(host(out), out_ref) <= TOL
    assert max_abs(host(out), gold.ravel()) <= TOL
    # the merge kernel itself against the oracle's merge, same partials
    ref_merge = oracle.merge_partials(acc.cpu().numpy(), m.cpu().numpy(), l.cpu().numpy())
    assert max_abs(host(out), ref_merge) <= 1e-3


def test_paged_decode_rejects_bad_arguments(mfk, foundry):
    import torch

    case = PagedCase(batch=2, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[5, 70], poison=False)
    dc = DeviceCase(mfk, case)
    plan = foundry.decode_plan(case.kv_lens, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16)
    out = torch.empty((2, 16 * 128), dtype=torch.float16, device="cuda")
    with pytest.raises(mfk.MetalError) as e:  # append without k/v
        foundry.paged_decode(plan, dc.desc, dc.q, out, n_heads=16, append=True)
    assert e.value.kind == "InputNotFound"
    with pytest.raises(mfk.MetalError) as e:  # geometry differs from the plan
        foundry.paged_decode(plan, dc.desc, dc.q, out, n_heads=8)
    assert e.value.kind == "InvalidShape"
    with pytest.raises(mfk.MetalError) as e:
        foundry.decode_plan(case.kv_lens, n_heads=16, n_kv_heads=2, head_dim=96, page_size=16)
    assert e.value.kind == "OperationNotSupported"
    plan.close()
    foundry.synchronize()


def test_overlapped_launches_give_the_same_bits(mfk, foundry):
    """MF_OPTION_OVERLAP_LAUNCHES: a chain of fused launches over several layers (separate pools,
    shared plan, partial slots and tickets) must equal the plainly serialised chain."""
    import torch

    layers = 6
    cases = [PagedCase(batch=5, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, seed=100 + i,
                       cached=[511, 1000, 2049, 3, 4095]) for i in range(layers)]
    results = {}
    for overlap in (0, 1):
        foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)
        dcs = [DeviceCase(mfk, c) for c in cases]
        plan = foundry.decode_plan(cases[0].kv_lens, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16)
        outs = [torch.zeros((5, 16 * 128), dtype=torch.float16, device="cuda") for _ in range(layers)]
        for _ in range(3):
            for c, dc, out in zip(cases, dcs, outs):
                foundry.paged_decode(plan, dc.desc, dc.q, out, n_heads=16, k=dc.k, v=dc.v, cos=dc.cos, sin=dc.sin,
                                     rope=True, append=True, scale=float(c.scale))
        foundry.synchronize()
        results[overlap] = [host(o) for o in outs] + [host(dc.k_pool) for dc in dcs]
        plan.close()
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    for a, b in zip(results[0], results[1]):
        assert np.array_equal(a, b)
    ref = cases[0].oracle_step()
    assert max_abs(results[1][0], ref[3]) <= TOL


def test_decode_chain_replays_from_a_cuda_graph(mfk):
    """A chain of fused launches (two layers sharing one plan) is captured once into a CUDA graph and
    replayed: the replay must give the bits of the eager chain.  The first (eager) pass also does the
    one-time work that does not belong inside a capture (function attributes, tensor-map encoding)."""
    import torch

    case = PagedCase(batch=5, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[300, 17, 2049, 64, 1000])
    ref = case.oracle_step()
    stream = torch.cuda.Stream()
    f = mfk.Foundry(0, stream.cuda_stream)
    f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 1)
    layers = [DeviceCase(mfk, case) for _ in range(2)]
    plan = f.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
    outs = [torch.full((case.B, case.Hq * case.D), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]

    def chain():
        for dc, out in zip(layers, outs):
            f.paged_decode(plan, dc.desc, dc.q, out, n_heads=case.Hq, k=dc.k, v=dc.v, cos=dc.cos, sin=dc.sin, rope=True,
                           rope_mode=case.rope_mode, append=True, scale=float(case.scale))

    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        chain()
    f.synchronize()
    eager = [host(o).copy() for o in outs]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        chain()
    for o in outs:
        o.fill_(float("nan"))
    torch.cuda.synchronize()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    f.synchronize()  # reads the device status word
    for o, e in zip(outs, eager):
        assert np.array_equal(host(o), e)
        assert max_abs(host(o), ref[3]) <= TOL
    for dc in layers:
        assert np.array_equal(host(dc.k_pool), ref[1]) and np.array_equal(host(dc.v_pool), ref[2])
    plan.close()
    f.close()


@pytest.mark.parametrize("n_layers", [4, 6])
@pytest.mark.parametrize("overlap", [1, 2])
def test_steps_in_a_row_on_rotating_pools(mfk, foundry, n_layers, overlap):
    """Several decode steps of a model whose layers each own a pool, short sequences (few CTAs per
    launch), overlapped launches: the launch that reads a pool comes `n_layers` launches after the
    one that appended the row before.  Pools bit-exact and every output checked, every step."""
    import torch

    from kvcases import normal

    base, steps = np.array([200, 37, 450], np.uint32), 12
    cfg = dict(batch=3, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16)
    cases = [PagedCase(cached=base + steps, seed=0x77 + 5 * layer, **cfg) for layer in range(n_layers)]
    for c in cases:
        # rows from `base` on are still to be appended: poison them
        for b in range(c.B):
            for t in range(int(base[b]), int(base[b]) + steps + 1):
                page = c.page_table[b, t // c.P]
                c.k_pool[page, :, t % c.P] = 0x7E00
                c.v_pool[page, :, t % c.P] = 0x7E00
        c.cached = base.copy()
        c.kv_lens = c.cached + 1
    dcs = [DeviceCase(mfk, c) for c in cases]
    c0 = cases[0]
    plan = foundry.decode_plan(c0.kv_lens, n_heads=c0.Hq, n_kv_heads=c0.Hkv, head_dim=c0.D, page_size=c0.P)
    n_q, n_kv = c0.B * c0.Hq * c0.D, c0.B * c0.Hkv * c0.D
    outs = torch.full((steps, n_layers, c0.B, c0.Hq * c0.D), float("nan"), dtype=torch.float16, device="cuda")
    step_in = []
    for s in range(steps):
        step_in.append([(normal(1000 + 10 * s + 100 * layer, n_q).reshape(c0.B, -1), normal(1001 + 10 * s + 100 * layer, n_kv).reshape(c0.B, -1),
                         normal(1002 + 10 * s + 100 * layer, n_kv).reshape(c0.B, -1)) for layer in range(n_layers)])
    dev_in = [[tuple(dev(x) for x in trio) for trio in row] for row in step_in]
    lens_dev = [dev_u32(base + 1 + s) for s in range(steps)]
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)
    for s in range(steps):
        plan.update(base + 1 + s)
        for dc in dcs:
            dc.kv_lens.copy_(lens_dev[s])
        for layer, dc in enumerate(dcs):
            q, k, v = dev_in[s][layer]
            foundry.paged_decode(plan, dc.desc, q, outs[s, layer], n_heads=c0.Hq, k=k, v=v, cos=dc.cos, sin=dc.sin,
                                 rope=True, rope_mode=0, append=True, scale=float(c0.scale))
    foundry.synchronize()
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    got = host(outs)
    for layer, c in enumerate(cases):
        for s in range(steps):
            c.cached = base + s
            c.kv_lens = c.cached + 1
            c.q, c.k, c.v = step_in[s][layer]
            _, kp, vp, out_ref, gold = c.oracle_step()
            c.k_pool, c.v_pool = kp, vp
            assert max_abs(got[s, layer], out_ref) <= TOL, (layer, s)
            assert max_abs(got[s, layer], gold.ravel()) <= TOL, (layer, s)
        assert np.array_equal(host(dcs[layer].k_pool), c.k_pool), layer
        assert np.array_equal(host(dcs[layer].v_pool), c.v_pool), layer
    plan.close()


def _case_with_spare_pages(spare=4):
    """A case whose pools hold `spare` pages more than the descriptor will declare: an access that a
    guard fails to stop still lands inside the allocation."""
    case = PagedCase(batch=4, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[100, 31, 15, 700],
                     extra_pages=spare)
    return case, case.n_pages - spare


def test_append_skips_a_page_id_outside_the_pool(mfk, foundry):
    """The page id of the new row comes from the caller's device-side table.  One that is not a page
    of the pool must not be written through: the store is skipped, mf_synchronize reports
    InvalidOperation, and the other sequences are unaffected."""
    import torch

    case, declared = _case_with_spare_pages()
    bad_seq, bad_page = 1, declared + 1  # inside the allocation, outside the declared pool
    ref = case.oracle_step()
    slot = int(case.cached[bad_seq]) // case.P
    # the valid pages of the case must all be inside the declared pool for this to be a fair test
    valid = case.page_table[case.page_table < 0x7FFFFFF0]
    remap = {int(p): i for i, p in enumerate(np.sort(valid))}
    assert len(remap) <= declared
    # the seeded permutation may have used the spare ids: renumber pages into [0, len(valid))
    new_k, new_v = case.k_pool.copy(), case.v_pool.copy()
    new_k[:], new_v[:] = 0x7E00, 0x7E00
    for old, new in remap.items():
        new_k[new], new_v[new] = case.k_pool[old], case.v_pool[old]
    pt = case.page_table.copy()
    for b in range(case.B):
        for j in range(pt.shape[1]):
            if pt[b, j] < 0x7FFFFFF0:
                pt[b, j] = remap[int(pt[b, j])]
    good_pt = pt.copy()
    pt[bad_seq, slot] = bad_page
    for fused in (True, False):
        k_pool, v_pool = dev(new_k), dev(new_v)
        table, lens = dev_u32(pt), dev_u32(case.kv_lens)
        desc = mfk.paged_kv(k_pool, v_pool, table, lens, n_kv_heads=case.Hkv, page_size=case.P, head_dim=case.D)
        desc.n_pages = declared
        out = torch.zeros((case.B, case.Hq * case.D), dtype=torch.float16, device="cuda")
        q_rot = torch.zeros_like(out)
        if fused:
            plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
            foundry.paged_decode(plan, desc, dev(case.q), out, n_heads=case.Hq, k=dev(case.k), v=dev(case.v), cos=dev(case.cos),
                                 sin=dev(case.sin), rope=True, rope_mode=0, append=True, scale=float(case.scale))
        else:
            foundry.paged_kv_append(desc, dev(case.q), dev(case.k), dev(case.v), q_rot, dev(case.cos), dev(case.sin),
                                    n_heads=case.Hq, rope_mode=0)
        with pytest.raises(mfk.MetalError) as e:
            foundry.synchronize()
        assert e.value.kind == "InvalidOperation", str(e.value)
        foundry.synchronize()  # the status word is cleared by the report
        kp, vp = host(k_pool), host(v_pool)
        assert np.all(kp[declared:] == 0x7E00) and np.all(vp[declared:] == 0x7E00)  # nothing beyond the declared pool
        # every other sequence's row was appended as the oracle says
        for b in range(case.B):
            if b == bad_seq:
                continue
            t = int(case.cached[b])
            page_old = int(case.page_table[b, t // case.P])
            page_new = int(good_pt[b, t // case.P])
            assert np.array_equal(kp[page_new, :, t % case.P], ref[1][page_old, :, t % case.P])
            assert np.array_equal(vp[page_new, :, t % case.P], ref[2][page_old, :, t % case.P])
            if fused:
                assert max_abs(host(out)[b], ref[3][b]) <= TOL
        if fused:
            plan.close()


def test_append_skips_an_empty_sequence_and_a_length_past_the_table(mfk, foundry):
    """kv_lens is device data too: a length of zero has no row to append (position -1), one past the
    table has no page entry.  Both are skipped with a status; the other sequences' rows are written."""
    import torch

    case, _ = _case_with_spare_pages()
    ref = case.oracle_step()
    bad = 2
    for bad_len in (0, case.pt_stride * case.P + 1):
        lens = case.kv_lens.copy()
        lens[bad] = bad_len
        k_pool, v_pool = dev(case.k_pool), dev(case.v_pool)
        table, dlens = dev_u32(case.page_table), dev_u32(lens)
        desc = mfk.paged_kv(k_pool, v_pool, table, dlens, n_kv_heads=case.Hkv, page_size=case.P, head_dim=case.D)
        q_rot = torch.zeros((case.B, case.Hq * case.D), dtype=torch.float16, device="cuda")
        foundry.paged_kv_append(desc, dev(case.q), dev(case.k), dev(case.v), q_rot, dev(case.cos), dev(case.sin),
                                n_heads=case.Hq, rope_mode=0)
        with pytest.raises(mfk.MetalError) as e:
            foundry.synchronize()
        assert e.value.kind == "InvalidOperation"
        want_k, want_v = case.k_pool.copy(), case.v_pool.copy()
        for b in range(case.B):
            if b == bad:
                continue
            t = int(case.cached[b])
            page = int(case.page_table[b, t // case.P])
            want_k[page, :, t % case.P] = ref[1][page, :, t % case.P]
            want_v[page, :, t % case.P] = ref[2][page, :, t % case.P]
        assert np.array_equal(host(k_pool), want_k) and np.array_equal(host(v_pool), want_v)


@pytest.mark.parametrize("cfg", [
    dict(batch=1, n_heads=24, n_kv_heads=8, head_dim=128, page_size=64, cached=[8191]),
    dict(batch=1, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[5000]),
    dict(batch=3, n_heads=14, n_kv_heads=2, head_dim=64, page_size=16, cached=[1023, 1023, 1023]),
    # 65 tiles per unit in 4 ranges of 17, 17, 17, 14 tiles for clusters of 16: two CTAs of the last cluster get no tile
    dict(batch=1, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[4159]),
])
def test_paged_decode_cluster_form(mfk, foundry, cfg):
    """One sequence (or equal lengths) on pages: the plan takes the cluster form; the same step in the plain
    form must agree with the oracle just the same."""
    case = PagedCase(**cfg)
    ref = case.oracle_step()
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
    assert plan.cluster in (8, 16) and plan.ctas % plan.cluster == 0
    plan.close()
    check(case, run_fused(mfk, foundry, case), ref)
    foundry.set_option(mfk.OPTION_DECODE_CLUSTERS, 1)
    try:
        plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
        assert plan.cluster == 0
        plan.close()
        check(case, run_fused(mfk, foundry, case), ref)
    finally:
        foundry.set_option(mfk.OPTION_DECODE_CLUSTERS, 0)


@pytest.mark.parametrize("cfg", [
    dict(batch=4, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[5567, 2751, 11455, 16255]),
    dict(batch=8, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16,
         cached=[5567, 2751, 11455, 16255, 12095, 4095, 6335, 10559]),
    dict(batch=2, n_heads=24, n_kv_heads=8, head_dim=128, page_size=64, cached=[700, 3000]),
    dict(batch=3, n_heads=14, n_kv_heads=2, head_dim=64, page_size=16, cached=[1500, 520, 4000]),
])
def test_short_batches_of_different_lengths_take_the_cluster_form(mfk, foundry, cfg):
    """A few sequences of different lengths (what a rank holds when one batch is split over eight GPUs): every unit is
    cut into ranges of about equal length, one cluster per range; same bits in the pools and in q_rot, same answer."""
    case = PagedCase(**cfg)
    ref = case.oracle_step()
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
    assert plan.cluster in (2, 4, 8) and plan.ctas % plan.cluster == 0
    plan.close()
    check(case, run_fused(mfk, foundry, case), ref)
    check(case, run_fused(mfk, foundry, case, repeats=2), ref)  # the step again on the same pools: idempotent
