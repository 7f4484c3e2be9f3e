"""GPU parity: the 8-bit (FP8 E4M3, one f32 scale per cached row) paged K/V cache.

The reference has no quantised cache (a roadmap only: docs/FLASH.md:121-186); format and arithmetic are this
project's and are restated in the oracle (oracle/mf_oracle.c, mfo_quantize_row_e4m3 and below).  Bars:
  * the quantiser is bit-exact with the oracle: pool bytes and row scales after an append are equal;
  * attention over a given quantised cache is within 2e-3 of the oracle's f32 online softmax and of the fp64
    gold computed over the SAME quantised data (the error of the kernel, not of the format);
  * the cost of the format itself - the 8-bit result against the f16-cache result on the same inputs - is
    measured and bounded at 3e-2 for N(0,1) inputs (three mantissa bits per element: relative 2^-4 per value,
    averaged over the keys a softmax mixes).
"""
import numpy as np
import pytest

import oracle
from kvcases import PagedCase, dev, dev_u32, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3
FORMAT_TOL = 3e-2


def quantised_pools(case, unwritten=None):
    """The case's f16 pools quantised row by row with the oracle: (k8, v8, ks, vs), V in the pool's byte order.
    `unwritten` ([n_pages, Hkv, P] bool): rows to fill with 0xFF bytes (an E4M3 NaN) and NaN scales."""
    L = oracle.lib()
    import ctypes as C

    n_rows = case.n_pages * case.Hkv * case.P
    out = []
    for pool in (case.k_pool, case.v_pool):
        q8 = np.zeros((n_rows, case.D), np.uint8)
        sc = np.zeros(n_rows, np.float32)
        rows = pool.reshape(n_rows, case.D)
        for r in range(n_rows):
            s = C.c_float()
            L.mfo_quantize_row_e4m3(np.ascontiguousarray(rows[r]), case.D, q8[r], C.byref(s))
            sc[r] = s.value
        out.append((q8.reshape(case.n_pages, case.Hkv, case.P, case.D), sc.reshape(case.n_pages, case.Hkv, case.P)))
    import importlib
    if unwritten is not None:
        for q8, sc in out:
            q8[unwritten] = 0xFF
            sc[unwritten] = np.nan
    v8 = importlib.import_module("test-burn_b200").kv8_v_pool_from_rows(out[1][0])  # V: dim-major 16-key blocks
    return out[0][0], v8, out[0][1], out[1][1]


def oracle_step(case, k8, v8, ks, vs):
    """Append + attend with the oracle on the quantised cache.  Returns (q_rot, k8', v8', ks', vs', out, gold)."""
    L = oracle.lib()
    k8, v8, ks, vs = k8.copy(), v8.copy(), ks.copy(), vs.copy()
    q_rot = np.empty_like(case.q)
    L.mfo_paged_kv8_append(case.q, case.k, case.v, q_rot, k8.reshape(-1), v8.reshape(-1), ks.reshape(-1), vs.reshape(-1),
                           case.cos, case.sin, case.page_table, case.pt_stride, case.cached, case.B, case.Hq, case.Hkv, case.D,
                           case.P, case.rope_mode, 1)
    out = np.empty((case.B, case.Hq * case.D), np.uint16)
    gold = np.empty((case.B, case.Hq * case.D), np.float64)
    for b in range(case.B):
        L.mfo_decode_kv8(q_rot[b], k8.reshape(-1), v8.reshape(-1), ks.reshape(-1), vs.reshape(-1), case.page_table[b],
                         int(case.kv_lens[b]), case.Hq, case.Hkv, case.D, case.P, float(case.scale), out[b],
                         gold[b].ctypes.data)
    return q_rot, k8, v8, ks, vs, out, gold


CASES = [
    dict(batch=6, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[0, 14, 15, 16, 63, 64]),
    dict(batch=5, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[511, 1000, 2049, 3, 4095]),
    dict(batch=4, n_heads=24, n_kv_heads=8, head_dim=128, page_size=64, cached=[0, 63, 64, 1337]),
    dict(batch=2, n_heads=4, n_kv_heads=4, head_dim=128, page_size=16, cached=[77, 130]),
    dict(batch=3, n_heads=8, n_kv_heads=1, head_dim=128, page_size=32, cached=[300, 127, 31]),
]


@pytest.mark.parametrize("cfg", CASES)
@pytest.mark.parametrize("rope_mode", [0, 1])
@pytest.mark.parametrize("max_ctas", [3, 296])
def test_fused_append_decode_on_the_8bit_cache(mfk, foundry, cfg, rope_mode, max_ctas):
    import torch

    case = PagedCase(rope_mode=rope_mode, poison=False, **cfg)
    # rows that were never written: NaN scales and 0xFF bytes (an E4M3 NaN), to prove they are never used
    written = np.zeros((case.n_pages, case.P), bool)
    for b in range(case.B):
        for t in range(int(case.cached[b])):
            written[case.page_table[b, t // case.P], t % case.P] = True
    k8, v8, ks, vs = quantised_pools(case, unwritten=~written[:, None, :].repeat(case.Hkv, 1))
    q_ref, k8_ref, v8_ref, ks_ref, vs_ref, out_ref, gold = oracle_step(case, k8, v8, ks, vs)
    d_k8, d_v8 = torch.from_numpy(k8).cuda(), torch.from_numpy(v8).cuda()
    d_ks, d_vs = torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda()
    pt, lens = dev_u32(case.page_table), dev_u32(case.kv_lens)
    desc = mfk.paged_kv8(d_k8, d_v8, d_ks, d_vs, pt, lens, n_kv_heads=case.Hkv, page_size=case.P)
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P,
                               max_ctas=max_ctas)
    out = torch.full((case.B, case.Hq * case.D), float("nan"), dtype=torch.float16, device="cuda")
    q_rot = torch.full_like(out, float("nan"))
    foundry.paged_decode_kv8(plan, desc, dev(case.q), out, n_heads=case.Hq, k=dev(case.k), v=dev(case.v), cos=dev(case.cos),
                             sin=dev(case.sin), rope=True, rope_mode=rope_mode, append=True, q_rot=q_rot, scale=float(case.scale))
    foundry.synchronize()
    plan.close()
    assert np.array_equal(host(q_rot), q_ref)
    # the appended rows, bit-exact, and nothing else touched (NaN != NaN: compare the bit patterns of the scales)
    assert np.array_equal(d_k8.cpu().numpy(), k8_ref) and np.array_equal(d_v8.cpu().numpy(), v8_ref)
    assert np.array_equal(d_ks.cpu().numpy().view(np.uint32), ks_ref.view(np.uint32))
    assert np.array_equal(d_vs.cpu().numpy().view(np.uint32), vs_ref.view(np.uint32))
    assert max_abs(host(out), out_ref) <= TOL
    assert max_abs(host(out), gold.ravel()) <= TOL


@pytest.mark.parametrize("cached", [[4999], [1500, 520, 4000], [4159]])  # 4159: two CTAs of the last cluster get no tile
def test_8bit_decode_on_a_plan_in_the_cluster_form(mfk, foundry, cached):
    """A plan made under the library's own CTA count for a short launch is in the cluster form (one range of a unit per
    cluster); the 8-bit kernel has no cluster form and runs every range as one CTA's item: same answer."""
    import torch

    case = PagedCase(batch=len(cached), n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=cached, poison=False)
    k8, v8, ks, vs = quantised_pools(case)
    q_ref, k8_ref, v8_ref, ks_ref, vs_ref, out_ref, gold = oracle_step(case, k8, v8, ks, vs)
    pools = [torch.from_numpy(x).cuda() for x in (k8, v8, ks, vs)]
    pt, lens = dev_u32(case.page_table), dev_u32(case.kv_lens)
    desc = mfk.paged_kv8(*pools, pt, lens, n_kv_heads=case.Hkv, page_size=case.P)
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P)
    assert plan.cluster > 1
    out = torch.full((case.B, case.Hq * case.D), float("nan"), dtype=torch.float16, device="cuda")
    foundry.paged_decode_kv8(plan, desc, dev(case.q), out, n_heads=case.Hq, k=dev(case.k), v=dev(case.v), cos=dev(case.cos),
                             sin=dev(case.sin), rope=True, rope_mode=case.rope_mode, append=True, scale=float(case.scale))
    foundry.synchronize()
    plan.close()
    assert np.array_equal(pools[0].cpu().numpy(), k8_ref) and np.array_equal(pools[1].cpu().numpy(), v8_ref)
    assert max_abs(host(out), out_ref) <= TOL and max_abs(host(out), gold.ravel()) <= TOL


@pytest.mark.parametrize("append_in_shard", [False, True])
@pytest.mark.parametrize("max_ctas", [296, 5, 0])
def test_8bit_partials_and_merge_equal_full_decode(mfk, foundry, append_in_shard, max_ctas):
    """Sequence-sharded decode over the 8-bit cache on one GPU: two shards of one long sequence emit (acc, m, l)
    with mf_paged_decode_kv8_partial, mf_merge_partials over them equals the oracle's unsharded result.  With
    append_in_shard the last shard ropes q and k and appends the new row itself (positions from rope_positions);
    the other shard gets the rotated q, as a rank without the token's keys would."""
    import torch

    Hq, Hkv, D, P, L = 24, 8, 128, 64, 2048 + 17
    case = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False, rope_mode=1)
    k8, v8, ks, vs = quantised_pools(case)
    q_ref, k8_ref, v8_ref, ks_ref, vs_ref, out_ref, gold = oracle_step(case, k8, v8, ks, vs)
    start = (k8, v8, ks, vs) if append_in_shard else (k8_ref, v8_ref, ks_ref, vs_ref)
    d_k8, d_v8, d_ks, d_vs = (torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in start)
    n_pages = case.page_table.shape[1]
    cut = n_pages // 2
    pos = dev_u32(np.array([L - 1], np.uint32))
    accs, ms, ls = [], [], []
    keep = []
    for (p0, p1) in [(0, cut), (cut, n_pages)]:
        pt = np.ascontiguousarray(case.page_table[:, p0:p1])
        lens = np.array([min(L, p1 * P) - p0 * P], np.uint32)
        d_pt, d_len = dev_u32(pt), dev_u32(lens)
        keep += [d_pt, d_len]
        desc = mfk.paged_kv8(d_k8, d_v8, d_ks, d_vs, d_pt, d_len, n_kv_heads=Hkv, page_size=P)
        plan = foundry.decode_plan(lens, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P,
                                   max_ctas=max_ctas)
        acc = torch.zeros((1, Hq, D), dtype=torch.float32, device="cuda")
        m = torch.full((1, Hq), -1e30, dtype=torch.float32, device="cuda")
        l = torch.zeros((1, Hq), dtype=torch.float32, device="cuda")
        if append_in_shard and p1 == n_pages:
            foundry.paged_decode_kv8_partial(plan, desc, dev(case.q), pos, acc, m, l, n_heads=Hq, k=dev(case.k), v=dev(case.v),
                                             cos=dev(case.cos), sin=dev(case.sin), rope=True, rope_mode=1, append=True,
                                             scale=float(case.scale))
        else:
            foundry.paged_decode_kv8_partial(plan, desc, dev(q_ref), pos, acc, m, l, n_heads=Hq, scale=float(case.scale))
        foundry.synchronize()
        plan.close()
        accs.append(acc.view(Hq, D))
        ms.append(m.view(Hq))
        ls.append(l.view(Hq))
    acc, m, l = torch.stack(accs).contiguous(), torch.stack(ms).contiguous(), torch.stack(ls).contiguous()
    out = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
    foundry.merge_partials(acc, m, l, out)
    foundry.synchronize()
    assert max_abs(host(out), out_ref) <= TOL
    assert max_abs(host(out), gold.ravel()) <= TOL
    if append_in_shard:  # the shard that owns the token wrote the same bytes and scales as the oracle's append
        assert np.array_equal(d_k8.cpu().numpy(), k8_ref) and np.array_equal(d_v8.cpu().numpy(), v8_ref)
        assert np.array_equal(d_ks.cpu().numpy().view(np.uint32), ks_ref.view(np.uint32))
        assert np.array_equal(d_vs.cpu().numpy().view(np.uint32), vs_ref.view(np.uint32))


def _kv8_shards(mfk, foundry, case, pools, L, cuts, max_ctas=296):
    """Shard descriptors over one set of 8-bit pools: [(desc, plan, keep-alive)] for the page ranges in `cuts`."""
    out = []
    for (p0, p1) in cuts:
        pt = np.ascontiguousarray(case.page_table[:, p0:p1])
        lens = np.array([max(0, min(L, p1 * case.P) - p0 * case.P)], np.uint32)
        d_pt, d_len = dev_u32(pt), dev_u32(lens)
        desc = mfk.paged_kv8(*pools, d_pt, d_len, n_kv_heads=case.Hkv, page_size=case.P)
        plan = foundry.decode_plan(lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P, max_ctas=max_ctas)
        out.append((desc, plan, (d_pt, d_len)))
    return out


@pytest.mark.parametrize("max_ctas", [296, 0])  # 0: the library's own count, which gives these shards the cluster form
def test_8bit_pushed_partials_two_shards_one_gpu(mfk, foundry, max_ctas):
    """The kernels' own exchange over the 8-bit cache, both shards on one GPU: two-launch form (both shards push,
    then each "rank" merges) against mf_paged_decode_kv8_partial + mf_merge_partials bit for bit and against the
    oracle's unsharded result; the one-launch form with a single pusher (a second rank's kernel could not run
    beside it on this one GPU) gives that shard's own normalised partial."""
    import torch

    Hq, Hkv, D, P, L = 24, 8, 128, 64, 2048 + 17
    case = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False, rope_mode=1)
    k8, v8, ks, vs = quantised_pools(case)
    q_ref, k8_ref, v8_ref, ks_ref, vs_ref, out_ref, gold = oracle_step(case, k8, v8, ks, vs)
    pools = [torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (k8_ref, v8_ref, ks_ref, vs_ref)]
    n_pages = case.page_table.shape[1]
    cut = n_pages // 3
    parts = _kv8_shards(mfk, foundry, case, pools, L, [(0, cut), (cut, n_pages)], max_ctas=max_ctas)
    assert all((plan.cluster > 1) == (max_ctas == 0) for (_, plan, _) in parts)
    q_rot = dev(q_ref)
    pxs = [foundry.peer_exchange_create(2, r, Hq, D)[0] for r in range(2)]
    for r in range(2):  # same process: the "peer" buffers are plain local pointers
        o = 1 - r
        pxs[r].recv[o], pxs[r].counters[o] = pxs[o].recv[o], pxs[o].counters[o]
    accs = torch.zeros((2, Hq, D), dtype=torch.float32, device="cuda")
    ms = torch.full((2, Hq), -1e30, dtype=torch.float32, device="cuda")
    ls = torch.zeros((2, Hq), dtype=torch.float32, device="cuda")
    for r, (desc, plan, _) in enumerate(parts):
        foundry.paged_decode_kv8_partial(plan, desc, q_rot, None, accs[r:r + 1], ms[r:r + 1], ls[r:r + 1], n_heads=Hq,
                                         scale=float(case.scale))
    want = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
    foundry.merge_partials(accs, ms, ls, want)
    foundry.synchronize()
    assert max_abs(host(want), out_ref) <= TOL and max_abs(host(want), gold.ravel()) <= TOL
    for step in range(3):
        outs = [torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
        for r, (desc, plan, _) in enumerate(parts):
            foundry.paged_decode_kv8_partial_push(plan, desc, q_rot, pxs[r], step, n_heads=Hq, scale=float(case.scale))
        for r in range(2):
            foundry.merge_pushed(pxs[r], [Hkv, Hkv], step, Hq, D, outs[r])
        foundry.synchronize()
        for o in outs:
            assert np.array_equal(host(o), host(want))
    for r, (desc, plan, _) in enumerate(parts):
        solo = torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda")
        foundry.paged_decode_kv8_push_merge(plan, desc, q_rot, solo, pxs[r], 3, 1 << r, n_heads=Hq, scale=float(case.scale))
        foundry.synchronize()
        one = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
        foundry.merge_partials(accs[r:r + 1], ms[r:r + 1], ls[r:r + 1], one)
        foundry.synchronize()
        assert np.array_equal(host(solo), host(one))
    for (_, plan, _) in parts:
        plan.close()
    for r in range(2):  # borrowed pointers are not this exchange's to release
        o = 1 - r
        pxs[r].recv[o] = pxs[r].counters[o] = None
        foundry.peer_exchange_destroy(pxs[r])


def _kv8_two_gpu_worker(rank, world, port, ret, max_ctas):
    import importlib
    import os
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    sys.path.insert(0, str(root / "tests"))
    import torch
    import torch.distributed as dist

    mfk = importlib.import_module("test-burn_b200")
    sharding = importlib.import_module("test-burn_b200.sharding")
    dist.init_process_group("gloo", init_method="file://" + port, rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    try:
        Hq, Hkv, D, P, L = 24, 8, 128, 64, 6000
        case = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False, rope_mode=1)
        k8, v8, ks, vs = quantised_pools(case)
        q_ref, k8_ref, v8_ref, ks_ref, vs_ref, out_ref, gold = oracle_step(case, k8, v8, ks, vs)
        f = mfk.Foundry(rank)
        pools = [torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (k8_ref, v8_ref, ks_ref, vs_ref)]
        n_pages = case.page_table.shape[1]
        b, e = sharding.shard_pages(n_pages, world, rank)
        (desc, plan, keep), = _kv8_shards(mfk, f, case, pools, L, [(b, e)], max_ctas=max_ctas)
        px, handle = f.peer_exchange_create(world, rank, Hq, D)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        for r in range(world):
            if r != rank:
                f.peer_exchange_attach(px, r, handles[r])
        ok = True
        q_rot = dev(q_ref)
        for step in range(6):
            f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, step // 3)
            f.set_option(mfk.OPTION_PUSH_TAGGED, 1 if step < 4 else 0)  # steps 1, 3: tagged words; step 5: counters
            out = torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda")
            if step % 2 == 0:  # two launches: push, then the waiting merge kernel
                f.paged_decode_kv8_partial_push(plan, desc, q_rot, px, step, n_heads=Hq, scale=float(case.scale))
                f.merge_pushed(px, [Hkv] * world, step, Hq, D, out)
            else:              # one launch: the decode kernel also waits for the peers and merges
                f.paged_decode_kv8_push_merge(plan, desc, q_rot, out, px, step, (1 << world) - 1, n_heads=Hq,
                                              scale=float(case.scale))
            f.synchronize()
            ok = ok and max_abs(host(out), out_ref) <= TOL and max_abs(host(out), gold.ravel()) <= TOL
        plan.close()
        dist.barrier()  # nobody unmaps while a peer may still store
        f.peer_exchange_destroy(px)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("max_ctas", [296, 0])  # 0: the cluster form
def test_8bit_pushed_partials_two_gpus(max_ctas):
    """One process per GPU: the 8-bit decode kernels exchange their partials over NVLink, two-launch and fused forms,
    tagged words and counters, against the oracle's unsharded result."""
    import os
    import tempfile

    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, os.path.join(tempfile.mkdtemp(prefix="mf_rdzv_"), "store")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_kv8_two_gpu_worker, args=(world, port, ret, max_ctas), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_8bit_append_kernel_and_gather(mfk, foundry):
    """The standalone quantising append (one token per sequence, and a chunk of rows of one sequence) against
    the oracle's quantiser, bit for bit; the dequantising gather against e4m3 * scale rounded to f16."""
    import torch

    case = PagedCase(batch=3, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[100, 31, 700], poison=False)
    k8, v8, ks, vs = quantised_pools(case)
    q_ref, k8_ref, v8_ref, ks_ref, vs_ref, _, _ = oracle_step(case, k8, v8, ks, vs)
    d = [torch.from_numpy(x).cuda() for x in (k8, v8, ks, vs)]
    pt, lens = dev_u32(case.page_table), dev_u32(case.kv_lens)
    desc = mfk.paged_kv8(*d, pt, lens, n_kv_heads=case.Hkv, page_size=case.P)
    q_rot = torch.zeros((case.B, case.Hq * case.D), dtype=torch.float16, device="cuda")
    for rope_mode in (0,):
        foundry.paged_kv8_append(desc, dev(case.q), dev(case.k), dev(case.v), q_rot, dev(case.cos), dev(case.sin), n_heads=case.Hq,
                                 rope_mode=rope_mode)
    foundry.synchronize()
    assert np.array_equal(host(q_rot), q_ref)
    assert np.array_equal(d[0].cpu().numpy(), k8_ref) and np.array_equal(d[1].cpu().numpy(), v8_ref)
    assert np.array_equal(d[2].cpu().numpy(), ks_ref) and np.array_equal(d[3].cpu().numpy(), vs_ref)
    # gather: the dequantised rows of sequence 2
    n = int(case.kv_lens[2])
    got = torch.zeros((case.Hkv, n, case.D), dtype=torch.float16, device="cuda")
    foundry.paged_kv8_gather(desc, False, 2, n, got)
    foundry.synchronize()
    L = oracle.lib()
    lut = np.array([L.mfo_e4m3_to_f32(b) for b in range(256)], np.float32)
    want = np.zeros((case.Hkv, n, case.D), np.float16)
    for t in range(n):
        page = case.page_table[2, t // case.P]
        for h in range(case.Hkv):
            want[h, t] = (lut[k8_ref[page, h, t % case.P]] * ks_ref[page, h, t % case.P]).astype(np.float16)
    assert np.array_equal(host(got), want.view(np.uint16))
    foundry.paged_kv8_gather(desc, True, 2, n, got)  # V: out of its dim-major blocks
    foundry.synchronize()
    v_rows = mfk.kv8_v_rows_from_pool(v8_ref)
    for t in range(n):
        page = case.page_table[2, t // case.P]
        for h in range(case.Hkv):
            want[h, t] = (lut[v_rows[page, h, t % case.P]] * vs_ref[page, h, t % case.P]).astype(np.float16)
    assert np.array_equal(host(got), want.view(np.uint16))
    # a chunk of 40 rows of sequence 1 at position 32 (a prefill chunk), both RoPE modes
    for rope_mode in (0, 1):
        chunk = PagedCase(batch=2, n_heads=8, n_kv_heads=2, head_dim=128, page_size=16, cached=[10, 71], poison=False,
                          rope_mode=rope_mode)
        m, off = 40, 32
        from kvcases import normal
        qc = normal(901, m * 8 * 128).reshape(m, -1)
        kc = normal(902, m * 2 * 128).reshape(m, -1)
        vc = normal(903, m * 2 * 128).reshape(m, -1)
        c8 = [np.zeros((chunk.n_pages, 2, 16, 128), np.uint8), np.zeros((chunk.n_pages, 2, 16, 128), np.uint8),
              np.zeros((chunk.n_pages, 2, 16), np.float32), np.zeros((chunk.n_pages, 2, 16), np.float32)]
        ref = [x.copy() for x in c8]
        q_rows = np.zeros((m, 8 * 128), np.uint16)
        # the oracle appends one token per "sequence": call it row by row for sequence 1
        for s in range(m):
            table = np.ascontiguousarray(chunk.page_table[1:2])
            one_q = np.zeros((1, 8 * 128), np.uint16)
            L.mfo_paged_kv8_append(qc[s:s + 1].copy(), kc[s:s + 1].copy(), vc[s:s + 1].copy(), one_q, ref[0].reshape(-1),
                                   ref[1].reshape(-1), ref[2].reshape(-1), ref[3].reshape(-1), chunk.cos, chunk.sin, table,
                                   chunk.pt_stride, np.array([off + s], np.uint32), 1, 8, 2, 128, 16, rope_mode, 1)
            q_rows[s] = one_q[0]
        dd = [torch.from_numpy(x).cuda() for x in c8]
        desc2 = mfk.paged_kv8(*dd, dev_u32(chunk.page_table), dev_u32(chunk.kv_lens), n_kv_heads=2, page_size=16)
        q_rot2 = torch.zeros((8, m, 128), dtype=torch.float16, device="cuda")
        foundry.paged_kv8_append(desc2, dev(qc), dev(kc), dev(vc), q_rot2, dev(chunk.cos), dev(chunk.sin), n_heads=8,
                                 rope_mode=rope_mode, seq=1, position_offset=off, seq_len=m)
        foundry.synchronize()
        for got8, want8 in zip(dd, ref):
            assert np.array_equal(got8.cpu().numpy(), want8)
        assert np.array_equal(host(q_rot2), q_rows.reshape(m, 8, 128).transpose(1, 0, 2))


@pytest.mark.parametrize("shape", [(8, 2, 16, 100, 40), (24, 8, 64, 512, 256), (16, 2, 32, 0, 130)])
def test_chunked_prefill_over_the_8bit_cache(mfk, foundry, shape):
    """A prefill chunk on the 8-bit cache: mf_paged_kv8_append of the chunk's rows, then mf_paged_prefill_kv8 =
    causal attention of the chunk's queries over the dequantised rows.  Checked against the oracle's f32 causal
    prefill and fp64 gold over the SAME dequantised cache (e4m3 * scale rounded to f16, the oracle's table)."""
    import torch

    from kvcases import normal

    hq, hkv, P, cached, m = shape
    d, L = 128, cached + m
    n_seq_pages = (L + P - 1) // P
    n_pages = n_seq_pages + 3
    rng = np.random.default_rng(cached * 7 + m)
    pages = rng.permutation(n_pages)[:n_seq_pages].astype(np.uint32)
    table = np.full((2, n_seq_pages), 0x7FFFFFF0, np.uint32)
    table[1] = pages
    lens = np.array([1, L], np.uint32)
    d_table, d_lens = dev_u32(table), dev_u32(lens)
    pools = [torch.zeros((n_pages, hkv, P, d), dtype=torch.uint8, device="cuda"), torch.zeros((n_pages, hkv, P, d), dtype=torch.uint8, device="cuda"),
             torch.full((n_pages, hkv, P), float("nan"), dtype=torch.float32, device="cuda"),
             torch.full((n_pages, hkv, P), float("nan"), dtype=torch.float32, device="cuda")]
    desc = mfk.paged_kv8(*pools, d_table, d_lens, n_kv_heads=hkv, page_size=P)
    cos, sin = oracle.rope_tables(1e6, d, L)
    # the cached rows arrive the way a model would have written them: earlier chunks through the same append
    q_rot = None
    for (off, rows, seed) in ([(0, cached, 50)] if cached else []) + [(cached, m, 60)]:
        qc, kc, vc = (normal(seed + i, rows * h * d).reshape(rows, h * d) for i, h in enumerate((hq, hkv, hkv)))
        q_rot = torch.full((hq, rows, d), float("nan"), dtype=torch.float16, device="cuda")
        foundry.paged_kv8_append(desc, dev(qc), dev(kc), dev(vc), q_rot, dev(cos), dev(sin), n_heads=hq, rope_mode=0, seq=1,
                                 position_offset=off, seq_len=rows)
    ws = torch.empty(mfk.paged_prefill_kv8_workspace_bytes(desc, L), dtype=torch.uint8, device="cuda")
    out = torch.full((m, hq * d), float("nan"), dtype=torch.float16, device="cuda")
    scale = np.float32(1.0) / np.sqrt(np.float32(d))
    foundry.paged_prefill_kv8(desc, q_rot, out, ws, seq=1, q_len=m, kv_len=L, query_offset=cached, n_heads=hq, scale=float(scale))
    foundry.synchronize()
    # the dequantised cache, restated on the host from the pool bytes and scales the append left
    lut = np.array([oracle.lib().mfo_e4m3_to_f32(b) for b in range(256)], np.float32)
    k8, ks, vs = pools[0].cpu().numpy(), pools[2].cpu().numpy(), pools[3].cpu().numpy()
    v_rows = mfk.kv8_v_rows_from_pool(pools[1].cpu().numpy())
    kc_f, vc_f = np.zeros((hkv, L, d), np.float16), np.zeros((hkv, L, d), np.float16)
    for t in range(L):
        pg, r = pages[t // P], t % P
        kc_f[:, t] = (lut[k8[pg, :, r]] * ks[pg, :, r, None]).astype(np.float16)
        vc_f[:, t] = (lut[v_rows[pg, :, r]] * vs[pg, :, r, None]).astype(np.float16)
    args = dict(n_heads=hq, cache_heads=hkv, head_dim=d, capacity=L, q_len=m, kv_len=L, query_offset=cached, scale=scale)
    q_host = host(q_rot).ravel()
    want = oracle.prefill_causal(q_host, kc_f.view(np.uint16).ravel(), vc_f.view(np.uint16).ravel(), **args)
    gold = oracle.prefill_gold(q_host, kc_f.view(np.uint16).ravel(), vc_f.view(np.uint16).ravel(), **args)
    assert max_abs(host(out), want) <= TOL
    assert max_abs(host(out), gold) <= TOL
    with pytest.raises(mfk.MetalError) as e:  # a workspace that is too small is refused, nothing is allocated behind the caller
        foundry.paged_prefill_kv8(desc, q_rot, out, ws[:256], seq=1, q_len=m, kv_len=L, query_offset=cached, n_heads=hq)
    assert e.value.kind == "InvalidOperation"


def test_cost_of_the_8bit_format(mfk, foundry):
    """The same step on the f16 cache and on its 8-bit quantisation: the difference is the format's cost."""
    import torch

    case = PagedCase(batch=4, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16, cached=[4095, 800, 12000, 300], poison=False)
    ref16 = case.oracle_step()
    k8, v8, ks, vs = quantised_pools(case)
    d = [torch.from_numpy(x).cuda() for x in (k8, v8, ks, vs)]
    desc = mfk.paged_kv8(*d, dev_u32(case.page_table), dev_u32(case.kv_lens), n_kv_heads=case.Hkv, page_size=case.P)
    plan = foundry.decode_plan(case.kv_lens, n_heads=case.Hq, n_kv_heads=case.Hkv, head_dim=case.D, page_size=case.P, max_ctas=296)
    out = torch.zeros((case.B, case.Hq * case.D), dtype=torch.float16, device="cuda")
    foundry.paged_decode_kv8(plan, desc, dev(case.q), out, n_heads=case.Hq, k=dev(case.k), v=dev(case.v), cos=dev(case.cos),
                             sin=dev(case.sin), rope=True, rope_mode=0, append=True, scale=float(case.scale))
    foundry.synchronize()
    plan.close()
    err = max_abs(host(out), ref16[4].ravel())  # against the fp64 gold over the UNquantised cache
    assert err <= FORMAT_TOL, err


def test_8bit_cache_refuses_what_it_does_not_support(mfk, foundry):
    import torch

    z8 = torch.zeros((4, 2, 16, 128), dtype=torch.uint8, device="cuda")
    zs = torch.zeros((4, 2, 16), dtype=torch.float32, device="cuda")
    pt, lens = dev_u32(np.zeros((1, 4), np.uint32)), dev_u32(np.array([5], np.uint32))
    desc = mfk.paged_kv8(z8, z8, zs, zs, pt, lens, n_kv_heads=2, page_size=16)
    desc.head_dim = 64
    q = torch.zeros((1, 16 * 64), dtype=torch.float16, device="cuda")
    with pytest.raises(mfk.MetalError) as e:
        foundry.paged_kv8_gather(desc, False, 0, 5, q)
    assert e.value.kind == "OperationNotSupported"
    desc.head_dim = 128
    desc.page_size = 8  # V lies in blocks of 16 keys: pages of 16, 32 or 64 rows
    with pytest.raises(mfk.MetalError) as e:
        foundry.paged_kv8_gather(desc, False, 0, 5, q)
    assert e.value.kind == "OperationNotSupported"
    foundry.synchronize()
