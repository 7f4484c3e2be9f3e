"""GPU parity: sequence-sharded decode whose exchange is done by the kernels themselves.

The decode kernel of each shard stores its (acc, m, l) into every rank's receive block and bumps an
arrival counter; the merge kernel waits for the counters and merges.  Cases:
  * two shards emulated on ONE GPU in one stream (every push precedes every merge in stream order,
    so no kernel ever waits on a later launch), three steps to cover both buffer parities;
  * a wait that nothing satisfies runs out and comes back as a Timeout status, context still usable;
  * two processes on two GPUs with buffers mapped through inter-process handles (skipped on one GPU).
"""
import importlib
import os
import sys
from pathlib import Path

import numpy as np
import pytest

import oracle
from kvcases import PagedCase, dev, dev_u32, host, max_abs

pytestmark = pytest.mark.gpu
TOL = 2e-3
ROOT = Path(__file__).resolve().parent.parent


def _shard_inputs(mfk, foundry, full, dk, dv, p0, p1, L):
    P = full.P
    pt = np.ascontiguousarray(full.page_table[:, p0:p1])
    lens = np.array([max(0, min(L, p1 * P) - p0 * P)], np.uint32)
    d_pt, d_len = dev_u32(pt), dev_u32(lens)
    desc = mfk.paged_kv(dk, dv, d_pt, d_len, n_kv_heads=full.Hkv, page_size=P, head_dim=full.D)
    plan = foundry.decode_plan(lens, n_heads=full.Hq, n_kv_heads=full.Hkv, head_dim=full.D, page_size=P)
    return desc, plan, (d_pt, d_len)


@pytest.mark.parametrize("overlap", [0, 1])
def test_pushed_partials_two_shards_one_gpu(mfk, foundry, overlap):
    import torch

    Hq, Hkv, D, P, L = 24, 8, 128, 64, 4096 + 17
    full = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False)
    q_ref, kp, vp, out_ref, gold = full.oracle_step()
    dk, dv, q_rot = dev(kp), dev(vp), dev(q_ref)
    n_pages = full.page_table.shape[1]
    cut = n_pages // 3
    shards = [(0, cut), (cut, n_pages)]
    pxs = [foundry.peer_exchange_create(2, r, Hq, D)[0] for r in range(2)]
    for r in range(2):  # same process: the "peer" buffers are plain local pointers
        o = 1 - r
        pxs[r].recv[o], pxs[r].counters[o] = pxs[o].recv[o], pxs[o].counters[o]
    parts = [_shard_inputs(mfk, foundry, full, dk, dv, p0, p1, L) for (p0, p1) in shards]
    # the library-collective path on the same shards, as the bits to match
    accs = torch.zeros((2, Hq, D), dtype=torch.float32, device="cuda")
    ms = torch.full((2, Hq), -1e30, dtype=torch.float32, device="cuda")
    ls = torch.zeros((2, Hq), dtype=torch.float32, device="cuda")
    for r, (desc, plan, _) in enumerate(parts):
        foundry.paged_decode_partial(plan, desc, q_rot, accs[r:r + 1], ms[r:r + 1], ls[r:r + 1], n_heads=Hq,
                                     scale=float(full.scale))
    want = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
    foundry.merge_partials(accs, ms, ls, want)
    foundry.synchronize()
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, overlap)  # programmatic dependent launches
    for step in range(3):
        outs = [torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
        for r, (desc, plan, _) in enumerate(parts):
            foundry.paged_decode_partial_push(plan, desc, q_rot, pxs[r], step, n_heads=Hq, scale=float(full.scale))
        for r in range(2):
            foundry.merge_pushed(pxs[r], [Hkv, Hkv], step, Hq, D, outs[r])
        foundry.synchronize()
        for o in outs:
            assert np.array_equal(host(o), host(want))
            assert max_abs(host(o), out_ref) <= TOL and max_abs(host(o), gold.ravel()) <= TOL
    # the one-launch form with a single pusher (a second rank's kernel could not run beside it on
    # this one GPU): pusher mask = this shard only, so the result is the shard's own normalised partial
    for r, (desc, plan, _) in enumerate(parts):
        solo = torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda")
        foundry.paged_decode_push_merge(plan, desc, q_rot, solo, pxs[r], 3, 1 << r, n_heads=Hq, scale=float(full.scale))
        foundry.synchronize()
        one = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
        foundry.merge_partials(accs[r:r + 1], ms[r:r + 1], ls[r:r + 1], one)
        foundry.synchronize()
        assert np.array_equal(host(solo), host(one))
    foundry.set_option(mfk.OPTION_OVERLAP_LAUNCHES, 0)
    for (_, plan, _) in parts:
        plan.close()
    for r in range(2):  # borrowed pointers are not this exchange's to release
        o = 1 - r
        pxs[r].recv[o] = pxs[r].counters[o] = None
        foundry.peer_exchange_destroy(pxs[r])


def test_merge_wait_runs_out_with_a_status(mfk, foundry):
    """Rank 1 never pushes: the merge kernel gives up after its limit, the status surfaces at
    synchronize as Timeout, and the context keeps working."""
    import torch

    Hq, D = 8, 128
    px, _ = foundry.peer_exchange_create(2, 0, Hq, D)
    silent, _ = foundry.peer_exchange_create(2, 1, Hq, D)
    px.recv[1], px.counters[1] = silent.recv[1], silent.counters[1]
    out = torch.zeros((Hq, D), dtype=torch.float16, device="cuda")
    foundry.merge_pushed(px, [0, 1], 0, Hq, D, out)
    with pytest.raises(mfk.MetalError) as e:
        foundry.synchronize()
    assert e.value.kind == "Timeout"
    assert not host(out).any()  # nothing was written
    foundry.merge_pushed(px, [0, 0], 0, Hq, D, out)  # nobody expected: merges nothing, at once
    foundry.synchronize()
    px.recv[1] = px.counters[1] = None
    foundry.peer_exchange_destroy(px)
    foundry.peer_exchange_destroy(silent)


def _two_gpu_worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist

    mfk = importlib.import_module("test-burn_b200")
    sharding = importlib.import_module("test-burn_b200.sharding")
    # host plumbing only; a file store: no port to collide with anything else on the box
    dist.init_process_group("gloo", init_method="file://" + port, rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    try:
        Hq, Hkv, D, P, L = 24, 8, 128, 64, 6000
        full = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False)
        q_ref, kp, vp, out_ref, gold = full.oracle_step()
        f = mfk.Foundry(rank)
        dk, dv, q_rot = dev(kp), dev(vp), dev(q_ref)
        n_pages = full.page_table.shape[1]
        b, e = sharding.shard_pages(n_pages, world, rank)
        desc, plan, keep = _shard_inputs(mfk, f, full, dk, dv, b, e, L)
        px, handle = f.peer_exchange_create(world, rank, Hq, D)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        for r in range(world):
            if r != rank:
                f.peer_exchange_attach(px, r, handles[r])
        ok = True
        for step in range(6):
            f.set_option(mfk.OPTION_OVERLAP_LAUNCHES, step // 3)
            f.set_option(mfk.OPTION_PUSH_TAGGED, 1 if step < 4 else 0)  # steps 1, 3: tagged words; step 5: counters
            out = torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda")
            if step % 2 == 0:  # two launches: push, then the waiting merge kernel
                f.paged_decode_partial_push(plan, desc, q_rot, px, step, n_heads=Hq, scale=float(full.scale))
                f.merge_pushed(px, [Hkv] * world, step, Hq, D, out)
            else:              # one launch: the decode kernel also waits for the peers and merges
                f.paged_decode_push_merge(plan, desc, q_rot, out, px, step, (1 << world) - 1, n_heads=Hq,
                                          scale=float(full.scale))
            f.synchronize()
            ok = ok and max_abs(host(out), out_ref) <= TOL and max_abs(host(out), gold.ravel()) <= TOL
        # the library-collective route on the same shards: partial blocks, ncclAllGather, merge
        lib = _nccl()
        if lib is not None:
            ids = [_nccl_comm(lib, -1, 0) if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            comm = _nccl_comm(lib, world, rank, ids[0])
            block = Hq * (D + 2)
            mine = torch.zeros(block, dtype=torch.float32, device="cuda")
            gathered = torch.zeros((world, block), dtype=torch.float32, device="cuda")
            out = torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda")
            f.paged_decode_partial(plan, desc, q_rot, mine[:Hq * D].view(1, Hq, D), mine[Hq * D:Hq * D + Hq], mine[Hq * D + Hq:],
                                   n_heads=Hq, scale=float(full.scale))
            f.allgather_merge(comm, mine, gathered, Hq, D, out)
            f.synchronize()
            ok = ok and max_abs(host(out), out_ref) <= TOL and max_abs(host(out), gold.ravel()) <= TOL
        plan.close()
        dist.barrier()  # nobody unmaps while a peer may still store
        f.peer_exchange_destroy(px)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_pushed_partials_two_gpus():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import tempfile

    world, port = 2, os.path.join(tempfile.mkdtemp(prefix="mf_rdzv_"), "store")
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_two_gpu_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_a_rank_that_only_merges_holds_the_pushers_back(mfk, foundry):
    """Rank 1 holds no keys: it never pushes, it only merges what rank 0 pushes to it.  Nothing in the
    pushers' own hand-shake waits for such a rank, so it is named in merge_only_mask: it counts the rows
    it has merged on the pusher's side, and the pusher's kernel of step s >= 2 waits for its merge of
    step s - 2 before overwriting that parity block.  Both ranks are emulated on one GPU in one stream,
    so the merging rank runs "on time" in the first part; in the second it skips a merge and the
    pusher's bounded wait runs out with a Timeout status instead of overwriting (or hanging)."""
    import torch

    Hq, Hkv, D, P, L = 24, 8, 128, 64, 1000
    full = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False)
    q_ref, kp, vp, out_ref, gold = full.oracle_step()
    dk, dv, q_rot = dev(kp), dev(vp), dev(q_ref)
    n_pages = full.page_table.shape[1]
    pxs = [foundry.peer_exchange_create(2, r, Hq, D)[0] for r in range(2)]
    for r in range(2):
        o = 1 - r
        pxs[r].recv[o], pxs[r].counters[o] = pxs[o].recv[o], pxs[o].counters[o]
        pxs[r].merge_only_mask = 0b10
    desc, plan, keep = _shard_inputs(mfk, foundry, full, dk, dv, 0, n_pages, L)
    units = [Hkv, 0]
    for step in range(5):
        outs = [torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
        foundry.paged_decode_partial_push(plan, desc, q_rot, pxs[0], step, n_heads=Hq, scale=float(full.scale))
        for r in range(2):
            foundry.merge_pushed(pxs[r], units, step, Hq, D, outs[r])
        foundry.synchronize()
        for o in outs:
            assert max_abs(host(o), out_ref) <= TOL and max_abs(host(o), gold.ravel()) <= TOL
    # the merging rank falls behind: steps 5 and 6 are pushed, rank 1 merges neither; the push of step 7
    # would overwrite the block of step 5 that rank 1 has not read yet
    for step in (5, 6, 7):
        foundry.paged_decode_partial_push(plan, desc, q_rot, pxs[0], step, n_heads=Hq, scale=float(full.scale))
        out0 = torch.zeros((Hq, D), dtype=torch.float16, device="cuda")
        foundry.merge_pushed(pxs[0], units, step, Hq, D, out0)
        if step < 7:
            foundry.synchronize()
    with pytest.raises(mfk.MetalError) as e:
        foundry.synchronize()
    assert e.value.kind == "Timeout"
    with pytest.raises(mfk.MetalError):  # a rank named as merge-only cannot push
        foundry.paged_decode_partial_push(plan, desc, q_rot, pxs[1], 8, n_heads=Hq, scale=float(full.scale))
    foundry.synchronize()
    plan.close()
    for r in range(2):
        o = 1 - r
        pxs[r].recv[o] = pxs[r].counters[o] = None
        foundry.peer_exchange_destroy(pxs[r])


def _nccl():
    """The NCCL library of this Python environment through ctypes (None if it cannot be found), loaded globally
    so that the product library's lookup of ncclAllGather finds the same instance."""
    import ctypes as C
    import glob

    try:
        import nvidia.nccl as pkg

        paths = glob.glob(os.path.join(list(pkg.__path__)[0], "lib", "libnccl.so*"))
    except Exception:
        paths = []
    for path in paths + ["libnccl.so.2"]:
        try:
            return C.CDLL(path, mode=C.RTLD_GLOBAL)
        except OSError:
            continue
    return None


def _nccl_comm(lib, world, rank, unique_id=None):
    import ctypes as C

    class UniqueId(C.Structure):
        _fields_ = [("internal", C.c_ubyte * 128)]

    uid = UniqueId()
    if unique_id is None:
        assert lib.ncclGetUniqueId(C.byref(uid)) == 0
    else:
        C.memmove(C.byref(uid), unique_id, 128)
    if world < 0:
        return C.string_at(C.byref(uid), 128)
    comm = C.c_void_p()
    lib.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
    assert lib.ncclCommInitRank(C.byref(comm), world, uid, rank) == 0
    return comm


def test_allgather_merge_route(mfk, foundry):
    """The library-collective route on one GPU: two shards' partial blocks, an all-gather and the merge.  The
    all-gather is (1) a test double installed with mf_context_set_allgather, which also lets the failure of
    the collective be produced on the host (an error code from the fake: NcclError, nothing written), and
    (2) the real ncclAllGather on a communicator of one rank."""
    import ctypes as C

    import torch

    Hq, Hkv, D, P, L = 24, 8, 128, 64, 3000
    full = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1], poison=False)
    q_ref, kp, vp, out_ref, gold = full.oracle_step()
    dk, dv, q_rot = dev(kp), dev(vp), dev(q_ref)
    n_pages = full.page_table.shape[1]
    cut = n_pages // 2
    block = Hq * (D + 2)
    blocks = torch.zeros((2, block), dtype=torch.float32, device="cuda")
    keep = []
    for r, (p0, p1) in enumerate([(0, cut), (cut, n_pages)]):
        desc, plan, k = _shard_inputs(mfk, foundry, full, dk, dv, p0, p1, L)
        keep.append((desc, plan, k))
        b = blocks[r]
        foundry.paged_decode_partial(plan, desc, q_rot, b[:Hq * D].view(1, Hq, D), b[Hq * D:Hq * D + Hq], b[Hq * D + Hq:],
                                     n_heads=Hq, scale=float(full.scale))
    foundry.synchronize()
    gathered = torch.zeros((2, block), dtype=torch.float32, device="cuda")
    out = torch.full((Hq, D), float("nan"), dtype=torch.float16, device="cuda")
    calls = []

    def fake(send, recv, count, comm, stream):
        calls.append((count, comm))
        assert send == blocks[0].data_ptr() and recv == gathered.data_ptr()
        gathered.copy_(blocks)  # what an all-gather over the two ranks delivers
        return 0

    cb = mfk.ALLGATHER_FN(fake)
    foundry.set_allgather(cb)
    foundry.allgather_merge(0x1234, blocks[0], gathered, Hq, D, out)
    foundry.synchronize()
    assert calls == [(block, 0x1234)]
    assert max_abs(host(out), out_ref) <= TOL and max_abs(host(out), gold.ravel()) <= TOL
    # the collective fails: the status names it, the output is not touched
    bad = mfk.ALLGATHER_FN(lambda send, recv, count, comm, stream: 5)
    foundry.set_allgather(bad)
    out.fill_(3.0)
    with pytest.raises(mfk.MetalError) as e:
        foundry.allgather_merge(0x1234, blocks[0], gathered, Hq, D, out)
    assert e.value.kind == "NcclError" and "code 5" in str(e.value)
    foundry.synchronize()
    assert bool((out == 3.0).all())
    foundry.set_allgather(None)
    # the real thing, one rank: gathering one block and merging it normalises that block
    lib = _nccl()
    if lib is not None:
        comm = _nccl_comm(lib, 1, 0)
        one = torch.zeros((1, block), dtype=torch.float32, device="cuda")
        foundry.allgather_merge(comm, blocks[1], one, Hq, D, out)
        foundry.synchronize()
        want = torch.empty((Hq, D), dtype=torch.float16, device="cuda")
        b = blocks[1]
        foundry.merge_partials(b[:Hq * D].view(1, Hq, D), b[Hq * D:Hq * D + Hq].view(1, Hq), b[Hq * D + Hq:].view(1, Hq), want)
        foundry.synchronize()
        assert torch.equal(one[0], blocks[1]) and np.array_equal(host(out), host(want))
        lib.ncclCommDestroy.argtypes = [C.c_void_p]
        lib.ncclCommDestroy(comm)
    for _, plan, _ in keep:
        plan.close()
