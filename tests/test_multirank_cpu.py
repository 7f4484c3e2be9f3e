"""World-size-2 tests of the multi-GPU host logic on CPU (gloo), with the oracle standing in for
the kernels: sequence sharding needs no collective; page sharding of one long sequence needs one
all-gather of (acc, m, l) followed by the merge; KV-head sharding of a batch-1 step or a prefill chunk
needs none (each rank appends to and attends over the caches of its own heads)."""
import importlib
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist

    import oracle
    from kvcases import PagedCase

    sharding = importlib.import_module("test-burn_b200.sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if mode == "sequences":
            case = PagedCase(batch=7, n_heads=16, n_kv_heads=2, head_dim=128, page_size=16,
                             cached=[511, 30, 2049, 3, 700, 64, 1500])
            full = case.oracle_step()[3]
            mine = sharding.shard_sequences(case.kv_lens, world, rank)
            sub = PagedCase(batch=len(mine), n_heads=16, n_kv_heads=2, head_dim=128, page_size=16,
                            cached=case.cached[mine])
            # same data as the owning sequences of the full batch
            sub.q, sub.k, sub.v = case.q[mine], case.k[mine], case.v[mine]
            sub.cos, sub.sin = case.cos, case.sin
            sub.page_table = case.page_table[mine]
            sub.pt_stride = case.pt_stride
            sub.k_pool, sub.v_pool = case.k_pool, case.v_pool
            out = sub.oracle_step()[3]
            outs = [None] * world
            dist.all_gather_object(outs, (mine.tolist(), out))  # verification only, not the data path
            merged = np.zeros_like(full)
            seen = []
            for idx, o in outs:
                merged[idx] = o
                seen += idx
            ret[rank] = bool(sorted(seen) == list(range(7)) and np.array_equal(merged, full))
        elif mode == "kv_heads":
            from kvcases import ContigCase

            Hq, Hkv, D, G = 24, 8, 64, 3
            full = ContigCase(n_heads=Hq, n_kv_heads=Hkv, head_dim=D, cached=37, m=5, capacity=48, rope_mode=1)
            q_all, k_all, v_all = full.oracle_append()
            want = oracle.prefill_causal(q_all, k_all.ravel(), v_all.ravel(), n_heads=Hq, cache_heads=Hkv, head_dim=D,
                                         capacity=48, q_len=5, kv_len=42, query_offset=37, scale=full.scale)
            h0, h1 = sharding.shard_kv_heads(Hkv, world, rank)
            sub = ContigCase(n_heads=(h1 - h0) * G, n_kv_heads=h1 - h0, head_dim=D, cached=37, m=5, capacity=48, rope_mode=1)
            # this rank's columns of q / k / v and its heads of the caches
            sub.q = np.ascontiguousarray(full.q.reshape(5, Hq, D)[:, h0 * G:h1 * G]).reshape(5, -1)
            sub.k = np.ascontiguousarray(full.k.reshape(5, Hkv, D)[:, h0:h1]).reshape(5, -1)
            sub.v = np.ascontiguousarray(full.v.reshape(5, Hkv, D)[:, h0:h1]).reshape(5, -1)
            sub.k_cache, sub.v_cache = full.k_cache[h0:h1].copy(), full.v_cache[h0:h1].copy()
            q_rot, kc, vc = sub.oracle_append()
            out = oracle.prefill_causal(q_rot, kc.ravel(), vc.ravel(), n_heads=(h1 - h0) * G, cache_heads=h1 - h0,
                                        head_dim=D, capacity=48, q_len=5, kv_len=42, query_offset=37, scale=full.scale)
            same_cache = np.array_equal(kc, k_all.reshape(Hkv, 48, D)[h0:h1]) and np.array_equal(vc, v_all.reshape(Hkv, 48, D)[h0:h1])
            outs = [None] * world
            dist.all_gather_object(outs, ((h0, h1), out.reshape(5, -1, D)))  # verification only, not the data path
            merged = np.concatenate([o for _, o in sorted(outs, key=lambda t: t[0][0])], axis=1)
            cover = sorted(r for r, _ in outs)
            ret[rank] = bool(same_cache and cover[0][0] == 0 and cover[-1][1] == Hkv and
                             np.array_equal(merged.reshape(5, Hq * D), want.reshape(5, Hq * D)))
        else:
            Hq, Hkv, D, P, L = 24, 8, 128, 64, 1000
            case = PagedCase(batch=1, n_heads=Hq, n_kv_heads=Hkv, head_dim=D, page_size=P, cached=[L - 1])
            q_rot, kp, vp, full, _ = case.oracle_step()
            n_pages = case.page_table.shape[1]
            b, e = sharding.shard_pages(n_pages, world, rank)
            n_local = sharding.shard_local_len(L, P, b, e)
            kc = np.empty((Hkv, L, D), np.uint16)
            vc = np.empty((Hkv, L, D), np.uint16)
            oracle.lib().mfo_paged_gather(kp, case.page_table[0], L, Hkv, P, D, kc)
            oracle.lib().mfo_paged_gather(vp, case.page_table[0], L, Hkv, P, D, vc)
            lo = min(L, b * P)
            _, acc, m, l = oracle.decode_online(q_rot[0], kc, vc, n_heads=Hq, cache_heads=Hkv, head_dim=D, capacity=L,
                                                key_begin=lo, kv_len=lo + n_local, scale=case.scale, partials=True)
            mine = sharding.pack_partials(torch.from_numpy(acc), torch.from_numpy(m), torch.from_numpy(l))
            gathered = torch.empty((world * Hq, D + 2), dtype=torch.float32)
            dist.all_gather_into_tensor(gathered, mine)
            a, mm, ll = sharding.unpack_partials(gathered.view(world, Hq, D + 2))
            merged = oracle.merge_partials(a.numpy(), mm.numpy(), ll.numpy())
            diff = np.abs(oracle.h2f(merged.ravel()) - oracle.h2f(full.ravel())).max()
            owner = sharding.tail_owner(L, P, n_pages, world)
            ret[rank] = bool(diff <= 1e-3 and owner == world - 1)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["sequences", "pages", "kv_heads"])
def test_two_ranks_gloo(mode):
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, mode, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_sequence_sharding_is_a_balanced_partition():
    sharding = importlib.import_module("test-burn_b200.sharding")
    rng = np.random.default_rng(3)
    lens = rng.integers(512, 16385, size=64)
    for world in (1, 2, 4, 8):
        parts = [sharding.shard_sequences(lens, world, r) for r in range(world)]
        assert sorted(np.concatenate(parts).tolist()) == list(range(64))
        totals = [int(lens[p].sum()) for p in parts]
        assert max(totals) - min(totals) <= 16384
    for world in (1, 2, 3, 4, 8, 16):
        heads = [sharding.shard_kv_heads(8, world, r) for r in range(world)]
        assert heads[0][0] == 0 and heads[-1][1] == 8
        assert all(heads[i][1] == heads[i + 1][0] for i in range(world - 1))
        assert max(e - b for b, e in heads) - min(e - b for b, e in heads) <= 1
    for world in (2, 4, 8):
        cover = [sharding.shard_pages(2048, world, r) for r in range(world)]
        assert cover[0][0] == 0 and cover[-1][1] == 2048
        assert all(cover[i][1] == cover[i + 1][0] for i in range(world - 1))
        assert sum(sharding.shard_local_len(131072, 64, b, e) for b, e in cover) == 131072
