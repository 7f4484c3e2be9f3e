"""Host-side partitioning of the decode path over the GPUs of one box.

Nothing here exists in the reference (single Apple GPU).  Three splits:

* batched decode: sequences are independent, so each rank owns whole sequences (their pages,
  page-table rows and plan) and no data crosses GPUs during a step;
* one long sequence: its page list is cut into contiguous ranges, every rank attends over its own
  pages and emits unnormalised f32 partials (acc, m, l) per query head; one all-gather of
  Hq*(D+2) floats per rank per layer followed by the log-sum-exp merge gives every rank the result;
* one sequence of ordinary length (a batch-1 step, a prefill chunk): KV heads are independent, so each
  rank owns a contiguous range of KV heads with their query groups, caches of [its heads, capacity, D]
  and the matching columns of q / k / v / output; nothing crosses GPUs inside the attention path.
"""
from __future__ import annotations

import numpy as np


def shard_sequences(kv_lens, world: int, rank: int) -> np.ndarray:
    """Indices of the sequences rank `rank` owns: longest first, dealt out in a snake so that the
    per-rank token totals stay close."""
    lens = np.asarray(kv_lens)
    order = np.argsort(-lens.astype(np.int64), kind="stable")
    mine = []
    for i, idx in enumerate(order):
        rnd, pos = divmod(i, world)
        owner = pos if rnd % 2 == 0 else world - 1 - pos
        if owner == rank:
            mine.append(int(idx))
    return np.array(sorted(mine), dtype=np.int64)


def shard_kv_heads(n_kv_heads: int, world: int, rank: int):
    """KV-head range [begin, end) of `rank` (query heads [begin*G, end*G)); ranks past the head
    count get an empty range."""
    begin = rank * n_kv_heads // world
    end = (rank + 1) * n_kv_heads // world
    return begin, end


def shard_pages(n_pages: int, world: int, rank: int):
    """Contiguous page range [begin, end) of one long sequence owned by `rank`."""
    begin = rank * n_pages // world
    end = (rank + 1) * n_pages // world
    return begin, end


def shard_local_len(kv_len: int, page_size: int, begin: int, end: int) -> int:
    """Number of keys of the sequence that fall into pages [begin, end)."""
    lo = min(kv_len, begin * page_size)
    hi = min(kv_len, end * page_size)
    return hi - lo


def tail_owner(kv_len: int, page_size: int, n_pages: int, world: int) -> int:
    """Rank whose range holds the page of position kv_len-1 (it performs the append)."""
    page = (kv_len - 1) // page_size
    for r in range(world):
        b, e = shard_pages(n_pages, world, r)
        if b <= page < e:
            return r
    raise ValueError("position outside the page list")


def pack_partials(acc, m, l):
    """(acc [H, D], m [H], l [H]) -> one [H, D+2] buffer for a single all-gather."""
    import torch

    return torch.cat([acc, m.unsqueeze(-1), l.unsqueeze(-1)], dim=-1).contiguous()


def unpack_partials(buf):
    """[world, H, D+2] -> acc [world, H, D], m [world, H], l [world, H] (contiguous)."""
    return buf[..., :-2].contiguous(), buf[..., -2].contiguous(), buf[..., -1].contiguous()
